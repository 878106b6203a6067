"""Compile the reference's own native module `computation_ops` (x86 variant).

TEST INFRASTRUCTURE.  The sources are compiled from where they lie in the
reference checkout (nothing is copied); the only output is
`oracle/_ref/computation_ops.so`, which is git-ignored.  The flags are those of the
reference's self_benchmark/a64fx/model/ops/setup.py:12-23 (AVX-512 + OpenMP, -O3).
The reference's own build system (setuptools BuildExtension) is not run; this is the
equivalent single g++ command.

usage: python oracle/build_ref.py [reference_root]
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "computation_ops.so")


def cpu_has_avx512() -> bool:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    flags = line.split()
                    need = ("avx512f", "avx512cd", "avx512bw", "avx512dq", "avx512vl", "avx512ifma", "avx512vbmi")
                    return all(x in flags for x in need)
    except OSError:
        pass
    return False


def build(ref_root: str, force: bool = False) -> str:
    src_dir = os.path.join(ref_root, "self_benchmark", "a64fx", "model", "ops", "src")
    srcs = [os.path.join(src_dir, f) for f in ("utils.cpp", "spmm.cpp", "ops.cpp", "quantization_x86.cpp")]
    for s in srcs:
        if not os.path.isfile(s):
            raise FileNotFoundError(s)
    if os.path.isfile(OUT) and not force and all(os.path.getmtime(OUT) >= os.path.getmtime(s) for s in srcs):
        return OUT
    if not cpu_has_avx512():
        raise RuntimeError("host CPU lacks the AVX-512 subsets the reference's x86 build enables")
    import torch
    from torch.utils import cpp_extension

    os.makedirs(OUT_DIR, exist_ok=True)
    inc = cpp_extension.include_paths() + [sysconfig.get_paths()["include"], src_dir]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    isa = ["-mavx512f", "-mavx512cd", "-mavx512bw", "-mavx512dq", "-mavx512vl", "-mavx512ifma", "-mavx512vbmi"]
    cmd = (
        ["/usr/bin/g++", "-O3", "-fopenmp", "-std=c++17", "-fPIC", "-shared", "-w"]
        + isa
        + ["-DTORCH_EXTENSION_NAME=computation_ops", "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
        + ["-I" + p for p in inc]
        + srcs
        + ["-o", OUT, "-L" + torch_lib, "-Wl,-rpath," + torch_lib,
           "-ltorch_python", "-ltorch", "-ltorch_cpu", "-lc10"]
    )
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    roots = [a for a in sys.argv[1:] if not a.startswith("--")]
    root = roots[0] if roots else os.environ.get("GNNAGG_REFERENCE_ROOT")
    if not root:
        raise SystemExit("usage: python oracle/build_ref.py <reference_root> [--force]  (or set GNNAGG_REFERENCE_ROOT)")
    print(build(root, force="--force" in sys.argv))
