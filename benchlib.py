"""Pieces shared by the benchmark drivers beside this file (bench.py, bench_multi.py, bench_epoch.py):
workload constants, roofline arithmetic, the nvidia-smi clock sampler and the three-stream host pipeline."""
import hashlib
import json
import os
import statistics
import subprocess
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))

# the benchmark workload; bench.py --scale / --widths choose a smaller case for a profiler capture and
# are echoed into the line's `config`
WIDTHS = (32, 128, 256)
SEED = 20261127
SCALE = 22
EDGE_FACTOR = 16
FALLBACK_HBM_GBS = 6650.0


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def spmm_algorithmic_bytes(M, nnz, F, accumulate=False, rowptr_bytes=8):
    """nnz*(4 col + 4 val + 4F gathered row) + (M+1)*rowptr + M*F*4 written (+ read when accumulating):
    the no-reuse gather model (every nonzero fetches its feature row from memory)."""
    return nnz * (8 + 4 * F) + (M + 1) * rowptr_bytes + M * F * 4 * (2 if accumulate else 1)


def spmm_compulsory_bytes(M, K, nnz, F, accumulate=False, rowptr_bytes=8):
    """Lower bound: the index and value streams, every feature row of the operand once, the output once."""
    return nnz * 8 + (M + 1) * rowptr_bytes + K * F * 4 + M * F * 4 * (2 if accumulate else 1)


def spmm_kernel_source_hash():
    """Identifies the SpMM kernel a DRAM-traffic capture belongs to: sha256 over its source files."""
    h = hashlib.sha256()
    for name in ("spmm.cu", "common.cuh", "codec.cuh"):
        with open(os.path.join(ROOT, "gnn_benchmark_b200", "csrc", name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


# dram__bytes_read.sum + dram__bytes_write.sum of ONE spmm_chunk_kernel launch (ncu), keyed by R-MAT scale
# and feature width, with the hash of the kernel source the capture was taken on.  A bench run on other
# kernel source reports `traffic: null` instead of a stale figure.
SPMM_DRAM_TRAFFIC = {
    "kernel_source": "de8b10505576fb26",
    "bytes_per_launch": {(22, 256): 75588076032, (22, 128): 30243030144, (22, 32): 4875673984},
}


def spmm_dram_traffic(scale, F):
    if SPMM_DRAM_TRAFFIC["kernel_source"] != spmm_kernel_source_hash():
        return None
    return SPMM_DRAM_TRAFFIC["bytes_per_launch"].get((scale, F))


class ClockSampler:
    """nvidia-smi clocks / throttle reasons every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def __enter__(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.path is None or not os.path.isfile(self.path):
            return out
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in open(self.path):
            p = [x.strip() for x in line.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1]))
                mx.append(float(p[2]))
            except ValueError:
                continue
            for name, v in zip(names, p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            # samples under load: the upper half of the observed clocks
            out["sm_mhz"] = statistics.median(sorted(sm)[len(sm) // 2:])
            out["sm_max_mhz"] = max(mx)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


def workload_config(n_gpus, scale=SCALE, widths=WIDTHS, A=None):
    cfg = {
        "workload": f"spmm_rmat{scale}" if n_gpus == 1 else f"aggregate_rmat{scale}_per_gpu",
        "graph": f"R-MAT scale {scale}{'' if n_gpus == 1 else ' per GPU'}, edge factor {EDGE_FACTOR}, "
                 "(a,b,c,d)=(0.57,0.19,0.19,0.05), symmetrised, deduplicated, self-loops, GCN-normalised",
        "widths": list(widths),
        "calls_per_step": "forward A.X + transposed A^T.G per width",
        "index_types": "int64 rowptr, int32 col, fp32 val",
        "l2_policy": "inputs_larger_than_L2 (X is 0.5-4.3 GB, CSR 1.1 GB; nothing flushed between steps)",
    }
    if A is not None:
        cfg["rows"] = A.sparse_size(0)
        cfg["nnz"] = A.nnz()
    return cfg


class HostPipeline:
    """Three streams and two device buffer pairs so that, call after call, the host->device copy of the
    next operand, the kernel on the current one and the device->host copy of the previous result run
    concurrently (PCIe is full duplex).  Every call still moves its own operand in and its own result
    out; nothing is skipped or cached."""

    def __init__(self, device, elems):
        self.dev = device
        self.s_in, self.s_k, self.s_out = (torch.cuda.Stream(device) for _ in range(3))
        self.din = [torch.empty(elems, device=device) for _ in range(2)]
        self.dout = [torch.empty(elems, device=device) for _ in range(2)]
        self.ev_in = [None, None]    # operand slot filled
        self.ev_k = [None, None]     # kernel on the slot finished (operand slot reusable, result ready)
        self.ev_out = [None, None]   # result slot copied out (result slot reusable)
        self.i = 0
        self.h2d = self.d2h = 0

    def call(self, host_in, host_out, shape, kernel):
        """kernel(x_dev, y_dev) on this call's slot; host_in / host_out are pinned views of `shape`."""
        slot = self.i & 1
        self.i += 1
        n = host_in.numel()
        x = self.din[slot][:n].view(shape)
        y = self.dout[slot][: host_out.numel()].view(host_out.shape)
        with torch.cuda.stream(self.s_in):
            if self.ev_k[slot] is not None:
                self.s_in.wait_event(self.ev_k[slot])
            x.copy_(host_in, non_blocking=True)
            self.ev_in[slot] = self.s_in.record_event()
        with torch.cuda.stream(self.s_k):
            self.s_k.wait_event(self.ev_in[slot])
            if self.ev_out[slot] is not None:
                self.s_k.wait_event(self.ev_out[slot])
            y = kernel(x, y)
            self.ev_k[slot] = self.s_k.record_event()
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_k[slot])
            host_out.copy_(y, non_blocking=True)
            y.record_stream(self.s_out)  # results allocated by the kernel stream stay alive until copied
            self.ev_out[slot] = self.s_out.record_event()
        self.h2d += n * 4
        self.d2h += host_out.numel() * 4

    def drain(self):
        for s in (self.s_in, self.s_k, self.s_out):
            s.synchronize()


