"""Single-kernel micro-benchmarks beside bench.py: the small cases the profiler captures under
profiles/ are taken on, and the per-kernel bandwidth / throughput figures quoted next to them.

    python bench_kernels.py codec [--rows 2097152] [--bits 2] [--widths 256,128,32] [--iters 10]
    python bench_kernels.py dense [--rows 2450000] [--shapes 256x256,256x100,48x256] [--iters 10]
    python bench_kernels.py halo  [--parts 2] [--scale 22] [--widths 256,128,32] [--bits 2]

codec: quantise+pack, gather+quantise+pack, unpack+dequantise on a halo-sized buffer, one JSON line
per feature width.  Algorithmic bytes per row: quantise 4F + F*bits/8 + 12 (fp32 row in; codes, fp32
and bf16 parameters out); dequantise F*bits/8 + 4 + 4F.  Peers: three segments, one of them empty and
none a multiple of the packing group, so that the ragged paths run.

dense: the tensor-core feature transform (forward / input gradient), the weight gradient, the fused
dropout-LayerNorm-ReLU pair and the row scaling, each beside the torch / cuBLAS fp32 call it replaces.
A shape NxK is a Linear layer with K inputs and N outputs; bytes counted: the transform reads
rows*K*4 and writes rows*N*4 (the weight is L2-resident); FLOPs 2*rows*N*K of fp32 product work (the
kernel issues three TF32 tensor-core products for each).
"""
import argparse
import json
import os
import sys

import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from gnn_benchmark_b200 import dense, norm  # noqa: E402
from gnn_benchmark_b200.quantizer import Quantizer_for_all_procs  # noqa: E402


def main_codec(argv):
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=1 << 21)
    ap.add_argument("--bits", type=int, default=2)
    ap.add_argument("--widths", type=str, default="256,128,32")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args(argv)
    dev = torch.device("cuda", 0)
    rows, bits = args.rows, args.bits
    epb = 8 // bits
    seg_list = [0, rows // 3, rows // 3, rows]
    seg = torch.tensor(seg_list, dtype=torch.int32, device=dev)
    q = Quantizer_for_all_procs(3, bits)
    prow = sum((b - a + epb - 1) // epb for a, b in zip(seg_list[:-1], seg_list[1:]))
    g = torch.Generator(device=dev).manual_seed(0)
    idx = torch.randint(0, rows, (rows,), device=dev, generator=g).to(torch.int32)

    def timed(fn):
        for _ in range(3):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / args.iters / 1e3

    for F in (int(w) for w in args.widths.split(",")):
        x = torch.randn(rows, F, device=dev, generator=g)
        codes = torch.empty(prow, F, dtype=torch.uint8, device=dev)
        params = torch.empty(rows, 2, device=dev)
        pb = torch.empty(rows, 2, dtype=torch.bfloat16, device=dev)
        y = torch.empty_like(x)
        tq = timed(lambda: q.quantize_fp32_to_intX(x, codes, params, seg, params_bf16=pb))
        tg = timed(lambda: q.quantize_fp32_to_intX(x, codes, params, seg, params_bf16=pb, gather_idx=idx))
        td = timed(lambda: q.dequantize_intX_to_fp32(codes, y, params, seg, params_bf16=pb))
        bq = rows * (4 * F + F * bits / 8 + 12)
        bd = rows * (F * bits / 8 + 4 + 4 * F)
        print(json.dumps({"F": F, "rows": rows, "bits": bits,
                          "quant_pack": {"ms": tq * 1e3, "gbs": bq / tq / 1e9},
                          "gather_quant_pack": {"ms": tg * 1e3, "gbs": (bq + 4 * rows) / tg / 1e9},
                          "unpack_dequant": {"ms": td * 1e3, "gbs": bd / td / 1e9}}), flush=True)



def main_dense(argv):
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=2_450_000)
    ap.add_argument("--shapes", type=str, default="256x256,256x100,48x256")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--only", type=str, default="", help="comma list of: linear,wgrad,norm,scale (default all)")
    ap.add_argument("--no-baseline", action="store_true", help="skip the torch / cuBLAS calls (profiling runs)")
    args = ap.parse_args(argv)
    only = set(args.only.split(",")) if args.only else {"linear", "wgrad", "norm", "scale"}
    dev = torch.device("cuda", 0)
    M = args.rows
    g = torch.Generator(device=dev).manual_seed(0)

    def timed(fn):
        for _ in range(3):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / args.iters

    for shape in args.shapes.split(","):
        N, K = (int(v) for v in shape.split("x"))
        x = torch.randn(M, K, device=dev, generator=g)
        w = torch.randn(N, K, device=dev, generator=g)
        b = torch.randn(N, device=dev, generator=g)
        gy = torch.randn(M, N, device=dev, generator=g)
        y = torch.empty(M, N, device=dev)
        line = {"rows": M, "N": N, "K": K}
        if "linear" in only:
            t = timed(lambda: dense.linear(x, w, b, out=y))
            line["linear_tf32x3"] = {"ms": t, "tflops": 2 * M * N * K / t / 1e9, "gbs": (M * K + M * N) * 4 / t / 1e6}
            if not args.no_baseline:
                t = timed(lambda: torch.addmm(b, x, w.t(), out=y))
                line["linear_cublas_fp32"] = {"ms": t, "tflops": 2 * M * N * K / t / 1e9}
        if "wgrad" in only and dense.wgrad_supported(gy, x):
            dw = torch.empty(N, K, device=dev)
            t = timed(lambda: dense.wgrad(gy, x, out=dw))
            line["wgrad_tf32x3"] = {"ms": t, "tflops": 2 * M * N * K / t / 1e9, "gbs": (M * K + M * N) * 4 / t / 1e6}
            if not args.no_baseline:
                t = timed(lambda: torch.mm(gy.t(), x, out=dw))
                line["wgrad_cublas_fp32"] = {"ms": t, "tflops": 2 * M * N * K / t / 1e9}
        if "norm" in only and norm.supported(gy):
            gamma = torch.rand(N, device=dev, generator=g).requires_grad_(True)
            beta = torch.randn(N, device=dev, generator=g).requires_grad_(True)
            h = gy.clone().requires_grad_(True)

            def fused():
                out = norm.dropout_ln_relu(h, gamma, beta, 0.5, True)
                out.backward(y)

            def plain():
                out = F.relu(F.layer_norm(F.dropout(h, 0.5, True), (N,), gamma, beta))
                out.backward(y)

            t = timed(fused)
            line["dropout_ln_relu_fwd_bwd_fused"] = {"ms": t, "gbs": 6 * M * N * 4 / t / 1e6}
            if not args.no_baseline:
                line["dropout_ln_relu_fwd_bwd_torch"] = {"ms": timed(plain)}
        if "scale" in only:
            s = torch.rand(M, 1, device=dev, generator=g) + 0.5
            t = timed(lambda: dense.scale_rows(gy, s, True, out=y))
            line["scale_rows"] = {"ms": t, "gbs": 2 * M * N * 4 / t / 1e6}
            if not args.no_baseline:
                line["scale_rows_torch"] = {"ms": timed(lambda: torch.div(gy, s, out=y))}
        dense.check_status()
        print(json.dumps(line), flush=True)



def main_halo(argv):
    """The kernels either side of a packed halo exchange on ONE rank's share of the benchmark graph (R-MAT,
    2^22 vertices per partition, randomly relabelled, partition 0 of --parts): forward gather+pack and
    fused-unpack remote SpMM, backward transposed SpMM with the packing epilogue (beside the two-call
    sequence it replaces: SpMM into an fp32 buffer, then quantise+pack) and the fused-unpack scatter-add."""
    from gnn_benchmark_b200 import SparseTensor, graphgen
    from gnn_benchmark_b200.aggregator import gather_rows
    from gnn_benchmark_b200.data_manager.DataLoader import _scatter_matrix
    from gnn_benchmark_b200.spmm_kernel import (SPMM_backward, SPMM_backward_quant_pack, SPMM_forward, SPMM_forward_packed)

    ap = argparse.ArgumentParser()
    ap.add_argument("--parts", type=int, default=2)
    ap.add_argument("--scale", type=int, default=22, help="log2 of the vertices per partition")
    ap.add_argument("--widths", type=str, default="256,128,32")
    ap.add_argument("--bits", type=int, default=2)
    ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args(argv)
    dev = torch.device("cuda", 0)
    P, bits = args.parts, args.bits
    scale = args.scale + (P - 1).bit_length()
    src, dst, begin = graphgen.partitioned_in_edges("rmat", 1 << scale, 16 << scale, 20261127, 0, P, dev, relabel=True,
                                                    scale=scale)
    n = int(begin[1])
    rem = src >= n
    halo_ids, slot = torch.unique(src[rem], return_inverse=True)
    A = SparseTensor(row=dst[rem], col=slot, sparse_sizes=(n, halo_ids.numel()))
    del src, dst, rem, slot
    K = halo_ids.numel()
    owner = torch.searchsorted(begin.to(dev), halo_ids, right=True) - 1
    counts = torch.bincount(owner, minlength=P)[:P].tolist()
    seg = torch.tensor([0] + list(torch.tensor(counts).cumsum(0).tolist()), dtype=torch.int32, device=dev)
    epb = 8 // bits
    prow = sum((c + epb - 1) // epb for c in counts)
    q = Quantizer_for_all_procs(P, bits)
    g = torch.Generator(device=dev).manual_seed(0)
    idx = torch.randint(0, n, (K,), device=dev, generator=g).to(torch.int32)
    S = _scatter_matrix(idx.to(torch.int64), n)

    def timed(fn):
        for _ in range(2):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / args.iters

    for F in (int(w) for w in args.widths.split(",")):
        x = torch.randn(n, F, device=dev, generator=g)
        out = torch.empty(n, F, device=dev)
        codes = torch.empty(prow, F, dtype=torch.uint8, device=dev)
        params = torch.empty(K, 2, device=dev)
        pb = torch.empty(K, 2, dtype=torch.bfloat16, device=dev)
        buf = torch.empty(K, F, device=dev)
        line = {"F": F, "rows": n, "halo_rows": K, "nnz_remote": A.nnz(), "bits": bits}
        line["gather_pack_ms"] = timed(lambda: q.quantize_fp32_to_intX(x, codes, params, seg, params_bf16=pb, gather_idx=idx))
        line["remote_spmm_fused_unpack_ms"] = timed(lambda: SPMM_forward_packed(A, codes, pb, seg, P, bits, out))

        def two_calls():
            SPMM_backward(A, x, buf, accumulate=False)
            q.quantize_fp32_to_intX(buf, codes, params, seg, params_bf16=pb)

        line["backward_spmm_then_pack_ms"] = timed(two_calls)
        line["backward_spmm_pack_fused_ms"] = timed(lambda: SPMM_backward_quant_pack(A, x, codes, params, pb, seg, P, bits))
        line["scatter_fused_unpack_ms"] = timed(lambda: SPMM_forward_packed(S, codes, pb, seg, P, bits, out))

        # the two-step forms the fused-unpack kernels replace: unpack into the fp32 halo buffer, then the SpMM
        def unpack_then(mat):
            q.dequantize_intX_to_fp32(codes, buf, params, seg, params_bf16=pb)
            SPMM_forward(mat, buf, out, accumulate=True)

        line["unpack_then_remote_spmm_ms"] = timed(lambda: unpack_then(A))
        line["unpack_then_scatter_ms"] = timed(lambda: unpack_then(S))
        line["gather_rows_ms"] = timed(lambda: gather_rows(x, idx, buf))
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    legs = {"codec": main_codec, "dense": main_dense, "halo": main_halo}
    if len(sys.argv) < 2 or sys.argv[1] not in legs:
        raise SystemExit("usage: python bench_kernels.py {codec|dense|halo} [options]")
    legs[sys.argv[1]](sys.argv[2:])
