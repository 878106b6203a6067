"""Micro-benchmark of the dense-side kernels around the aggregation: the tensor-core feature
transform (forward / input gradient), the weight gradient, the fused dropout-LayerNorm-ReLU pair and
the row scaling, each beside the torch / cuBLAS fp32 call it replaces.  One JSON line per shape.

    python -m gnn_benchmark_b200.bench_dense [--rows 2450000] [--shapes 256x256,256x100,48x256] [--iters 10]

A shape NxK is a Linear layer with K inputs and N outputs.  Bytes counted for the roofline: the
transform reads rows*K*4 and writes rows*N*4 (the weight is L2-resident); FLOPs 2*rows*N*K of fp32
product work (the kernel issues three TF32 tensor-core products for each).
"""
import argparse
import json

import torch
import torch.nn.functional as F

from . import dense, norm


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=2_450_000)
    ap.add_argument("--shapes", type=str, default="256x256,256x100,48x256")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--only", type=str, default="", help="comma list of: linear,wgrad,norm,scale (default all)")
    ap.add_argument("--no-baseline", action="store_true", help="skip the torch / cuBLAS calls (profiling runs)")
    args = ap.parse_args()
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


if __name__ == "__main__":
    main()
