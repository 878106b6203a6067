"""Micro-benchmark of the halo codec kernels (K3): quantise+pack, gather+quantise+pack,
unpack+dequantise, on a halo-sized buffer.  One JSON line per feature width.

    python -m gnn_benchmark_b200.bench_codec [--rows 2097152] [--bits 2] [--widths 256,128,32] [--iters 10]

Algorithmic bytes per row: quantise 4F + F*bits/8 + 12 (fp32 row in; codes, fp32 and bf16 parameters
out); dequantise F*bits/8 + 4 + 4F.  Peers: three segments, one of them empty and none a multiple of
the packing group, so that the ragged paths run.
"""
import argparse
import json

import torch

from .quantizer import Quantizer_for_all_procs


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=1 << 21)
    ap.add_argument("--bits", type=int, default=2)
    ap.add_argument("--widths", type=str, default="256,128,32")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
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


if __name__ == "__main__":
    main()
