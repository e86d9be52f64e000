"""Isolated benchmark of the row kernels either side of the projections (CUDA-event timing,
L2 flushed by a read of a 256 MB buffer between iterations).

    python -m weightshared_torchtitan_b200.rowbench                 # all kernels, 32768 tokens
    python -m weightshared_torchtitan_b200.rowbench --what rmsnorm --iters 1 --tokens 8192

Prints one JSON line per kernel and shape: microseconds and GB/s over the algorithmic bytes
(RMSNorm forward 2 passes, backward 3; SwiGLU 3 / 5; cross-entropy 3; optimizer step 4 B per
parameter for the norm, 30 B for clip + AdamW + bf16 copy). `--what` / `--iters`
give the small single-launch runs that ncu captures are taken from.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import ops
from .decoder import rope_tables


def time_us(fn, iters, warmup=2):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    total = 0.0
    for _ in range(iters):
        flush.sum()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--what", default="all", choices=["all", "rmsnorm", "swiglu", "ce", "adamw", "embed"])
    args = ap.parse_args()
    M, S = args.tokens, args.seq
    bf = torch.bfloat16
    if args.what in ("all", "rmsnorm"):
        # hidden rows (configurations 1 to 4) and head rows with the rotary embedding (16 and 8 heads)
        for rows, D, heads in [(M, 1024, 0), (M, 2048, 0), (M // 2, 2560, 0), (M // 2, 4096, 0), (M * 16, 128, 16),
                               (M * 8, 128, 8)]:
            x = torch.randn(rows, D, device="cuda").to(bf)
            dy = torch.randn(rows, D, device="cuda").to(bf)
            w = torch.ones(D, device="cuda")
            dw = torch.zeros(D, device="cuda")
            rope = None
            if heads:
                cos, sin = rope_tables(D, S, 1e6, "cuda")
                rope = (cos.contiguous(), sin.contiguous(), heads, S)
            _, rstd = ops.rmsnorm_fwd(x, w, 1e-6, rope)
            tf = time_us(lambda: ops.rmsnorm_fwd(x, w, 1e-6, rope), args.iters, args.warmup)
            tb = time_us(lambda: ops.rmsnorm_bwd(dy, x, w, rstd, dw, rope), args.iters, args.warmup)
            nb = rows * D * 2
            print(json.dumps({"kernel": "rmsnorm", "rows": rows, "D": D, "heads": heads,
                              "fwd_us": tf, "fwd_gbs": 2 * nb / tf / 1e3,
                              "bwd_us": tb, "bwd_gbs": 3 * nb / tb / 1e3}), flush=True)
    if args.what in ("all", "swiglu"):
        g = torch.randn(M, 3072, device="cuda").to(bf)
        u = torch.randn(M, 3072, device="cuda").to(bf)
        d = torch.randn(M, 3072, device="cuda").to(bf)
        nb = g.numel() * 2
        tf = time_us(lambda: ops.swiglu_fwd(g, u), args.iters, args.warmup)
        tb = time_us(lambda: ops.swiglu_bwd(d, g, u), args.iters, args.warmup)
        print(json.dumps({"kernel": "swiglu", "rows": M, "D": 3072, "fwd_us": tf, "fwd_gbs": 3 * nb / tf / 1e3,
                          "bwd_us": tb, "bwd_gbs": 5 * nb / tb / 1e3}), flush=True)
    if args.what in ("all", "ce"):
        rows, V = min(M, 8192), 151936
        logits = torch.randn(rows, V, device="cuda").to(bf)
        labels = torch.randint(0, V, (rows,), device="cuda")
        nb = logits.numel() * 2
        t = time_us(lambda: ops.ce_fwd_bwd(logits, labels, 1.0 / rows), args.iters, args.warmup)
        print(json.dumps({"kernel": "ce_fwd_bwd", "rows": rows, "V": V, "us": t, "gbs": 3 * nb / t / 1e3}), flush=True)


    if args.what in ("all", "embed"):
        # factorized embedding of configuration 1: gather from E_small [V, r_e] alone, and fused
        # into the projection GEMM (rows fetched by TMA gather4 inside the producer)
        V, r_e, d = 151936, 256, 1024
        tok = torch.randint(0, V, (M,), device="cuda")
        E = torch.randn(V, r_e, device="cuda").to(bf)
        P = (torch.randn(d, r_e, device="cuda") * 0.02).to(bf)
        tg = time_us(lambda: ops.embed_gather(tok, E), args.iters, args.warmup)
        tf = time_us(lambda: ops.embed_fwd(tok, E, P), args.iters, args.warmup)
        print(json.dumps({"kernel": "embedding", "tokens": M, "V": V, "r_e": r_e, "d": d,
                          "gather_us": tg, "gather_gbs": (8.0 * M + 4.0 * M * r_e) / tg / 1e3,
                          "fused_fwd_us": tf, "fused_fwd_gbs": (8.0 * M + 2.0 * M * (r_e + d)) / tf / 1e3,
                          "fused_fwd_tflops": 2.0 * M * r_e * d / tf / 1e6}), flush=True)
    if args.what in ("all", "adamw"):
        n = 64 * 1024 * 1024 if args.what == "adamw" and args.iters == 1 else 268 * 1000 * 1000
        p = torch.randn(n, device="cuda")
        g = torch.randn(n, device="cuda")
        m, v = torch.zeros_like(p), torch.zeros_like(p)
        copy = torch.empty(n, device="cuda", dtype=bf)
        part = torch.empty(ops.SUMSQ_PARTIALS, device="cuda")
        ts = time_us(lambda: ops.grad_sumsq_partials(g, part), args.iters, args.warmup)
        ta = time_us(lambda: ops.adamw_flat_step(p, g, m, v, copy, 3e-4, 0.9, 0.95, 1e-8, 0.1, 5, part, 1.0),
                     args.iters, args.warmup)
        print(json.dumps({"kernel": "flat optimizer step", "n": n, "sumsq_us": ts, "sumsq_gbs": 4.0 * n / ts / 1e3,
                          "adamw_us": ta, "adamw_gbs": 30.0 * n / ta / 1e3}), flush=True)


if __name__ == "__main__":
    main()
