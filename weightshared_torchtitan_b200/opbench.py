"""Isolated benchmark of the fused projection kernels (one shape, CUDA-event timing).

    python -m weightshared_torchtitan_b200.opbench --M 16384 --N 12288 --K 4096 --r 64
    python -m weightshared_torchtitan_b200.opbench --sweep-r            # r in {8..128}, M = 32768

Prints one JSON line per shape with per-kernel milliseconds, TFLOP/s (tensor-bound GEMMs)
and GB/s (rank-r pre-passes), using algorithmic FLOPs 6MNK + 6Mr(K+N) and bytes
2(MK + rK + Mr). Also the command that ncu captures are taken from (--what, --iters).
"""
from __future__ import annotations

import argparse
import json

import torch

from . import ops


def make_inputs(M, N, K, r, seed=1238):
    g = torch.Generator(device="cuda").manual_seed(seed)
    bf = torch.bfloat16
    x = torch.randn(M, K, device="cuda", generator=g).to(bf)
    W = (torch.randn(N, K, device="cuda", generator=g) * 0.02).to(bf)
    A = ((torch.rand(r, K, device="cuda", generator=g) * 2 - 1) / K ** 0.5).to(bf)
    B = (torch.randn(N, r, device="cuda", generator=g) * 0.02).to(bf)
    dY = torch.randn(M, N, device="cuda", generator=g).to(bf)
    return x, W, A, B, dY


def time_ms(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def bench_shape(M, N, K, r, iters, what="all", warmup=3):
    x, W, A, B, dY = make_inputs(M, N, K, r)
    dW = torch.zeros(N, K, device="cuda")
    dA = torch.zeros(r, K, device="cuda")
    dB = torch.zeros(N, r, device="cuda")
    T = ops.lora_prepass(x, A, 2.0)
    U = ops.lora_bwd_prepass(dY, B, 2.0)
    parts = {
        "prepass_T": lambda: ops.lora_prepass(x, A, 2.0),
        "fwd": lambda: ops.lora_linear_fwd(x, W, T, B),
        "prepass_U": lambda: ops.lora_bwd_prepass(dY, B, 2.0),
        "dx": lambda: ops.lora_linear_bwd_dx([dY], [U], [W], [A]),
        "dw": lambda: ops.lora_linear_bwd_dw(dY, U, x, T, dW, dA, dB),
    }
    # the backward through the layer's own weight gradient (what the autograd Function runs when
    # the shared weight is trained): merged weight -> dX, dW with a bf16 copy, adapters from it
    Weff = ops.lora_merge_weight([W], [A], [B], 2.0)[0]
    G = ops.bwd_dw_layer_group([dY], x, [dW])
    via_dw = {
        "merge": lambda: ops.lora_merge_weight([W], [A], [B], 2.0),
        "dx_merged": lambda: ops.lora_linear_bwd_dx([dY], [None], [Weff], [None]),
        "dw_copy": lambda: ops.bwd_dw_layer_group([dY], x, [dW]),
        "adapter_grads": lambda: ops.lora_adapter_grads_from_dw(G, [A], [B], [dA], [dB], 2.0),
    }
    res = {"M": M, "N": N, "K": K, "r": r}
    if what != "all":
        res[what + "_ms"] = time_ms({**parts, **via_dw}[what], iters, warmup)
        return res

    def whole():
        for f in parts.values():
            f()

    def whole_via_dw():
        parts["prepass_T"]()
        parts["fwd"]()
        for f in via_dw.values():
            f()

    ms = {k: time_ms(f, iters, warmup) for k, f in {**parts, **via_dw}.items()}
    total_direct = time_ms(whole, iters, warmup)
    total = time_ms(whole_via_dw, iters, warmup)
    flops = 6.0 * M * N * K + 6.0 * M * r * (K + N)
    res.update({
        "total_ms": total, "tflops": flops / total / 1e9, "frac_of_2.25PF": flops / total / 1e9 / 2250.0,
        "total_ms_direct": total_direct, "tflops_direct": flops / total_direct / 1e9,
        "ms": ms,
        "dx_merged_tflops": 2.0 * M * K * N / ms["dx_merged"] / 1e9,
        "dw_copy_tflops": 2.0 * M * N * K / ms["dw_copy"] / 1e9,
        "fwd_tflops": 2.0 * M * N * (K + r) / ms["fwd"] / 1e9,
        "dx_tflops": 2.0 * M * K * (N + r) / ms["dx"] / 1e9,
        "dw_tflops": 2.0 * M * (N * K + r * K + N * r) / ms["dw"] / 1e9,
        "prepass_T_gbs": 2.0 * (M * K + r * K + M * r) / ms["prepass_T"] / 1e6,
        "prepass_U_gbs": 2.0 * (M * N + r * N + M * r) / ms["prepass_U"] / 1e6,
        "torch_mm_tflops": 2.0 * M * N * K / time_ms(lambda: torch.mm(x, W.T), iters, warmup) / 1e9,
    })
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--M", type=int, default=16384)
    ap.add_argument("--N", type=int, default=12288)
    ap.add_argument("--K", type=int, default=4096)
    ap.add_argument("--r", type=int, default=64)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--what", default="all", choices=["all", "prepass_T", "fwd", "prepass_U", "dx", "dw", "merge",
                                                      "dx_merged", "dw_copy", "adapter_grads"])
    ap.add_argument("--sweep-r", action="store_true", help="baseline config 3 sweep: r in {8,16,32,64,128}, M=32768")
    args = ap.parse_args()
    if args.sweep_r:
        for r in (8, 16, 32, 64, 128):
            print(json.dumps(bench_shape(32768, 9728, 2560, r, args.iters)), flush=True)
        return
    print(json.dumps(bench_shape(args.M, args.N, args.K, args.r, args.iters, args.what, args.warmup)), flush=True)


if __name__ == "__main__":
    main()
