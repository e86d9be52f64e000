"""Benchmark of the shared-W + LoRA linear hot path inside its training step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
    torchrun --nnodes=1 --nproc-per-node N ... bench.py --gpus N --steps K --warmup W

Workload (default, every N, weak scaling): baseline configuration 4, the Qwen3-8B-shape
weight-shared decoder the headline metric is quoted on (hidden 4096, SwiGLU 12288, 36 layers
over 4 shared blocks, 32/8 heads of 128, LoRA r=64 on all seven projections, factorized
embedding r_e=1024, vocab 151936), sequence 8192, micro-batch 2 per GPU, uniform token ids,
random-init weights, AdamW step. `--workload` selects configurations 1-3 instead. A "step"
is one full optimisation step (forward, loss, backward, gradient all-reduce, clip, AdamW)
over one batch. Synthetic token ids stand in for the C4 stream the reference trains on.

One JSON line on stdout (rank 0). `value` = whole-job tokens/s with tokens already resident
in HBM; `e2e` = the same step driven from pinned host buffers (H2D of tokens/labels and D2H
of the loss inside the timed region); `roofline` = the dominant kernel of this library by
device time inside the timed region (CUDA events on the launching stream around every launch
of one step in four: events between kernels switch their programmatic overlap off, so the
other steps run without them), against the measured bf16 tensor peak; `op_headline` = the isolated fused projection fwd+bwd at the
configuration-4 MLP shapes (M = 16384) with its own clock record; `gpu_eager_baseline` = the
reference's eager composition (nn.Linear + LoRA + add under bf16 autocast) at the same shape
on the same GPU; `cpu_baseline` = the CPU oracle (eager PyTorch restatement of the reference
path) on the host cores for a bounded sample, and `parity` = this library's loss and sampled
gradients against that oracle on the same sample; at N > 1 `dp_parity` (N ranks on shards
+ all-reduce against one rank on the whole batch) and `replicas_identical`.

`--impl reference` times that CPU eager path alone (the reference has no other
implementation of this path that runs without a GPU-side rewrite).

Kernel-level modes (one JSON line per shape; also the commands profiler captures are taken
from): `--op M,N,K,r [--what KERNEL]` isolated projection kernels, `--op-sweep` the rank sweep
of configuration 3 (r in 8..128 at M = 32768), `--rows [--what KIND]` the row kernels and the
factorized embedding.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# (sequence length, micro-batch per GPU, baseline configuration number)
WORKLOAD_SHAPES = {"qwen3-0.6b-ws": (4096, 8, 1), "qwen3-1.7b-ws": (4096, 8, 2), "qwen3-4b-ws": (8192, 4, 3),
                   "qwen3-8b-ws": (8192, 2, 4)}
WORKLOAD = "qwen3-8b-ws"
SEQ_LEN, MICRO_BATCH, CONFIG_NO = WORKLOAD_SHAPES[WORKLOAD]
METRIC = "step_tokens_per_s"
UNIT = "tokens/s"
TIMING_EVERY = 4             # steps between two steps that carry per-launch CUDA events
PEAK_NOMINAL_TF = 2250.0     # B200 dense bf16, the constant the reference's MFU uses (torchtitan/tools/utils.py:96-98)

# Measured DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) over algorithmic bytes
# of one launch, from profiler captures of the three GEMM kinds at M=N=8192, K=4096, r=64. The
# step's launches are too many and too varied to capture one by one; traffic of these
# kernels grows with the operand sizes, so the bench scales the ratio by the algorithmic
# bytes of its own average launch.
NCU_TRAFFIC_OVER_ALGORITHMIC = {"fwd": 1.76, "dx": 2.50, "dw": 1.78}   # dw: the launch with the bf16 copy


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "tf_burst": p["bf16_tflops"], "tf_sustained": p["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tf_burst": 1590.0, "tf_sustained": 1400.0, "source": "fallback"}


def config_block(world: int) -> dict:
    """`config` of the JSON line; identical for both arms."""
    return {"workload": f"{WORKLOAD} decoder training step (baseline config {CONFIG_NO})",
            "seq_len": SEQ_LEN, "micro_batch_per_gpu": MICRO_BATCH, "global_batch": MICRO_BATCH * world,
            "parallelism": f"dp{world}",
            "l2": "per-step activations and weights (tens of GB) exceed the 126 MB L2; no flush needed"}


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled during a timed region."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, interval_ms: int = 200):
        self.gpu = gpu_index
        self.interval_ms = interval_ms
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms",
                 str(self.interval_ms), "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [c.strip() for c in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                pw.append(float(f[3]))
            except ValueError:
                continue
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------- CPU baseline
def _oracle_setup(sample_tokens: int):
    """Oracle arguments, bf16-representable fp32 parameters (so that a bf16 GPU run of the same
    values computes with exactly these numbers) and one seeded sample of token ids / labels."""
    import torch
    from oracle import lora_oracle as O
    from weightshared_torchtitan_b200.decoder import CONFIGS
    c = CONFIGS[WORKLOAD]
    a = O.DecoderArgs(dim=c.dim, hidden_dim=c.hidden_dim, n_layers=c.n_layers, n_unique=c.n_unique,
                      n_heads=c.n_heads, n_kv_heads=c.n_kv_heads, head_dim=c.head_dim, rank=c.rank,
                      vocab_size=c.vocab_size, embed_rank=c.embed_rank, max_seq_len=sample_tokens)
    p = {k: v.to(torch.bfloat16).float() for k, v in O.init_decoder_params(a, seed=1235).items()}
    g = torch.Generator().manual_seed(1)
    tokens = torch.randint(0, a.vocab_size, (1, 256), generator=g)
    labels = torch.randint(0, a.vocab_size, (1, 256), generator=g)
    return O, a, p, tokens, labels


def _oracle_step(O, a, p, tokens, labels):
    """One eager fwd + loss + bwd of the oracle; returns (seconds, loss)."""
    for v in p.values():
        v.grad = None
    t0 = time.perf_counter()
    loss = O.decoder_loss(a, p, tokens, labels)
    loss.backward()
    return time.perf_counter() - t0, float(loss.item())


# Tokens of the one-sequence sample the in-line CPU baseline of the GPU arm times (about 10-30 s
# of host work per configuration on 16-32 cores).
CPU_SAMPLE_TOKENS = {"qwen3-0.6b-ws": 256, "qwen3-1.7b-ws": 128, "qwen3-4b-ws": 64, "qwen3-8b-ws": 64}


def cpu_reference(steps: int, warmup: int, budget_s=None, keep_grads: bool = False):
    """The oracle's eager decoder step (fwd + loss + bwd, fp32, all host threads) on ONE sequence.
    With `budget_s` the sequence length (16..256 tokens) is chosen so that warmup + steps
    repetitions fit that many seconds (two short probe steps measure the host first); without,
    the configuration's fixed sample is used after one 16-token step that touches every page.
    Returns a dict with tokens/s, the sample and, if asked, what the parity check needs."""
    import torch
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    O, a, p, tokens, labels = _oracle_setup(256)
    p = {k: v.requires_grad_(True) for k, v in p.items()}
    _oracle_step(O, a, p, tokens[:, :16], labels[:, :16])     # touches every page once
    if budget_s is None:
        n = CPU_SAMPLE_TOKENS[WORKLOAD]
    else:
        t16, _ = _oracle_step(O, a, p, tokens[:, :16], labels[:, :16])
        t32, _ = _oracle_step(O, a, p, tokens[:, :32], labels[:, :32])
        per_tok = max((t32 - t16) / 16.0, 1e-4)
        fixed = max(t16 - 16 * per_tok, 0.0)
        n = 16
        for cand in (32, 64, 128, 256):
            if (warmup + steps) * (fixed + cand * per_tok) <= budget_s:
                n = cand
    tk, lb = tokens[:, :n], labels[:, :n]
    times, loss = [], None
    for i in range(warmup + steps):
        dt, loss = _oracle_step(O, a, p, tk, lb)
        if i >= warmup:
            times.append(dt)
    sec = sum(times) / len(times)
    c = a
    out = {"tokens_per_s": n / sec, "s_per_step": sec, "threads": threads, "sample_tokens": n, "loss": loss,
           "sample": f"1 sequence x {n} tokens of the {WORKLOAD} decoder, all {c.n_layers} layers + head, "
                     f"fwd+loss+bwd, fp32 eager oracle, {steps} timed step(s) after {warmup} warm-up"}
    if keep_grads:
        out["params"] = p
        out["tokens"], out["labels"], out["args"], out["oracle"] = tk, lb, a, O
    return out


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    r = cpu_reference(steps, warmup, budget_s=150.0)
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    line = {
        "impl": "reference", "metric": METRIC, "value": r["tokens_per_s"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": r["s_per_step"] * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_block(world),
        "cpu_baseline": {"value": r["tokens_per_s"], "unit": UNIT, "cores": r["threads"], "kind": "port",
                         "sample": r["sample"]},
        "e2e": {"value": r["tokens_per_s"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# --------------------------------------------------------------- isolated kernels
def make_projection_inputs(torch, M, N, K, r, seed=1238):
    g = torch.Generator(device="cuda").manual_seed(seed)
    bf = torch.bfloat16
    x = torch.randn(M, K, device="cuda", generator=g).to(bf)
    W = (torch.randn(N, K, device="cuda", generator=g) * 0.02).to(bf)
    A = ((torch.rand(r, K, device="cuda", generator=g) * 2 - 1) / K ** 0.5).to(bf)
    B = (torch.randn(N, r, device="cuda", generator=g) * 0.02).to(bf)
    dY = torch.randn(M, N, device="cuda", generator=g).to(bf)
    return x, W, A, B, dY


def time_ms(torch, fn, iters, warmup=3):
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


def headline_op(torch, peaks, gpu_index):
    """Isolated fused projection fwd+bwd through the autograd Function (pre-pass T, forward; dX,
    dW, dA, dB) at the configuration-4 MLP shapes, M = 16384, r = 64; inputs (>= 670 MB) exceed
    the 126 MB L2. Two figures per shape with the SM clock sampled meanwhile: the first 10
    repetitions after an idle second (burst clocks) and 200 repetitions after 100 more
    (sustained, power-capped clocks)."""
    from weightshared_torchtitan_b200 import functional as Fn
    out = {}
    for name, (M, N, K, r) in {"gate_up_12288x4096": (16384, 12288, 4096, 64),
                               "down_4096x12288": (16384, 4096, 12288, 64)}.items():
        x, W, A, B, dY = make_projection_inputs(torch, M, N, K, r)
        dW = torch.zeros(N, K, device="cuda")
        dA = torch.zeros(r, K, device="cuda")
        dB = torch.zeros(N, r, device="cuda")
        x.requires_grad_(True)

        def run():
            # the product's own call: the autograd Function with in-place fp32 gradient buffers
            y = Fn.lora_linear(x, W, A, B, 2.0, (dW, dA, dB))
            y.backward(dY)
            x.grad = None

        for _ in range(3):
            run()
        torch.cuda.synchronize()
        time.sleep(1.0)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        sampler = ClockSampler(gpu_index, interval_ms=50)
        sampler.start()
        ev[0].record()
        for _ in range(10):
            run()
        ev[1].record()
        for _ in range(100):
            run()
        ev[2].record()
        for _ in range(200):
            run()
        ev[3].record()
        torch.cuda.synchronize()
        clocks = sampler.stop()
        ms_burst = ev[0].elapsed_time(ev[1]) / 10
        ms = ev[2].elapsed_time(ev[3]) / 200
        flops = 6.0 * M * N * K + 6.0 * M * r * (K + N)
        tf, tf_b = flops / ms / 1e9, flops / ms_burst / 1e9
        mhz = clocks.get("sm_mhz")
        out[name] = {"ms": ms, "tflops": tf, "frac_of_2.25PF": tf / PEAK_NOMINAL_TF,
                     "frac_of_measured_sustained": tf / peaks["tf_sustained"],
                     "burst_first_10_reps": {"ms": ms_burst, "tflops": tf_b, "frac_of_2.25PF": tf_b / PEAK_NOMINAL_TF,
                                             "frac_of_measured_burst": tf_b / peaks["tf_burst"]},
                     "reps": 200, "clocks": clocks,
                     "ms_x_sm_mhz": ms * mhz if mhz else None,
                     "tflops_at_max_sm_clock": tf * clocks["sm_max_mhz"] / mhz if mhz else None}
        del x, W, A, B, dY, dW, dA, dB
    return out


def gpu_eager_projection(torch, ours):
    """What the reference itself would run on this GPU for one projection: fp32 master weights,
    nn.Linear base + LoRAModule.forward + add under torch.autocast(bfloat16), autograd backward
    (torchtitan/models/llama3/model/model.py:189-192,392-398; distributed/utils.py:219-239),
    at the headline shapes. Timed like the fused op; the speed-up is eager ms / fused ms."""
    import torch.nn.functional as F
    out = {}
    for name, (M, N, K, r) in {"gate_up_12288x4096": (16384, 12288, 4096, 64),
                               "down_4096x12288": (16384, 4096, 12288, 64)}.items():
        x, W, A, B, dY = make_projection_inputs(torch, M, N, K, r)
        Wm, Am, Bm = (t.float().requires_grad_(True) for t in (W, A, B))
        x.requires_grad_(True)
        del W, A, B

        def run():
            with torch.autocast("cuda", dtype=torch.bfloat16):
                y = F.linear(x, Wm) + F.linear(F.linear(x, Am), Bm) * 2.0
            y.backward(dY)
            x.grad = None      # parameter grads keep accumulating in fp32, as in a training step

        ms = time_ms(torch, run, 20, 3)
        flops = 6.0 * M * N * K + 6.0 * M * r * (K + N)
        out[name] = {"ms": ms, "tflops": flops / ms / 1e9, "speedup_of_fused": ms / ours[name]["ms"]}
        del x, Wm, Am, Bm, dY
    return out


def bench_projection(torch, M, N, K, r, iters, what="all", warmup=3):
    """Per-kernel times of one projection: direct backward (pre-pass U, dX with the rank-r
    segment, dW|dB|dA regions) and the backward through the layer's weight gradient (merged
    weight, dX, dW with a bf16 copy, adapter gradients from it)."""
    from weightshared_torchtitan_b200 import ops
    x, W, A, B, dY = make_projection_inputs(torch, M, N, K, r)
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
    via_dw = {}
    if r in ops.MERGE_RANKS:
        Weff = ops.lora_merge_weight([W], [A], [B], 2.0)[0]
        G = ops.bwd_dw_layer_group([dY], x, [dW])
        via_dw = {
            "merge": lambda: ops.lora_merge_weight([W], [A], [B], 2.0),
            "dx_merged": lambda: ops.lora_linear_bwd_dx([dY], [None], [Weff], [None]),
            "dw_copy": lambda: ops.bwd_dw_layer_group([dY], x, [dW]),
            "adapter_grads": lambda: ops.lora_adapter_grads_from_dw(G, [A], [B], [dA], [dB], 2.0),
        }
    # the MLP launches that carry the activation in their epilogues, with this shape as the gate / up
    # projection (N = inner width): gate|up + SwiGLU forward, and the down projection's input gradient
    # (contraction over K = model width, output width N) with the SwiGLU backward
    mlp = {}
    if N >= K and ops.lora_swiglu_supported(M, N, K, r) and ops.swiglu_bwd_in_dx_supported(M, K, N, r):
        A_cat = torch.cat((A, A))
        T_cat = ops.lora_prepass(x, A_cat, 2.0)
        g_, u_, _ = ops.lora_swiglu_fwd(x, W, W, T_cat, B, B)
        Wd = W.t().contiguous()                       # [K, N]: the down projection's weight
        dYd = dY[:, :K].contiguous()                  # its output gradient [M, K]
        Ad = A[:, :1].expand(r, N).contiguous()       # [r, N]
        Ud = ops.lora_bwd_prepass(dYd, B[:K], 2.0)    # [M, r]
        mlp = {
            "mlp_fwd": lambda: ops.lora_swiglu_fwd(x, W, W, T_cat, B, B),
            "mlp_fwd_unfused": lambda: ops.swiglu_fwd(*ops.lora_linear_fwd_group(
                x, [W, W], [T_cat[:, :r], T_cat[:, r:]], [B, B])),
            "mlp_dx": lambda: ops.lora_linear_bwd_dx_swiglu(dYd, Ud, Wd, Ad, g_, u_),
            "mlp_dx_unfused": lambda: ops.swiglu_bwd(ops.lora_linear_bwd_dx([dYd], [Ud], [Wd], [Ad]), g_, u_),
        }
    res = {"M": M, "N": N, "K": K, "r": r}
    if what != "all":
        res[what + "_ms"] = time_ms(torch, {**parts, **via_dw, **mlp}[what], iters, warmup)
        return res

    def whole():
        for f in parts.values():
            f()

    def whole_via_dw():
        parts["prepass_T"]()
        parts["fwd"]()
        for f in via_dw.values():
            f()

    ms = {k: time_ms(torch, f, iters, warmup) for k, f in {**parts, **via_dw, **mlp}.items()}
    flops = 6.0 * M * N * K + 6.0 * M * r * (K + N)
    total_direct = time_ms(torch, whole, iters, warmup)
    res.update({
        "total_ms_direct": total_direct, "tflops_direct": flops / total_direct / 1e9,
        "frac_of_2.25PF_direct": flops / total_direct / 1e9 / PEAK_NOMINAL_TF,
        "ms": ms,
        "fwd_tflops": 2.0 * M * N * (K + r) / ms["fwd"] / 1e9,
        "dx_tflops": 2.0 * M * K * (N + r) / ms["dx"] / 1e9,
        "dw_tflops": 2.0 * M * (N * K + r * K + N * r) / ms["dw"] / 1e9,
        "prepass_T_gbs": 2.0 * (M * K + r * K + M * r) / ms["prepass_T"] / 1e6,
        "prepass_U_gbs": 2.0 * (M * N + r * N + M * r) / ms["prepass_U"] / 1e6,
        "torch_mm_tflops": 2.0 * M * N * K / time_ms(torch, lambda: torch.mm(x, W.T), iters, warmup) / 1e9,
    })
    if via_dw:
        total = time_ms(torch, whole_via_dw, iters, warmup)
        res.update({"total_ms_through_layer_gradient": total, "tflops_through_layer_gradient": flops / total / 1e9,
                    "dx_merged_tflops": 2.0 * M * K * N / ms["dx_merged"] / 1e9,
                    "dw_copy_tflops": 2.0 * M * N * K / ms["dw_copy"] / 1e9,
                    "merge_gbs": 4.0 * N * K / ms["merge"] / 1e6})
    return res


def time_us_flushed(torch, fn, iters, warmup=2):
    """Per-call microseconds with the L2 flushed (a 256 MB buffer is read) before each call."""
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


def run_rows(args):
    """Row kernels either side of the projections and the factorized embedding, one JSON line per
    kernel and shape: microseconds and GB/s over the algorithmic bytes (RMSNorm forward 2 passes,
    backward 3; SwiGLU 3 / 5; cross-entropy 3; optimizer 4 B per parameter for the norm, 30 B for
    clip + AdamW + bf16 copy; embedding 8 M + 2 (M r_e + r_e d + M d))."""
    import torch
    from weightshared_torchtitan_b200 import ops
    from weightshared_torchtitan_b200.decoder import CONFIGS, rope_tables
    M, S = args.tokens, args.seq
    bf = torch.bfloat16
    what, iters, warmup = args.what, args.iters, args.warmup
    if what in ("all", "rmsnorm"):
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
            tf = time_us_flushed(torch, lambda: ops.rmsnorm_fwd(x, w, 1e-6, rope), iters, warmup)
            tb = time_us_flushed(torch, lambda: ops.rmsnorm_bwd(dy, x, w, rstd, dw, rope), iters, warmup)
            nb = rows * D * 2
            print(json.dumps({"kernel": "rmsnorm", "rows": rows, "D": D, "heads": heads,
                              "fwd_us": tf, "fwd_gbs": 2 * nb / tf / 1e3,
                              "bwd_us": tb, "bwd_gbs": 3 * nb / tb / 1e3}), flush=True)
    if what in ("all", "swiglu"):
        g = torch.randn(M, 3072, device="cuda").to(bf)
        u = torch.randn(M, 3072, device="cuda").to(bf)
        d = torch.randn(M, 3072, device="cuda").to(bf)
        nb = g.numel() * 2
        tf = time_us_flushed(torch, lambda: ops.swiglu_fwd(g, u), iters, warmup)
        tb = time_us_flushed(torch, lambda: ops.swiglu_bwd(d, g, u), iters, warmup)
        print(json.dumps({"kernel": "swiglu", "rows": M, "D": 3072, "fwd_us": tf, "fwd_gbs": 3 * nb / tf / 1e3,
                          "bwd_us": tb, "bwd_gbs": 5 * nb / tb / 1e3}), flush=True)
    if what in ("all", "ce"):
        rows, V = min(M, 8192), 151936
        logits = torch.randn(rows, V, device="cuda").to(bf)
        labels = torch.randint(0, V, (rows,), device="cuda")
        nb = logits.numel() * 2
        t = time_us_flushed(torch, lambda: ops.ce_fwd_bwd(logits, labels, 1.0 / rows), iters, warmup)
        print(json.dumps({"kernel": "ce_fwd_bwd", "rows": rows, "V": V, "us": t, "gbs": 3 * nb / t / 1e3}), flush=True)
    if what in ("all", "embed", "embed_fwd", "embed_dproj"):
        # factorized embedding at the sizes of a baseline configuration (--workload): the gather
        # from E_small [V, r_e] runs inside the GEMM's TMA producer, forward and backward
        c = CONFIGS[args.workload]
        Me = min(M, args.embed_tokens)
        V, r_e, d = c.vocab_size, c.embed_rank, c.dim
        tok = torch.randint(0, V, (Me,), device="cuda")
        E = torch.randn(V, r_e, device="cuda").to(bf)
        P = (torch.randn(d, r_e, device="cuda") * 0.02).to(bf)
        dH = torch.randn(Me, d, device="cuda").to(bf)
        dP = torch.zeros(d, r_e, device="cuda")
        line = {"kernel": "factorized embedding", "tokens": Me, "V": V, "r_e": r_e, "d": d}
        alg = 8.0 * Me + 2.0 * (Me * r_e + r_e * d + Me * d)
        if what != "embed_dproj":
            tf = time_us_flushed(torch, lambda: ops.embed_fwd(tok, E, P), iters, warmup)
            line.update({"fwd_us": tf, "fwd_gbs": alg / tf / 1e3, "fwd_tflops": 2.0 * Me * r_e * d / tf / 1e6})
        if what != "embed_fwd":
            tb = time_us_flushed(torch, lambda: ops.embed_bwd_dproj(tok, dH, E, dP), iters, warmup)
            line.update({"dproj_us": tb, "dproj_tflops": 2.0 * Me * r_e * d / tb / 1e6,
                         "dproj_gbs": (8.0 * Me + 2.0 * Me * (r_e + d) + 8.0 * r_e * d) / tb / 1e3})
        if what in ("all", "embed"):
            tg = time_us_flushed(torch, lambda: ops.embed_gather(tok, E), iters, warmup)
            line.update({"gather_alone_us": tg, "gather_alone_gbs": (8.0 * Me + 4.0 * Me * r_e) / tg / 1e3})
            # the two-kernel form (row-gather kernel, then the plain GEMMs) the module takes for wide outputs
            G = ops.embed_gather(tok, E)
            t2f = time_us_flushed(torch, lambda: ops.linear_fwd(ops.embed_gather(tok, E), P), iters, warmup)
            t2b = time_us_flushed(torch, lambda: ops.lora_linear_bwd_dw(dH, None, G, None, dP, None, None), iters, warmup)
            line.update({"two_kernel_fwd_us": t2f, "two_kernel_fwd_tflops": 2.0 * Me * r_e * d / t2f / 1e6,
                         "two_kernel_dproj_us": t2b, "two_kernel_dproj_tflops": 2.0 * Me * r_e * d / t2b / 1e6,
                         "module_takes": "gather inside the GEMM" if ops.embed_gather_in_gemm_pays(d) else "two kernels"})
        print(json.dumps(line), flush=True)
    if what in ("all", "adamw"):
        n = 64 * 1024 * 1024 if what == "adamw" and iters == 1 else 268 * 1000 * 1000
        p = torch.randn(n, device="cuda")
        g = torch.randn(n, device="cuda")
        m, v = torch.zeros_like(p), torch.zeros_like(p)
        copy = torch.empty(n, device="cuda", dtype=bf)
        part = torch.empty(ops.SUMSQ_PARTIALS, device="cuda")
        ts = time_us_flushed(torch, lambda: ops.grad_sumsq_partials(g, part), iters, warmup)
        ta = time_us_flushed(torch, lambda: ops.adamw_flat_step(p, g, m, v, copy, 3e-4, 0.9, 0.95, 1e-8, 0.1, 5,
                                                                part, 1.0), iters, warmup)
        print(json.dumps({"kernel": "flat optimizer step", "n": n, "sumsq_us": ts, "sumsq_gbs": 4.0 * n / ts / 1e3,
                          "adamw_us": ta, "adamw_gbs": 30.0 * n / ta / 1e3}), flush=True)


def run_routes(args):
    """Both backward formulations of every projection group (q|k|v, o, gate|up, down) of every
    baseline configuration at its own token count, fwd+bwd through the autograd Function with
    in-place gradient buffers: the measurements functional.ROUTE_TABLE is filled from."""
    import torch
    from weightshared_torchtitan_b200 import functional as Fn
    from weightshared_torchtitan_b200.decoder import CONFIGS, proj_shapes
    saved = Fn.DERIVED_ADAPTER_GRADS
    bf = torch.bfloat16
    for name, (seq, mb, _) in WORKLOAD_SHAPES.items():
        c = CONFIGS[name]
        M, r = seq * mb, c.rank
        shp = proj_shapes(c)
        for gname, names in (("qkv", ("wq", "wk", "wv")), ("o", ("wo",)), ("gate_up", ("w1", "w3")), ("down", ("w2",))):
            K = shp[names[0]][1]
            Ns = [shp[n][0] for n in names]
            g = torch.Generator(device="cuda").manual_seed(7)
            x = torch.randn(M, K, device="cuda", generator=g).to(bf).requires_grad_(True)
            Ws = [(torch.randn(n, K, device="cuda", generator=g) * 0.02).to(bf) for n in Ns]
            As = [((torch.rand(r, K, device="cuda", generator=g) * 2 - 1) / K ** 0.5).to(bf) for _ in Ns]
            Bs = [(torch.randn(n, r, device="cuda", generator=g) * 0.02).to(bf) for n in Ns]
            dYs = [torch.randn(M, n, device="cuda", generator=g).to(bf) for n in Ns]
            sinks = [(torch.zeros(n, K, device="cuda"), torch.zeros(r, K, device="cuda"), torch.zeros(n, r, device="cuda"))
                     for n in Ns]
            line = {"config": name, "group": gname, "M": M, "K": K, "Ns": Ns, "r": r}

            def run():
                ys = Fn.lora_linear_group(x, Ws, As, Bs, 2.0, sinks)
                torch.autograd.backward(ys, dYs)
                x.grad = None

            # the two formulations alternate rep by rep, so that both see the same clocks (the
            # SM clock under the power cap drifts by tens of percent within seconds)
            samples = {False: [], True: []}
            try:
                for flag in (False, True):
                    Fn.DERIVED_ADAPTER_GRADS = flag
                    run()
                torch.cuda.synchronize()
                for _ in range(args.iters):
                    for flag in (False, True):
                        Fn.DERIVED_ADAPTER_GRADS = flag
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record()
                        run()
                        run()
                        e1.record()
                        torch.cuda.synchronize()
                        samples[flag].append(e0.elapsed_time(e1) / 2)
            finally:
                Fn.DERIVED_ADAPTER_GRADS = saved
            line["direct_ms"] = statistics.median(samples[False])
            line["through_layer_gradient_ms"] = statistics.median(samples[True])
            line["auto_picks_through_layer_gradient"] = bool(Fn.derived_route_pays(M, K, Ns, r))
            print(json.dumps(line), flush=True)
            del x, Ws, As, Bs, dYs, sinks
            torch.cuda.empty_cache()


def run_op(args):
    import torch
    if args.op_sweep:
        for r in (8, 16, 32, 64, 128):
            print(json.dumps(bench_projection(torch, 32768, 9728, 2560, r, args.iters)), flush=True)
        return
    M, N, K, r = (int(v) for v in args.op.split(","))
    print(json.dumps(bench_projection(torch, M, N, K, r, args.iters, args.what, args.warmup)), flush=True)


# ------------------------------------------------------------------------ our arm
def reference_formula_flops_per_token(model, seq_len: int):
    """get_nparams_and_flops of the reference (torchtitan/models/llama3/model/args.py:71-93,
    torchtitan/experiments/qwen3/model/args.py:51-67): 6 (nparams - nparams_embedding) +
    12 l h q t with q = dim // n_heads and parameters counted as model.parameters() lists them,
    i.e. a base weight shared by several layers ONCE. The lookup table of the factorized
    embedding is what the rule's nn.Embedding exclusion means here."""
    c = model.config
    nparams = sum(p.numel() for p in model.parameters())
    nemb = model.tok_embeddings.embed.weight.numel()
    l, h, q, t = c.n_layers, c.n_heads, c.dim // c.n_heads, seq_len
    return nparams, nemb, 6 * (nparams - nemb) + 12 * l * h * q * t


def section_rel_err(torch, arena, got, want):
    """max|a-b| / max|b| over the whole arena and per kind of parameter."""
    out = {"all": float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))}
    kinds = {"shared_W": lambda n: n.startswith("blocks."), "adapters": lambda n: "_offset." in n,
             "embedding": lambda n: n.startswith("tok_embeddings."), "head": lambda n: n.startswith("output."),
             "norms": lambda n: "norm" in n}
    for kind, pred in kinds.items():
        worst = 0.0
        for n, p, off in zip(arena.names, arena.params, arena.offsets):
            if pred(n):
                a, b = got[off:off + p.numel()], want[off:off + p.numel()]
                worst = max(worst, float((a - b).abs().max() / b.abs().max().clamp_min(1e-30)))
        out[kind] = worst
    return out


def dp_parity_probe(torch, dist, model, step, rank, world):
    """N ranks on their shards + gradient exchange against ONE rank on the whole probe batch
    (world sequences of 256 tokens): the data-parallel semantics of the reference (gradient mean
    over ranks, torchtitan/models/llama3/infra/parallelize.py:442; per-rank token-mean loss,
    torchtitan/components/loss.py:18-22). Run with both backward formulations of the projections."""
    from weightshared_torchtitan_b200 import functional as Fn
    c = model.config
    g = torch.Generator().manual_seed(77)
    tokens = torch.randint(0, c.vocab_size, (world, 256), generator=g).cuda()
    labels = torch.randint(0, c.vocab_size, (world, 256), generator=g).cuda()
    out = {}
    saved = Fn.DERIVED_ADAPTER_GRADS
    try:
        for route, flag, bar in (("direct", False, 1e-4), ("through_layer_gradient", True, 1e-2)):
            Fn.DERIVED_ADAPTER_GRADS = flag
            loss_full = step.gradients(tokens, labels, exchange=False)
            full = step.arena.buffer.clone()
            loss_shard = step.gradients(tokens[rank:rank + 1], labels[rank:rank + 1], exchange=True)
            dist.all_reduce(loss_shard, op=dist.ReduceOp.AVG)
            err = section_rel_err(torch, step.arena, step.arena.buffer, full)
            worst = torch.tensor([err["all"]], device="cuda")
            dist.all_reduce(worst, op=dist.ReduceOp.MAX)
            out[route] = {"max_rel": float(worst.item()), "max_rel_by_kind_rank0": err, "bar": bar,
                          "ok": bool(worst.item() <= bar),
                          "loss_whole_batch": float(loss_full.item()), "loss_mean_of_shards": float(loss_shard.item())}
            del full
    finally:
        Fn.DERIVED_ADAPTER_GRADS = saved
    return out


def parity_against_oracle(torch, ref):
    """This library's bf16 loss and sampled gradients against the CPU oracle on the SAME sample
    (same parameters, already bf16-representable, same token ids). The loss is held to 1e-2. The
    1e-2 bar of the gradients is a per-operation bar (bf16 inputs, fp32 accumulation); through
    all the layers of the stack any bf16 implementation drifts from an fp32 one by rounding its
    activations after every operation, so beside this library's distance from the fp32 oracle
    the block gives the distance of the reference's own path on this GPU (the oracle under
    torch.autocast(bfloat16)), and `ok` asks for no more than twice that."""
    from weightshared_torchtitan_b200.decoder import CONFIGS, WeightSharedDecoder
    import dataclasses
    O, a, p = ref["oracle"], ref["args"], ref["params"]
    c = dataclasses.replace(CONFIGS[WORKLOAD], loss_chunk=max(32, ref["sample_tokens"] // 2))
    m = WeightSharedDecoder(c).cuda()
    m.load_named_params({k: v.detach().cuda() for k, v in p.items()})
    loss = m.loss(ref["tokens"].cuda(), ref["labels"].cuda())
    loss.backward()
    L, U = c.n_layers, c.n_unique

    def rel(got, want):
        got, want = got.detach().double().cpu(), want.detach().double().cpu()
        return float((got - want).abs().max() / want.abs().max().clamp_min(1e-300))

    names = ["blocks.0.wq.weight", f"blocks.{U - 1}.w2.weight", "layers.0.w1.w_a", f"layers.{L - 1}.w2.w_b",
             "embed.P", f"layers.{L // 2}.ffn_norm", "output"]
    grads = {
        "blocks.0.wq.weight": m.blocks[0].wq.weight.grad,
        f"blocks.{U - 1}.w2.weight": m.blocks[U - 1].w2.weight.grad,
        "layers.0.w1.w_a": m.layers[0].w1_offset.w_a.weight.grad,
        f"layers.{L - 1}.w2.w_b": m.layers[L - 1].w2_offset.w_b.weight.grad,
        "embed.P": m.tok_embeddings.proj.weight.grad,
        f"layers.{L // 2}.ffn_norm": m.layers[L // 2].ffn_norm.weight.grad,
        "output": m.output.weight.grad,
    }
    errs = {k: rel(grads[k][::97] if k == "output" else grads[k], p[k].grad[::97] if k == "output" else p[k].grad)
            for k in names}
    lg, lo = float(loss.item()), ref["loss"]
    del m, grads, loss
    torch.cuda.empty_cache()
    # the reference's own mixed-precision eager path on this GPU, same values
    pe = {k: v.detach().cuda().requires_grad_(True) for k, v in p.items()}
    with torch.autocast("cuda", dtype=torch.bfloat16):
        le = O.decoder_loss(a, pe, ref["tokens"].cuda(), ref["labels"].cuda())
    le.backward()
    floor = {k: rel(pe[k].grad[::97] if k == "output" else pe[k].grad, p[k].grad[::97] if k == "output" else p[k].grad)
             for k in names}
    del pe
    torch.cuda.empty_cache()
    loss_ok = abs(lg - lo) / abs(lo) <= 1e-2
    grads_ok = all(errs[k] <= 1e-2 or (errs[k] <= 2.0 * floor[k] and floor[k] < 0.1) for k in names)
    return {"sample_tokens": ref["sample_tokens"], "loss_gpu": lg, "loss_oracle": lo,
            "loss_rel_err": abs(lg - lo) / abs(lo), "loss_bar": 1e-2,
            "grad_max_rel_err_vs_fp32_oracle": errs,
            "reference_eager_bf16_autocast_on_this_gpu_vs_fp32_oracle": floor,
            "grad_bar": "1e-2, or 2 x the reference eager bf16 path's own distance (depth of the stack)",
            "ok": bool(loss_ok and grads_ok)}


def run_ours(args):
    import torch
    import torch.distributed as dist
    from weightshared_torchtitan_b200 import _lib, dp, ops
    from weightshared_torchtitan_b200.decoder import CONFIGS, WeightSharedDecoder, flops_per_token
    from weightshared_torchtitan_b200.train_step import TrainStep

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the wsl path has no CPU implementation "
                         "(use --impl reference for the CPU baseline)")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        opts = None
        if args.allreduce == "overlap":
            # the buckets run beside the backward kernels: give their stream priority
            opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
            if args.nccl_ctas > 0:
                opts.config.max_ctas = args.nccl_ctas
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), pg_options=opts)
    _lib.lib()
    peaks = load_peaks()

    c = CONFIGS[WORKLOAD]
    model = WeightSharedDecoder(c).cuda()
    model.init_weights(seed=1235)
    if world > 1:
        dp.broadcast_parameters(model, src=0)      # replicas identical by construction AND by exchange
    overlap = args.allreduce == "overlap" and world > 1
    step = TrainStep(model, lr=3e-4, overlap=overlap, bucket_bytes=args.bucket_mb << 20,
                     reserved_sms=args.reserve_sms, link_gbs=args.link_gbs, status_every=0)
    tokens_per_step = MICRO_BATCH * SEQ_LEN
    g = torch.Generator().manual_seed(1235 + 1000 * rank)

    def host_batch():
        t = torch.randint(0, c.vocab_size, (MICRO_BATCH, SEQ_LEN), generator=g).pin_memory()
        l = torch.randint(0, c.vocab_size, (MICRO_BATCH, SEQ_LEN), generator=g).pin_memory()
        return t, l

    nbatch = 4
    host = [host_batch() for _ in range(nbatch)]
    dev = [(t.cuda(), l.cuda()) for t, l in host]

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    dp_parity = None
    if world > 1 and not args.no_extras:
        dp_parity = dp_parity_probe(torch, dist, model, step, rank, world)

    for i in range(args.warmup):
        step(*dev[i % nbatch])
    sync_all()

    # ---- timed region 1: device-resident inputs, per-launch kernel timing on
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # A pair of CUDA events around every launch of this library sits between consecutive
    # kernels and so switches their programmatic overlap off; one step in TIMING_EVERY carries
    # them (the sample the kernel table and the roofline are computed from), the others run as
    # a user's step does.
    records = []
    instrumented = [i for i in range(args.steps) if i % TIMING_EVERY == 0]
    step.timing = {}
    n0 = _lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    e0.record()
    for i in range(args.steps):
        ops.set_timing(records if i % TIMING_EVERY == 0 else None)
        loss = step(*dev[i % nbatch])
    e1.record()
    sync_all()
    ops.set_timing(None)
    launches = _lib.launch_count() - n0
    ms_dev = e0.elapsed_time(e1)
    ar_wait = [a.elapsed_time(b) for a, b in step.timing.get("allreduce_wait", [])]
    step.timing = None

    # ---- timed region 2: end to end from pinned host buffers, loss read back every step
    sync_all()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    last = 0.0
    for i in range(args.steps):
        t, l = host[i % nbatch]
        last = step(t.cuda(non_blocking=True), l.cuda(non_blocking=True)).item()
    f1.record()
    sync_all()
    ms_e2e = f0.elapsed_time(f1)
    clocks = sampler.stop() if rank == 0 else None

    ar_ms = sum(ar_wait) / max(len(ar_wait), 1)
    times = torch.tensor([ms_dev, ms_e2e, ar_ms], device="cuda", dtype=torch.float64)
    replicas_identical = None
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        # after all the steps every replica must hold bit-identical master weights
        chk = torch.stack([step.arena.master.double().sum(), step.arena.master.double().abs().sum()])
        allc = [torch.zeros_like(chk) for _ in range(world)]
        dist.all_gather(allc, chk)
        replicas_identical = all(torch.equal(allc[0], t) for t in allc)
    ms_dev, ms_e2e, ar_ms = times.tolist()
    st, words = _lib.poll_status()
    if st != 0:
        raise SystemExit(f"bench.py: device status {st} {words}")

    if rank == 0:
        # per-kind device time of this library's kernels inside timed region 1
        kinds = {}
        for kind, fl, nb, a, b in records:
            k = kinds.setdefault(kind, {"launches": 0, "ms": 0.0, "flops": 0.0, "bytes": 0.0})
            k["launches"] += 1
            k["ms"] += a.elapsed_time(b)
            k["flops"] += fl
            k["bytes"] += nb
        top = max(kinds, key=lambda k: kinds[k]["ms"])
        tk = kinds[top]
        tensor_bound = tk["flops"] / max(tk["bytes"], 1.0) > 280.0
        if tensor_bound:
            achieved = tk["flops"] / tk["ms"] / 1e9
            peak, unit = peaks["tf_sustained"], "TFLOP/s"
        else:
            achieved = tk["bytes"] / tk["ms"] / 1e6
            peak, unit = peaks["hbm_gbs"], "GB/s"
        roofline = {"kernel": f"block_gemm_kernel ({top})", "bound": "tensor" if tensor_bound else "hbm",
                    "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                    "peak_source": peaks["source"] + (" sustained bf16" if tensor_bound else " copy"),
                    "avg_launch_ms": tk["ms"] / tk["launches"], "launches_timed": tk["launches"],
                    "algorithmic_bytes_per_launch": tk["bytes"] / tk["launches"],
                    "traffic": (NCU_TRAFFIC_OVER_ALGORITHMIC[top] * tk["bytes"] / tk["launches"]
                                if top in NCU_TRAFFIC_OVER_ALGORITHMIC else None),
                    "traffic_source": "ncu ratio at M=N=8192,K=4096 scaled by algorithmic bytes"}
        kernel_ms = sum(k["ms"] for k in kinds.values())
        fpt = flops_per_token(c, SEQ_LEN)
        total_tokens = world * tokens_per_step * args.steps
        value = total_tokens / (ms_dev / 1e3)
        e2e_v = total_tokens / (ms_e2e / 1e3)
        tps_gpu = value / world
        nparams, nemb, ref_fpt = reference_formula_flops_per_token(model, SEQ_LEN)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_dev / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_block(world),
            "e2e": {"value": e2e_v, "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": 2 * MICRO_BATCH * SEQ_LEN * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches) * world,
            "roofline": roofline,
            "kernels_timed_in_steps": instrumented,
            "kernels": {k: {"launches": v["launches"], "ms_per_step": v["ms"] / len(instrumented),
                            "tflops": v["flops"] / v["ms"] / 1e9 if v["flops"] else None,
                            "gbs": v["bytes"] / v["ms"] / 1e6} for k, v in sorted(kinds.items())},
            "wsl_kernel_share_of_step": (kernel_ms / len(instrumented)) / (ms_dev / args.steps),
            "model_tflops_per_gpu": fpt["total"] * tps_gpu / 1e12,
            "linear_tflops_per_gpu_in_step": fpt["linear"] * tokens_per_step * len(instrumented) / (kernel_ms / 1e3) / 1e12,
            # executed algorithmic FLOPs per token (every layer's projections counted, shared or
            # not) against the nominal dense bf16 peak, linears alone and the full step
            "step_roofline": {
                "flops_per_token": fpt, "terms_included": ["linear", "attention", "head", "embed"],
                "tokens_per_s_per_gpu": tps_gpu,
                "roofline_tokens_per_s_2.25PF_linear_only": PEAK_NOMINAL_TF * 1e12 / fpt["linear"],
                "frac_of_linear_only_roofline_2.25PF": tps_gpu / (PEAK_NOMINAL_TF * 1e12 / fpt["linear"]),
                "roofline_tokens_per_s_2.25PF_full_step": PEAK_NOMINAL_TF * 1e12 / fpt["total"],
                "frac_of_full_step_roofline_2.25PF": tps_gpu / (PEAK_NOMINAL_TF * 1e12 / fpt["total"]),
                "frac_of_full_step_roofline_measured_sustained": tps_gpu / (peaks["tf_sustained"] * 1e12 / fpt["total"]),
            },
            # the reference's own MFU definition (torchtitan/components/metrics.py:366-376): its
            # FLOP count sees a weight shared by several layers once, so it undercounts the work
            # this model executes; both are given
            "mfu_reference_formula": {
                "nparams": nparams, "nparams_embedding": nemb, "flops_per_token": ref_fpt,
                "tflops": ref_fpt * tps_gpu / 1e12, "mfu_pct": 100.0 * ref_fpt * tps_gpu / (PEAK_NOMINAL_TF * 1e12),
                "mfu_pct_executed_flops": 100.0 * fpt["total"] * tps_gpu / (PEAK_NOMINAL_TF * 1e12)},
            "allreduce": {"mode": "overlap" if overlap else ("blocking" if world > 1 else "none"),
                          "arena_bytes": step.arena.nbytes,
                          # device time the step's stream spent waiting for the exchange after
                          # backward (blocking: the whole all-reduce; overlap: what stayed exposed)
                          "exposed_ms_per_step": ar_ms,
                          "bucket_mb": args.bucket_mb if overlap else None,
                          "reserved_sms": args.reserve_sms if overlap else None,
                          "nccl_max_ctas": args.nccl_ctas if world > 1 else None},
            "allreduce_ms_per_step": ar_ms,
            "clocks": clocks, "final_loss": last, "device_status": st,
        }
        if dp_parity is not None:
            line["dp_parity"] = dp_parity
        if replicas_identical is not None:
            line["replicas_identical"] = bool(replicas_identical)
        if world == 1 and not args.no_extras:
            del model, step, dev
            torch.cuda.empty_cache()
            line["op_headline"] = headline_op(torch, peaks, local)
            torch.cuda.empty_cache()
            line["gpu_eager_baseline"] = gpu_eager_projection(torch, line["op_headline"])
            torch.cuda.empty_cache()
            ref = cpu_reference(1, 0, keep_grads=True)
            line["cpu_baseline"] = {"value": ref["tokens_per_s"], "unit": UNIT, "cores": ref["threads"],
                                    "kind": "port", "sample": ref["sample"], "s_per_step": ref["s_per_step"]}
            line["parity"] = parity_against_oracle(torch, ref)
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


_OUT_FD = 1


def claim_stdout() -> None:
    """File descriptor 1 carries the one JSON line and nothing else: whatever a library prints
    to stdout from here on (NCCL's version banner, for one) is sent to stderr instead."""
    global _OUT_FD
    sys.stdout.flush()
    _OUT_FD = os.dup(1)
    os.dup2(2, 1)


def emit(line: dict) -> None:
    os.write(_OUT_FD, (json.dumps(line) + "\n").encode())


def main():
    global WORKLOAD, SEQ_LEN, MICRO_BATCH, CONFIG_NO
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true",
                    help="skip op_headline, gpu_eager_baseline, cpu_baseline, parity and the DP probe")
    ap.add_argument("--workload", default=WORKLOAD, choices=sorted(WORKLOAD_SHAPES),
                    help="baseline configuration to step (default: configuration 4, the one the metric is quoted on)")
    ap.add_argument("--allreduce", default="overlap", choices=["overlap", "blocking"],
                    help="N > 1: exchange gradients in buckets during backward, or once after it")
    ap.add_argument("--bucket-mb", type=int, default=256)
    ap.add_argument("--reserve-sms", type=int, default=0,
                    help="SMs the library's kernels leave free while a bucket is in flight (0 = none)")
    ap.add_argument("--nccl-ctas", type=int, default=0, help="NCCL max CTAs per collective (0 = NCCL's default)")
    ap.add_argument("--link-gbs", type=float, default=300.0,
                    help="all-reduce rate (GB/s of arena bytes) assumed when sizing the reservation window")
    # kernel-level modes
    ap.add_argument("--op", default=None, metavar="M,N,K,r", help="isolated projection kernels at one shape")
    ap.add_argument("--op-sweep", action="store_true", help="configuration 3 rank sweep: r in {8..128}, M=32768")
    ap.add_argument("--rows", action="store_true", help="row kernels and the factorized embedding")
    ap.add_argument("--routes", action="store_true",
                    help="both backward formulations of every projection group of every configuration")
    ap.add_argument("--what", default="all", help="--op: one kernel (prepass_T, fwd, prepass_U, dx, dw, merge, "
                    "dx_merged, dw_copy, adapter_grads, mlp_fwd, mlp_fwd_unfused, mlp_dx, mlp_dx_unfused); --rows: rmsnorm, swiglu, ce, adamw, embed, embed_fwd, embed_dproj")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--embed-tokens", type=int, default=16384)
    ap.add_argument("--seq", type=int, default=4096)
    args = ap.parse_args()
    WORKLOAD = args.workload
    SEQ_LEN, MICRO_BATCH, CONFIG_NO = WORKLOAD_SHAPES[WORKLOAD]
    if args.op or args.op_sweep:
        return run_op(args)
    if args.rows:
        return run_rows(args)
    if args.routes:
        return run_routes(args)
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        # launched without torchrun: start one rank per GPU ourselves
        port = 29500 + os.getpid() % 1000
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.abspath(__file__)] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    claim_stdout()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
