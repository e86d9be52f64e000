"""Benchmark of the shared-W + LoRA linear hot path inside its training step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    torchrun --nnodes=1 --nproc-per-node N ... bench.py --gpus N --steps K --warmup W

Workload (N = 1 and every N, weak scaling): baseline configuration 1, the Qwen3-0.6B-shape
weight-shared decoder (hidden 1024, SwiGLU 3072, 28 layers over 4 shared blocks, 16/8 heads
of 128, LoRA r=16 on all seven projections, factorized embedding r_e=256, vocab 151936),
sequence 4096, micro-batch 8 per GPU, uniform token ids, random-init weights, AdamW step.
A "step" is one full optimisation step (forward, loss, backward, gradient all-reduce, clip,
AdamW) over one batch. Synthetic token ids stand in for the C4 stream the reference trains on.

One JSON line on stdout (rank 0). `value` = whole-job tokens/s with tokens already resident
in HBM; `e2e` = the same step driven from pinned host buffers (H2D of tokens/labels and D2H
of the loss inside the timed region); `roofline` = the dominant kernel of this library by
device time inside the timed region (CUDA events on the launching stream), against the
measured bf16 tensor peak; `op_headline` = the isolated fused projection fwd+bwd at the
configuration-4 MLP shapes (M = 16384), the figure the baseline's target is quoted on;
`cpu_baseline` = the CPU oracle (eager PyTorch restatement of the reference path) on the
host cores for a bounded sample.

`--impl reference` times that CPU eager path alone (the reference has no other
implementation of this path that runs without a GPU-side rewrite).
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

WORKLOAD = "qwen3-0.6b-ws"
SEQ_LEN = 4096
MICRO_BATCH = 8
# (sequence length, micro-batch per GPU) of the other baseline configurations, for --workload
WORKLOAD_SHAPES = {"qwen3-0.6b-ws": (4096, 8), "qwen3-1.7b-ws": (4096, 8), "qwen3-4b-ws": (8192, 4),
                   "qwen3-8b-ws": (8192, 2)}
METRIC = "step_tokens_per_s"
UNIT = "tokens/s"

# Measured DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) over algorithmic bytes
# of one launch, from the ncu captures summarised in
# profiles/block_gemm_pair_fwd_dx_dw_M8192_N8192_K4096_r64.md (M=N=8192, K=4096, r=64). The
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


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms during the timed region."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
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
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [c.strip() for c in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for nm, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------- CPU baseline
def cpu_reference_step(sample_tokens: int, steps: int, warmup: int):
    """The oracle's eager decoder step (fwd + loss + bwd, fp32, all host threads) on one
    sequence of `sample_tokens` tokens. Returns (tokens/s, seconds per step, threads)."""
    import torch
    from oracle import lora_oracle as O
    from weightshared_torchtitan_b200.decoder import CONFIGS
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    c = CONFIGS[WORKLOAD]
    a = O.DecoderArgs(dim=c.dim, hidden_dim=c.hidden_dim, n_layers=c.n_layers, n_unique=c.n_unique,
                      n_heads=c.n_heads, n_kv_heads=c.n_kv_heads, head_dim=c.head_dim, rank=c.rank,
                      vocab_size=c.vocab_size, embed_rank=c.embed_rank, max_seq_len=sample_tokens)
    p = {k: v.requires_grad_(True) for k, v in O.init_decoder_params(a, seed=1235).items()}
    g = torch.Generator().manual_seed(1)
    tokens = torch.randint(0, a.vocab_size, (1, sample_tokens), generator=g)
    labels = torch.randint(0, a.vocab_size, (1, sample_tokens), generator=g)
    times = []
    for i in range(warmup + steps):
        for v in p.values():
            v.grad = None
        t0 = time.perf_counter()
        loss = O.decoder_loss(a, p, tokens, labels)
        loss.backward()
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    sec = sum(times) / len(times)
    return sample_tokens / sec, sec, threads


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = 256
    tps, sec, threads = cpu_reference_step(sample, max(1, min(args.steps, 3)), 1)
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus,
        "steps": max(1, min(args.steps, 3)), "warmup": 1, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{WORKLOAD} decoder step (baseline config 1) on host cores",
                   "seq_len": sample, "micro_batch": 1},
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"1 sequence x {sample} tokens, all 28 layers + head, fwd+loss+bwd, fp32 eager"},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# ------------------------------------------------------------------------ our arm
def headline_op(ops, torch, peaks):
    """Isolated fused projection fwd+bwd through the autograd Function (pre-pass T, forward;
    merged weight, dX, dW, dA, dB) at the configuration-4 MLP shapes, M = 16384, r = 64; inputs
    (>= 670 MB) exceed the 126 MB L2."""
    from weightshared_torchtitan_b200 import functional as Fn
    out = {}
    for name, (M, N, K, r) in {"gate_up_12288x4096": (16384, 12288, 4096, 64),
                               "down_4096x12288": (16384, 4096, 12288, 64)}.items():
        g = torch.Generator(device="cuda").manual_seed(1238)
        bf = torch.bfloat16
        x = torch.randn(M, K, device="cuda", generator=g).to(bf)
        W = (torch.randn(N, K, device="cuda", generator=g) * 0.02).to(bf)
        A = ((torch.rand(r, K, device="cuda", generator=g) * 2 - 1) / K ** 0.5).to(bf)
        B = (torch.randn(N, r, device="cuda", generator=g) * 0.02).to(bf)
        dY = torch.randn(M, N, device="cuda", generator=g).to(bf)
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
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        e0.record()
        for _ in range(reps):
            run()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        flops = 6.0 * M * N * K + 6.0 * M * r * (K + N)
        tf = flops / ms / 1e9
        out[name] = {"ms": ms, "tflops": tf, "frac_of_2.25PF": tf / 2250.0,
                     "frac_of_measured_burst": tf / peaks["tf_burst"]}
        del x, W, A, B, dY, dW, dA, dB
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist
    from weightshared_torchtitan_b200 import _lib, ops
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
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    _lib.lib()
    peaks = load_peaks()

    c = CONFIGS[WORKLOAD]
    model = WeightSharedDecoder(c).cuda()
    model.init_weights(seed=1235)
    step = TrainStep(model, lr=3e-4)
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

    for i in range(args.warmup):
        step(*dev[i % nbatch])
    sync_all()

    # ---- timed region 1: device-resident inputs, per-launch kernel timing on
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    records = []
    ops.set_timing(records)
    n0 = _lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    e0.record()
    for i in range(args.steps):
        loss = step(*dev[i % nbatch])
    e1.record()
    sync_all()
    ops.set_timing(None)
    launches = _lib.launch_count() - n0
    ms_dev = e0.elapsed_time(e1)

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

    times = torch.tensor([ms_dev, ms_e2e], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_dev, ms_e2e = times.tolist()

    if rank == 0:
        st, words = _lib.poll_status()
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
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_dev / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{WORKLOAD} decoder training step (baseline config "
                                   f"{list(WORKLOAD_SHAPES).index(WORKLOAD) + 1})",
                       "seq_len": SEQ_LEN,
                       "micro_batch_per_gpu": MICRO_BATCH, "global_batch": MICRO_BATCH * world,
                       "parallelism": f"dp{world}",
                       "l2": "per-step activations and weights (tens of GB) exceed the 126 MB L2; no flush needed"},
            "e2e": {"value": e2e_v, "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": 2 * MICRO_BATCH * SEQ_LEN * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches) * world,
            "roofline": roofline,
            "kernels": {k: {"launches": v["launches"], "ms_per_step": v["ms"] / args.steps,
                            "tflops": v["flops"] / v["ms"] / 1e9 if v["flops"] else None,
                            "gbs": v["bytes"] / v["ms"] / 1e6} for k, v in sorted(kinds.items())},
            "wsl_kernel_share_of_step": kernel_ms / ms_dev,
            "model_tflops_per_gpu": fpt["total"] * tokens_per_step * args.steps / (ms_dev / 1e3) / 1e12,
            "linear_tflops_per_gpu_in_step": fpt["linear"] * tokens_per_step * args.steps / (kernel_ms / 1e3) / 1e12,
            "frac_of_linear_only_roofline_2.25PF": value / world / (2.25e15 / fpt["linear"]),
            "clocks": clocks, "final_loss": last, "device_status": st,
        }
        if world == 1 and not args.no_extras:
            line["op_headline"] = headline_op(ops, torch, peaks)
            del model, step
            tps, sec, threads = cpu_reference_step(256, 1, 1)
            line["cpu_baseline"] = {"value": tps, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": "1 sequence x 256 tokens, all 28 layers + head, fwd+loss+bwd, "
                                              "fp32 eager oracle", "s_per_step": sec}
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
    global WORKLOAD, SEQ_LEN, MICRO_BATCH
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip op_headline and cpu_baseline (N=1)")
    ap.add_argument("--workload", default=WORKLOAD, choices=sorted(WORKLOAD_SHAPES),
                    help="baseline configuration to step (default: configuration 1, the contract workload)")
    args = ap.parse_args()
    WORKLOAD = args.workload
    SEQ_LEN, MICRO_BATCH = WORKLOAD_SHAPES[WORKLOAD]
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
