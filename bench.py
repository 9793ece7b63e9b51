"""Benchmark of the RL step (trainer/rl.go driven by cmd/chat_rl) on B200.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N --steps K ...  # the CPU path, timed on the host cores

One "step" is one whole RL step on the dense d12 workload: rollout of 64 prompts x G=8 rows
(128 prompt tokens, 256 new tokens, temperature 1.0, top-k 50), Bernoulli(0.5) rewards, group
advantages, the teacher-forced policy-gradient loss with its backward, the gradient
all-reduce and the optimizer step with ZeroGrad (trainer/rl.go:62-67; chat_rl's MuonAdamW:
Sinkhorn for lm_head / wte / value embeddings, Muon for the block matrices, AdamW for the
scalars).  With N GPUs the 64 prompts are split into N contiguous shards (strong scaling: the
total work is fixed), one process per GPU, a full policy replica each.

Prints ONE JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from gonano_b200 import synthetic  # noqa: E402

_STDOUT_FD = None


def emit(line: dict) -> None:
    data = (json.dumps(line) + "\n").encode()
    if _STDOUT_FD is None:
        sys.stdout.write(data.decode()); sys.stdout.flush()
    else:
        os.write(_STDOUT_FD, data)


GEMM_TRAFFIC_BYTES = 277851136   # 120.4 MB read + 157.5 MB written: ncu capture of `profile_cli kernel gemm_nt 16384 3072 768` (profiles/gemm_tc_timeline.md)
WORKLOAD = dict(name="d12", n_prompts=64, prompt_len=128, group=8, max_tokens=256, temperature=1.0, top_k=50, seed=0)
METRIC, UNIT = "rl_steps_per_s_d12", "steps/s"


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        p = json.loads(path.read_text())
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"], source="measured (MEASURED_PEAKS.json)")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi during the timed region."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ---------------------------------------------------------------------------------------------
# CPU baseline: the oracle's SIMD-structured flavour (restatement of kernels/simd), all host
# threads, on a bounded sample of the same workload, extrapolated linearly to one full step.
# ---------------------------------------------------------------------------------------------
def cpu_baseline(sample_scale: int = 1):
    from oracle import oracle
    w = WORKLOAD
    cfg = synthetic.dense_config(w["name"])
    # every host thread this process may use: a launcher such as torchrun sets OMP_NUM_THREADS=1, which would
    # otherwise time the CPU path on one core
    try:
        avail = len(os.sched_getaffinity(0))
    except AttributeError:
        avail = os.cpu_count() or 1
    oracle.set_threads(max(1, avail))
    threads = oracle.num_threads()
    om = oracle.Model(mode=1, **cfg)
    for name, value in synthetic.fill_weights(om.names, om.shape, w["seed"]):
        om.param(name)[:] = value
    G, plen, new = w["group"], w["prompt_len"], w["max_tokens"]
    prompt = synthetic.prompts(1, plen, cfg["vocab_size"], w["seed"])
    t0 = time.perf_counter()
    cache0 = om.cache(1, plen)
    logits = om.forward_cached(cache0, prompt)
    t_prefill = time.perf_counter() - t0
    cache = om.cache(G, plen + new)
    cache.replicate_from(cache0)
    ids = oracle.sample_next_token(np.repeat(logits[:, -1], G, axis=0), w["temperature"], w["top_k"], seeds=[0], group=G, step=0)
    n_dec = 4 * sample_scale
    t0 = time.perf_counter()
    for step in range(n_dec):
        logits = om.forward_cached(cache, ids.reshape(G, 1))
        ids = oracle.sample_next_token(logits[:, 0], w["temperature"], w["top_k"], seeds=[0], group=G, step=step + 1)
    t_decode = (time.perf_counter() - t0) / n_dec
    T = plen + new - 1
    rng = np.random.default_rng(0)
    inputs = rng.integers(0, cfg["vocab_size"] - 11, (1, T), dtype=np.int32)
    targets = np.roll(inputs, -1, axis=1).copy(); targets[:, :plen] = -1
    t0 = time.perf_counter()
    om.policy_gradient_step(inputs, targets, np.array([0.5], np.float32), float(T + 1))
    t_train_row = time.perf_counter() - t0
    # optimizer step (optimizer/muon.go, sinkhorn.go): one update of each distinct matrix shape, scaled by how many the model has
    d, L, V, KV = cfg["embed_dim"], cfg["n_layer"], om.padded_vocab(), cfg["n_kv_head"] * (cfg["embed_dim"] // cfg["n_head"])

    def t_muon(rows, cols):
        p = (rng.standard_normal(rows * cols) * 0.02).astype(np.float32); g = (rng.standard_normal(rows * cols) * 0.01).astype(np.float32)
        t = time.perf_counter()
        oracle.muon_step(p, g, np.zeros_like(p), np.zeros(max(rows, cols), np.float32), rows, cols, lr=0.001, mode=1)
        return time.perf_counter() - t

    def t_sink(rows, cols):
        p = np.zeros(rows * cols, np.float32); g = (rng.standard_normal(rows * cols) * 0.01).astype(np.float32)
        t = time.perf_counter()
        oracle.sinkhorn_step(p, g, np.zeros_like(p), rows, cols, lr=0.001)
        return time.perf_counter() - t

    n_ve = sum(1 for n in om.names if n.startswith("value_embeds."))
    t_opt = L * (2 * t_muon(d, d) + 2 * t_muon(KV, d) + t_muon(4 * d, d) + t_muon(d, 4 * d)) + t_sink(V, KV) * (2.0 * d / KV + n_ve)
    P = w["n_prompts"]
    # decode cost grows with the context; the sample sits at the start of the rollout, so this is a lower bound
    step_s = P * (t_prefill + new * t_decode) + P * G * t_train_row + t_opt
    return {"value": 1.0 / step_s, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": (f"extrapolated: 1 prompt prefill ({t_prefill:.3f}s) + {n_dec} decode steps of {G} rows ({t_decode:.4f}s each) + "
                       f"train/loss/backward of 1 row x {T} tokens ({t_train_row:.2f}s), scaled to {P} prompts x {G} rows x {new} tokens; "
                       f"optimizer: one Muon update per matrix shape and one Sinkhorn update of a value-embedding table, scaled by count ({t_opt:.1f}s); "
                       f"oracle mode 1 (kernels/simd structure), {oracle.isa()}, {threads} threads"),
            "step_seconds_extrapolated": step_s}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    steps = []
    for i in range(max(1, min(args.steps, 2))):
        steps.append(cpu_baseline())
    best = max(steps, key=lambda s: s["value"])
    line = {"impl": "reference", "metric": METRIC, "value": best["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1000.0 / best["value"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": "dense d12 RL step: 64 prompts x G=8, 128 prompt tokens, 256 new tokens, vocab 32768 (bounded sample, extrapolated)"},
            "cpu_baseline": best, "e2e": {"value": best["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(line)
    return 0


# ---------------------------------------------------------------------------------------------
def kernel_rooflines(ctx, pk, tf32_tflops):
    """Each hot kernel beside the roofline that bounds it (CUDA events, synthetic data larger than L2)."""
    out = []
    hbm = pk["hbm_gbs"]
    gemm_peak = tf32_tflops / 3.0 if tf32_tflops else None

    def hbm_entry(name, dims, bytes_, workload):
        ms = ctx.profile_kernel(name, dims, 10)
        gbs = bytes_ / (ms * 1e-3) / 1e9
        out.append({"kernel": name, "workload": workload, "bound": "hbm", "ms": ms, "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm})

    def gemm_entry(name, m, n, k, workload):
        ms = ctx.profile_kernel(name, [m, n, k], 5)
        tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        out.append({"kernel": name, "workload": workload, "bound": "tensor", "ms": ms, "achieved": tf, "peak": gemm_peak, "unit": "TFLOP/s",
                    "frac": tf / gemm_peak if gemm_peak else None})

    gemm_entry("gemm_nt", 16384, 3072, 768, "train c_fc forward, 16384 tokens")
    gemm_entry("gemm_nt", 512, 32768, 768, "decode lm_head, 512 rows")
    gemm_entry("gemm_tn", 32768, 768, 16384, "lm_head weight gradient")
    # loss: C5 shape, half the rows valid: 4*V*(2*valid + masked) bytes
    rows, vocab = 16384, 65536
    hbm_entry("loss", [rows, vocab, 50], 4.0 * vocab * (2 * rows * 0.5 + rows * 0.5), "loss microbench 16384 x 65536, 50% valid")
    rows, vocab = 8192, 32768
    hbm_entry("loss", [rows, vocab, 67], 4.0 * vocab * (2 * rows * 0.67 + rows * 0.33), "d12 train pass 8192 x 32768, 67% valid")
    hbm_entry("sampler", [512, 32768, 50], 4.0 * 512 * 32768, "d12 decode step, 512 rows")
    r, hq, hkv, d, c = 512, 6, 2, 128, 320
    hbm_entry("decode_attention", [r, hq, hkv, d, c], r * (2.0 * hkv * d * 4 * c + 2 * hq * d * 4), "d12 one layer, 512 rows, context 320")
    # a long prompt (1024 positions) shared by each group of 8 rows: the prompt's keys are read once per group by the
    # shared-prefix pass, so the algorithmic bytes drop (short prompts such as d12's 128 tokens keep the per-row kernel)
    r2, c2, p2 = 256, 1088, 1024
    hbm_entry("decode_attention", [r2, hq, hkv, d, c2, 8, p2], (r2 / 8) * 2.0 * hkv * d * 4 * p2 + r2 * (2.0 * hkv * d * 4 * (c2 - p2) + 2 * hq * d * 4),
              "one layer, 256 rows, context 1088, shared 1024-token prefix per group of 8")
    hbm_entry("advantage", [64, 8], 8.0 * 512, "64 groups of 8 (latency-bound)")

    # attention of one training pass (32 x 383 tokens, causal): 2 products forward, 7 backward (S and dP are recomputed
    # in both backward kernels), each 2*T^2/2*D flop per (row, head), on the legacy mma.sync pipe in 3xTF32
    B, T = 32, 383
    unit = B * hq * (T * (T + 1) / 2.0) * d * 2.0
    for name, products, label in (("attention_fwd", 2, "forward"), ("attention_bwd", 7, "backward (dK/dV + dQ)")):
        ms = ctx.profile_kernel(name, [B, hq, hkv, d, T], 10)
        tf = products * unit / (ms * 1e-3) / 1e12
        out.append({"kernel": name, "workload": f"d12 one layer of a training pass, {B} x {T} tokens, {label}", "bound": "tensor", "ms": ms,
                    "achieved": tf, "peak": gemm_peak, "unit": "TFLOP/s", "frac": tf / gemm_peak if gemm_peak else None,
                    "note": "mma.sync m16n8k8 tf32; a dense loop of that instruction reaches 278/3 = 92 TFLOP/s useful on this GPU"})
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist
    from gonano_b200 import dist as gdist
    from gonano_b200.session import Context, Model, rl_step

    rank, world, local = gdist.env_rank_world()
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    w = WORKLOAD
    cfg = synthetic.dense_config(w["name"])
    stream = torch.cuda.Stream(device=local)
    ctx = Context(local, stream.cuda_stream)
    model = Model(ctx, **cfg)
    for name, value in synthetic.fill_weights(model.names, model.shape, w["seed"]):
        model.upload(name, value)
    P, G = w["n_prompts"], w["group"]
    lo, hi = gdist.shard_range(P, rank, world)
    prompts_all = synthetic.prompts(P, w["prompt_len"], cfg["vocab_size"], w["seed"])
    prompts = prompts_all[lo:hi]
    rewards_all = synthetic.bernoulli_rewards(P * G, w["seed"])

    def reward_fn(tokens, lengths):
        return rewards_all[lo * G:hi * G]

    model.optimizer_init()   # cmd/chat_rl/main.go:68-72
    all_reduce = gdist.GradAllReduce(model, local, stream) if world > 1 else None
    phases = ["prefill", "decode", "train_forward", "loss", "train_backward", "allreduce", "optimizer"]
    state = {"step": 0}

    def one_step():
        seeds = np.arange(lo, hi, dtype=np.uint64) + np.uint64(1000 * state["step"])   # cmd/chat_rl seeds rollouts by step
        state["step"] += 1
        res = rl_step(model, prompts, G, w["max_tokens"], w["temperature"], w["top_k"], seeds, reward_fn, advantage_mode=0,
                      all_reduce=all_reduce, max_len_fn=gdist.global_max_len if world > 1 else None, optimizer=True,
                      shard=(rank, world))
        ph = {p: model.phase_ms(p) for p in phases if p != "allreduce"}
        ph["allreduce"] = all_reduce.last_ms() if all_reduce is not None else 0.0
        return res, ph

    for _ in range(args.warmup):
        one_step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = ctx.launch_count()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    phase_sum = {p: 0.0 for p in phases}
    tokens = 0
    t_wall = time.perf_counter()
    with torch.cuda.stream(stream):
        start.record(stream)
        for _ in range(args.steps):
            res, ph = one_step()
            tokens += res.rollout_tokens
            for p in phases:
                phase_sum[p] += ph[p]
        end.record(stream)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t_wall = time.perf_counter() - t_wall
    clocks = sampler.stop()
    launches = ctx.launch_count() - launches0
    ms = start.elapsed_time(end)
    t = torch.tensor([ms, sum(phase_sum.values())], dtype=torch.float64, device=f"cuda:{local}")
    tok = torch.tensor([tokens], dtype=torch.int64, device=f"cuda:{local}")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(tok, op=dist.ReduceOp.SUM)
    ms_total, ms_resident = float(t[0]), float(t[1])
    tokens_total = int(tok[0])
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0

    pk = peaks()
    # TF32 dense peak by the same method the bf16 figure was measured with (a library GEMM, used
    # only as a roofline denominator): 8192^3, best of 10.
    tf32 = None
    try:
        if args.lean:
            raise RuntimeError("lean run")
        torch.backends.cuda.matmul.allow_tf32 = True
        a = torch.randn(8192, 8192, device=f"cuda:{local}"); b = torch.randn(8192, 8192, device=f"cuda:{local}")
        best = 1e9
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); torch.matmul(a, b); e1.record(); torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        tf32 = 2 * 8192 ** 3 / (best * 1e-3) / 1e12
        del a, b
    except Exception:
        pass
    kernels = kernel_rooflines(ctx, pk, tf32) if not args.lean else [{"kernel": "gemm_nt", "workload": "not measured (--lean)"}]
    dominant = dict(kernels[0])
    # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this product under ncu (profiles/gemm_tc_timeline.md);
    # algorithmic: operands hi+lo 2 * 4 * (M*K + N*K) = 119.5 MB read, output 201.3 MB written
    dominant["traffic"] = GEMM_TRAFFIC_BYTES
    dominant["peak_source"] = f"TF32 8192^3 torch.matmul measured in this run ({tf32:.1f} TFLOP/s) / 3 for the 3xTF32 split" if tf32 else "unavailable"
    cpu = None
    if world == 1 and not args.no_cpu_baseline and not args.lean:
        try:
            cpu = cpu_baseline()
        except Exception as exc:  # the oracle is test infrastructure: its absence must not hide the GPU number
            cpu = {"value": None, "unit": UNIT, "cores": None, "kind": "port", "sample": f"unavailable: {exc}"}
    steps_per_s_e2e = args.steps / (ms_total * 1e-3)
    steps_per_s_resident = args.steps / (ms_resident * 1e-3)
    rows = P * G
    T = w["prompt_len"] + w["max_tokens"] - 1
    h2d = P * w["prompt_len"] * 4 + P * 8 + 2 * rows * T * 4 + rows * 4 + rows * 4
    d2h = rows * w["max_tokens"] * 4 + rows * 4 + 8 + rows * 4
    line = {
        "metric": METRIC, "value": steps_per_s_resident, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "dense d12 RL step: 64 prompts x G=8 (512 rows), 128 prompt tokens, 256 new tokens, T=1.0, top-k 50, "
                               "vocab 32768, d768 L12 Hq6 Hkv2; rollout + advantage + policy-gradient loss/backward + gradient all-reduce + "
                               "optimizer step (Sinkhorn / Muon / AdamW as cmd/chat_rl) + ZeroGrad",
                   "parallelism": f"dp{world}", "l2": "working set (705 MB weights, 4.8 GB KV cache, GBs of activations) is far larger than L2; no flush",
                   "gemm": "tcgen05 3xTF32" if os.environ.get("GN_GEMM", "") != "simt" else "simt"},
        "e2e": {"value": steps_per_s_e2e, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "rollout_tokens_per_s": tokens_total / (ms_total * 1e-3),
        "phase_ms_per_step": {p: phase_sum[p] / args.steps for p in phases},
        "wall_s": t_wall,
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": dominant,
        "kernels": kernels,
        "cpu_baseline": cpu,
        "peaks": pk,
    }
    emit(line)
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    # Libraries (NCCL prints its version) write to stdout; the contract is ONE JSON line there,
    # so everything else goes to stderr and the line is written to the original descriptor.
    global _STDOUT_FD
    sys.stdout.flush()
    _STDOUT_FD = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--lean", action="store_true", help="steps only: no per-kernel microbenchmarks, TF32 peak or CPU baseline (for ncu launch lists)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
