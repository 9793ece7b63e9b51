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

Sub-workloads for profiling (each prints one small JSON line; `ncu` wraps these, never the whole benchmark):

    python bench.py --only decode --prompts 8 --tokens 4 [--eager]     # prefill + a few decode steps of the d12 model
    python bench.py --only train --rows 32                             # one training pass (forward, loss, backward)
    python bench.py --only kernel --kernel gemm_nt --dims 16384 3072 768   # one kernel on synthetic device data
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


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the 16384 x 3072 x 768 product under ncu
# (`bench.py --only kernel --kernel gemm_nt --dims 16384 3072 768`): 120.4 MB read + 157.5 MB written
GEMM_TRAFFIC_BYTES = 277851136
WORKLOAD = dict(name="d12", n_prompts=64, prompt_len=128, group=8, max_tokens=256, temperature=1.0, top_k=50, seed=0)
# the latent preset's workload (absorbed MLA rollout, un-absorbed MLA + DeepSeekMoE training): `--workload c3`, one GPU line
WORKLOAD_C3 = dict(name="c3", n_prompts=32, prompt_len=256, group=8, max_tokens=256, temperature=1.0, top_k=50, seed=0)
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
# threads.  The d12 step is far too long to run on the host (about an hour), so it is timed on a
# bounded sample and extrapolated linearly, labelled so; the plumbing step and the loss
# microbenchmark are small enough to run IN FULL on both arms and are reported as measured pairs.
# ---------------------------------------------------------------------------------------------
def _host_threads():
    # every host thread this process may use: a launcher such as torchrun sets OMP_NUM_THREADS=1, which would
    # otherwise time the CPU path on one core
    from oracle import oracle
    try:
        avail = len(os.sched_getaffinity(0))
    except AttributeError:
        avail = os.cpu_count() or 1
    oracle.set_threads(max(1, avail))
    return oracle.num_threads()


def cpu_baseline():
    from oracle import oracle
    w = WORKLOAD
    cfg = synthetic.dense_config(w["name"])
    threads = _host_threads()
    om = oracle.Model(mode=1, **cfg)
    for name, value in synthetic.fill_weights(om.names, om.shape, w["seed"]):
        om.param(name)[:] = value
    G, plen, new = w["group"], w["prompt_len"], w["max_tokens"]
    V = cfg["vocab_size"]
    prompt = synthetic.prompts(1, plen, V, w["seed"])
    t0 = time.perf_counter()
    cache0 = om.cache(1, plen)
    logits = om.forward_cached(cache0, prompt)
    t_prefill = time.perf_counter() - t0
    # decode at three context lengths (start, middle, end of the rollout), two steps each, median per length
    rng = np.random.default_rng(0)
    t_ctx = []
    for ctx_len in (plen, plen + new // 2, plen + new - 2):
        cache = om.cache(G, plen + new)
        cache.replicate_from(cache0)
        if ctx_len > plen:      # grow the cache to the wanted context with one batched forward (untimed)
            filler = rng.integers(0, V - 11, (G, ctx_len - plen), dtype=np.int32)
            om.forward_cached(cache, filler)
        ids = rng.integers(0, V - 11, (G, 1), dtype=np.int32)
        samples = []
        for step in range(2):
            t0 = time.perf_counter()
            lg = om.forward_cached(cache, ids)
            ids = oracle.sample_next_token(lg[:, 0], w["temperature"], w["top_k"], seeds=[0], group=G, step=step + 1).reshape(G, 1)
            samples.append(time.perf_counter() - t0)
        t_ctx.append(float(np.median(samples)))
    t_decode = float(np.mean(t_ctx))       # the context grows linearly over the rollout: mean of start / middle / end
    T = plen + new - 1
    n_train = 2
    inputs = rng.integers(0, V - 11, (n_train, T), dtype=np.int32)
    targets = np.roll(inputs, -1, axis=1).copy(); targets[:, :plen] = -1
    t0 = time.perf_counter()
    om.policy_gradient_step(inputs, targets, np.array([0.5, -0.5], np.float32), float(T + 1))
    t_train_row = (time.perf_counter() - t0) / n_train
    # optimizer step (optimizer/muon.go, sinkhorn.go): one update of each distinct matrix shape, scaled by how many the model has
    d, L, Vp, KV = cfg["embed_dim"], cfg["n_layer"], om.padded_vocab(), cfg["n_kv_head"] * (cfg["embed_dim"] // cfg["n_head"])

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
    t_opt = L * (2 * t_muon(d, d) + 2 * t_muon(KV, d) + t_muon(4 * d, d) + t_muon(d, 4 * d)) + t_sink(Vp, KV) * (2.0 * d / KV + n_ve)
    P = w["n_prompts"]
    step_s = P * (t_prefill + new * t_decode) + P * G * t_train_row + t_opt
    return {"value": 1.0 / step_s, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": (f"extrapolated, not measured whole: 1 prompt prefill ({t_prefill:.3f}s) + decode steps of {G} rows at contexts {plen}, "
                       f"{plen + new // 2}, {plen + new - 2} (medians {t_ctx[0]:.4f} / {t_ctx[1]:.4f} / {t_ctx[2]:.4f}s, mean used) + "
                       f"train/loss/backward of {n_train} rows x {T} tokens ({t_train_row:.2f}s per row), scaled linearly to {P} prompts x {G} rows x "
                       f"{new} tokens; optimizer: one Muon update per matrix shape and one Sinkhorn update of a value-embedding table, scaled by "
                       f"count ({t_opt:.1f}s); oracle mode 1 (a C++ restatement of the structure of kernels/simd, not the reference's own "
                       f"binary), {oracle.isa()}, {threads} threads"),
            "step_seconds_extrapolated": step_s}


def plumbing_step_cpu():
    """The plumbing RL step (depth 2, d128, vocab 8192; 8 prompts x 32, G = 4, 32 new tokens, reward = contains id 7,
    std advantage, one optimizer step) IN FULL on the host: seconds for one step."""
    from oracle import oracle
    _host_threads()
    cfg = synthetic.dense_config("c1")
    om = oracle.Model(mode=1, **cfg)
    for name, value in synthetic.fill_weights(om.names, om.shape, 0):
        om.param(name)[:] = value
    V, P, PLEN, G, NEW = cfg["vocab_size"], 8, 32, 4, 32
    prompts = synthetic.prompts(P, PLEN, V, 1)
    opt = oracle.Optimizer(om)
    from gonano_b200.session import build_batch
    t0 = time.perf_counter()
    toks, lens = [], []
    for p in range(P):
        t, l, _, _ = om.generate(prompts[p], G, NEW, 1.0, 50, seed=40 + p)
        toks.append(t); lens.append(l)
    tokens, lengths = np.concatenate(toks), np.concatenate(lens)
    adv = oracle.advantage(synthetic.contains_token_rewards(tokens, lengths, 7), G, 1)
    inputs, targets, max_len = build_batch(prompts, G, tokens, lengths, V - 7)
    om.zero_grad()
    om.policy_gradient_step(inputs, targets, adv, float(max_len))
    opt.step()
    return time.perf_counter() - t0


def loss_microbench_cpu(rows=16384, vocab=65536, block=2048):
    """The loss microbenchmark (16384 x 65536 logits, 50% of the positions valid) IN FULL on the host, as passes over one
    `block`-row buffer of logits (every row is processed; the buffer is far larger than the caches): seconds."""
    from oracle import oracle
    _host_threads()
    rng = np.random.default_rng(0)
    z = rng.standard_normal((block, vocab), dtype=np.float32) * np.float32(3)
    logits = (np.float32(15) * np.tanh(z / np.float32(15))).astype(np.float32)
    del z
    total = 0.0
    for b0 in range(0, rows, block):
        targets = rng.integers(0, vocab, block).astype(np.int32)
        targets[rng.random(block) < 0.5] = -1
        adv = rng.standard_normal(block // 512).astype(np.float32)
        t0 = time.perf_counter()
        oracle.pg_loss_backward(logits, targets, adv, 512, float(rows // 2), mode=1)
        total += time.perf_counter() - t0
    return total


def measured_pairs(ctx):
    """Workloads small enough to run whole on both arms: (config, cpu seconds, gpu seconds)."""
    from gonano_b200.session import Model, rl_step
    pairs = []
    # plumbing step on the GPU through the public call
    cfg = synthetic.dense_config("c1")
    gm = Model(ctx, **cfg)
    for name, value in synthetic.fill_weights(gm.names, gm.shape, 0):
        gm.upload(name, value)
    gm.optimizer_init()
    prompts = synthetic.prompts(8, 32, cfg["vocab_size"], 1)
    seeds = np.arange(8, dtype=np.uint64) + 40
    reward_fn = lambda t, l: synthetic.contains_token_rewards(t, l, 7)
    times = []
    for _ in range(4):
        t0 = time.perf_counter()
        rl_step(gm, prompts, 4, 32, 1.0, 50, seeds, reward_fn, advantage_mode=1, optimizer=True)
        ctx.sync()
        times.append(time.perf_counter() - t0)
    gm.close()
    pairs.append({"config": "plumbing RL step (depth 2, d128, vocab 8192; 8 prompts x 32, G=4, 32 new tokens, one optimizer step), whole step, host buffers",
                  "cpu_s": plumbing_step_cpu(), "gpu_s": float(np.median(times[1:]))})
    ms = ctx.profile_kernel("loss", [16384, 65536, 50], 5)
    pairs.append({"config": "loss microbenchmark 16384 x 65536, 50% valid: log-probs, loss and dlogits (device-resident on the GPU arm)",
                  "cpu_s": loss_microbench_cpu(), "gpu_s": ms * 1e-3})
    for p in pairs:
        p["ratio"] = p["cpu_s"] / p["gpu_s"] if p["gpu_s"] else None
    return pairs


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    steps = [cpu_baseline() for _ in range(max(1, min(args.steps, 3)))]
    steps.sort(key=lambda s: s["value"])
    mid = steps[len(steps) // 2]     # the median sample
    line = {"impl": "reference", "metric": METRIC, "value": mid["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1000.0 / mid["value"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": "dense d12 RL step: 64 prompts x G=8, 128 prompt tokens, 256 new tokens, vocab 32768 (bounded sample, extrapolated)"},
            "cpu_baseline": mid, "e2e": {"value": mid["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
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

    # attention of one layer of a training pass (128 x 383 tokens, causal): 2 products forward; backward 5 products over
    # the causal half (S and dP in the score kernel, dV, dK, dQ as batched products), each 2*T^2/2*D flop per (row, head),
    # on tcgen05 in 3xTF32.  The backward is bound by the HBM traffic of the materialised P and dS, not by the tensor pipe.
    B, T = 128, 383
    unit = B * hq * (T * (T + 1) / 2.0) * d * 2.0
    for name, products, label, note in (
            ("attention_fwd", 2, "forward", "tcgen05: Q as the A operand in tensor memory, K/V by TMA, P through shared memory"),
            ("attention_bwd", 5, "backward (pack, P, dS, dV, dK, dQ)", "tcgen05 score kernel + batched products; 3.6 GB of P / dS traffic per call")):
        ms = ctx.profile_kernel(name, [B, hq, hkv, d, T], 10)
        tf = products * unit / (ms * 1e-3) / 1e12
        out.append({"kernel": name, "workload": f"d12 one layer of a training pass, {B} x {T} tokens, {label}", "bound": "tensor", "ms": ms,
                    "achieved": tf, "peak": gemm_peak, "unit": "TFLOP/s", "frac": tf / gemm_peak if gemm_peak else None, "note": note})
    # the global branch of a compressed attention layer at the flash preset's shape (8 192-token prompt + 512 new tokens, 8 query heads
    # on one kv head of 128, ratio 4): every query sees the blocks before its own, (T / ratio) / 2 on average; two products
    Bc, Hc, Tc, ratio = 4, 8, 8704, 4
    ms = ctx.profile_kernel("compressed_attention_fwd", [Bc, Hc, 1, d, Tc, ratio], 3)
    tf = 2 * Bc * Hc * Tc * ((Tc // ratio) / 2.0) * d * 2.0 / (ms * 1e-3) / 1e12
    out.append({"kernel": "compressed_attention_fwd", "workload": f"flash preset, one layer, {Bc} x {Tc} tokens over {Tc // ratio} compressed blocks, forward",
                "bound": "tensor", "ms": ms, "achieved": tf, "peak": gemm_peak, "unit": "TFLOP/s", "frac": tf / gemm_peak if gemm_peak else None,
                "note": "tcgen05 attention forward with the keys counted in blocks of `ratio` positions"})
    return out


def step_flop(cfg, w):
    """Useful floating-point work of one RL step: 2*M*N*K per product (the 3xTF32 split issues three times as many
    tensor-core flop), attention by the reference's own accounting (model/flops.go:107-117: 4*T_q*T_k*d per layer)."""
    d, L, Vp = cfg["embed_dim"], cfg["n_layer"], (cfg["vocab_size"] + 63) // 64 * 64
    D = d // cfg["n_head"]
    kv = cfg["n_kv_head"] * D
    per_layer = d * (d + 2 * kv) + d * d + 8 * d * d          # q,k,v, c_proj, c_fc + mlp c_proj
    p_mm = L * per_layer + Vp * d
    rows, plen, new = w["n_prompts"] * w["group"], w["prompt_len"], w["max_tokens"]
    T = plen + new - 1
    decode = 2.0 * p_mm * rows * new
    prefill = 2.0 * p_mm * w["n_prompts"] * plen
    train = 6.0 * p_mm * rows * T
    attn_train = 3.0 * L * rows * 4.0 * (T * (T + 1) / 2.0) * d      # forward + backward (2x)
    attn_decode = L * rows * 4.0 * d * sum(range(plen + 1, plen + new + 1))
    return decode + prefill + train + attn_train + attn_decode


def run_only(args):
    """Sub-workloads for profiling: one small JSON line each."""
    from gonano_b200.session import Context, Model
    ctx = Context(0)
    for item in args.option:
        name, value = item.split("=")
        ctx.set_option(name, int(value))
    if args.only == "kernel":
        ms = ctx.profile_kernel(args.kernel, args.dims, args.iters)
        emit({"only": "kernel", "kernel": args.kernel, "dims": args.dims, "ms": ms})
        return 0
    cfg = synthetic.latent_config(args.model) if args.model in ("c3", "latent-small", "latent-tiny") else synthetic.dense_config(args.model)
    model = Model(ctx, **cfg)
    for name, value in synthetic.fill_weights(model.names, model.shape, 0):
        model.upload(name, value)
    V = cfg["vocab_size"]
    if args.only == "decode":
        if args.eager:
            ctx.set_option("decode_graph", 0)
        prompts = synthetic.prompts(args.prompts, 128, V, 1)
        seeds = np.arange(args.prompts, dtype=np.uint64)
        for _ in range(2):
            tokens, lengths, steps, _ = model.generate_batch(prompts, 8, args.tokens, 1.0, 50, seeds)
        emit({"only": "decode", "rows": args.prompts * 8, "steps": steps, "prefill_ms": model.phase_ms("prefill"), "decode_ms": model.phase_ms("decode"),
              "ms_per_decode_step": model.phase_ms("decode") / max(steps - 1, 1)})
    else:
        rng = np.random.default_rng(0)
        T = 383
        ids = rng.integers(0, V - 11, (args.rows, T), dtype=np.int32)
        tg = np.roll(ids, -1, axis=1).copy(); tg[:, : T // 3] = -1
        adv = rng.standard_normal(args.rows).astype(np.float32)
        for _ in range(2):
            model.zero_grad()
            loss, _, _, _ = model.policy_gradient_step(ids, tg, adv, float(T + 1), rows_per_pass=args.rows)
        emit({"only": "train", "rows": args.rows, "seq": T, "loss": loss, "ms": {p: model.phase_ms(p) for p in ["train_forward", "loss", "train_backward"]}})
    model.close(); ctx.close()
    return 0


def run_ours(args):
    import torch
    import torch.distributed as dist
    from gonano_b200 import dist as gdist
    from gonano_b200.session import Context, Model, rl_step, build_batch
    from gonano_b200.backend import group_advantage

    rank, world, local = gdist.env_rank_world()
    torch.cuda.set_device(local)
    latent = args.workload == "c3"
    w = WORKLOAD_C3 if latent else WORKLOAD
    cfg = synthetic.latent_config(w["name"]) if latent else synthetic.dense_config(w["name"])
    if latent:
        args.lean = True      # the per-kernel rooflines, the CPU sample and the flop model below describe the dense d12 step
    stream = torch.cuda.Stream(device=local)
    ctx = Context(local, stream.cuda_stream)
    for item in args.option:
        name, value = item.split("=")
        ctx.set_option(name, int(value))
    if world > 1:
        # torch.distributed is the rendezvous (it hands rank 0's communicator id to the others) and the clock's
        # barrier; the gradient exchange itself runs inside the library (gn_model_grad_allreduce, NCCL)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
        box = [Context.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        ctx.comm_init(box[0], rank, world)
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
    phases = ["prefill", "decode", "train_forward", "loss", "train_backward", "allreduce", "optimizer"]
    state = {"step": 0}

    def one_step():
        seeds = np.arange(lo, hi, dtype=np.uint64) + np.uint64(1000 * state["step"])   # cmd/chat_rl seeds rollouts by step
        state["step"] += 1
        res = rl_step(model, prompts, G, w["max_tokens"], w["temperature"], w["top_k"], seeds, reward_fn, advantage_mode=0,
                      optimizer=True, data_parallel=world > 1)
        ph = {p: model.phase_ms(p) for p in phases if p != "allreduce"}
        ph["allreduce"] = model.phase_ms("allreduce") if world > 1 else 0.0
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

    # ---- untimed verification of the data-parallel run: replicas and the reduced gradient
    verify = {}
    if world > 1 and not args.lean:
        psum, _ = model.checksum()
        sums = [None] * world
        dist.all_gather_object(sums, psum)
        verify["replicas_identical"] = bool(all(v == sums[0] for v in sums))
        verify["replica_param_checksums"] = sums
        # one more rollout + policy-gradient step without the optimizer: the all-reduced gradient of the N shards against
        # the gradient rank 0 computes alone over all rows (same parameters, same rollouts, same padded length)
        seeds = np.arange(lo, hi, dtype=np.uint64) + np.uint64(777)
        tk, ln, _, _ = model.generate_batch(prompts, G, w["max_tokens"], w["temperature"], w["top_k"], seeds)
        gathered = [None] * world
        dist.all_gather_object(gathered, (tk, ln))
        tk_all = np.concatenate([g[0] for g in gathered]); ln_all = np.concatenate([g[1] for g in gathered])
        adv_all = group_advantage(rewards_all, G, 0)
        pad = cfg["vocab_size"] - 7
        max_len = w["prompt_len"] + int(ln_all.max())
        inputs, targets, _ = build_batch(prompts, G, tk, ln, pad, max_len)
        model.zero_grad()
        model.policy_gradient_step(inputs, targets, adv_all[lo * G:hi * G], float(max_len))
        model.grad_allreduce()
        address, count = model.grad_buffer()
        g_n = gdist.device_tensor(address, count, local).clone()
        dist.barrier()
        if rank == 0:
            inputs, targets, _ = build_batch(prompts_all, G, tk_all, ln_all, pad, max_len)
            model.zero_grad()
            model.policy_gradient_step(inputs, targets, adv_all, float(max_len))
            g_1 = gdist.device_tensor(address, count, local)
            verify["grad_vs_single_rank"] = float((g_n - g_1).abs().max() / g_1.abs().max())
        model.zero_grad()
        dist.barrier()
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
    if not args.lean and not latent:
        # the decode step itself, event-timed over a rollout of 64 tokens replayed from the CUDA graph: the full batch and the
        # shard an 8-GPU run gives each rank; bytes = the float32 weights once per step (what a step must at least stream)
        weight_bytes = 4.0 * sum(int(np.prod(model.shape(n))) for n in model.names if n.startswith("transformer.h.") and model.shape(n)[-1] > 1 and "ve" not in n) \
            + 4.0 * int(np.prod(model.shape("lm_head.weight")))
        for prompts_n in (64, 8):
            pp = synthetic.prompts(prompts_n, w["prompt_len"], cfg["vocab_size"], seed=77)
            sd = np.arange(prompts_n, dtype=np.uint64) + 900
            for _ in range(2):
                _, _, nsteps, _ = model.generate_batch(pp, w["group"], 64, w["temperature"], w["top_k"], sd)
            ms = model.phase_ms("decode") / max(nsteps - 1, 1)
            gbs = weight_bytes / (ms * 1e-3) / 1e9
            kernels.append({"kernel": "decode_step", "workload": f"d12, {prompts_n * w['group']} rows, 64 new tokens after a {w['prompt_len']}-token prompt (whole step, graph replay)",
                            "bound": "hbm", "ms": ms, "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"],
                            "note": "latency-bound chain of ~100 dependent launches; bytes counted = the float32 matmul weights once"})
    dominant = dict(kernels[0])
    # algorithmic bytes of that product: operands hi+lo 2 * 4 * (M*K + N*K) = 119.5 MB read, output 201.3 MB written
    dominant["traffic"] = GEMM_TRAFFIC_BYTES
    dominant["peak_source"] = f"TF32 8192^3 torch.matmul measured in this run ({tf32:.1f} TFLOP/s) / 3 for the 3xTF32 split" if tf32 else "unavailable"
    cpu, pairs = None, None
    if world == 1 and not args.no_cpu_baseline and not args.lean:
        try:
            cpu = cpu_baseline()
            pairs = measured_pairs(ctx)
            cpu["measured"] = pairs
        except Exception as exc:  # the oracle is test infrastructure: its absence must not hide the GPU number
            cpu = {"value": None, "unit": UNIT, "cores": None, "kind": "port", "sample": f"unavailable: {exc}"}
    steps_per_s_e2e = args.steps / (ms_total * 1e-3)
    steps_per_s_resident = args.steps / (ms_resident * 1e-3)
    rows = P * G
    T = w["prompt_len"] + w["max_tokens"] - 1
    h2d = P * w["prompt_len"] * 4 + P * 8 + 2 * rows * T * 4 + rows * 4 + rows * 4
    d2h = rows * w["max_tokens"] * 4 + rows * 4 + 8 + rows * 4
    flop = step_flop(cfg, w) if not latent else None
    step_tflops = flop / (ms_total / args.steps * 1e-3) / 1e12 if flop else None
    line = {
        "metric": METRIC if not latent else "rl_steps_per_s_c3", "value": steps_per_s_resident, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": ("latent preset RL step: 32 prompts x G=8 (256 rows), 256 prompt tokens, 256 new tokens, T=1.0, top-k 50, vocab 32768, "
                                "d1024 L8 Hq8, latent 256, 1 shared + 16 routed experts of hidden 512, top-2; absorbed-MLA rollout, un-absorbed MLA + MoE "
                                "training pass with the balance loss, optimizer step (per-expert Muon views)") if latent else
                               "dense d12 RL step: 64 prompts x G=8 (512 rows), 128 prompt tokens, 256 new tokens, T=1.0, top-k 50, "
                               "vocab 32768, d768 L12 Hq6 Hkv2; rollout + advantage + policy-gradient loss/backward + gradient all-reduce + "
                               "optimizer step (Sinkhorn / Muon / AdamW as cmd/chat_rl) + ZeroGrad",
                   "parallelism": f"dp{world}", "l2": "working set (705 MB weights, 4.8 GB KV cache, GBs of activations) is far larger than L2; no flush",
                   "gemm": "tcgen05 3xTF32"},
        "e2e": {"value": steps_per_s_e2e, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "rollout_tokens_per_s": tokens_total / (ms_total * 1e-3),
        "phase_ms_per_step": {p: phase_sum[p] / args.steps for p in phases},
        "wall_s": t_wall,
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": dominant,
        # the whole step against the same tensor roof: useful flop of one step / step time (all N GPUs) / (N x peak)
        "step_roofline": {"flop": flop, "tflops": step_tflops, "peak": (tf32 / 3.0 * world) if tf32 else None,
                          "frac": step_tflops / (tf32 / 3.0 * world) if (tf32 and step_tflops) else None,
                          "note": "useful flop of one whole step (products 2*M*N*K, attention 4*Tq*Tk*d per layer) / step time; the `roofline` object is one kernel"},
        "kernels": kernels,
        "cpu_baseline": cpu,
        "peaks": pk,
    }
    line.update(verify)
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
    ap.add_argument("--lean", action="store_true", help="steps only: no per-kernel microbenchmarks, TF32 peak, CPU baseline or replica checks")
    ap.add_argument("--workload", default="d12", choices=["d12", "c3"], help="d12: the dense step the metric is quoted on; c3: the latent preset's step")
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE", help="a gn_ctx_set_option switch, e.g. head_chunk_rows=8192 (repeatable)")
    ap.add_argument("--only", choices=["decode", "train", "kernel"], help="run one sub-workload for profiling instead of the benchmark")
    ap.add_argument("--model", default="d12"); ap.add_argument("--prompts", type=int, default=64); ap.add_argument("--tokens", type=int, default=4)
    ap.add_argument("--rows", type=int, default=32); ap.add_argument("--eager", action="store_true", help="--only decode: no CUDA-graph replay, so that a profiler sees every launch")
    ap.add_argument("--kernel", default="gemm_nt"); ap.add_argument("--dims", type=int, nargs="+", default=[16384, 3072, 768]); ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.only:
        return run_only(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
