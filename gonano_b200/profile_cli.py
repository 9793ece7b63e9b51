"""Small driver for profiling runs (the commands quoted in profiles/*.md):

    python -m gonano_b200.profile_cli kernel gemm_nt 8192 3072 768      # one kernel on synthetic data
    python -m gonano_b200.profile_cli train  --rows 32                   # one training pass of the d12 model
    python -m gonano_b200.profile_cli decode --prompts 64 --steps 4      # prefill + a few decode steps

Each mode prints timings measured with CUDA events; under ``ncu`` the same commands give the
launch list and the per-kernel counters.
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from . import synthetic
from .session import Context, Model


def make_model(ctx, name="d12", seed=0):
    cfg = synthetic.latent_config(name) if name in ("c3", "latent-tiny", "latent-small") else synthetic.dense_config(name)
    model = Model(ctx, **cfg)
    for pname, value in synthetic.fill_weights(model.names, model.shape, seed):
        model.upload(pname, value)
    return model, cfg


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="mode", required=True)
    k = sub.add_parser("kernel"); k.add_argument("name"); k.add_argument("dims", nargs="+", type=int); k.add_argument("--iters", type=int, default=3)
    t = sub.add_parser("train"); t.add_argument("--rows", type=int, default=32); t.add_argument("--seq", type=int, default=383)
    t.add_argument("--config", default="d12"); t.add_argument("--gemm", type=int, default=1)
    d = sub.add_parser("decode"); d.add_argument("--prompts", type=int, default=64); d.add_argument("--group", type=int, default=8)
    d.add_argument("--prompt-len", type=int, default=128); d.add_argument("--steps", type=int, default=4); d.add_argument("--config", default="d12")
    d.add_argument("--gemm", type=int, default=1)
    args = ap.parse_args()
    ctx = Context(0)
    if args.mode == "kernel":
        ms = ctx.profile_kernel(args.name, args.dims, args.iters)
        print(json.dumps({"kernel": args.name, "dims": args.dims, "ms": ms}))
        return
    ctx.set_gemm(args.gemm)
    model, cfg = make_model(ctx, args.config)
    V = cfg["vocab_size"]
    rng = np.random.default_rng(0)
    if args.mode == "train":
        ids = rng.integers(0, V - 11, (args.rows, args.seq), dtype=np.int32)
        tg = np.roll(ids, -1, axis=1).copy(); tg[:, : args.seq // 3] = -1
        adv = rng.standard_normal(args.rows).astype(np.float32)
        for _ in range(2):
            model.zero_grad()
            loss, _, _, _ = model.policy_gradient_step(ids, tg, adv, float(args.seq + 1), rows_per_pass=args.rows)
        print(json.dumps({"mode": "train", "rows": args.rows, "seq": args.seq, "loss": loss,
                          "ms": {p: model.phase_ms(p) for p in ["train_forward", "loss", "train_backward"]}}))
    else:
        prompts = synthetic.prompts(args.prompts, args.prompt_len, V, 0)
        seeds = np.arange(args.prompts, dtype=np.uint64)
        for _ in range(2):
            tokens, lengths, steps, _ = model.generate_batch(prompts, args.group, args.steps, 1.0, 50, seeds)
        print(json.dumps({"mode": "decode", "rows": args.prompts * args.group, "steps": steps,
                          "ms": {p: model.phase_ms(p) for p in ["prefill", "decode"]}}))


if __name__ == "__main__":
    main()
