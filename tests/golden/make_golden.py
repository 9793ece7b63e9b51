"""Writes tests/golden/rl_step_golden.npz: seeded inputs of the RL step's stages with the outputs of the scalar
oracle (oracle mode 0, the restatement of kernels/scalar and of the dense / latent model).

The reference is pure Go and cannot run in the build image, so these vectors are not reference outputs; they freeze
the oracle's answers, which are themselves pinned to the reference's known-answer tests (tests/test_oracle_golden.py).
The CPU suite checks the oracle against this file (it must not drift); the GPU suite checks the CUDA library against it
without needing the oracle build.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from gonano_b200 import synthetic  # noqa: E402
from oracle import oracle as O      # noqa: E402


def main():
    out = {}
    rng = np.random.default_rng(20240607)
    # ---- sampler (inference/sampler.go:16-77): logits + explicit uniforms -> indices
    logits = (rng.standard_normal((6, 517)) * 3).astype(np.float32)
    logits[2, 100:110] = logits[2, 100]                      # ties at the top-k threshold keep every tied entry
    uniforms = rng.random((6, 517), dtype=np.float32)
    out["sampler_logits"], out["sampler_uniforms"] = logits, uniforms
    out["sampler_topk50_T1"] = O.sample_next_token(logits, 1.0, 50, uniforms=uniforms)
    out["sampler_topk0_T07"] = O.sample_next_token(logits, 0.7, 0, uniforms=uniforms)
    out["sampler_greedy"] = O.sample_next_token(logits, 0.0, 0, uniforms=uniforms)
    out["sampler_philox_seeded"] = O.sample_next_token(logits, 1.0, 50, seeds=np.array([11, 12], np.uint64), group=3, step=5)
    # ---- group-relative advantage (cmd/chat_rl/main.go:137-154), both normalisations
    rewards = rng.integers(0, 2, 24).astype(np.float32)
    out["adv_rewards"] = rewards
    out["adv_mean"] = O.advantage(rewards, 4, mode=0)
    out["adv_std"] = O.advantage(rewards, 4, mode=1)
    # ---- policy-gradient loss and dlogits (trainer/rl.go:14-60) on softcapped logits
    B, T, V = 3, 7, 203
    z = (15.0 * np.tanh(rng.standard_normal((B * T, V)) * 3 / 15.0)).astype(np.float32)
    tg = rng.integers(0, V, B * T).astype(np.int32); tg[[0, 1, 9, 20]] = -1
    adv = rng.standard_normal(B).astype(np.float32)
    loss, nll, grad = O.pg_loss_backward(z, tg, adv, T, float(T))
    out["pg_logits"], out["pg_targets"], out["pg_adv"] = z, tg, adv
    out["pg_loss"], out["pg_nll"], out["pg_grad"] = np.float32(loss), nll, grad
    # ---- dense model forward (tiny) and latent model forward (latent-tiny)
    for tag, cfg in (("dense", synthetic.dense_config("tiny")), ("latent", synthetic.latent_config("latent-tiny"))):
        m = O.Model(mode=0, **cfg)
        for name, value in synthetic.fill_weights(m.names, m.shape, 5, std=0.12):
            m.param(name)[:] = value
        ids = rng.integers(0, cfg["vocab_size"], (2, 10)).astype(np.int32)
        out[f"{tag}_ids"] = ids
        out[f"{tag}_logits"] = m.forward(ids)
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "rl_step_golden.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
