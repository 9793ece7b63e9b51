"""Seeded synthetic weights, prompts and rewards for the RL-step workloads.

There is no dataset or checkpoint: every benchmark and parity case runs on
inputs generated here.  Weights follow the configured workloads' rule "every
matrix ~ N(0, 0.02) from the seed"; the scalar parameters keep the values the
reference's ``InitWeights`` gives them (model/transformer.go:177-186) except
``smear_lambda``, which the reference initialises to 0 and its own smear tests
raise to 0.7 (model/smear_test.go:15) so that the smear path is exercised.
"""
from __future__ import annotations

import numpy as np

SPECIAL_TOKENS = 11  # tokenizer/special.go:19-31: the last 11 ids of the vocabulary


def dense_config(name: str) -> dict:
    """The dense-preset workloads (model/config.go:574-603 ConfigForDepthRatio shapes)."""
    if name == "c1":  # CPU-runnable plumbing step
        return dict(sequence_len=256, vocab_size=8192, n_layer=2, n_head=2, n_kv_head=1, embed_dim=128, rotary_dims=64,
                    window_pattern="L")
    if name == "d12":  # ConfigForDepthRatio(12, 32768, 64, 128, 2048, "SSSL", 3)
        return dict(sequence_len=2048, vocab_size=32768, n_layer=12, n_head=6, n_kv_head=2, embed_dim=768, rotary_dims=64,
                    window_pattern="SSSL")
    if name == "h128":  # small model with the d12 head geometry (head_dim 128, 2:1 grouped queries, partial rotary, a binding window)
        return dict(sequence_len=512, vocab_size=1024, n_layer=2, n_head=2, n_kv_head=1, embed_dim=256, rotary_dims=64,
                    window_pattern="SL")
    if name == "tiny":  # model/gradcheck_test.go:14-31 tinyTrainModel shape, GQA 2:1
        return dict(sequence_len=16, vocab_size=16, n_layer=2, n_head=2, n_kv_head=1, embed_dim=32, rotary_dims=0,
                    window_pattern="L")
    raise KeyError(name)


def latent_config(name: str) -> dict:
    """Latent-preset workloads (model/preset.go:120-128: absorbed MLA + DeepSeekMoE, grouped queries 2:1)."""
    if name == "latent-tiny":  # the scale of the reference's own MLA / MoE unit-test models
        return dict(sequence_len=32, vocab_size=96, n_layer=2, n_head=4, n_kv_head=2, embed_dim=64, window_pattern="L",
                    n_experts=4, experts_per_token=2, expert_hidden=32, shared_hidden=32, mla_latent=24, mla_rotary_dims=8)
    if name == "latent-small":  # head_dim 64, 8 experts: exercises the tensor-core products of the latent blocks
        return dict(sequence_len=256, vocab_size=2048, n_layer=3, n_head=4, n_kv_head=2, embed_dim=256, window_pattern="L",
                    n_experts=8, experts_per_token=2, expert_hidden=128, shared_hidden=128, mla_latent=128)
    if name == "c3":  # d_model 1024, 8 heads, latent 256, 8 layers, 1 shared + 16 routed experts of hidden 512, top-2
        return dict(sequence_len=1024, vocab_size=32768, n_layer=8, n_head=8, n_kv_head=4, embed_dim=1024, window_pattern="L",
                    n_experts=16, experts_per_token=2, expert_hidden=512, shared_hidden=512, mla_latent=256)
    raise KeyError(name)


def fill_weights(names, shape_of, seed: int, std: float = 0.02, smear_lambda: float = 0.7):
    """Yield (name, float32 array) for every parameter name, deterministically."""
    n_layer = max((int(n.split(".")[2]) for n in names if n.startswith("transformer.h.")), default=-1) + 1
    for index, name in enumerate(sorted(names)):
        rows, cols = shape_of(name)
        count = rows * cols
        if name == "resid_lambdas":
            value = np.array([1.15 - 0.10 * np.float32(l) / np.float32(max(n_layer - 1, 1)) for l in range(n_layer)], np.float32)
        elif name == "x0_lambdas":
            value = np.array([0.20 - 0.15 * np.float32(l) / np.float32(max(n_layer - 1, 1)) for l in range(n_layer)], np.float32)
        elif name == "smear_lambda":
            value = np.array([smear_lambda], np.float32)
        elif name == "backout_lambda":
            value = np.array([0.2], np.float32)
        else:
            gen = np.random.Generator(np.random.Philox(key=[seed, index]))
            value = (gen.standard_normal(count, dtype=np.float32) * np.float32(std)).astype(np.float32)
        yield name, value


def prompts(n_prompts: int, prompt_len: int, vocab: int, seed: int) -> np.ndarray:
    """Uniform-random prompt ids that avoid the special ids (a prompt never starts inside a tool/think span)."""
    gen = np.random.Generator(np.random.Philox(key=[seed, 0xC0FFEE]))
    return gen.integers(0, vocab - SPECIAL_TOKENS, size=(n_prompts, prompt_len), dtype=np.int32)


def bernoulli_rewards(n_rollouts: int, seed: int) -> np.ndarray:
    """One Bernoulli(0.5) reward per rollout, drawn from the seed."""
    gen = np.random.Generator(np.random.Philox(key=[seed, 0xBEEF]))
    return (gen.random(n_rollouts, dtype=np.float32) < 0.5).astype(np.float32)


def contains_token_rewards(tokens: np.ndarray, lengths: np.ndarray, token_id: int = 7) -> np.ndarray:
    """Reward 1 when the generated part of a rollout contains ``token_id`` (what chat_rl scores, cmd/chat_rl/main.go:107)."""
    out = np.zeros(len(lengths), np.float32)
    for row, length in enumerate(lengths):
        out[row] = 1.0 if np.any(tokens[row, :length] == token_id) else 0.0
    return out
