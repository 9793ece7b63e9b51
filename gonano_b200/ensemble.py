"""Blended generation over several models (inference/ensemble.go:10-243): every member keeps its own KV cache, the
next-token logits are the weighted sum of the members' logits, and one token is sampled from the combined row.

Built on the step-wise rollout calls of the C-ABI: each member prefills and forwards on its own; the blend is an
axpy chain over the members' device-resident logits (`gn_scale` / `gn_add_scaled`), the first member samples from the
blended logits through its engine state machine, and the others follow its column.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import check


def normalized_weights(weights) -> np.ndarray:
    """Ensemble.normalizedWeights (inference/ensemble.go:38-60): negative weights count as zero; weights without mass
    become uniform."""
    w = np.maximum(np.asarray(weights, np.float32), np.float32(0))
    total = np.float32(0)
    for v in w:
        total = np.float32(total + v)
    if total <= 0:
        return np.full(len(w), np.float32(1) / np.float32(len(w)), np.float32)
    return (w / total).astype(np.float32)


class Ensemble:
    def __init__(self, members):
        """``members``: list of (session.Model, weight).  All members share one vocabulary and one context."""
        assert members, "inference: ensemble has no models"
        self.models = [m for m, _ in members]
        self.weights = normalized_weights([w for _, w in members])
        self.lib = _lib.load()

    def generate_batch(self, prompts, group, max_tokens, temperature, top_k, seeds, thinking=False, thinking_budget=0):
        """Ensemble.GenerateBatchWith for many prompts: kept tokens, lengths, masks, steps."""
        import torch
        lead = self.models[0]
        for m in self.models:
            m.rollout_begin(prompts, group, max_tokens, seeds, thinking=thinking, thinking_budget=thinking_budget)
        vocab = lead.vocab
        steps = 0
        blended = None
        while steps < max_tokens:
            address, rows, div = lead.rollout_logits()
            n = rows * vocab
            if blended is None or blended.numel() < n:
                blended = torch.empty(n, dtype=torch.float32, device=f"cuda:{lead.ctx.device}")
            # combined = sum_i w_i * logits_i, accumulated member by member in float32 (inference/ensemble.go:141-150)
            check(self.lib.gn_scale(C.c_void_p(blended.data_ptr()), C.c_void_p(address), float(self.weights[0]), n))
            for m, w in zip(self.models[1:], self.weights[1:]):
                a, r, d = m.rollout_logits()
                assert (r, d) == (rows, div)
                check(self.lib.gn_add_scaled(C.c_void_p(blended.data_ptr()), C.c_void_p(blended.data_ptr()), C.c_void_p(a), float(w), n))
            column, _, done = lead.rollout_sample(temperature, top_k, logits_device=blended.data_ptr())
            steps += 1
            if done or steps >= max_tokens:
                break
            lead.rollout_forward()
            for m in self.models[1:]:
                m.rollout_forward(column)
        tokens, lengths, masks = lead.rollout_end()
        for m in self.models[1:]:
            m.rollout_end()
        return tokens, lengths, masks, steps
