"""Reward shaping of the RL loop (host scalars): the effort-conditioned length penalty of
``trainer/effort.go`` and the format bonus of ``cmd/chat_rl/main.go:226-237``.

Everything here is per-rollout scalar arithmetic in float32 with the exponential taken in
float64, as the reference does; it runs on the host between the rollout and the advantage
kernel.  Token ids follow the reference's convention: the special tokens are the last eleven
ids of the vocabulary in the order of ``tokenizer/special.go:19-31``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

SPECIAL_TOKENS = ("<|bos|>", "<|user_start|>", "<|user_end|>", "<|assistant_start|>", "<|assistant_end|>", "<|tool_start|>",
                  "<|tool_end|>", "<|tool_output_start|>", "<|tool_output_end|>", "<|think_start|>", "<|think_end|>")


def special_id(vocab_size: int, name: str) -> int:
    """Id of a special token: they are appended after the mergeable ranks (tokenizer/tokenizer.go:33-56)."""
    return vocab_size - len(SPECIAL_TOKENS) + SPECIAL_TOKENS.index(name)


@dataclass
class EffortPenaltyConfig:
    """trainer/effort.go:8-22."""
    k0: float = 0.0
    lam: float = 0.0
    cap: float = 0.0
    norm: float = 0.0
    min_effort: int = 50
    mean_delta_effort: float = 25.0

    @classmethod
    def for_efforts(cls, efforts, k0, lam, cap, norm):
        """The configuration chat_rl derives from its effort list (cmd/chat_rl/main.go:75-85)."""
        cfg = cls(k0, lam, cap, norm)
        if efforts:
            cfg.min_effort = int(efforts[0])
            if len(efforts) > 1:
                cfg.mean_delta_effort = float(np.float32(efforts[-1] - efforts[0]) / np.float32(len(efforts) - 1))
        return cfg


def effort_penalty_coefficient(effort: int, config: EffortPenaltyConfig) -> np.float32:
    """k(b) = K0 * exp(-(b - b_min) / tau), tau = Lambda * MeanDeltaEffort; tau <= 0 disables the decay
    (trainer/effort.go:24-33)."""
    tau = np.float32(config.lam) * np.float32(config.mean_delta_effort)
    if tau <= 0:
        return np.float32(config.k0)
    delta = float(effort - config.min_effort) / float(tau)
    return np.float32(config.k0) * np.float32(math.exp(-delta))


def exponential_token_penalty(effort: int, length: int, config: EffortPenaltyConfig) -> np.float32:
    """r_len = -min(Cap, k(b) * length / Norm); zero when Norm, Cap or the length is not positive
    (trainer/effort.go:35-50)."""
    if config.norm <= 0 or config.cap <= 0 or length <= 0:
        return np.float32(0.0)
    penalty = effort_penalty_coefficient(effort, config) * np.float32(length) / np.float32(config.norm)
    if penalty > np.float32(config.cap):
        penalty = np.float32(config.cap)
    return np.float32(-penalty)


def reasoning_token_count(ids, vocab_size: int) -> int:
    """Tokens strictly inside <|think_start|> ... <|think_end|> spans (tokenizer/render.go:93-109)."""
    start, end = special_id(vocab_size, "<|think_start|>"), special_id(vocab_size, "<|think_end|>")
    count, inside = 0, False
    for token in ids:
        if token == start:
            inside = True
        elif token == end:
            inside = False
        elif inside:
            count += 1
    return count


def format_trace_reward(rollout, vocab_size: int, thinking: bool, bonus: float) -> np.float32:
    """The bonus for a well-formed, non-empty reasoning trace: format only (cmd/chat_rl/main.go:226-237)."""
    if not thinking or bonus == 0:
        return np.float32(0.0)
    if reasoning_token_count(rollout, vocab_size) == 0:
        return np.float32(0.0)
    if special_id(vocab_size, "<|think_end|>") not in [int(t) for t in rollout]:
        return np.float32(0.0)
    return np.float32(bonus)


def shaped_rewards(task_rewards, rollouts, prompt_lengths, vocab_size: int, efforts=None, penalty: EffortPenaltyConfig | None = None,
                   thinking: bool = False, format_bonus: float = 0.0) -> np.ndarray:
    """Reward of every rollout as chat_rl sums it (cmd/chat_rl/main.go:104-129): task reward + length penalty at the
    rollout's effort level (when effort conditioning is on) + format bonus.  ``rollouts`` are full id sequences
    (prompt + kept tokens); ``efforts`` is None or one effort level per rollout."""
    out = np.zeros(len(rollouts), np.float32)
    for i, rollout in enumerate(rollouts):
        reward = np.float32(task_rewards[i])
        if efforts is not None and penalty is not None:
            length = reasoning_token_count(rollout, vocab_size) if thinking else len(rollout) - int(prompt_lengths[i])
            reward = np.float32(reward + exponential_token_penalty(int(efforts[i]), length, penalty))
        reward = np.float32(reward + format_trace_reward(rollout, vocab_size, thinking, format_bonus))
        out[i] = reward
    return out
