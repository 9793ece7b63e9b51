"""Reward shaping (host scalars) against the reference's own checks: trainer/effort_test.go:8-41 and the format
bonus of cmd/chat_rl/main.go:226-237."""
import math

import numpy as np

from gonano_b200 import rewards as R


def test_effort_penalty_coefficient_decreases_with_effort():
    cfg = R.EffortPenaltyConfig(k0=1, lam=1, min_effort=50, mean_delta_effort=25)
    low, mid, high = (R.effort_penalty_coefficient(e, cfg) for e in (50, 75, 100))
    assert low > mid > high
    assert abs(float(mid / low) - math.exp(-1)) <= 1e-4          # tau = 25: +25 effort multiplies by e^-1
    assert R.effort_penalty_coefficient(90, R.EffortPenaltyConfig(k0=0.7, lam=0)) == np.float32(0.7)   # tau <= 0: no decay


def test_exponential_token_penalty():
    cfg = R.EffortPenaltyConfig(k0=1, lam=1, min_effort=50, mean_delta_effort=25, cap=0.5, norm=100)
    short, long_ = R.exponential_token_penalty(50, 10, cfg), R.exponential_token_penalty(50, 90, cfg)
    assert short > long_ and long_ < 0
    assert short == np.float32(-0.1)
    assert R.exponential_token_penalty(50, 100000, cfg) == np.float32(-0.5)      # the cap saturates the deduction
    assert R.exponential_token_penalty(100, 50, cfg) > R.exponential_token_penalty(50, 50, cfg)
    assert R.exponential_token_penalty(50, 0, cfg) == 0
    assert R.exponential_token_penalty(50, 10, R.EffortPenaltyConfig(k0=1, lam=1, cap=0.5, norm=0)) == 0


def test_config_from_effort_list():
    cfg = R.EffortPenaltyConfig.for_efforts([50, 75, 100], 0.1, 1.0, 0.5, 32)
    assert cfg.min_effort == 50 and cfg.mean_delta_effort == 25.0
    assert R.EffortPenaltyConfig.for_efforts([], 0.1, 1.0, 0.5, 32).min_effort == 50


def test_reasoning_count_and_format_bonus():
    V = 1000
    ts, te, ae = R.special_id(V, "<|think_start|>"), R.special_id(V, "<|think_end|>"), R.special_id(V, "<|assistant_end|>")
    assert (R.special_id(V, "<|bos|>"), ae, ts, te) == (V - 11, V - 7, V - 2, V - 1)
    rollout = [1, 2, ts, 5, 6, 7, te, 9, ae]
    assert R.reasoning_token_count(rollout, V) == 3
    assert R.format_trace_reward(rollout, V, True, 0.25) == np.float32(0.25)
    assert R.format_trace_reward(rollout, V, False, 0.25) == 0             # thinking off
    assert R.format_trace_reward([1, ts, te, 4], V, True, 0.25) == 0        # empty trace
    assert R.format_trace_reward([1, ts, 5, 6], V, True, 0.25) == 0         # never closed
    assert R.format_trace_reward(rollout, V, True, 0.0) == 0


def test_shaped_rewards_sum_like_chat_rl():
    V = 1000
    cfg = R.EffortPenaltyConfig.for_efforts([50, 100], 1.0, 1.0, 0.5, 10)
    rollouts = [[1, 2, 3, 4, 5, 6], [1, 2, 3, 4]]
    got = R.shaped_rewards([1.0, 0.0], rollouts, [2, 2], V, efforts=[50, 100], penalty=cfg)
    want0 = np.float32(1.0) + R.exponential_token_penalty(50, 4, cfg)
    want1 = np.float32(0.0) + R.exponential_token_penalty(100, 2, cfg)
    assert got[0] == want0 and got[1] == want1
    assert np.array_equal(R.shaped_rewards([1.0, 0.0], rollouts, [2, 2], V), np.array([1.0, 0.0], np.float32))
