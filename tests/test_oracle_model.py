"""Self-consistency of the oracle's dense model, following the reference's own invariants."""
import numpy as np
import pytest

from gonano_b200 import synthetic


def make(oracle, name, seed=1, std=0.1, mode=0, **over):
    cfg = dict(synthetic.dense_config(name)); cfg.update(over)
    m = oracle.Model(mode=mode, **cfg)
    for pname, value in synthetic.fill_weights(m.names, m.shape, seed, std=std):
        m.param(pname)[:] = value
    return m, cfg


# model/smear_test.go:30-80: a batched forward equals token-by-token decode within 1e-4
def test_batched_forward_matches_sequential_decode(oracle):
    m, cfg = make(oracle, "tiny")
    ids = np.array([[1, 5, 2, 8, 3, 7], [4, 4, 9, 0, 11, 2]], np.int32)
    full = m.forward(ids)
    cache = m.cache(2, 6)
    for t in range(6):
        step = m.forward_cached(cache, ids[:, t:t + 1])
        assert np.max(np.abs(step[:, 0] - full[:, t])) <= 1e-4
    assert cache.position() == 6


# model/moe_test.go:221-258 pattern for the dense model: train-forward == inference-forward
def test_train_forward_matches_inference_forward(oracle):
    m, cfg = make(oracle, "tiny")
    ids = np.array([[1, 5, 2, 8, 3, 7]], np.int32)
    assert np.max(np.abs(m.train_forward(ids).reshape(1, 6, -1) - m.forward(ids))) <= 1e-5


# inference/inference_test.go:110-123,412-440: prefill + replicate + decode equals naive recompute (greedy)
def test_engine_matches_naive_recompute(oracle):
    m, cfg = make(oracle, "tiny", sequence_len=32)
    prompt = np.array([1, 5, 2, 8], np.int32)
    toks, lens, steps, _ = m.generate(prompt, 2, 6, 0.0, 0, seed=3)
    seq = list(prompt)
    for t in range(int(lens[0])):
        nxt = int(np.argmax(m.forward(np.array([seq + [0]], np.int32)[:, :len(seq)] if len(seq) > 1 else None)[0, -1]))
        assert nxt == toks[0, t]
        seq.append(nxt)
    assert np.array_equal(toks[0, :lens[0]], toks[1, :lens[1]])


# model/gradcheck_test.go:193-236: directional finite-difference check of the whole model
@pytest.mark.parametrize("name", ["tiny"])
def test_directional_gradient_check(oracle, name):
    m, cfg = make(oracle, name)
    ids = np.array([[1, 5, 2, 8, 3, 7]], np.int32)
    tg = np.array([[5, 2, 8, 3, 7, 4]], np.int32)
    adv = np.array([1.0], np.float32)

    def loss():
        logits = m.train_forward(ids)
        l, _, _ = oracle.pg_loss_backward(logits, tg.reshape(-1), adv, 6, 6.0, want_grad=False)
        return l

    m.zero_grad()
    m.policy_gradient_step(ids, tg, adv, 6.0)
    rng = np.random.default_rng(0)
    dirs = {n: rng.standard_normal(m.param(n).size).astype(np.float32) for n in m.names}
    analytic = sum(float(np.dot(m.grad(n).astype(np.float64), dirs[n])) for n in m.names)
    eps = 1e-3
    for n in m.names: m.param(n)[:] += eps * dirs[n]
    lp = loss()
    for n in m.names: m.param(n)[:] -= 2 * eps * dirs[n]
    lm = loss()
    for n in m.names: m.param(n)[:] += eps * dirs[n]
    numeric = (lp - lm) / (2 * eps)
    assert abs(analytic - numeric) <= 0.05 * max(abs(analytic), abs(numeric)) + 1e-4, (analytic, numeric)


# model/gradcheck_test.go:394-443: per-element checks on named weights
@pytest.mark.parametrize("pname", ["resid_lambdas", "x0_lambdas", "backout_lambda", "transformer.h.0.attn.c_k.weight",
                                   "transformer.h.1.attn.ve_gate.weight", "value_embeds.1.weight", "transformer.h.0.mlp.c_fc.weight",
                                   "lm_head.weight", "transformer.wte.weight"])
def test_per_element_gradient_check(oracle, pname):
    m, cfg = make(oracle, "tiny")
    ids = np.array([[1, 5, 2, 8, 3, 7], [2, 2, 5, 1, 5, 9]], np.int32)
    tg = np.array([[5, 2, 8, 3, 7, 4], [-1, -1, 1, 5, 9, 3]], np.int32)
    adv = np.array([1.0, -0.5], np.float32)

    def loss():
        l, _, _ = oracle.pg_loss_backward(m.train_forward(ids), tg.reshape(-1), adv, 6, 8.0, want_grad=False)
        return l

    m.zero_grad()
    m.policy_gradient_step(ids, tg, adv, 8.0)
    g = m.grad(pname).copy()
    p = m.param(pname)
    idxs = np.argsort(-np.abs(g))[:3]
    for i in idxs:
        old = p[i]; eps = 1e-2 if abs(old) > 0.5 else 2e-3
        p[i] = old + eps; lp = loss(); p[i] = old - eps; lm = loss(); p[i] = old
        numeric = (lp - lm) / (2 * eps)
        assert abs(numeric - g[i]) <= 0.05 * max(abs(numeric), abs(g[i])) + 2e-4, (pname, i, numeric, g[i])


# trainer/sft_rl_test.go:53-87: B x T = 2 x 4, adv {1, -0.5}, norm 8: finite, some gradient non-zero
def test_policy_gradient_step_finite(oracle):
    m, cfg = make(oracle, "tiny")
    ids = np.array([[1, 2, 3, 4], [5, 6, 7, 8]], np.int32)
    tg = np.array([[2, 3, 4, 5], [6, 7, 8, 9]], np.int32)
    loss, _, _, _ = m.policy_gradient_step(ids, tg, np.array([1.0, -0.5], np.float32), 8.0)
    assert np.isfinite(loss)
    assert any(np.any(m.grad(n) != 0) for n in m.names)
    assert all(np.all(np.isfinite(m.grad(n))) for n in m.names)


def test_advantage_and_batch_assembly(oracle):
    r = np.array([1, 0, 0, 1, 1, 1, 0, 0], np.float32)
    a = oracle.advantage(r, 4, 0)
    assert np.allclose(a, [0.5, -0.5, -0.5, 0.5, 0.5, 0.5, -0.5, -0.5])
    a = oracle.advantage(r, 4, 1)
    assert np.allclose(a, np.array([0.5, -0.5, -0.5, 0.5, 0.5, 0.5, -0.5, -0.5]) / (0.5 + 1e-6), rtol=1e-6)
    toks = np.array([[1, 2, 3, 4, 5, 0], [1, 2, 3, 9, 0, 0]], np.int32)
    inputs, targets, max_len = oracle.build_batch(toks, [5, 4], [3, 3], 99)
    assert max_len == 5
    assert inputs.tolist() == [[1, 2, 3, 4], [1, 2, 3, 9]]
    # cmd/chat_rl/main.go:171-179: target index < prompt length is masked, pads are trained on
    assert targets.tolist() == [[-1, -1, -1, 5], [-1, -1, -1, 99]]
