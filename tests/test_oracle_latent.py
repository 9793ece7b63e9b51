"""The oracle's latent preset (absorbed MLA + DeepSeekMoE) against the properties the reference's own
tests assert for it; the reference pins no numeric value for these blocks, so the pins are the
equivalences below plus an independent numpy restatement of the routed experts.

  model/mla_test.go:279-293   absorbed inference == un-absorbed training construction   (1e-3)
  model/mla_test.go:297-317   decode through the latent cache == prefill                (1e-3)
  model/mla_test.go:403-415   nil-cache forward == cached forward                       (1e-5)
  model/moe_test.go:238-259   MoE decode == prefill                                     (1e-3)
  model/moe_test.go:409-441   scalar backend == simd backend
"""
import numpy as np
import pytest

from gonano_b200 import synthetic


def build(oracle, name="latent-tiny", mode=0, seed=3, std=0.15, **over):
    cfg = dict(synthetic.latent_config(name)); cfg.update(over)
    m = oracle.Model(mode=mode, **cfg)
    for pname, value in synthetic.fill_weights(m.names, m.shape, seed, std=std):
        m.param(pname)[:] = value
    return m, cfg


def test_parameter_table(oracle):
    m, cfg = build(oracle)
    lat, rope, hd = cfg["mla_latent"], cfg["mla_rotary_dims"], cfg["embed_dim"] // cfg["n_head"]
    assert m.shape("transformer.h.0.attn.mla_q_down.weight") == (lat, cfg["embed_dim"])
    assert m.shape("transformer.h.0.attn.mla_q_up.weight") == (cfg["n_head"] * (hd - rope), lat)
    assert m.shape("transformer.h.0.attn.mla_k_rope.weight") == (cfg["n_kv_head"] * rope, cfg["embed_dim"])
    assert m.shape("transformer.h.0.attn.mla_v_up.weight") == (cfg["n_kv_head"] * hd, lat)
    assert m.shape("transformer.h.1.moe.experts.down.weight") == (cfg["n_experts"] * cfg["embed_dim"], cfg["expert_hidden"])
    assert not any(n.startswith("value_embeds") for n in m.names)          # model/transformer.go:73
    assert not any(".attn.c_q." in n for n in m.names)


def test_absorbed_matches_unabsorbed(oracle):
    m, cfg = build(oracle)
    ids = np.random.default_rng(0).integers(0, cfg["vocab_size"], (2, 9)).astype(np.int32)
    a, b = m.forward(ids), m.forward_unabsorbed(ids)
    assert np.max(np.abs(a - b)) <= 1e-3 and np.max(np.abs(a)) > 0.1


def test_decode_matches_prefill_and_nil_cache(oracle):
    m, cfg = build(oracle)
    ids = np.random.default_rng(1).integers(0, cfg["vocab_size"], (2, 9)).astype(np.int32)
    full = m.forward(ids)
    cache = m.cache(2, 16)
    pre = m.forward_cached(cache, ids[:, :8]); dec = m.forward_cached(cache, ids[:, 8:9])
    assert np.max(np.abs(pre - full[:, :8])) <= 1e-5          # nil cache == cached
    assert np.max(np.abs(dec[:, 0] - full[:, 8])) <= 1e-3     # decode == prefill
    assert cache.position() == 9


def test_cache_replication(oracle):
    m, cfg = build(oracle)
    ids = np.random.default_rng(2).integers(0, cfg["vocab_size"], (1, 9)).astype(np.int32)
    c1 = m.cache(1, 16); m.forward_cached(c1, ids[:, :8])
    c3 = m.cache(3, 16); c3.replicate_from(c1)
    out = m.forward_cached(c3, np.repeat(ids[:, 8:9], 3, 0))
    assert np.array_equal(out[0], out[1]) and np.array_equal(out[0], out[2])
    assert np.max(np.abs(out[0, 0] - m.forward(ids)[0, 8])) <= 1e-3


def test_scalar_matches_simd(oracle):
    m0, cfg = build(oracle, mode=0); m1, _ = build(oracle, mode=1)
    ids = np.random.default_rng(3).integers(0, cfg["vocab_size"], (2, 12)).astype(np.int32)
    assert np.max(np.abs(m0.forward(ids) - m1.forward(ids))) <= 1e-3


def test_routed_experts_against_numpy(oracle):
    """model/moe.go:118-169 restated in numpy (float64): select on logits + bias, weight by softmax(logits)."""
    m, cfg = build(oracle)
    d, E, K, eh = cfg["embed_dim"], cfg["n_experts"], cfg["experts_per_token"], cfg["expert_hidden"]
    m.param("transformer.h.0.moe.router_bias")[:] = np.array([0.3, -0.2, 0.0, 0.1], np.float32)
    x = np.random.default_rng(4).normal(0, 1, (11, d)).astype(np.float32)
    got, sel = m.moe_forward(0, x)
    wr = m.param("transformer.h.0.moe.router.weight").reshape(E, d).astype(np.float64)
    bias = m.param("transformer.h.0.moe.router_bias").astype(np.float64)
    wg = m.param("transformer.h.0.moe.experts.gate.weight").reshape(E, eh, d).astype(np.float64)
    wu = m.param("transformer.h.0.moe.experts.up.weight").reshape(E, eh, d).astype(np.float64)
    wd = m.param("transformer.h.0.moe.experts.down.weight").reshape(E, d, eh).astype(np.float64)
    logits = x.astype(np.float64) @ wr.T
    probs = np.exp(logits - logits.max(1, keepdims=True)); probs /= probs.sum(1, keepdims=True)
    want = np.zeros((11, d))
    for r in range(11):
        order = sorted(range(E), key=lambda e: (-(logits[r, e] + bias[e]), e))[:K]
        assert list(sel[r]) == order
        for e in order:
            g = np.minimum(wg[e] @ x[r], 10.0); u = np.clip(wu[e] @ x[r], -10.0, 10.0)
            want[r] += probs[r, e] * (wd[e] @ (g / (1.0 + np.exp(-g)) * u))
    assert np.max(np.abs(got - want)) <= 1e-4 * max(1.0, np.max(np.abs(want)))
