"""The oracle's training pass through latent attention and routed experts, held to the reference's own checks:
finite-difference gradient checks (model/moe_test.go:261-362, model/mla_test.go:190-234) and train-forward ==
inference-forward (model/moe_test.go:221-258, model/mla_test.go:279-318).  The reference pins no value here; these
are the invariants its tests assert."""
import numpy as np
import pytest

from gonano_b200 import synthetic

VARIANTS = {
    "latent": {},
    "moe-only": dict(mla_latent=0, mla_rotary_dims=0),
    "mla-only": dict(n_experts=0, experts_per_token=0, expert_hidden=0, shared_hidden=0),
}


def build(oracle, variant, seed=3, std=0.15):
    cfg = dict(synthetic.latent_config("latent-tiny")); cfg.update(VARIANTS[variant])
    om = oracle.Model(**cfg)
    for n, v in synthetic.fill_weights(om.names, om.shape, seed, std=std):
        om.param(n)[:] = v
    return om, cfg


def batch(cfg, B=2, T=8):
    rng = np.random.default_rng(1)
    V = cfg["vocab_size"]
    ids = rng.integers(0, V - 11, (B, T), dtype=np.int32)
    tg = rng.integers(0, V, (B, T)).astype(np.int32); tg[:, :2] = -1
    return ids, tg, np.array([1.0, -0.7], np.float32)


@pytest.mark.parametrize("variant", list(VARIANTS))
def test_train_forward_equals_inference_forward(oracle, variant):
    om, cfg = build(oracle, variant)
    ids, _, _ = batch(cfg)
    a = om.train_forward(ids).reshape(ids.shape + (-1,))
    b = om.forward(ids)
    assert np.max(np.abs(a - b)) <= 1e-3 * np.max(np.abs(b))      # MLA: absorbed vs un-absorbed construction, 1e-3 as mla_test.go:279-318


@pytest.mark.parametrize("variant", list(VARIANTS))
def test_directional_gradient_check(oracle, variant):
    """Every matrix that the latent preset adds (latent projections, shared SwiGLU expert, router, packed experts)
    plus the block's output projection, one random direction per tensor, central differences.  The step is 3e-4:
    expert selection is piecewise constant, and a larger step flips a top-k choice on this model.  The router
    correction bias is excluded (selection is piecewise constant in it, as the reference's test says)."""
    om, cfg = build(oracle, variant)
    ids, tg, adv = batch(cfg)
    T = ids.shape[1]
    om.zero_grad()
    om.policy_gradient_step(ids, tg, adv, float(T))
    grads = {n: om.grad(n).copy() for n in om.names}
    names = [n for n in om.names if (".mla_" in n or ".moe." in n or ".mlp." in n or n.endswith("attn.c_proj.weight")) and not n.endswith("router_bias")]
    assert names
    rng = np.random.default_rng(7)
    eps = 3e-4
    for n in names:
        p = om.param(n)
        direction = rng.standard_normal(p.size).astype(np.float32)
        base = p.copy()
        p[:] = base + eps * direction; plus = om.policy_gradient_step(ids, tg, adv, float(T))[0]
        p[:] = base - eps * direction; minus = om.policy_gradient_step(ids, tg, adv, float(T))[0]
        p[:] = base
        numeric = (plus - minus) / (2 * eps)
        analytic = float(np.dot(grads[n].astype(np.float64), direction.astype(np.float64)))
        assert abs(numeric - analytic) <= 5e-2 * (abs(analytic) + 1e-6) + 2e-3, (n, numeric, analytic)


def test_router_bias_gets_no_gradient_and_no_update(oracle):
    om, cfg = build(oracle, "latent")
    ids, tg, adv = batch(cfg)
    om.zero_grad()
    om.policy_gradient_step(ids, tg, adv, float(ids.shape[1]))
    bias_names = [n for n in om.names if n.endswith("router_bias")]
    before = {n: om.param(n).copy() for n in om.names}
    assert all(not np.any(om.grad(n)) for n in bias_names)
    oracle.Optimizer(om).step()
    for n in om.names:
        moved = np.any(om.param(n) != before[n])
        assert moved != n.endswith("router_bias"), n       # every tensor but the correction bias is updated (model/optimizer.go:83-93)
