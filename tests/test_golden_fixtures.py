"""tests/golden/rl_step_golden.npz (made by tests/golden/make_golden.py) against both sides:
the oracle must still produce it (CPU), and the CUDA library must match it through the C-ABI (GPU)
without the oracle being involved.  Integer results are exact; floating point within the RL step's
tolerances (logits 1e-3 max relative, log-probs / advantages / loss / gradients 1e-4)."""
import os

import numpy as np
import pytest

from gonano_b200 import synthetic

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "rl_step_golden.npz"))


def rel(got, want):
    got = np.asarray(got, np.float64); want = np.asarray(want, np.float64)
    return float(np.max(np.abs(got - want)) / max(np.max(np.abs(want)), 1e-30))


# ------------------------------------------------------------------ oracle vs fixture (CPU)
def test_oracle_reproduces_fixture(oracle):
    lg, un = G["sampler_logits"], G["sampler_uniforms"]
    assert np.array_equal(oracle.sample_next_token(lg, 1.0, 50, uniforms=un), G["sampler_topk50_T1"])
    assert np.array_equal(oracle.sample_next_token(lg, 0.7, 0, uniforms=un), G["sampler_topk0_T07"])
    assert np.array_equal(oracle.sample_next_token(lg, 0.0, 0, uniforms=un), G["sampler_greedy"])
    assert np.array_equal(oracle.sample_next_token(lg, 1.0, 50, seeds=np.array([11, 12], np.uint64), group=3, step=5), G["sampler_philox_seeded"])
    assert np.array_equal(oracle.advantage(G["adv_rewards"], 4, mode=0), G["adv_mean"])
    assert np.array_equal(oracle.advantage(G["adv_rewards"], 4, mode=1), G["adv_std"])
    loss, nll, grad = oracle.pg_loss_backward(G["pg_logits"], G["pg_targets"], G["pg_adv"], 7, 7.0)
    assert np.float32(loss) == G["pg_loss"] and np.array_equal(nll, G["pg_nll"]) and np.array_equal(grad, G["pg_grad"])
    for tag, cfg in (("dense", synthetic.dense_config("tiny")), ("latent", synthetic.latent_config("latent-tiny"))):
        m = oracle.Model(mode=0, **cfg)
        for name, value in synthetic.fill_weights(m.names, m.shape, 5, std=0.12):
            m.param(name)[:] = value
        assert np.array_equal(m.forward(G[f"{tag}_ids"]), G[f"{tag}_logits"])


def test_fixture_is_well_formed():
    assert G["sampler_topk50_T1"].dtype == np.int32 and G["sampler_logits"].shape == (6, 517)
    assert np.all(G["sampler_greedy"] == np.argmax(G["sampler_logits"], axis=1))      # T <= 0 is argmax (sampler.go:27-30)
    adv = G["adv_mean"].reshape(-1, 4)
    assert np.max(np.abs(adv.sum(1))) < 1e-5                                          # reward - group mean sums to zero
    ignored = G["pg_targets"] < 0
    assert np.all(G["pg_nll"][ignored] == 0) and np.all(G["pg_grad"][ignored] == 0)   # ignored rows carry nothing


# ------------------------------------------------------------------ CUDA library vs fixture (GPU)
@pytest.mark.gpu
def test_cuda_sampler_and_advantage_match_fixture():
    from gonano_b200 import backend
    lg, un = G["sampler_logits"], G["sampler_uniforms"]
    assert np.array_equal(backend.sample_next_token(lg, 1.0, 50, uniforms=un), G["sampler_topk50_T1"])
    assert np.array_equal(backend.sample_next_token(lg, 0.7, 0, uniforms=un), G["sampler_topk0_T07"])
    assert np.array_equal(backend.sample_next_token(lg, 0.0, 0, uniforms=un), G["sampler_greedy"])
    assert np.array_equal(backend.sample_next_token(lg, 1.0, 50, seeds=np.array([11, 12], np.uint64), group=3, step=5), G["sampler_philox_seeded"])
    assert rel(backend.group_advantage(G["adv_rewards"], 4, mode=0), G["adv_mean"]) <= 1e-6
    assert rel(backend.group_advantage(G["adv_rewards"], 4, mode=1), G["adv_std"]) <= 1e-4


@pytest.mark.gpu
def test_cuda_loss_matches_fixture():
    from gonano_b200 import backend
    loss, nll, grad = backend.pg_loss_backward(G["pg_logits"], G["pg_targets"], G["pg_adv"], 7, 7.0)
    scale = float(np.sum(np.abs(G["pg_nll"].reshape(3, 7) * G["pg_adv"][:, None])) / 7.0)
    assert abs(loss - float(G["pg_loss"])) <= 1e-4 * scale
    assert rel(nll, G["pg_nll"]) <= 1e-4 and rel(grad, G["pg_grad"]) <= 1e-4


@pytest.mark.gpu
@pytest.mark.parametrize("tag", ["dense", "latent"])
def test_cuda_forward_matches_fixture(tag):
    from gonano_b200.session import Context, Model
    cfg = synthetic.dense_config("tiny") if tag == "dense" else synthetic.latent_config("latent-tiny")
    ctx = Context(0)
    m = Model(ctx, **cfg)
    for name, value in synthetic.fill_weights(m.names, m.shape, 5, std=0.12):
        m.upload(name, value)
    assert rel(m.forward(G[f"{tag}_ids"]), G[f"{tag}_logits"]) <= 1e-3
    m.close(); ctx.close()
