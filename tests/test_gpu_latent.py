"""The latent preset (absorbed MLA + DeepSeekMoE) of the resident session against the oracle:
forward logits and rollouts by teacher forcing, at the RL step's tolerances (logits <= 1e-3 max
relative error; sampled tokens bit-exact given the logits).  Training a latent-preset model is
outside this library and must be refused, not approximated.
"""
import numpy as np
import pytest

from gonano_b200 import synthetic

pytestmark = pytest.mark.gpu


def rel_err(got, want):
    got = np.asarray(got, np.float64); want = np.asarray(want, np.float64)
    return float(np.max(np.abs(got - want)) / max(np.max(np.abs(want)), 1e-30))


@pytest.fixture(scope="module")
def ctx():
    from gonano_b200.session import Context
    c = Context(0)
    yield c
    c.close()


def make_pair(oracle, ctx, name, seed=1, std=0.1, **over):
    from gonano_b200.session import Model
    cfg = dict(synthetic.latent_config(name)); cfg.update(over)
    om = oracle.Model(**cfg)
    gm = Model(ctx, **cfg)
    assert sorted(gm.names) == sorted(om.names)
    for pname, value in synthetic.fill_weights(om.names, om.shape, seed, std=std):
        assert gm.shape(pname) == om.shape(pname), pname
        om.param(pname)[:] = value
        gm.upload(pname, value)
    return om, gm, cfg


VARIANTS = {
    "latent": {},
    "moe-only": dict(mla_latent=0, mla_rotary_dims=0),                                       # routed experts over dense attention
    "mla-only": dict(n_experts=0, experts_per_token=0, expert_hidden=0, shared_hidden=0),    # latent attention over the dense MLP
}


@pytest.mark.parametrize("name,variant,std,B,T", [("latent-tiny", "latent", 0.15, 2, 9), ("latent-tiny", "moe-only", 0.15, 3, 12),
                                                  ("latent-tiny", "mla-only", 0.15, 2, 16), ("latent-small", "latent", 0.05, 2, 70),
                                                  ("latent-small", "latent", 0.05, 1, 200)])
def test_forward_logits(oracle, ctx, name, variant, std, B, T):
    om, gm, cfg = make_pair(oracle, ctx, name, std=std, **VARIANTS[variant])
    ids = np.random.default_rng(0).integers(0, cfg["vocab_size"] - 11, (B, T), dtype=np.int32)
    assert rel_err(gm.forward(ids), om.forward(ids)) <= 1e-3
    gm.close()


@pytest.mark.parametrize("name,std,P,plen,G,maxtok", [("latent-tiny", 0.15, 2, 5, 3, 6), ("latent-small", 0.05, 2, 40, 4, 10)])
def test_rollout_by_teacher_forcing(oracle, ctx, name, std, P, plen, G, maxtok):
    om, gm, cfg = make_pair(oracle, ctx, name, std=std)
    V = cfg["vocab_size"]
    prompts = synthetic.prompts(P, plen, V, seed=4)
    seeds = np.arange(P, dtype=np.uint64) + 100
    tokens, lengths, steps, slog = gm.generate_batch(prompts, G, maxtok, 1.0, 50, seeds, want_logits=True)
    assert steps >= 1 and np.all(lengths <= maxtok)
    for p in range(P):
        cache0 = om.cache(1, plen)
        last = om.forward_cached(cache0, prompts[p:p + 1])[:, -1]
        cache = om.cache(G, plen + maxtok)
        cache.replicate_from(cache0)
        cur = np.repeat(last, G, axis=0)
        done = np.zeros(G, bool)
        kept = [[] for _ in range(G)]
        for step in range(steps):
            rows = slice(p * G, (p + 1) * G)
            assert rel_err(slog[step, rows], cur) <= 1e-3, (p, step)
            drawn = oracle.sample_next_token(slog[step, rows], 1.0, 50, seeds=seeds[p:p + 1], group=G, step=step)
            for g in range(G):
                if not done[g]:
                    if drawn[g] in (V - 11, V - 7): done[g] = True
                    else: kept[g].append(int(drawn[g]))
            if step + 1 == steps: break
            cur = om.forward_cached(cache, drawn.reshape(G, 1))[:, 0]
        for g in range(G):
            r = p * G + g
            assert kept[g] == tokens[r, :lengths[r]].tolist(), (p, g)
    gm.close()


def test_graph_replayed_rollout_matches_eager(oracle, ctx):
    """Without the logits tap the decode loop is replayed from a CUDA graph: same tokens."""
    om, gm, cfg = make_pair(oracle, ctx, "latent-small", std=0.05)
    prompts = synthetic.prompts(2, 24, cfg["vocab_size"], seed=5)
    seeds = np.array([7, 8], np.uint64)
    t1, l1, s1, _ = gm.generate_batch(prompts, 3, 12, 1.0, 50, seeds, want_logits=True)
    t2, l2, s2, _ = gm.generate_batch(prompts, 3, 12, 1.0, 50, seeds)
    assert np.array_equal(l1, l2)
    for r in range(6):
        assert np.array_equal(t1[r, :l1[r]], t2[r, :l2[r]])
    gm.close()


@pytest.mark.parametrize("name,variant,std,B,T,rpp", [("latent-tiny", "latent", 0.15, 2, 8, 0), ("latent-tiny", "moe-only", 0.15, 3, 12, 2),
                                                       ("latent-tiny", "mla-only", 0.15, 2, 16, 0), ("latent-small", "latent", 0.05, 2, 70, 0),
                                                       ("latent-small", "latent", 0.05, 3, 40, 2)])
def test_policy_gradient_step(oracle, ctx, name, variant, std, B, T, rpp):
    """trainer.PolicyGradientStep through latent attention (un-absorbed training construction) and the routed experts
    (with the sequence-level balance loss): logits, log-probs, loss, the gradient at the logits and every parameter
    gradient against the oracle; the router correction bias gets no gradient."""
    from parity import GRAD_REL, assert_gradients_close, close_elementwise
    om, gm, cfg = make_pair(oracle, ctx, name, std=std, **VARIANTS[variant])
    V = cfg["vocab_size"]
    rng = np.random.default_rng(B * T + 1)
    ids = rng.integers(0, V - 11, (B, T), dtype=np.int32)
    ids[:, 1] = ids[:, 0]
    tg = rng.integers(0, V, (B, T)).astype(np.int32)
    tg[:, : T // 3] = -1
    adv = rng.standard_normal(B).astype(np.float32)
    om.zero_grad()
    want_loss, want_nll, want_dl, want_lg = om.policy_gradient_step(ids, tg, adv, float(T + 1), taps=True)
    gm.zero_grad()
    loss, nll, dl, lg = gm.policy_gradient_step(ids, tg, adv, float(T + 1), rows_per_pass=rpp, taps=True)
    assert rel_err(lg, want_lg) <= 1e-3
    terms = np.abs(want_nll.reshape(B, T) * adv[:, None]) / float(T + 1)
    assert abs(loss - want_loss) <= 1e-4 * float(terms.sum())
    assert close_elementwise(nll, want_nll, 1e-4, 1e-5)
    assert close_elementwise(dl, want_dl, GRAD_REL, 1e-6)
    assert_gradients_close(gm, om)
    for n in gm.names:
        if n.endswith("router_bias"):
            assert not np.any(gm.grad(n))
    gm.close()


def test_optimizer_step_of_a_latent_model(oracle, ctx):
    """chat_rl's optimizer on a latent-preset model from identical gradients: Muon on every latent-attention matrix,
    on the router and on each expert's view of the packed weights; the router correction bias stays put
    (model/optimizer.go:25-36,83-93)."""
    om, gm, cfg = make_pair(oracle, ctx, "latent-tiny", std=0.1)
    oopt = oracle.Optimizer(om); gm.optimizer_init()
    rng = np.random.default_rng(3)
    before = {n: om.param(n).copy() for n in om.names}
    for n in om.names:
        g = (rng.standard_normal(om.param(n).size) * 0.01).astype(np.float32)
        om.grad(n)[:] = g; gm.upload_grad(n, g)
    oopt.step(); gm.optimizer_step()
    for n in om.names:
        got, want = gm.download(n), om.param(n)
        if n.endswith("router_bias"):
            assert np.array_equal(got, before[n]) and np.array_equal(want, before[n])
            continue
        upd = float(np.max(np.abs(want.astype(np.float64) - before[n])))
        assert upd > 0, n
        assert float(np.max(np.abs(got.astype(np.float64) - want))) <= 1e-4 * upd + float(np.max(np.abs(want))) * 2.0 ** -23, n
        assert not np.any(gm.grad(n)), n
    gm.close()
