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


def test_training_is_refused(oracle, ctx):
    om, gm, cfg = make_pair(oracle, ctx, "latent-tiny")
    ids = np.zeros((2, 6), np.int32)
    with pytest.raises(Exception, match="inference-only"):
        gm.policy_gradient_step(ids, ids, np.ones(2, np.float32), 6.0)
    gm.close()
