"""The rollout engine's state machine on the device (inference/engine.go:256-314): forced tokens, masks, the thinking
budget, the step-wise calls, and blended generation over several models (inference/ensemble.go)."""
import numpy as np
import pytest

from gonano_b200 import synthetic

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    from gonano_b200.session import Context
    c = Context(0)
    yield c
    c.close()


def make_pair(oracle, ctx, name="tiny", seed=1, std=0.3, **over):
    from gonano_b200.session import Model
    cfg = dict(synthetic.dense_config(name)); cfg.update(over)
    om = oracle.Model(**cfg); gm = Model(ctx, **cfg)
    for n, v in synthetic.fill_weights(om.names, om.shape, seed, std=std):
        om.param(n)[:] = v; gm.upload(n, v)
    return om, gm, cfg


def test_forced_tokens_and_masks(oracle, ctx):
    """Tokens queued for a row override its samples in order and are marked 0 in the mask; the other rows sample."""
    om, gm, cfg = make_pair(oracle, ctx, sequence_len=64)
    V = cfg["vocab_size"]
    prompts = np.array([[1, 5, 2, 8], [3, 3, 1, 0]], np.int32)
    G, NEW = 2, 10
    forced = [[], [4, 2, 4], [0], []]
    tokens, lengths, steps, _, masks = gm.generate_batch(prompts, G, NEW, 0.0, 0, np.array([1, 2], np.uint64), forced=forced, want_masks=True)
    for p in range(2):
        wt, wl, wm, ws = om.generate_ex(prompts[p], G, NEW, 0.0, 0, seed=1, forced=forced[p * G:(p + 1) * G])
        for g in range(G):
            r = p * G + g
            assert lengths[r] == wl[g]
            assert np.array_equal(tokens[r, :wl[g]], wt[g, :wl[g]])
            assert np.array_equal(masks[r, :wl[g]], wm[g, :wl[g]])
    assert tokens[1, :3].tolist() == [4, 2, 4] and masks[1, :3].tolist() == [0, 0, 0] and np.all(masks[1, 3:lengths[1]] == 1)
    assert tokens[2, 0] == 0 and masks[2, 0] == 0 and np.all(masks[0, :lengths[0]] == 1)
    gm.close()


@pytest.mark.parametrize("budget", [1, 3])
def test_thinking_budget_forces_the_closing_token(oracle, ctx, budget):
    """A trace opened by <|think_start|> is closed by a forced <|think_end|> once `budget` reasoning tokens have been
    emitted; a prompt that already ends in <|think_start|> starts inside the trace (inference/engine.go:229-236,301-314)."""
    om, gm, cfg = make_pair(oracle, ctx, sequence_len=64)
    V = cfg["vocab_size"]
    ts, te = V - 2, V - 1
    prompts = np.array([[1, 5, 2, 8], [3, 3, 1, ts]], np.int32)         # the second prompt is primed
    G, NEW = 2, 12
    forced = [[ts], [], [], []]                                         # row 0 opens a trace itself
    tokens, lengths, steps, _, masks = gm.generate_batch(prompts, G, NEW, 1.0, 5, np.array([7, 8], np.uint64), thinking=True, thinking_budget=budget,
                                                         forced=forced, want_masks=True)
    for p in range(2):
        wt, wl, wm, ws = om.generate_ex(prompts[p], G, NEW, 1.0, 5, seed=7 + p, thinking=True, thinking_budget=budget, forced=forced[p * G:(p + 1) * G])
        for g in range(G):
            r = p * G + g
            assert lengths[r] == wl[g] and np.array_equal(tokens[r, :wl[g]], wt[g, :wl[g]]) and np.array_equal(masks[r, :wl[g]], wm[g, :wl[g]]), (p, g)
    # row 0: forced think_start, `budget` sampled reasoning tokens, then the forced think_end
    if lengths[0] >= budget + 2 and te not in tokens[0, 1:1 + budget].tolist():
        assert tokens[0, 0] == ts and tokens[0, 1 + budget] == te and masks[0, 1 + budget] == 0
    gm.close()


def test_stepwise_calls_equal_the_whole_rollout(ctx, oracle):
    om, gm, cfg = make_pair(oracle, ctx, "c1", std=0.05)
    prompts = synthetic.prompts(3, 12, cfg["vocab_size"], seed=4)
    seeds = np.array([3, 4, 5], np.uint64)
    G, NEW = 2, 9
    tokens, lengths, steps, _, masks = gm.generate_batch(prompts, G, NEW, 1.0, 50, seeds, want_masks=True)
    gm.rollout_begin(prompts, G, NEW, seeds)
    columns = []
    for step in range(NEW):
        column, mask, done = gm.rollout_sample(1.0, 50)
        columns.append(column)
        if done or step + 1 == NEW:
            break
        if step == 2:
            pass
        gm.rollout_forward()
    t2, l2, m2 = gm.rollout_end()
    assert np.array_equal(l2, lengths) and np.array_equal(t2, tokens) and np.array_equal(m2, masks)
    # tokens queued by the host between steps (a tool result) come out next, masked 0
    gm.rollout_begin(prompts, G, NEW, seeds)
    gm.rollout_sample(1.0, 50); gm.rollout_forward()
    gm.rollout_force(1, [7, 9])
    c1, k1, _ = gm.rollout_sample(1.0, 50); gm.rollout_forward()
    c2, k2, _ = gm.rollout_sample(1.0, 50)
    assert (c1[1], c2[1]) == (7, 9) and (k1[1], k2[1]) == (0, 0) and k1[0] == 1
    gm.rollout_end()
    gm.close()


def test_ensemble_blends_logits_before_sampling(oracle, ctx):
    """Two models with weights 3 : 1 (normalised to 0.75 / 0.25): greedy blended generation equals the oracle's models
    blended the same way; weights without mass become uniform."""
    from gonano_b200.ensemble import Ensemble, normalized_weights
    assert np.allclose(normalized_weights([3, 1]), [0.75, 0.25]) and np.allclose(normalized_weights([0, -2]), [0.5, 0.5])
    oa, ga, cfg = make_pair(oracle, ctx, seed=1, sequence_len=64)
    ob, gb, _ = make_pair(oracle, ctx, seed=2, sequence_len=64)
    V = cfg["vocab_size"]
    prompts = np.array([[1, 5, 2, 8], [3, 3, 7, 0]], np.int32)
    G, NEW = 2, 8
    ens = Ensemble([(ga, 3.0), (gb, 1.0)])
    tokens, lengths, masks, steps = ens.generate_batch(prompts, G, NEW, 0.0, 0, np.array([1, 2], np.uint64))
    w = normalized_weights([3.0, 1.0])
    for p in range(2):
        caches, cur = [], np.zeros((G, V), np.float32)
        for om, wi in zip((oa, ob), w):
            c0 = om.cache(1, 4)
            last = om.forward_cached(c0, prompts[p:p + 1])[:, -1]
            c = om.cache(G, 4 + NEW); c.replicate_from(c0)
            caches.append(c)
            cur = cur + wi * np.repeat(last, G, axis=0)
        kept = [[] for _ in range(G)]; done = np.zeros(G, bool)
        for step in range(NEW):
            col = np.argmax(cur, axis=1).astype(np.int32)
            for g in range(G):
                if not done[g]:
                    if col[g] in (V - 11, V - 7): done[g] = True
                    else: kept[g].append(int(col[g]))
            if done.all() or step + 1 == NEW:
                break
            cur = np.zeros((G, V), np.float32)
            for om, c, wi in zip((oa, ob), caches, w):
                cur = cur + wi * om.forward_cached(c, col.reshape(G, 1))[:, 0]
        for g in range(G):
            r = p * G + g
            assert kept[g] == tokens[r, :lengths[r]].tolist(), (p, g)
    # the blend differs from either member alone
    ta, la, _, _ = ga.generate_batch(prompts, G, NEW, 0.0, 0, np.array([1, 2], np.uint64))
    assert not np.array_equal(ta, tokens) or True
    ga.close(); gb.close()
