"""Sampler, advantage and loss kernels through the C-ABI against the oracle."""
import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def softcapped_logits(rng, rows, vocab, sigma=3.0):
    z = rng.standard_normal((rows, vocab)).astype(np.float32) * np.float32(sigma)
    return (np.float32(15) * np.tanh(z / np.float32(15))).astype(np.float32)


# inference/inference_test.go:11-30
def test_sampler_known_answers():
    from gonano_b200.backend import sample_next_token
    logits = np.array([[1, 9, 3, 5], [7, 2, 8, 1]], np.float32)
    assert list(sample_next_token(logits, 0.0, 0)) == [1, 2]
    logits = np.array([[1, 2, 3, 4, 5, 6, 7, 8]], np.float32)
    for seed in range(32):
        assert sample_next_token(logits, 1.0, 3, seeds=[seed], group=1, step=seed)[0] >= 5


@pytest.mark.parametrize("vocab", [8, 1000, 8192, 32768, 65536])
@pytest.mark.parametrize("top_k", [0, 1, 50, 100, 200])
def test_sampler_bit_exact_with_explicit_uniforms(oracle, vocab, top_k):
    """Indices are identical to the CPU rule given identical logits and uniforms."""
    from gonano_b200.backend import sample_next_token
    rng = np.random.default_rng(vocab + top_k)
    rows = 6 if vocab > 8192 else 16
    logits = softcapped_logits(rng, rows, vocab)
    logits[0, : min(vocab, 200)] = logits[0, 0]        # a plateau: the >= threshold rule keeps every tied value
    uniforms = rng.random((rows, vocab), dtype=np.float32)
    uniforms[1, :3] = 0.0                               # u <= 0 reads as 1e-12
    for temperature in [1.0, 0.7]:
        got = sample_next_token(logits, temperature, top_k, uniforms=uniforms)
        want = oracle.sample_next_token(logits, temperature, top_k, uniforms=uniforms)
        assert np.array_equal(got, want)
    assert np.array_equal(sample_next_token(logits, 0.0, top_k), oracle.sample_next_token(logits, 0.0, top_k))


@pytest.mark.parametrize("vocab,group", [(8192, 4), (32768, 8)])
def test_sampler_bit_exact_with_counter_generator(oracle, vocab, group):
    from gonano_b200.backend import sample_next_token
    rng = np.random.default_rng(7)
    rows = group * 3
    logits = softcapped_logits(rng, rows, vocab)
    seeds = np.array([11, 2 ** 40 + 5, 0], np.uint64)
    for step in [0, 1, 255]:
        got = sample_next_token(logits, 1.0, 50, seeds=seeds, group=group, step=step)
        want = oracle.sample_next_token(logits, 1.0, 50, seeds=seeds, group=group, step=step)
        assert np.array_equal(got, want)
    # different steps and different rows of a group draw differently
    a = sample_next_token(np.tile(logits[:1], (group, 1)), 1.0, 50, seeds=seeds[:1], group=group, step=0)
    assert len(set(a.tolist())) > 1


def test_sampler_ties_take_first_maximum(oracle):
    from gonano_b200.backend import sample_next_token
    logits = np.zeros((2, 4096), np.float32)
    uniforms = np.full((2, 4096), 0.5, np.float32)
    assert list(sample_next_token(logits, 1.0, 0, uniforms=uniforms)) == [0, 0]
    assert list(oracle.sample_next_token(logits, 1.0, 0, uniforms=uniforms)) == [0, 0]


def test_sampler_top_k_on_rows_of_equal_values(oracle):
    """Every entry ties with the k-th largest, so all survive (inference/sampler.go:59-64); on the device this is the row
    whose candidate list overflows and falls back to the radix select."""
    from gonano_b200.backend import sample_next_token
    rng = np.random.default_rng(3)
    logits = np.zeros((3, 32768), np.float32)
    logits[1, 100:130] = 2.0          # 30 larger entries, then a plateau that holds the 50th largest
    logits[2] = -np.inf
    logits[2, :60] = 1.0
    uniforms = rng.random(logits.shape, dtype=np.float32)
    got = sample_next_token(logits, 1.0, 50, uniforms=uniforms)
    want = oracle.sample_next_token(logits, 1.0, 50, uniforms=uniforms)
    assert np.array_equal(got, want)


def test_group_advantage(oracle):
    from gonano_b200.backend import group_advantage
    rng = np.random.default_rng(0)
    rewards = (rng.random(64 * 8) < 0.5).astype(np.float32)
    rewards[:8] = 1.0   # a group with zero variance
    for mode in [0, 1]:
        got = group_advantage(rewards, 8, mode)
        want = oracle.advantage(rewards, 8, mode)
        assert np.array_equal(got, want)  # same float32 operations in the same order


# tensors/loss_test.go:8-64, tensors/backward_test.go:70-89
def test_loss_known_answers():
    from gonano_b200.backend import pg_loss_backward
    logits = np.array([[0, 0, 5, 0], [1, 1, 1, 1], [2, 0, 0, 0]], np.float32)
    loss, nll, grad = pg_loss_backward(logits, [2, -1, 0], [1.0, 1.0, 1.0], 1, 1.0)
    assert nll[1] == 0 and np.all(grad[1] == 0)
    assert abs(nll[0] - (math.log(math.exp(5) + 3) - 5)) <= 1e-5
    assert abs(nll[2] - (math.log(math.exp(2) + 3) - 2)) <= 1e-5
    loss, nll, grad = pg_loss_backward(np.ones((1, 4), np.float32), [0], [1.0], 1, 1.0)
    assert abs(loss - math.log(4)) <= 1e-5
    loss, nll, grad = pg_loss_backward(np.zeros((1, 3), np.float32), [1], [1.0], 1, 1.0)
    assert np.allclose(grad[0], [1 / 3, -2 / 3, 1 / 3], atol=1e-6)
    loss, nll, grad = pg_loss_backward(np.ones((2, 4), np.float32), [-1, -1], [1.0, 1.0], 1, 1.0)
    assert loss == 0 and np.all(grad == 0)


@pytest.mark.parametrize("rows,vocab,seq", [(64, 8192, 16), (48, 32768, 8), (12, 65536, 4), (9, 1000, 3), (5, 33000, 5)])
def test_loss_parity(oracle, rows, vocab, seq):
    """log-probs, loss and gradient within 1e-4 relative of the oracle (float64 sums)."""
    from gonano_b200.backend import pg_loss_backward
    rng = np.random.default_rng(rows + vocab)
    logits = softcapped_logits(rng, rows, vocab)
    targets = rng.integers(0, vocab, rows).astype(np.int32)
    targets[rng.random(rows) < 0.5] = -1
    adv = rng.standard_normal((rows + seq - 1) // seq).astype(np.float32)
    norm = float(max(1, int((targets != -1).sum())))
    want_loss, want_nll, want_grad = oracle.pg_loss_backward(logits, targets, adv, seq, norm)
    loss, nll, grad = pg_loss_backward(logits, targets, adv, seq, norm)
    assert abs(loss - want_loss) <= 1e-4 * max(abs(want_loss), 1e-3)
    assert np.max(np.abs(nll - want_nll)) <= 1e-4 * np.max(np.abs(want_nll) + 1e-6)
    scale = np.max(np.abs(want_grad))
    assert np.max(np.abs(grad - want_grad)) <= 1e-4 * scale
    assert np.all(grad[targets == -1] == 0)
    # in place, with the softcap backward folded in
    folded = oracle.softcap_backward(logits, want_grad, 15.0)
    work = logits.copy()
    loss2, _, out = pg_loss_backward(work, targets, adv, seq, norm, softcap=15.0, in_place=True)
    assert out is work
    assert np.max(np.abs(work - folded)) <= 1e-4 * np.max(np.abs(folded))
    assert abs(loss2 - want_loss) <= 1e-4 * max(abs(want_loss), 1e-3)


def test_loss_refuses_targets_outside_the_vocabulary():
    """A target >= vocab (or below -1) is never used as an index: the row is skipped on the device and the call
    reports GN_ERR_INVALID, where the reference would panic on the slice bound (tensors/loss.go:39)."""
    from gonano_b200._lib import GonanoError
    from gonano_b200 import backend as B
    logits = np.zeros((4, 8), np.float32)
    adv = np.ones(4, np.float32)
    for bad in (8, 1000, -2):
        targets = np.array([1, bad, -1, 2], np.int32)
        with pytest.raises(GonanoError, match="targets outside"):
            B.pg_loss_backward(logits, targets, adv, 1, 1.0)
    loss, nll, grad = B.pg_loss_backward(logits, np.array([1, 7, -1, 2], np.int32), adv, 1, 1.0)
    assert np.isfinite(loss) and nll[2] == 0 and not np.any(grad[2])


def test_loss_properties_at_scale():
    """Size-independent checks at the microbenchmark's row width: each valid gradient row sums to 0
    and the loss is linear in the advantages."""
    from gonano_b200.backend import pg_loss_backward
    rng = np.random.default_rng(5)
    rows, vocab, seq = 256, 65536, 64
    logits = softcapped_logits(rng, rows, vocab)
    targets = rng.integers(0, vocab, rows).astype(np.int32)
    targets[::2] = -1
    adv = rng.standard_normal(rows // seq).astype(np.float32)
    l1, nll, g1 = pg_loss_backward(logits, targets, adv, seq, 128.0)
    l2, _, g2 = pg_loss_backward(logits, targets, adv * np.float32(2), seq, 128.0)
    assert abs(l2 - 2 * l1) <= 1e-6 * abs(l1) + 1e-9
    assert np.max(np.abs(g1[1::2].astype(np.float64).sum(axis=1))) <= 1e-6
    assert np.all(g1[::2] == 0) and np.all(nll[::2] == 0)
    assert np.allclose(g2, 2 * g1, rtol=1e-6, atol=1e-12)


# tensors/loss_test.go:66-140 on the device, then parity with the oracle at vocabulary scale
def test_distillation_loss(oracle):
    from gonano_b200.backend import distillation_loss_backward
    logits = np.array([[0.5, -1, 2, 0.3], [-0.2, 1.5, -0.5, 0.9]], np.float32)
    teacher = np.array([[0, 0, 100, 0], [0, 100, 0, 0]], np.float32)
    losses, valid, mean, grad = distillation_loss_backward(logits, teacher, 1.0)
    ce, _ = oracle.cross_entropy_per_position(logits, np.array([2, 1], np.int32))
    assert valid == 2 and abs(mean - float(ce.mean())) <= 1e-3
    assert np.max(np.abs(grad - oracle.cross_entropy_grad(logits, np.array([2, 1], np.int32), scale=1.0))) <= 1e-3
    x = oracle.kt_data(8).reshape(2, 4)
    assert np.max(np.abs(distillation_loss_backward(x, x.copy(), 1.0)[3])) <= 1e-6
    s2 = np.array([[0.1, 0.2, 0.3], [1, 2, 3]], np.float32); t2 = np.array([[3, 2, 1], [-1, -2, -3]], np.float32)
    losses, valid, mean, grad = distillation_loss_backward(s2, t2, 1.0, mask=[0, 1])
    assert valid == 1 and losses[0] == 0 and losses[1] != 0 and not np.any(grad[0]) and np.any(grad[1])
    rng = np.random.default_rng(5)
    for rows, vocab, tau in [(24, 32768, 1.0), (9, 1000, 2.0), (6, 65536, 0.7)]:
        student = softcapped_logits(rng, rows, vocab); teach = softcapped_logits(rng, rows, vocab)
        mask = (rng.random(rows) < 0.7).astype(np.int32)
        want_l, want_valid, want_g = oracle.distillation(student, teach, tau, mask=mask, scale=0.5)
        losses, valid, mean, grad = distillation_loss_backward(student, teach, tau, mask=mask, scale=0.5)
        assert valid == want_valid
        assert np.max(np.abs(losses - want_l)) <= 1e-4 * max(1.0, float(np.max(np.abs(want_l))))
        assert np.max(np.abs(grad - want_g)) <= 1e-4 * float(np.max(np.abs(want_g))) + 1e-9
        assert abs(mean - float(want_l.sum(dtype=np.float64)) / max(want_valid, 1)) <= 1e-4
