"""Pins the CPU oracle against the known answers held by the reference's own tests.

Each test names the reference test whose expectation it restates.
"""
import math

import numpy as np
import pytest


def close(got, want, rel, floor):
    got = np.asarray(got, np.float32); want = np.asarray(want, np.float32)
    return bool(np.all(np.abs(got - want) <= floor + rel * np.maximum(np.abs(want), 1.0)))


# kernels/scalar/scalar_test.go:12-38
def test_elementwise(oracle):
    bk = oracle.Backend(0)
    l, r = [1, 2, 3], [4, 5, 6]
    assert close(bk.add(l, r), [5, 7, 9], 1e-6, 1e-6)
    assert close(bk.subtract(r, l), [3, 3, 3], 1e-6, 1e-6)
    assert close(bk.multiply(l, r), [4, 10, 18], 1e-6, 1e-6)
    assert close(bk.divide(r, l), [4, 2.5, 2], 1e-6, 1e-6)
    assert close(bk.scale(l, 2), [2, 4, 6], 1e-6, 1e-6)
    assert close(bk.add_scaled(l, r, 0.5), [3, 4.5, 6], 1e-6, 1e-6)
    assert close(bk.negate(l), [-1, -2, -3], 1e-6, 1e-6)
    assert close(bk.abs([-1, 2, -3]), [1, 2, 3], 1e-6, 1e-6)
    assert close(bk.square(l), [1, 4, 9], 1e-6, 1e-6)
    assert close(bk.relu_squared([-1, 2, -3]), [0, 4, 0], 1e-6, 1e-6)


# kernels/scalar/scalar_test.go:40-94
def test_swiglu(oracle):
    bk = oracle.Backend(0)
    silu = lambda x: np.float32(x) / (np.float32(1) + np.float32(math.exp(-x)))
    got = bk.swiglu([0, 1, -1, 2], [1, 1, 2, -3], 0)
    assert close(got, [silu(0) * 1, silu(1) * 1, silu(-1) * 2, silu(2) * -3], 1e-5, 1e-6)
    got = bk.swiglu([20, 1, 1, 2], [1, 20, -20, 1], 10)
    assert close(got, [silu(10) * 1, silu(1) * 10, silu(1) * -10, silu(2) * 1], 1e-5, 1e-6)
    gate, up, og = [0.5, 1.5], [2.0, -1.0], [1.0, 2.0]
    gg, ug = bk.swiglu_backward(gate, up, og, 10)
    for i in range(2):
        g, u, d = gate[i], up[i], og[i]
        s = 1.0 / (1.0 + math.exp(-g))
        assert close(gg[i], d * u * s * (1 + g * (1 - s)), 1e-5, 1e-6)
        assert close(ug[i], d * g * s, 1e-5, 1e-6)


# kernels/scalar/scalar_test.go:96-108
def test_transcendentals(oracle):
    bk = oracle.Backend(0)
    assert close(bk.exp([1]), [math.e], 1e-6, 1e-6)
    assert close(bk.sigmoid([0]), [0.5], 1e-6, 1e-6)
    assert close(bk.tanh([0]), [0], 1e-6, 1e-6)
    assert close(bk.rsqrt([4]), [0.5], 1e-6, 1e-6)


# kernels/scalar/scalar_test.go:110-137
def test_reductions_and_linear_algebra(oracle):
    bk = oracle.Backend(0)
    assert bk.sum([1, 2, 3, 4]) == 10
    assert bk.max([1, 9, 3]) == 9
    assert bk.max([]) == 0
    assert bk.argmax([1, 9, 3]) == 1
    left, right = [1, 2, 3, 4, 5, 6], [7, 8, 9, 10, 11, 12]
    assert close(bk.matmul(left, right, 2, 2, 3), [58, 64, 139, 154], 1e-5, 1e-5)
    assert close(bk.matmul_transposed(left, right, 2, 2, 3), [50, 68, 122, 167], 1e-5, 1e-5)
    assert close(bk.dot_product([1, 2, 3], [4, 5, 6]), 32, 1e-6, 1e-6)


# kernels/scalar/scalar_test.go:139-151
def test_rows(oracle):
    bk = oracle.Backend(0)
    sm = bk.softmax_last_dim([1, 2, 3, 4], 2, 2)
    assert abs(float(sm.astype(np.float64).sum()) - 2) < 1e-6
    assert close(bk.rmsnorm_last_dim([1, 1, 1, 1], 2, 2, 1e-6), [1, 1, 1, 1], 1e-5, 1e-5)


# kernels/scalar/scalar_test.go:153-186
def test_attention_reference(oracle):
    bk = oracle.Backend(0)
    q = k = v = [1, 0, 0, 1]
    out, lse = bk.attention_forward(q, k, v, 2, 2, 2, 0, -1)
    assert close(out[:2], [1, 0], 1e-5, 1e-6)
    dq, dk, dv = bk.attention_backward(q, k, v, [1, 1, 1, 1], lse, 2, 2, 2, 0, -1)
    assert np.all(np.isfinite(dq)) and np.all(np.isfinite(dk)) and np.all(np.isfinite(dv))


# kernels/scalar/scalar_test.go:188-205
def test_moe_gate_topk(oracle):
    bk = oracle.Backend(0)
    probs, sel, w = bk.moe_gate_topk([0, 0, 0], [0, 1, 2], 1, 3, 2)
    assert close(probs, [1 / 3] * 3, 1e-6, 1e-6)
    assert list(sel) == [2, 1]
    assert close(w, [1 / 3, 1 / 3], 1e-6, 1e-6)


# kernels/scalar/scalar_test.go:207-222
def test_topk_indices(oracle):
    bk = oracle.Backend(0)
    got = bk.topk_indices([0.1, 0.9, 0.3, 0.7, 0.5, 0.2, 0.5, 0.2], 2, 4, 3)
    assert list(got) == [1, 3, 2, 0, 2, 1]


# kernels/scalar/scalar_test.go:224-235
def test_grouped_matmul_transposed(oracle):
    bk = oracle.Backend(0)
    got = bk.grouped_matmul_transposed([1, 2, 3, 4, 5, 6], [1, 0, 0, 1, 2, 0, 0, 3], [2, 1], 2, 2, 2)
    assert close(got, [1, 2, 3, 4, 10, 18], 1e-6, 1e-6)


# tensors/loss_test.go:8-32
def test_cross_entropy_per_position(oracle):
    logits = np.array([[0, 0, 5, 0], [1, 1, 1, 1], [2, 0, 0, 0]], np.float32)
    losses, valid = oracle.cross_entropy_per_position(logits, [2, -1, 0])
    assert valid == 2
    assert losses[1] == 0
    assert abs(losses[0] - np.float32(math.log(math.exp(5) + 3) - 5)) <= 1e-5
    assert abs(losses[2] - np.float32(math.log(math.exp(2) + 3) - 2)) <= 1e-5


# tensors/loss_test.go:34-64
def test_cross_entropy_known_values(oracle):
    losses, valid = oracle.cross_entropy_per_position(np.ones((1, 4), np.float32), [0])
    assert abs(losses.sum() / valid - np.float32(math.log(4))) <= 1e-5
    losses, _ = oracle.cross_entropy_per_position(np.ones((2, 4), np.float32), [0, 1])
    assert abs(losses.sum() - 2 * np.float32(math.log(4))) <= 1e-4
    losses, valid = oracle.cross_entropy_per_position(np.ones((2, 4), np.float32), [-1, -1])
    assert valid == 0 and losses.sum() == 0


# tensors/backward_test.go:70-89
def test_cross_entropy_grad(oracle):
    g = oracle.cross_entropy_grad(np.zeros((1, 3), np.float32), [1], -1, 1.0)
    assert close(g[0], [1 / 3, -2 / 3, 1 / 3], 1e-5, 1e-6)
    g = oracle.cross_entropy_grad(np.zeros((2, 3), np.float32), [-1, 0], -1, 1.0)
    assert np.all(g[0] == 0)


# tensors/backward_test.go:118-158
def test_backward_primitives(oracle):
    assert close(oracle.relu_squared_backward([-1, 2, -3, 4], [1, 1, 1, 1]), [0, 4, 0, 8], 1e-5, 1e-6)
    g = oracle.rmsnorm_backward(np.array([[1, 2, 3, 4]], np.float32), np.ones((1, 4), np.float32), 1e-6)
    assert g.size == 4 and np.all(np.isfinite(g))
    assert np.all(np.isfinite(oracle.softcap_backward([0.5, -0.5], [1, 1], 15)))
    assert close(oracle.sigmoid_backward([0.5, -0.5], [1, 1])[0], 0.25, 1e-5, 1e-6)


# inference/inference_test.go:11-30
def test_sample_next_token(oracle):
    logits = np.array([[1, 9, 3, 5], [7, 2, 8, 1]], np.float32)
    assert list(oracle.sample_next_token(logits, 0.0, 0)) == [1, 2]
    logits = np.array([[1, 2, 3, 4, 5, 6, 7, 8]], np.float32)
    for seed in range(64):
        got = oracle.sample_next_token(logits, 1.0, 3, seeds=[seed], group=1, step=seed % 5)
        assert got[0] >= 5


# tensors/random_test.go:67-86 (the Gumbel sampler favours a dominant logit; argmax at T<=0)
def test_sample_multinomial_statistics(oracle):
    logits = np.array([[0, 0, 10, 0]], np.float32)
    hits = sum(int(oracle.sample_next_token(logits, 1.0, 0, seeds=[s], group=1)[0] == 2) for s in range(200))
    assert hits > 180
    assert oracle.sample_next_token(np.array([[0.1, 0.7, 0.2]], np.float32), 0.0, 0)[0] == 1


# model/model_test.go:196-211, 283-301
def test_rotary_quarter_turn(oracle):
    cos = np.array([[1], [0]], np.float32); sin = np.array([[0], [1]], np.float32)
    assert list(oracle.rotary_tables([3, 4], cos, sin, 1, 1, 1, 2, 1)) == [4, -3]
    assert list(oracle.rotary_tables([10, 20, 3, 4], cos, sin, 1, 1, 1, 4, 1)) == [10, 20, 4, -3]


# model/model_test.go:158-194
def test_window_sizes_and_padded_vocab(oracle):
    m = oracle.Model(2048, 32, 4, 2, 2, 8, 0, "SSSL")
    assert list(m.window_sizes()) == [512, 512, 512, 2048]
    assert m.padded_vocab() == 64
    assert oracle.Model(64, 65, 2, 2, 2, 8).padded_vocab() == 128


# kernels/simd/parity_test.go:263-310 and model/model_test.go:232-253: split-K shards recombine to the full pass
@pytest.mark.parametrize("ql,kl,hd,off,win", [(6, 6, 8, 0, -1), (1, 10, 8, 9, -1), (6, 6, 8, 0, 2), (1, 10, 4, 9, 3), (1, 700, 16, 699, -1)])
@pytest.mark.parametrize("splits", [1, 2, 3, 5])
def test_attention_split_combines_to_full(oracle, ql, kl, hd, off, win, splits):
    bk = oracle.Backend(0)
    q, k, v = oracle.kt_data(ql * hd), oracle.kt_data(kl * hd), oracle.kt_data_b(kl * hd)
    want_o, want_l = bk.attention_forward(q, k, v, ql, kl, hd, off, win)
    per = (kl + splits - 1) // splits
    parts = [bk.attention_forward_split(q, k, v, ql, kl, hd, off, win, s * per, min((s + 1) * per, kl)) for s in range(splits)]
    got_o, got_l = bk.attention_combine([p[0] for p in parts], [p[1] for p in parts], [p[2] for p in parts], ql, hd)
    assert close(got_o, want_o, 2e-3, 1e-5)
    assert close(got_l, want_l, 2e-3, 1e-5)


# kernels/simd/parity_test.go:15-223: the SIMD-structured port stays within the
# reference's own simd-vs-scalar tolerances.
def test_simd_port_within_reference_tolerances(oracle):
    sc, sp = oracle.Backend(0), oracle.Backend(1)
    for rows, cols, inner in [(3, 5, 17), (4, 6, 13), (64, 129, 200), (97, 131, 256), (400, 128, 512)]:
        left = oracle.kt_data(rows * inner)
        assert close(sp.matmul(left, oracle.kt_data_b(inner * cols), rows, cols, inner),
                     sc.matmul(left, oracle.kt_data_b(inner * cols), rows, cols, inner), 2e-3, 1e-4)
        assert close(sp.matmul_transposed(left, oracle.kt_data_b(cols * inner), rows, cols, inner),
                     sc.matmul_transposed(left, oracle.kt_data_b(cols * inner), rows, cols, inner), 2e-3, 1e-4)
    for n in [1, 7, 31, 64, 513, 1031]:
        x = oracle.kt_data(n)
        assert close(sp.softmax_last_dim(x, 1, n), sc.softmax_last_dim(x, 1, n), 1e-4, 1e-6)
        assert close(sp.rmsnorm_last_dim(x, 1, n, 1e-6), sc.rmsnorm_last_dim(x, 1, n, 1e-6), 1e-5, 1e-6)
    ql = kl = 200; hd = 32
    q, k, v = oracle.kt_data(ql * hd), oracle.kt_data(kl * hd), oracle.kt_data_b(kl * hd)
    o1, l1 = sp.attention_forward(q, k, v, ql, kl, hd, 0, -1)
    o0, l0 = sc.attention_forward(q, k, v, ql, kl, hd, 0, -1)
    assert close(o1, o0, 5e-3, 1e-5) and close(l1, l0, 5e-3, 1e-5)


# tensors/loss_test.go:66-140: the distillation loss's own known answers
def test_distillation_known_answers(oracle):
    logits = np.array([[0.5, -1, 2, 0.3], [-0.2, 1.5, -0.5, 0.9]], np.float32)
    teacher = np.array([[0, 0, 100, 0], [0, 100, 0, 0]], np.float32)             # effectively one-hot
    losses, valid, grad = oracle.distillation(logits, teacher, 1.0)
    ce, _ = oracle.cross_entropy_per_position(logits, np.array([2, 1], np.int32))
    assert valid == 2 and abs(float(losses.mean()) - float(ce.mean())) <= 1e-3
    assert np.max(np.abs(grad - oracle.cross_entropy_grad(logits, np.array([2, 1], np.int32), scale=1.0))) <= 1e-3
    student = np.array([[0.3, -0.7, 1.1]], np.float32); teach = np.array([[0.8, 0.2, -0.4]], np.float32)
    _, _, g = oracle.distillation(student, teach, 1.0)
    for i in range(3):                                                            # numeric gradient, eps 1e-3
        p = student.copy(); p[0, i] += 1e-3; q = student.copy(); q[0, i] -= 1e-3
        numeric = (oracle.distillation(p, teach, 1.0)[0][0] - oracle.distillation(q, teach, 1.0)[0][0]) / 2e-3
        assert abs(numeric - g[0, i]) <= 1e-3
    x = oracle.kt_data(8).reshape(2, 4)
    assert np.max(np.abs(oracle.distillation(x, x.copy(), 1.0)[2])) <= 1e-6          # self-distillation: zero gradient
    s2 = np.array([[0.1, 0.2, 0.3], [1, 2, 3]], np.float32); t2 = np.array([[3, 2, 1], [-1, -2, -3]], np.float32)
    losses, valid, grad = oracle.distillation(s2, t2, 1.0, mask=[0, 1])
    assert valid == 1 and losses[0] == 0 and losses[1] != 0 and not np.any(grad[0]) and np.any(grad[1])


# model/compress_test.go:10-26: zero logits give a uniform softmax, so a complete block is the mean of its rows and a
# trailing partial block keeps its single row
def test_compressor_means_blocks(oracle):
    out, prob = oracle.compressor_forward(np.zeros((1, 3, 1)), np.array([2, 4, 6], np.float32).reshape(1, 3, 1), np.zeros((1, 1)), np.zeros((2, 1)), 2)
    assert out.shape == (1, 2, 1) and out[0, 0, 0] == 3.0 and out[0, 1, 0] == 6.0
    assert prob[0, 0, :, 0].tolist() == [0.5, 0.5] and prob[0, 1, :, 0].tolist() == [1.0, 0.0]


# model/indexer_test.go:318-325 (three equal maxima: the smallest indices win, in order), 437-470 (TopK orders and
# breaks ties; k clamps to the block count), 413-435 (causality: a token takes only blocks before its own)
def test_select_blocks_known_answers(oracle):
    sel, cnt = oracle.select_blocks(np.array([[5, 5, 5, 1, 2]], np.float32), 10, 1, 2)
    assert sel[0].tolist() == [0, 1] and cnt[0] == 2
    scores = np.array([[1, 9, 3, 9, 2], [4, 5, 6, 7, 8]], np.float32)
    sel, cnt = oracle.select_blocks(scores, 100, 1, 2)          # every block allowed: TopK
    assert sel[0].tolist() == [1, 3] and sel[1].tolist() == [4, 3]
    sel, cnt = oracle.select_blocks(np.array([[1, 2, 3]], np.float32), 100, 1, 10)
    assert cnt[0] == 3 and sel[0, :3].tolist() == [2, 1, 0] and np.all(sel[0, 3:] == -1)
    sel, cnt = oracle.select_blocks(np.tile(np.arange(6, dtype=np.float32), (8, 1)), 0, 2, 2)   # token t: blocks [0, t // 2)
    assert cnt.tolist() == [0, 0, 1, 1, 2, 2, 2, 2]
    assert sel[2].tolist() == [0, -1] and sel[4].tolist() == [1, 0] and sel[7].tolist() == [2, 1]


# the merge of two branches equals attention over the union of their keys (the purpose stated at
# model/compress_attention.go:434-439)
def test_merge_branches_equals_joint_softmax(oracle):
    rng = np.random.default_rng(0)
    bk = oracle.Backend(0)
    hd, na, nb = 8, 5, 7
    q = rng.standard_normal(hd).astype(np.float32); k = rng.standard_normal((na + nb, hd)).astype(np.float32); v = rng.standard_normal((na + nb, hd)).astype(np.float32)
    oa, la = bk.attention_forward(q, k[:na], v[:na], 1, na, hd, na, -1)
    ob, lb = bk.attention_forward(q, k[na:], v[na:], 1, nb, hd, nb, -1)
    want_o, want_l = bk.attention_forward(q, k, v, 1, na + nb, hd, na + nb, -1)
    got_o, got_l = oracle.merge_branches(oa.reshape(1, hd), la.reshape(1), ob.reshape(1, hd), lb.reshape(1))
    assert np.allclose(got_o.ravel(), want_o.ravel(), rtol=1e-5, atol=1e-6) and np.allclose(got_l.ravel(), want_l.ravel(), rtol=1e-5)
    empty = np.full(1, -np.inf, np.float32)
    o2, l2 = oracle.merge_branches(np.zeros((1, hd)), empty, ob.reshape(1, hd), lb.reshape(1))
    assert np.array_equal(o2.ravel(), ob.ravel()) and l2[0] == lb.ravel()[0]
    o3, l3 = oracle.merge_branches(np.zeros((1, hd)), empty, np.zeros((1, hd)), empty)
    assert np.all(o3 == 0) and l3[0] == -np.inf


# model/compress_test.go:28-110: the compressor's backward against a central finite difference along random directions of
# every input and parameter (the reference's own check, same shapes: d 4, C 3, ratio 2, B 2, T 5)
def test_compressor_gradient_matches_finite_difference(oracle):
    rng = np.random.default_rng(7)
    B, T, d, C_, ratio = 2, 5, 4, 3, 2
    w = (rng.standard_normal((C_, d)) * 0.5).astype(np.float32); bias = (rng.standard_normal((ratio, C_)) * 0.5).astype(np.float32)
    hidden = rng.standard_normal((B, T, d)).astype(np.float32); value = rng.standard_normal((B, T, C_)).astype(np.float32)
    gc = rng.standard_normal((B, 3, C_)).astype(np.float32)
    gh, gv, gw, gb = oracle.compressor_backward(hidden, value, w, bias, ratio, gc)
    dirs = [rng.standard_normal(x.shape).astype(np.float32) for x in (hidden, value, w, bias)]
    analytic = sum(float(np.sum(g.astype(np.float64) * dr)) for g, dr in zip((gh, gv, gw, gb), dirs))
    def loss(eps):
        out, _ = oracle.compressor_forward(hidden + eps * dirs[0], value + eps * dirs[1], w + eps * dirs[2], bias + eps * dirs[3], ratio)
        return float(np.sum(out.astype(np.float64) * gc))
    eps = 1e-3
    numeric = (loss(eps) - loss(-eps)) / (2 * eps)
    assert abs(analytic - numeric) <= 2e-3 * max(1.0, abs(numeric)), (analytic, numeric)


# compressedAttentionBackward (model/compress_attention.go:735-781) against a central difference of its forward
def test_compressed_attention_gradient_matches_finite_difference(oracle):
    rng = np.random.default_rng(11)
    B, Hq, Hkv, T, D, ratio = 1, 4, 2, 11, 6, 3
    blocks = (T + ratio - 1) // ratio
    q = (rng.standard_normal((B, Hq, T, D)) * 0.5).astype(np.float32)
    kc = (rng.standard_normal((B, Hkv, blocks, D)) * 0.5).astype(np.float32); vc = rng.standard_normal((B, Hkv, blocks, D)).astype(np.float32)
    dout = rng.standard_normal((B, Hq, T, D)).astype(np.float32)
    _, lse = oracle.compressed_attention_forward(q, kc, vc, ratio)
    gq, gk, gv = oracle.compressed_attention_backward(q, kc, vc, dout, lse, ratio)
    assert np.all(gq[:, :, :ratio] == 0) and np.all(gk[:, :, (T - 1) // ratio:] == 0)
    dirs = [rng.standard_normal(x.shape).astype(np.float32) for x in (q, kc, vc)]
    analytic = sum(float(np.sum(g.astype(np.float64) * dr)) for g, dr in zip((gq, gk, gv), dirs))
    def loss(eps):
        out, _ = oracle.compressed_attention_forward(q + eps * dirs[0], kc + eps * dirs[1], vc + eps * dirs[2], ratio)
        return float(np.sum(out.astype(np.float64) * dout))
    eps = 1e-3
    numeric = (loss(eps) - loss(-eps)) / (2 * eps)
    assert abs(analytic - numeric) <= 2e-3 * max(1.0, abs(numeric)), (analytic, numeric)


# compressedAttentionBackwardSparse (model/compress_attention.go:376-433) against a central difference of its forward
def test_sparse_attention_gradient_matches_finite_difference(oracle):
    rng = np.random.default_rng(13)
    B, Hq, Hkv, T, D, ratio, topk = 1, 4, 2, 13, 6, 2, 3
    blocks = (T + ratio - 1) // ratio
    q = (rng.standard_normal((B, Hq, T, D)) * 0.5).astype(np.float32)
    kc = (rng.standard_normal((B, Hkv, blocks, D)) * 0.5).astype(np.float32); vc = rng.standard_normal((B, Hkv, blocks, D)).astype(np.float32)
    dout = rng.standard_normal((B, Hq, T, D)).astype(np.float32)
    sel = np.zeros((B * Hkv, T, topk), np.int32); cnt = np.zeros((B * Hkv, T), np.int32)
    for i in range(B * Hkv):
        sel[i], cnt[i] = oracle.select_blocks(rng.standard_normal((T, blocks)).astype(np.float32), 0, ratio, topk)
    sel = np.maximum(sel, 0)
    _, lse = oracle.compressed_attention_sparse_forward(q, kc, vc, sel, cnt)
    grads = oracle.compressed_attention_sparse_backward(q, kc, vc, dout, lse, sel, cnt)
    dirs = [rng.standard_normal(x.shape).astype(np.float32) for x in (q, kc, vc)]
    analytic = sum(float(np.sum(g.astype(np.float64) * dr)) for g, dr in zip(grads, dirs))
    def loss(eps):
        out, _ = oracle.compressed_attention_sparse_forward(q + eps * dirs[0], kc + eps * dirs[1], vc + eps * dirs[2], sel, cnt)
        return float(np.sum(out.astype(np.float64) * dout))
    eps = 1e-3
    numeric = (loss(eps) - loss(-eps)) / (2 * eps)
    assert abs(analytic - numeric) <= 2e-3 * max(1.0, abs(numeric)), (analytic, numeric)


# One heavily-compressed attention layer assembled from the blocks: both branches are differentiated with the merged
# log-sum-exp and the merged row correction dO . O (model/train.go:211-226, 289-301); the assembled gradient must be the
# gradient of the assembled forward.
def test_heavily_compressed_layer_gradient_matches_finite_difference(oracle):
    from test_gpu_compress import _hca_layer
    rng = np.random.default_rng(17)
    B, Hq, Hkv, T, D, d, ratio, window = 1, 2, 1, 11, 4, 5, 3, 4
    x = rng.standard_normal((B, T, d)).astype(np.float32)
    q = (rng.standard_normal((B, Hq, T, D)) * 0.5).astype(np.float32)
    k = (rng.standard_normal((B, Hkv, T, D)) * 0.5).astype(np.float32); v = rng.standard_normal((B, Hkv, T, D)).astype(np.float32)
    wk = (rng.standard_normal((D, d)) * 0.3).astype(np.float32); bias = (rng.standard_normal((ratio, D)) * 0.3).astype(np.float32)
    dout = rng.standard_normal((B, Hq, T, D)).astype(np.float32)
    ref = oracle.Backend(0)

    def attn_bwd(q_, k_, v_, out_, dout_, lse_, ql, kl, hd, off, win, row_correction=None, dq=None, dk=None, dv=None):
        return ref.attention_backward(q_, k_, v_, dout_, lse_, ql, kl, hd, off, win, row_correction=row_correction, dq=dq, dk=dk, dv=dv)

    ops = (oracle.compressor_forward, oracle.compressor_backward, oracle.compressed_attention_forward, oracle.compressed_attention_backward,
           oracle.merge_branches, ref.attention_forward, attn_bwd)
    _, grads = _hca_layer(ops, x, q, k, v, wk, bias, ratio, window, dout)
    args = (q, k, v, x, wk, bias)
    dirs = [rng.standard_normal(a.shape).astype(np.float32) for a in args]
    analytic = sum(float(np.sum(g.astype(np.float64) * dr)) for g, dr in zip(grads, dirs))
    def loss(eps):
        q2, k2, v2, x2, w2, b2 = [a + np.float32(eps) * dr for a, dr in zip(args, dirs)]
        out, _ = _hca_layer(ops, x2, q2, k2, v2, w2, b2, ratio, window)
        return float(np.sum(out.astype(np.float64) * dout))
    eps = 1e-3
    numeric = (loss(eps) - loss(-eps)) / (2 * eps)
    assert abs(analytic - numeric) <= 3e-3 * max(1.0, abs(numeric)), (analytic, numeric)


# model/indexer_test.go:351-365 (super-blocks are ranked by their maximum, not their mean), :327-349 (an unbounded budget gives the
# flat selection), :212-244 (candidates bounded by the budget and causal), :183-210 (re-selecting inside the candidates)
def test_hierarchical_selection_known_answers(oracle):
    sel, cnt, cand, cc = oracle.select_blocks_hierarchical(np.array([[4, 0, 3, 3]], np.float32), 4, 1, 1, 2, 2)
    assert cand[0].tolist() == [0, 1] and cc[0] == 2 and sel[0].tolist() == [0] and cnt[0] == 1
    rng = np.random.default_rng(3)
    scores = rng.standard_normal((48, 32)).astype(np.float32)
    flat, flat_c = oracle.select_blocks(scores, 0, 2, 2)
    for pool in (1, 2, 3):
        sel, cnt, _, _ = oracle.select_blocks_hierarchical(scores, 0, 2, 2, pool, 1000)
        assert np.array_equal(sel, flat) and np.array_equal(cnt, flat_c)
    sel, cnt, cand, cc = oracle.select_blocks_hierarchical(scores, 0, 2, 4, 4, 8)
    assert cand.shape[1] == 8 and cc.max() <= 8
    allowed = np.minimum(np.arange(48) // 2, 32)
    assert np.all((cand < allowed[:, None]) | (cand == -1)) and cnt[0] == 0 and cnt[1] == 0
    again, again_c = oracle.select_blocks_within_pool(scores, 0, 2, 4, cand, cc)
    assert np.array_equal(again, sel) and np.array_equal(again_c, cnt)


# SparseIndexer.Backward's score part against a central difference of the scores (model/indexer_test.go:86-181 checks the same way)
def test_indexer_scores_gradient_matches_finite_difference(oracle):
    rng = np.random.default_rng(23)
    rows, blocks, heads, dim = 6, 5, 3, 4
    bk = oracle.Backend(0)
    q = rng.standard_normal((rows, heads, dim)).astype(np.float32); k = rng.standard_normal((blocks, heads, dim)).astype(np.float32)
    w = rng.standard_normal(heads).astype(np.float32); gs = rng.standard_normal((rows, blocks)).astype(np.float32)
    gq, gk, gw = oracle.indexer_scores_backward(gs, q, k, w)
    dirs = [rng.standard_normal(x.shape).astype(np.float32) for x in (q, k, w)]
    analytic = sum(float(np.sum(g.astype(np.float64) * d)) for g, d in zip((gq, gk, gw), dirs))
    def loss(eps):
        s = bk.indexer_scores(q + eps * dirs[0], k + eps * dirs[1], w + eps * dirs[2], rows, blocks, heads, dim)
        return float(np.sum(np.asarray(s, np.float64).reshape(rows, blocks) * gs))
    eps = 1e-3
    numeric = (loss(eps) - loss(-eps)) / (2 * eps)
    assert abs(analytic - numeric) <= 5e-3 * max(1.0, abs(numeric)), (analytic, numeric)


# model/indexer_test.go:367-396: restricting to a candidate list masks the scores outside it and renormalises the target inside.
# With weight 1 the gradient is softmax(masked scores) - restricted target, which exposes both.
def test_distillation_restricted_to_candidates_known_answer(oracle):
    scores = np.array([[[1, 2, 3, 4], [5, 6, 7, 8]]], np.float32)
    target = np.array([[[0.1, 0.2, 0.3, 0.4], [0.25, 0.25, 0.25, 0.25]]], np.float32)
    cand = np.array([[1, 3], [0, 2]], np.int32); cc = np.array([2, 2], np.int32)
    # ratio 1 and a sequence of 2 would allow 0 / 1 blocks; rows here stand for late tokens, so place them at positions >= 4
    big_s = np.zeros((1, 6, 4), np.float32); big_t = np.zeros((1, 6, 4), np.float32)
    big_s[0, 4:] = scores[0]; big_t[0, 4:] = target[0]
    big_c = np.full((6, 2), -1, np.int32); big_n = np.zeros(6, np.int32); big_c[4:] = cand; big_n[4:] = cc
    g = oracle.indexer_distillation_grad(big_s, big_t, 1, 1.0, big_c, big_n)[0, 4:]
    p0 = np.exp(np.array([2.0, 4.0]) - 4.0); p0 /= p0.sum()
    assert np.allclose(g[0], [0, p0[0] - 1 / 3, 0, p0[1] - 2 / 3], atol=1e-6)
    p1 = np.exp(np.array([5.0, 7.0]) - 7.0); p1 /= p1.sum()
    assert np.allclose(g[1], [p1[0] - 0.5, 0, p1[1] - 0.5, 0], atol=1e-6)
    # the free form: the gradient of KL(target || softmax(scores)) with respect to the scores
    rng = np.random.default_rng(2)
    s = rng.standard_normal((1, 9, 4)).astype(np.float32)
    t = oracle.indexer_distillation_target(rng.standard_normal((1, 2, 9, 4)).astype(np.float32), rng.standard_normal((1, 1, 4, 4)).astype(np.float32), 2)
    g = oracle.indexer_distillation_grad(s, t, 2, 1.0)
    d = rng.standard_normal(s.shape).astype(np.float32)
    def loss(eps):
        total = 0.0
        for tok in range(9):
            a = min(tok // 2, 4)
            if a == 0: continue
            z = (s[0, tok, :a] + eps * d[0, tok, :a]).astype(np.float64)
            logp = z - z.max() - np.log(np.exp(z - z.max()).sum())
            total -= float(np.sum(t[0, tok, :a] * logp))
        return total
    numeric = (loss(1e-3) - loss(-1e-3)) / 2e-3
    assert abs(float(np.sum(g.astype(np.float64) * d)) - numeric) <= 1e-3 * max(1.0, abs(numeric))


def _merge_contract(attn_fwd, attn_bwd, merge, rng):
    """model/swa_test.go:14-113: two branches merged through their log-sum-exps equal one attention over the concatenated keys,
    forward and backward (each branch differentiated with the merged log-sum-exp and the merged row correction dO . O)."""
    ql, hd, na, nb = 5, 8, 6, 4
    q = rng.standard_normal((ql, hd)).astype(np.float32)
    ka, va = rng.standard_normal((na, hd)).astype(np.float32), rng.standard_normal((na, hd)).astype(np.float32)
    kb, vb = rng.standard_normal((nb, hd)).astype(np.float32), rng.standard_normal((nb, hd)).astype(np.float32)
    off = ql + na + nb                                           # past every key: no causal or window cut
    oa, la = attn_fwd(q, ka, va, ql, na, hd, off, -1); ob, lb = attn_fwd(q, kb, vb, ql, nb, hd, off, -1)
    om, lm = merge(np.asarray(oa).reshape(ql, hd), np.asarray(la), np.asarray(ob).reshape(ql, hd), np.asarray(lb))
    om = np.asarray(om).reshape(ql, hd); lm = np.asarray(lm).reshape(ql)
    k = np.concatenate([ka, kb]); v = np.concatenate([va, vb])
    oref, lref = attn_fwd(q, k, v, ql, na + nb, hd, off, -1)
    oref = np.asarray(oref).reshape(ql, hd); lref = np.asarray(lref).reshape(ql)
    tol = lambda got, want: np.all(np.abs(got - want) <= 1e-3 * (np.abs(want) + 1e-4))
    assert tol(om, oref) and tol(lm, lref)
    dout = rng.standard_normal((ql, hd)).astype(np.float32)
    rc = np.sum(dout.astype(np.float64) * om.astype(np.float64), axis=1).astype(np.float32)
    gqa, gka, gva = attn_bwd(q, ka, va, oa, dout, lm, ql, na, hd, off, -1, rc)
    gqb, gkb, gvb = attn_bwd(q, kb, vb, ob, dout, lm, ql, nb, hd, off, -1, rc)
    gq, gk, gv = attn_bwd(q, k, v, oref, dout, lref, ql, na + nb, hd, off, -1, None)
    gq, gk, gv = np.asarray(gq), np.asarray(gk).reshape(na + nb, hd), np.asarray(gv).reshape(na + nb, hd)
    assert tol(np.asarray(gqa) + np.asarray(gqb), gq)
    assert tol(np.asarray(gka).reshape(na, hd), gk[:na]) and tol(np.asarray(gkb).reshape(nb, hd), gk[na:])
    assert tol(np.asarray(gva).reshape(na, hd), gv[:na]) and tol(np.asarray(gvb).reshape(nb, hd), gv[na:])


def test_merged_branches_equal_concatenated_attention_forward_and_backward(oracle):
    bk = oracle.Backend(0)
    bwd = lambda q, k, v, o, dout, lse, ql, kl, hd, off, win, rc: bk.attention_backward(q, k, v, dout, lse, ql, kl, hd, off, win, row_correction=rc)
    _merge_contract(bk.attention_forward, bwd, oracle.merge_branches, np.random.default_rng(7))


# the cached inference form against the full-sequence pass (the invariant inference/inference_test.go:306-440 holds the reference's
# engine to): the last rows of a full pass equal the continuation computed from the cached blocks at their positions
def test_cached_compressed_attention_equals_full_pass(oracle):
    rng = np.random.default_rng(19)
    B, Hq, Hkv, T, D, ratio, T0 = 2, 4, 2, 23, 8, 4, 9
    blocks = (T + ratio - 1) // ratio
    q = (rng.standard_normal((B, Hq, T, D)) * 0.5).astype(np.float32)
    kc = (rng.standard_normal((B, Hkv, blocks, D)) * 0.5).astype(np.float32); vc = rng.standard_normal((B, Hkv, blocks, D)).astype(np.float32)
    full, full_l = oracle.compressed_attention_forward(q, kc, vc, ratio)
    again, again_l = oracle.compressed_attention_forward_at(q, kc, vc, ratio, 0)
    assert np.array_equal(full, again) and np.array_equal(full_l, again_l)
    tail, tail_l = oracle.compressed_attention_forward_at(q[:, :, T0:], kc, vc, ratio, T0)
    assert np.array_equal(tail, full[:, :, T0:]) and np.array_equal(tail_l, full_l[:, :, T0:])
    for t in range(T0, T):                                     # token by token with only the blocks complete at that time
        have = (t + 1) // ratio
        one, one_l = oracle.compressed_attention_forward_at(q[:, :, t:t + 1], kc[:, :, :have], vc[:, :, :have], ratio, t)
        assert np.allclose(one[:, :, 0], full[:, :, t], atol=1e-6) and np.allclose(one_l[:, :, 0], full_l[:, :, t], atol=1e-6)
