"""Tier-A conformance on the GPU: every kernels.Backend method through the C-ABI against the
CPU oracle, on the reference's own fixtures, shapes and tolerances
(kernels/simd/parity_test.go:15-679, kernels/kerneltest/compare.go:12-51)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

AWKWARD = [1, 7, 31, 64, 513, 1031]


@pytest.fixture(scope="module")
def bk():
    import os
    from gonano_b200 import _lib
    from gonano_b200.backend import CudaBackend
    b = CudaBackend()
    if os.environ.get("GN_TEST_GEMM_PERSISTENT_CTAS"):   # set by the test that re-runs the product tests on a small persistent grid
        one = np.ones(4, np.float32)
        b.add(one, one)                                   # the stand-alone calls' stream exists after their first call
        _lib.check(_lib.load().gn_ctx_set_option(None, b"gemm_persistent_ctas", int(os.environ["GN_TEST_GEMM_PERSISTENT_CTAS"])))
    return b


@pytest.fixture(scope="module")
def ref(oracle):
    return oracle.Backend(0)


def close(oracle, got, want, rel, floor):
    ok = oracle.kt_close(got, want, rel, floor)
    if not np.all(ok):
        i = int(np.argmin(ok))
        raise AssertionError(f"mismatch at {i}: got {np.asarray(got).ravel()[i]} want {np.asarray(want).ravel()[i]}")


# parity_test.go:15-111
@pytest.mark.parametrize("n", AWKWARD)
def test_elementwise_parity(oracle, bk, ref, n):
    a, b = oracle.kt_data(n), oracle.kt_data_b(n)
    for name in ["add", "subtract", "multiply", "divide"]:
        close(oracle, getattr(bk, name)(a, b), getattr(ref, name)(a, b), 1e-5, 1e-6)
    for name in ["negate", "abs", "square", "relu_squared", "sigmoid", "tanh"]:
        close(oracle, getattr(bk, name)(a), getattr(ref, name)(a), 1e-5, 1e-6)
    small = a * np.float32(0.25)
    close(oracle, bk.exp(small), ref.exp(small), 1e-5, 1e-6)
    close(oracle, bk.rsqrt(b), ref.rsqrt(b), 1e-5, 1e-6)
    close(oracle, bk.scale(a, 0.37), ref.scale(a, 0.37), 1e-5, 1e-6)
    close(oracle, bk.add_scaled(a, b, -1.25), ref.add_scaled(a, b, -1.25), 1e-5, 1e-6)
    for clamp in [0.0, 2.0, 10.0]:
        close(oracle, bk.swiglu(a, b, clamp), ref.swiglu(a, b, clamp), 1e-5, 1e-6)
        gg, ug = bk.swiglu_backward(a, b, b, clamp)
        wg, wu = ref.swiglu_backward(a, b, b, clamp)
        close(oracle, gg, wg, 1e-5, 1e-6); close(oracle, ug, wu, 1e-5, 1e-6)


# parity_test.go:115-132
@pytest.mark.parametrize("n", AWKWARD)
def test_reduction_parity(oracle, bk, ref, n):
    a = oracle.kt_data(n)
    assert oracle.kt_close(bk.sum(a), ref.sum(a), 1e-4, 1e-4)
    assert bk.max(a) == ref.max(a)
    assert bk.argmax(a) == ref.argmax(a)


def test_reductions_empty_and_ties(bk):
    assert bk.max([]) == 0 and bk.sum([]) == 0 and bk.argmax([]) == 0
    assert bk.argmax([1, 9, 3, 9]) == 1  # first maximum


# parity_test.go:134-170
@pytest.mark.parametrize("rows,cols,inner", [(3, 5, 17), (4, 6, 13), (64, 129, 200), (97, 131, 256), (400, 128, 512)])
def test_linear_algebra_parity(oracle, bk, ref, rows, cols, inner):
    left = oracle.kt_data(rows * inner)
    right = oracle.kt_data_b(inner * cols)
    close(oracle, bk.matmul(left, right, rows, cols, inner), ref.matmul(left, right, rows, cols, inner), 2e-3, 1e-4)
    rt = oracle.kt_data_b(cols * inner)
    close(oracle, bk.matmul_transposed(left, rt, rows, cols, inner), ref.matmul_transposed(left, rt, rows, cols, inner), 2e-3, 1e-4)


def test_dot_product_parity(oracle, bk, ref):
    a, b = oracle.kt_data(257), oracle.kt_data_b(257)
    assert oracle.kt_close(bk.dot_product(a, b), ref.dot_product(a, b), 1e-4, 1e-4)


def test_matmul_random_tight(oracle, bk, ref):
    """float32 accumulation stays within 1e-4 relative of the float64-accumulating oracle (the RL step's gradient bar)."""
    rng = np.random.default_rng(3)
    rows, cols, inner = 200, 264, 768
    left = rng.standard_normal(rows * inner).astype(np.float32)
    right = rng.standard_normal(cols * inner).astype(np.float32)
    got = bk.matmul_transposed(left, right, rows, cols, inner)
    want = ref.matmul_transposed(left, right, rows, cols, inner)
    assert np.max(np.abs(got - want)) <= 1e-4 * np.max(np.abs(want))


# parity_test.go:174-201
@pytest.mark.parametrize("cols", AWKWARD)
def test_row_parity(oracle, bk, ref, cols):
    rows = 5
    x = oracle.kt_data(rows * cols)
    close(oracle, bk.softmax_last_dim(x, rows, cols), ref.softmax_last_dim(x, rows, cols), 1e-5, 1e-6)
    close(oracle, bk.rmsnorm_last_dim(x, rows, cols, 1e-6), ref.rmsnorm_last_dim(x, rows, cols, 1e-6), 1e-5, 1e-6)


ATTN_CASES = [("causal", 6, 6, 8, 0, -1), ("decode", 1, 10, 8, 9, -1), ("sliding", 6, 6, 8, 0, 2), ("sliding-decode", 1, 10, 4, 9, 3),
              ("wide-head", 5, 5, 16, 0, -1), ("d64", 70, 70, 64, 0, -1), ("d128-window", 150, 150, 128, 0, 40), ("offset", 40, 100, 32, 60, -1),
              ("d128-train", 383, 383, 128, 0, -1), ("d128-offset", 70, 200, 128, 130, -1), ("d128-decode", 1, 300, 128, 299, 64)]


# parity_test.go:350-431 (forward + backward), 203-223 (large)
@pytest.mark.parametrize("name,ql,kl,hd,off,win", ATTN_CASES + [("large", 200, 200, 32, 0, -1)])
def test_attention_parity(oracle, bk, ref, name, ql, kl, hd, off, win):
    if hd >= 64:
        rng = np.random.default_rng(1)
        q = (rng.standard_normal(ql * hd) * 0.3).astype(np.float32); k = (rng.standard_normal(kl * hd) * 0.3).astype(np.float32)
        v = rng.standard_normal(kl * hd).astype(np.float32)
    else:
        q, k, v = oracle.kt_data(ql * hd), oracle.kt_data(kl * hd), oracle.kt_data_b(kl * hd)
    want_o, want_l = ref.attention_forward(q, k, v, ql, kl, hd, off, win)
    got_o, got_l = bk.attention_forward(q, k, v, ql, kl, hd, off, win)
    close(oracle, got_o, want_o, 2e-3, 1e-5); close(oracle, got_l, want_l, 2e-3, 1e-5)
    dout = oracle.kt_data(ql * hd)
    wq, wk, wv = ref.attention_backward(q, k, v, dout, want_l, ql, kl, hd, off, win)
    gq, gk, gv = bk.attention_backward(q, k, v, want_o, dout, want_l, ql, kl, hd, off, win)
    close(oracle, gq, wq, 5e-3, 1e-5); close(oracle, gk, wk, 5e-3, 1e-5); close(oracle, gv, wv, 5e-3, 1e-5)


def test_attention_backward_accumulates(oracle, bk, ref):
    """Gradients add into the destination slices (kernels/backend.go:217-220)."""
    ql = kl = 6; hd = 8
    q, k, v = oracle.kt_data(ql * hd), oracle.kt_data(kl * hd), oracle.kt_data_b(kl * hd)
    o, l = ref.attention_forward(q, k, v, ql, kl, hd, 0, -1)
    dout = oracle.kt_data(ql * hd)
    base = np.ones(ql * hd, np.float32)
    gq, gk, gv = bk.attention_backward(q, k, v, o, dout, l, ql, kl, hd, 0, -1, dq=base, dk=base, dv=base)
    wq, wk, wv = ref.attention_backward(q, k, v, dout, l, ql, kl, hd, 0, -1, dq=base, dk=base, dv=base)
    close(oracle, gq, wq, 5e-3, 1e-5); close(oracle, gk, wk, 5e-3, 1e-5); close(oracle, gv, wv, 5e-3, 1e-5)


# parity_test.go:315-346
def test_attention_backward_row_correction(oracle, bk, ref):
    ql = kl = 6; hd = 8
    q, k, v = oracle.kt_data(ql * hd), oracle.kt_data(kl * hd), oracle.kt_data_b(kl * hd)
    o, l = ref.attention_forward(q, k, v, ql, kl, hd, 0, -1)
    dout = oracle.kt_data(ql * hd)
    rc = oracle.kt_data_b(ql) * np.float32(0.1)
    wq, wk, wv = ref.attention_backward(q, k, v, dout, l, ql, kl, hd, 0, -1, row_correction=rc)
    gq, gk, gv = bk.attention_backward(q, k, v, o, dout, l, ql, kl, hd, 0, -1, row_correction=rc)
    close(oracle, gq, wq, 5e-3, 1e-5); close(oracle, gk, wk, 5e-3, 1e-5); close(oracle, gv, wv, 5e-3, 1e-5)


# parity_test.go:263-310
@pytest.mark.parametrize("name,ql,kl,hd,off,win", ATTN_CASES[:5])
@pytest.mark.parametrize("splits", [1, 2, 3, 5])
def test_attention_split_parity(oracle, bk, ref, name, ql, kl, hd, off, win, splits):
    q, k, v = oracle.kt_data(ql * hd), oracle.kt_data(kl * hd), oracle.kt_data_b(kl * hd)
    want_o, want_l = ref.attention_forward(q, k, v, ql, kl, hd, off, win)
    per = (kl + splits - 1) // splits
    parts = [bk.attention_forward_split(q, k, v, ql, kl, hd, off, win, s * per, min((s + 1) * per, kl)) for s in range(splits)]
    got_o, got_l = bk.attention_combine([p[0] for p in parts], [p[1] for p in parts], [p[2] for p in parts], ql, hd)
    close(oracle, got_o, want_o, 2e-3, 1e-5); close(oracle, got_l, want_l, 2e-3, 1e-5)
    # shard statistics agree with the scalar shard statistics up to the per-shard maximum convention
    rparts = [ref.attention_forward_split(q, k, v, ql, kl, hd, off, win, s * per, min((s + 1) * per, kl)) for s in range(splits)]
    ro, rl = ref.attention_combine([p[0] for p in rparts], [p[1] for p in rparts], [p[2] for p in rparts], ql, hd)
    close(oracle, got_o, ro, 2e-3, 1e-5)


# parity_test.go:433-519
def test_attention_segment_mask_parity(oracle, bk, ref):
    ql = kl = 12; hd = 8
    q, k, v = oracle.kt_data(ql * hd), oracle.kt_data(kl * hd), oracle.kt_data_b(kl * hd)
    seg = np.array([0, 0, 0, 0, 1, 1, 1, 2, 2, 2, 2, 2], np.int32)
    want_o, want_l = ref.attention_forward(q, k, v, ql, kl, hd, 0, -1, segments=seg)
    got_o, got_l = bk.attention_forward(q, k, v, ql, kl, hd, 0, -1, segments=seg)
    close(oracle, got_o, want_o, 2e-3, 1e-5); close(oracle, got_l, want_l, 2e-3, 1e-5)
    dout = oracle.kt_data(ql * hd)
    wq, wk, wv = ref.attention_backward(q, k, v, dout, want_l, ql, kl, hd, 0, -1, segments=seg)
    gq, gk, gv = bk.attention_backward(q, k, v, want_o, dout, want_l, ql, kl, hd, 0, -1, segments=seg)
    close(oracle, gq, wq, 5e-3, 1e-5); close(oracle, gk, wk, 5e-3, 1e-5); close(oracle, gv, wv, 5e-3, 1e-5)


# parity_test.go:521-568
def test_indexer_parity(oracle, bk, ref):
    rows, blocks, heads, dim = 9, 13, 3, 24
    q, k, w = oracle.kt_data(rows * heads * dim), oracle.kt_data(blocks * heads * dim), oracle.kt_data_b(heads)
    want = ref.indexer_scores(q, k, w, rows, blocks, heads, dim)
    close(oracle, bk.indexer_scores(q, k, w, rows, blocks, heads, dim), want, 1e-4, 1e-4)
    for group in [1, 4, 5, 13, 20]:
        assert np.array_equal(bk.indexer_block_max(want, rows, blocks, group), ref.indexer_block_max(want, rows, blocks, group))


# parity_test.go:570-612, 648-679: exact indices on tie-heavy inputs
@pytest.mark.parametrize("rows,count,k", [(256, 16, 2), (7, 4, 3), (33, 64, 8), (5, 3, 5), (3, 1500, 4)])
def test_topk_and_gate_exact_indices(oracle, bk, ref, rows, count, k):
    scores = (np.arange(rows * count) % 5).astype(np.float32) * np.float32(0.25)   # many ties
    assert np.array_equal(bk.topk_indices(scores, rows, count, k), ref.topk_indices(scores, rows, count, k))
    logits = oracle.kt_data(rows * count)
    bias = (np.arange(count) % 3).astype(np.float32) * np.float32(0.5)
    gp, gs, gw = bk.moe_gate_topk(logits, bias, rows, count, k)
    wp, ws, ww = ref.moe_gate_topk(logits, bias, rows, count, k)
    assert np.array_equal(gs, ws)
    close(oracle, gp, wp, 1e-5, 1e-6); close(oracle, gw, ww, 1e-5, 1e-6)


# parity_test.go:614-646: empty experts
def test_grouped_matmul_parity(oracle, bk, ref):
    counts = np.array([3, 0, 5, 1, 0, 7], np.int32)
    experts, cols, inner = 6, 24, 40
    inp = oracle.kt_data(int(counts.sum()) * inner); w = oracle.kt_data_b(experts * cols * inner)
    close(oracle, bk.grouped_matmul_transposed(inp, w, counts, experts, cols, inner),
          ref.grouped_matmul_transposed(inp, w, counts, experts, cols, inner), 2e-3, 1e-4)


# Expert shapes large enough for the grouped tensor-core product (each 128-row tile of an expert is one CTA):
# empty experts, experts smaller and larger than a tile, a ragged last tile.
@pytest.mark.parametrize("counts,cols,inner", [([130, 0, 5, 257, 0, 64, 1, 300], 128, 256), ([40, 90], 512, 128), ([0, 0, 700], 192, 64)])
def test_grouped_matmul_tensor_core(oracle, bk, ref, counts, cols, inner):
    counts = np.array(counts, np.int32); experts = len(counts)
    rng = np.random.default_rng(3)
    inp = rng.standard_normal(int(counts.sum()) * inner).astype(np.float32)
    w = rng.standard_normal(experts * cols * inner).astype(np.float32)
    got = bk.grouped_matmul_transposed(inp, w, counts, experts, cols, inner)
    want = ref.grouped_matmul_transposed(inp, w, counts, experts, cols, inner)
    assert np.max(np.abs(got - want)) <= 2e-5 * np.max(np.abs(want))


# The tensor-core path (tcgen05, 3xTF32) serves the large aligned products; these shapes reach it
# through the same entry points, tails included, and must stay float32-faithful.
@pytest.mark.parametrize("rows,cols,inner", [(128, 128, 32), (128, 128, 256), (256, 384, 768), (200, 264, 768), (130, 70, 100), (1000, 3072, 768),
                                             (512, 768, 3072)])
def test_tensor_core_matmul_faithful(oracle, bk, ref, rows, cols, inner):
    rng = np.random.default_rng(rows * 7 + cols)
    left = rng.standard_normal(rows * inner).astype(np.float32)
    rt = rng.standard_normal(cols * inner).astype(np.float32)
    want = ref.matmul_transposed(left, rt, rows, cols, inner)
    got = bk.matmul_transposed(left, rt, rows, cols, inner)
    assert np.max(np.abs(got - want)) <= 2e-5 * np.max(np.abs(want))
    right = rng.standard_normal(inner * cols).astype(np.float32)      # stored [inner, cols]: the transposing operand split
    want = ref.matmul(left, right, rows, cols, inner)
    got = bk.matmul(left, right, rows, cols, inner)
    assert np.max(np.abs(got - want)) <= 2e-5 * np.max(np.abs(want))


# The decode step's products have few rows (the rollout batch) against a weight matrix; they take the weight-streaming
# form of the tensor-core kernel (weights read raw and split on chip, K split over CTAs).  Every row count class, slab
# tails, K tails, K splits with and without remainder, one and two row blocks.
@pytest.mark.parametrize("rows,cols,inner", [(1, 128, 32), (7, 64, 128), (16, 256, 768), (64, 1280, 768), (64, 768, 3072), (100, 200, 100),
                                             (128, 3072, 768), (256, 768, 768), (12, 8192, 128), (40, 1000, 2052)])
def test_few_row_products(oracle, bk, ref, rows, cols, inner):
    rng = np.random.default_rng(rows * 13 + cols)
    left = rng.standard_normal(rows * inner).astype(np.float32)
    rt = rng.standard_normal(cols * inner).astype(np.float32)
    want = ref.matmul_transposed(left, rt, rows, cols, inner)
    got = bk.matmul_transposed(left, rt, rows, cols, inner)
    assert np.max(np.abs(got - want)) <= 2e-5 * np.max(np.abs(want))
    again = bk.matmul_transposed(left, rt, rows, cols, inner)
    assert np.array_equal(got, again)          # fixed summation order: bit-reproducible


def test_wide_product_with_512_rows(bk):
    """x W^T with 512 rows against a very wide weight matrix (the shape of the decode step's lm_head), and a ragged row count."""
    rng = np.random.default_rng(5)
    M, N, K = 512, 16384, 160
    x = rng.standard_normal((M, K)).astype(np.float32); w = rng.standard_normal((N, K)).astype(np.float32)
    got = np.asarray(bk.matmul_transposed(x, w, M, N, K)).reshape(M, N)
    want = x.astype(np.float64) @ w.astype(np.float64).T
    assert np.max(np.abs(got - want)) <= 1e-5 * np.sqrt(K) * 4
    M2 = 300                                                   # a ragged last row block
    got2 = np.asarray(bk.matmul_transposed(x[:M2], w, M2, N, K)).reshape(M2, N)
    assert np.max(np.abs(got2 - want[:M2])) <= 1e-5 * np.sqrt(K) * 4
