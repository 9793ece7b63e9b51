"""Building blocks of the compressed attention layers on the device against the oracle (oracle/flash.h): the channel
compressor, attention over the preceding compressed blocks, the merge of two softmax branches, block selection, and the
three composed into the forward of one heavily-compressed attention layer (compressed global branch + sliding-window
local branch, model/compress_attention.go:440-484,562-673)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def bk():
    from gonano_b200.backend import CudaBackend
    return CudaBackend()


def close(got, want, rel, floor):
    got = np.asarray(got, np.float64); want = np.asarray(want, np.float64)
    fin = np.isfinite(want)
    assert np.array_equal(np.isfinite(got), fin) and np.array_equal(got[~fin], want[~fin])
    assert np.all(np.abs(got[fin] - want[fin]) <= floor + rel * np.maximum(np.abs(want[fin]), 1.0))


@pytest.mark.parametrize("B,T,d,C,ratio", [(1, 3, 1, 1, 2), (2, 17, 24, 16, 4), (1, 130, 96, 128, 8), (3, 64, 128, 64, 64), (1, 5, 8, 4, 1)])
def test_compressor_forward(oracle, bk, B, T, d, C, ratio):
    rng = np.random.default_rng(B * 100 + T)
    hidden = rng.standard_normal((B, T, d)).astype(np.float32); value = rng.standard_normal((B, T, C)).astype(np.float32)
    weight = (rng.standard_normal((C, d)) * 0.3).astype(np.float32); bias = (rng.standard_normal((ratio, C)) * 0.5).astype(np.float32)
    want, want_p = oracle.compressor_forward(hidden, value, weight, bias, ratio)
    got, got_p = bk.compressor_forward(hidden, value, weight, bias, ratio)
    close(got_p, want_p, 1e-5, 1e-6); close(got, want, 1e-5, 1e-6)
    blocks = (T + ratio - 1) // ratio
    full = (T // ratio)
    assert np.allclose(got_p[:, :full].sum(axis=2), 1.0, atol=1e-5) and got.shape == (B, blocks, C)


def test_compressor_known_answer(bk):
    out, _ = bk.compressor_forward(np.zeros((1, 3, 1)), np.array([2, 4, 6], np.float32).reshape(1, 3, 1), np.zeros((1, 1)), np.zeros((2, 1)), 2)
    assert out.ravel().tolist() == [3.0, 6.0]                     # model/compress_test.go:10-26


@pytest.mark.parametrize("B,Hq,Hkv,T,D,ratio", [(1, 1, 1, 9, 8, 2), (2, 6, 2, 70, 128, 4), (1, 4, 4, 33, 64, 8), (1, 2, 1, 40, 32, 64),
                                                (2, 8, 1, 300, 128, 4), (1, 4, 2, 1030, 128, 8), (1, 2, 2, 257, 128, 2)])   # the last three: tensor-core path
def test_compressed_attention_forward(oracle, bk, B, Hq, Hkv, T, D, ratio):
    rng = np.random.default_rng(T + D)
    blocks = (T + ratio - 1) // ratio
    q = (rng.standard_normal((B, Hq, T, D)) * 0.4).astype(np.float32)
    kc = (rng.standard_normal((B, Hkv, blocks, D)) * 0.4).astype(np.float32); vc = rng.standard_normal((B, Hkv, blocks, D)).astype(np.float32)
    want, want_l = oracle.compressed_attention_forward(q, kc, vc, ratio)
    got, got_l = bk.compressed_attention_forward(q, kc, vc, ratio)
    close(got, want, 1e-4, 1e-5); close(got_l, want_l, 1e-4, 1e-5)
    assert np.all(got[:, :, :min(ratio, T)] == 0)                 # block 0 has no preceding block


def test_attention_merge(oracle, bk):
    rng = np.random.default_rng(3)
    rows, D = 257, 128
    oa = rng.standard_normal((rows, D)).astype(np.float32); ob = rng.standard_normal((rows, D)).astype(np.float32)
    la = (rng.standard_normal(rows) * 3).astype(np.float32); lb = (rng.standard_normal(rows) * 3).astype(np.float32)
    la[:5] = -np.inf; lb[3:8] = -np.inf
    want, want_l = oracle.merge_branches(oa, la, ob, lb)
    got, got_l = bk.attention_merge(oa, la, ob, lb)
    close(got, want, 1e-6, 1e-7); close(got_l, want_l, 1e-6, 1e-7)


@pytest.mark.parametrize("tokens,blocks,offset,ratio,topk", [(8, 6, 0, 2, 2), (50, 40, 7, 4, 8), (33, 300, 1000, 4, 16), (5, 3, 0, 1, 10), (4, 4, 0, 2, 0)])
def test_select_blocks(oracle, bk, tokens, blocks, offset, ratio, topk):
    rng = np.random.default_rng(tokens + blocks)
    scores = np.round(rng.standard_normal((tokens, blocks)) * 4).astype(np.float32)      # quantised: many ties (model/indexer_test.go:295-316)
    want, want_c = oracle.select_blocks(scores, offset, ratio, topk)
    got, got_c = bk.select_blocks(scores, offset, ratio, topk)
    assert np.array_equal(got_c, want_c) and np.array_equal(got, want)
    sel, cnt = bk.select_blocks(np.array([[5, 5, 5, 1, 2]], np.float32), 10, 1, 2)       # model/indexer_test.go:318-325
    assert sel[0].tolist() == [0, 1]


def test_heavily_compressed_layer_forward(oracle, bk):
    """One HCA attention forward: K and V compressed per kv head from the layer input, the global branch over the
    preceding compressed blocks, the local sliding-window branch over the raw keys, merged by their log-sum-exps."""
    rng = np.random.default_rng(11)
    B, Hq, Hkv, T, D, d, ratio, window = 2, 4, 2, 45, 64, 96, 4, 6
    x = rng.standard_normal((B, T, d)).astype(np.float32)
    q = (rng.standard_normal((B, Hq, T, D)) * 0.4).astype(np.float32)
    k = (rng.standard_normal((B, Hkv, T, D)) * 0.4).astype(np.float32); v = rng.standard_normal((B, Hkv, T, D)).astype(np.float32)
    wk = (rng.standard_normal((D, d)) * 0.2).astype(np.float32); bias = (rng.standard_normal((ratio, D)) * 0.3).astype(np.float32)
    ref = oracle.Backend(0)

    def layer(comp, catt, merge, attn):
        blocks = (T + ratio - 1) // ratio
        kc = np.zeros((B, Hkv, blocks, D), np.float32); vc = np.zeros_like(kc)
        for b in range(B):
            for h in range(Hkv):      # compressForward: the same compressor serves keys and values of every kv head
                kc[b, h] = comp(x[b:b + 1], k[b, h][None], wk, bias, ratio)[0][0]
                vc[b, h] = comp(x[b:b + 1], v[b, h][None], wk, bias, ratio)[0][0]
        og, lg = catt(q, kc, vc, ratio)
        ol = np.zeros_like(q); ll = np.zeros((B, Hq, T), np.float32)
        for b in range(B):
            for h in range(Hq):
                o, l = attn(q[b, h], k[b, h // (Hq // Hkv)], v[b, h // (Hq // Hkv)], T, T, D, 0, window)
                ol[b, h] = np.asarray(o).reshape(T, D); ll[b, h] = np.asarray(l).reshape(T)
        return merge(og.reshape(-1, D), lg.reshape(-1), ol.reshape(-1, D), ll.reshape(-1))

    want, want_l = layer(oracle.compressor_forward, oracle.compressed_attention_forward, oracle.merge_branches, ref.attention_forward)
    got, got_l = layer(bk.compressor_forward, bk.compressed_attention_forward, bk.attention_merge, bk.attention_forward)
    close(got, want, 1e-4, 1e-5); close(got_l, want_l, 1e-4, 1e-5)


def test_compressed_attention_sparse_forward(oracle, bk):
    """Attention over the selected blocks only (model/compress_attention.go:321-374), with the selection the block
    selector made from quantised scores (ties) for every (sequence, kv head)."""
    rng = np.random.default_rng(21)
    B, Hq, Hkv, T, D, ratio, topk = 2, 4, 2, 37, 64, 4, 3
    blocks = (T + ratio - 1) // ratio
    q = (rng.standard_normal((B, Hq, T, D)) * 0.4).astype(np.float32)
    kc = (rng.standard_normal((B, Hkv, blocks, D)) * 0.4).astype(np.float32); vc = rng.standard_normal((B, Hkv, blocks, D)).astype(np.float32)
    sel = np.zeros((B * Hkv, T, topk), np.int32); cnt = np.zeros((B * Hkv, T), np.int32)
    for i in range(B * Hkv):
        scores = np.round(rng.standard_normal((T, blocks)) * 3).astype(np.float32)
        sel[i], cnt[i] = bk.select_blocks(scores, 0, ratio, topk)
        want_s, want_c = oracle.select_blocks(scores, 0, ratio, topk)
        assert np.array_equal(sel[i], want_s) and np.array_equal(cnt[i], want_c)
    want, want_l = oracle.compressed_attention_sparse_forward(q, kc, vc, np.maximum(sel, 0), cnt)
    got, got_l = bk.compressed_attention_sparse_forward(q, kc, vc, np.maximum(sel, 0), cnt)
    close(got, want, 1e-4, 1e-5); close(got_l, want_l, 1e-4, 1e-5)
    assert np.all(got[:, :, :ratio] == 0) and np.all(np.isneginf(got_l[:, :, :ratio]))       # no block precedes block 0
    # with every allowed block selected the sparse form equals the dense one (model/indexer_test.go:327-349, the
    # unbounded selection)
    full = np.zeros((B * Hkv, T, blocks), np.int32); fc = np.zeros((B * Hkv, T), np.int32)
    for t in range(T):
        fc[:, t] = min(t // ratio, blocks); full[:, t, :fc[0, t]] = np.arange(fc[0, t])
    dense, dense_l = bk.compressed_attention_forward(q, kc, vc, ratio)
    sparse, sparse_l = bk.compressed_attention_sparse_forward(q, kc, vc, full, fc)
    close(sparse, dense, 1e-6, 1e-7); close(sparse_l, dense_l, 1e-6, 1e-7)


def test_sparse_compressed_layer_forward(oracle, bk):
    """One sparse compressed attention layer, inference forward, composed from the entry points the way
    model/compress_attention.go does it: K and V compressed per kv head (compressForward), index scores
    I[t, s] = sum_h w_h relu(q_t,h . k_s,h) from the hidden state and the compressed keys (SparseIndexer.Scores,
    model/indexer.go:58-99: two Linear forwards + Backend.IndexerScores per sequence), the top-k preceding blocks per
    token (SelectBlocks), attention over them, the sliding-window branch over the raw keys, merged by log-sum-exp.
    Selection must agree exactly; the outputs within float32 rounding."""
    rng = np.random.default_rng(31)
    B, Hq, Hkv, T, D, d, ratio, window, topk, ih, idim = 2, 4, 2, 53, 64, 96, 4, 5, 3, 2, 16
    blocks = (T + ratio - 1) // ratio
    x = rng.standard_normal((B, T, d)).astype(np.float32)
    q = (rng.standard_normal((B, Hq, T, D)) * 0.4).astype(np.float32)
    k = (rng.standard_normal((B, Hkv, T, D)) * 0.4).astype(np.float32); v = rng.standard_normal((B, Hkv, T, D)).astype(np.float32)
    wc = (rng.standard_normal((D, d)) * 0.2).astype(np.float32); bias = (rng.standard_normal((ratio, D)) * 0.3).astype(np.float32)
    wq = (rng.standard_normal((ih * idim, d)) * 0.2).astype(np.float32); wk = (rng.standard_normal((ih * idim, D)) * 0.3).astype(np.float32)
    hw = np.array([0.7, 1.3], np.float32)
    ref = oracle.Backend(0)

    def layer(be, comp, sparse, merge, select):
        kc = np.zeros((B, Hkv, blocks, D), np.float32); vc = np.zeros_like(kc)
        sel = np.zeros((B * Hkv, T, topk), np.int32); cnt = np.zeros((B * Hkv, T), np.int32)
        for b in range(B):
            iq = be.matmul_transposed(x[b], wq, T, ih * idim, d)                       # indexer queries [T, heads * dim]
            for h in range(Hkv):
                kc[b, h] = comp(x[b:b + 1], k[b, h][None], wc, bias, ratio)[0][0]
                vc[b, h] = comp(x[b:b + 1], v[b, h][None], wc, bias, ratio)[0][0]
                ik = be.matmul_transposed(kc[b, h], wk, blocks, ih * idim, D)          # indexer keys [blocks, heads * dim]
                scores = np.asarray(be.indexer_scores(iq, ik, hw, T, blocks, ih, idim)).reshape(T, blocks)
                sel[b * Hkv + h], cnt[b * Hkv + h] = select(scores, 0, ratio, topk)
        og, lg = sparse(q, kc, vc, np.maximum(sel, 0), cnt)
        ol = np.zeros_like(q); ll = np.zeros((B, Hq, T), np.float32)
        for b in range(B):
            for h in range(Hq):
                o, l = be.attention_forward(q[b, h], k[b, h // (Hq // Hkv)], v[b, h // (Hq // Hkv)], T, T, D, 0, window)
                ol[b, h] = np.asarray(o).reshape(T, D); ll[b, h] = np.asarray(l).reshape(T)
        out, lse = merge(og.reshape(-1, D), lg.reshape(-1), ol.reshape(-1, D), ll.reshape(-1))
        return out, lse, sel, cnt

    want, want_l, want_sel, want_cnt = layer(ref, oracle.compressor_forward, oracle.compressed_attention_sparse_forward, oracle.merge_branches, oracle.select_blocks)
    got, got_l, got_sel, got_cnt = layer(bk, bk.compressor_forward, bk.compressed_attention_sparse_forward, bk.attention_merge, bk.select_blocks)
    assert np.array_equal(got_cnt, want_cnt)
    same = np.all(got_sel == want_sel, axis=(1, 2))
    assert same.all(), "block selection differs"       # scores agree to rounding; a flipped near-tie would show here
    close(got, want, 1e-4, 1e-5); close(got_l, want_l, 1e-4, 1e-5)


@pytest.mark.parametrize("B,T,d,C,ratio", [(2, 5, 4, 3, 2), (2, 37, 48, 32, 4), (1, 130, 96, 128, 8)])
def test_compressor_backward(oracle, bk, B, T, d, C, ratio):
    """ChannelCompressor.Backward (model/compress.go:182-237) against the oracle, whose own backward is held to the
    reference's finite-difference check (tests/test_oracle_golden.py); parameter gradients accumulate."""
    rng = np.random.default_rng(B * 10 + T)
    hidden = rng.standard_normal((B, T, d)).astype(np.float32); value = rng.standard_normal((B, T, C)).astype(np.float32)
    weight = (rng.standard_normal((C, d)) * 0.4).astype(np.float32); bias = (rng.standard_normal((ratio, C)) * 0.5).astype(np.float32)
    blocks = (T + ratio - 1) // ratio
    gc = rng.standard_normal((B, blocks, C)).astype(np.float32)
    want = oracle.compressor_backward(hidden, value, weight, bias, ratio, gc)
    got = bk.compressor_backward(hidden, value, weight, bias, ratio, gc)
    for g, w in zip(got, want):
        close(g, w, 1e-4, 1e-5 * max(1.0, float(np.max(np.abs(w)))))
    gw0 = rng.standard_normal(weight.shape).astype(np.float32); gb0 = rng.standard_normal(bias.shape).astype(np.float32)
    acc = bk.compressor_backward(hidden, value, weight, bias, ratio, gc, grad_weight=gw0, grad_bias=gb0)
    close(acc[2], got[2] + gw0, 1e-5, 1e-5); close(acc[3], got[3] + gb0, 1e-5, 1e-5)


# compressedAttentionBackward (model/compress_attention.go:735-781): with and without a row correction, grouped heads,
# a ragged last block, and accumulation into gradients that already hold values
@pytest.mark.parametrize("B,Hq,Hkv,T,D,ratio,corr", [(1, 1, 1, 9, 8, 2, False), (2, 6, 2, 70, 128, 4, False), (1, 4, 4, 33, 64, 8, True),
                                                    (1, 2, 1, 40, 32, 64, False), (2, 6, 2, 130, 128, 4, True),
                                                    (2, 8, 1, 300, 128, 4, True), (1, 4, 2, 530, 128, 8, False), (1, 3, 3, 257, 128, 2, True)])   # the last three: mma.sync path
def test_compressed_attention_backward(oracle, bk, B, Hq, Hkv, T, D, ratio, corr):
    rng = np.random.default_rng(T * 3 + D)
    blocks = (T + ratio - 1) // ratio
    q = (rng.standard_normal((B, Hq, T, D)) * 0.4).astype(np.float32)
    kc = (rng.standard_normal((B, Hkv, blocks, D)) * 0.4).astype(np.float32); vc = rng.standard_normal((B, Hkv, blocks, D)).astype(np.float32)
    dout = rng.standard_normal((B, Hq, T, D)).astype(np.float32)
    _, lse = oracle.compressed_attention_forward(q, kc, vc, ratio)
    rc = rng.standard_normal((B, Hq, T)).astype(np.float32) if corr else None
    if corr:
        lse = (lse + np.abs(rng.standard_normal(lse.shape)).astype(np.float32)).astype(np.float32)     # a merged row's lse exceeds the branch's own
    want = oracle.compressed_attention_backward(q, kc, vc, dout, lse, ratio, rc)
    got = bk.compressed_attention_backward(q, kc, vc, dout, lse, ratio, rc)
    # an entry of dkc / dvc sums thousands of terms of the size of the tensor's largest entries (with an arbitrary row correction
    # they do not cancel), so the floor scales with that size; the relative part stays element-wise
    for g, w in zip(got, want):
        close(g, w, 2e-4, 2e-5 * max(1.0, float(np.max(np.abs(w)))))
    assert np.all(got[0][:, :, :min(ratio, T)] == 0) and np.all(got[1][:, :, (T - 1) // ratio:] == 0)   # no preceding block / no later token
    seed = [rng.standard_normal(x.shape).astype(np.float32) for x in (q, kc, vc)]
    acc = bk.compressed_attention_backward(q, kc, vc, dout, lse, ratio, rc, *seed)
    for a, s0, w in zip(acc, seed, want):
        close(a, s0 + w, 2e-4, 2e-5 * max(1.0, float(np.max(np.abs(w)))))


# compressedAttentionBackwardSparse (model/compress_attention.go:376-433)
@pytest.mark.parametrize("B,Hq,Hkv,T,D,ratio,topk,corr", [(2, 4, 2, 37, 64, 4, 3, False), (1, 6, 2, 130, 128, 4, 8, True), (1, 2, 2, 21, 32, 2, 40, False)])
def test_compressed_attention_sparse_backward(oracle, bk, B, Hq, Hkv, T, D, ratio, topk, corr):
    rng = np.random.default_rng(T + topk)
    blocks = (T + ratio - 1) // ratio
    q = (rng.standard_normal((B, Hq, T, D)) * 0.4).astype(np.float32)
    kc = (rng.standard_normal((B, Hkv, blocks, D)) * 0.4).astype(np.float32); vc = rng.standard_normal((B, Hkv, blocks, D)).astype(np.float32)
    dout = rng.standard_normal((B, Hq, T, D)).astype(np.float32)
    sel = np.zeros((B * Hkv, T, topk), np.int32); cnt = np.zeros((B * Hkv, T), np.int32)
    for i in range(B * Hkv):
        sel[i], cnt[i] = oracle.select_blocks(np.round(rng.standard_normal((T, blocks)) * 3).astype(np.float32), 0, ratio, topk)
    sel = np.maximum(sel, 0)
    _, lse = oracle.compressed_attention_sparse_forward(q, kc, vc, sel, cnt)
    rc = rng.standard_normal((B, Hq, T)).astype(np.float32) if corr else None
    if corr:
        lse = (lse + np.abs(rng.standard_normal(lse.shape)).astype(np.float32)).astype(np.float32)
    want = oracle.compressed_attention_sparse_backward(q, kc, vc, dout, lse, sel, cnt, rc)
    got = bk.compressed_attention_sparse_backward(q, kc, vc, dout, lse, sel, cnt, rc)
    for g, w in zip(got, want):
        close(g, w, 2e-4, 2e-5)
    # every allowed block selected: the dense backward
    full = np.zeros((B * Hkv, T, blocks), np.int32); fc = np.zeros((B * Hkv, T), np.int32)
    for t in range(T):
        fc[:, t] = min(t // ratio, blocks); full[:, t, :fc[0, t]] = np.arange(fc[0, t])
    _, dl = oracle.compressed_attention_forward(q, kc, vc, ratio)
    dense = bk.compressed_attention_backward(q, kc, vc, dout, dl, ratio)
    sparse = bk.compressed_attention_sparse_backward(q, kc, vc, dout, dl, full, fc)
    for a, b_ in zip(sparse, dense):      # the dense form may run on the tensor cores (3xTF32), the selected-block form does not
        close(a, b_, 2e-4, 2e-5 * max(1.0, float(np.max(np.abs(b_)))))


def _hca_layer(ops, x, q, k, v, wk, bias, ratio, window, dout=None):
    """Forward (and, with dout, backward) of one heavily-compressed attention layer from the blocks: compressor per kv head,
    compressed global branch, sliding-window local branch, merge; the backward hands both branches the merged log-sum-exp
    and the merged row correction dO . O (model/train.go:211-226, 289-301)."""
    comp, comp_bwd, catt, catt_bwd, merge, attn, attn_bwd = ops
    B, Hq, T, D = q.shape; Hkv = k.shape[1]; hr = Hq // Hkv
    blocks = (T + ratio - 1) // ratio
    kc = np.zeros((B, Hkv, blocks, D), np.float32); vc = np.zeros_like(kc)
    for b in range(B):
        for h in range(Hkv):
            kc[b, h] = comp(x[b:b + 1], k[b, h][None], wk, bias, ratio)[0][0]
            vc[b, h] = comp(x[b:b + 1], v[b, h][None], wk, bias, ratio)[0][0]
    og, lg = catt(q, kc, vc, ratio)
    ol = np.zeros_like(q); ll = np.zeros((B, Hq, T), np.float32)
    for b in range(B):
        for h in range(Hq):
            o, l = attn(q[b, h], k[b, h // hr], v[b, h // hr], T, T, D, 0, window)
            ol[b, h] = np.asarray(o).reshape(T, D); ll[b, h] = np.asarray(l).reshape(T)
    out, lse = merge(og.reshape(-1, D), lg.reshape(-1), ol.reshape(-1, D), ll.reshape(-1))
    out = np.asarray(out).reshape(B, Hq, T, D); lse = np.asarray(lse).reshape(B, Hq, T)
    if dout is None:
        return out, lse
    rc = np.sum(dout.astype(np.float64) * out.astype(np.float64), axis=-1).astype(np.float32)
    dq, dkc, dvc = catt_bwd(q, kc, vc, dout, lse, ratio, rc)
    dk = np.zeros_like(k); dv = np.zeros_like(v)
    for b in range(B):
        for h in range(Hq):
            g = attn_bwd(q[b, h], k[b, h // hr], v[b, h // hr], out[b, h], dout[b, h], lse[b, h], T, T, D, 0, window, row_correction=rc[b, h],
                         dq=dq[b, h].ravel(), dk=dk[b, h // hr].ravel(), dv=dv[b, h // hr].ravel())
            dq[b, h] = g[0].reshape(T, D); dk[b, h // hr] = g[1].reshape(T, D); dv[b, h // hr] = g[2].reshape(T, D)
    dx = np.zeros_like(x); dw = np.zeros_like(wk); db = np.zeros_like(bias)
    for b in range(B):
        for h in range(Hkv):
            for val, gc, gval in ((k, dkc, dk), (v, dvc, dv)):
                gh, gv_, gw, gb = comp_bwd(x[b:b + 1], val[b, h][None], wk, bias, ratio, gc[b, h][None])
                dx[b] += gh[0]; gval[b, h] += gv_[0]; dw += gw; db += gb
    return out, (dq, dk, dv, dx, dw, db)


def test_heavily_compressed_layer_backward(oracle, bk):
    rng = np.random.default_rng(12)
    B, Hq, Hkv, T, D, d, ratio, window = 2, 4, 2, 45, 64, 48, 4, 6
    x = rng.standard_normal((B, T, d)).astype(np.float32)
    q = (rng.standard_normal((B, Hq, T, D)) * 0.4).astype(np.float32)
    k = (rng.standard_normal((B, Hkv, T, D)) * 0.4).astype(np.float32); v = rng.standard_normal((B, Hkv, T, D)).astype(np.float32)
    wk = (rng.standard_normal((D, d)) * 0.2).astype(np.float32); bias = (rng.standard_normal((ratio, D)) * 0.3).astype(np.float32)
    dout = rng.standard_normal((B, Hq, T, D)).astype(np.float32)
    ref = oracle.Backend(0)

    def ref_attn_bwd(q_, k_, v_, out_, dout_, lse_, ql, kl, hd, off, win, row_correction=None, dq=None, dk=None, dv=None):
        return ref.attention_backward(q_, k_, v_, dout_, lse_, ql, kl, hd, off, win, row_correction=row_correction, dq=dq, dk=dk, dv=dv)

    want_o, want = _hca_layer((oracle.compressor_forward, oracle.compressor_backward, oracle.compressed_attention_forward, oracle.compressed_attention_backward,
                               oracle.merge_branches, ref.attention_forward, ref_attn_bwd), x, q, k, v, wk, bias, ratio, window, dout)
    got_o, got = _hca_layer((bk.compressor_forward, bk.compressor_backward, bk.compressed_attention_forward, bk.compressed_attention_backward,
                             bk.attention_merge, bk.attention_forward, bk.attention_backward), x, q, k, v, wk, bias, ratio, window, dout)
    close(got_o, want_o, 1e-4, 1e-5)
    for g, w in zip(got, want):
        close(g, w, 3e-4, 3e-5)


# the two-level selection (model/indexer.go:442-513) and the selection inside a published candidate list (:547-613)
@pytest.mark.parametrize("tokens,blocks,offset,ratio,topk,pool,budget", [(1, 4, 4, 1, 1, 2, 2), (40, 30, 0, 2, 4, 4, 8), (50, 300, 900, 4, 16, 8, 64),
                                                                         (33, 70, 5, 1, 8, 3, 10), (20, 20, 0, 2, 2, 1, 1000), (9, 16, 64, 4, 64, 8, 0)])
def test_select_blocks_hierarchical(oracle, bk, tokens, blocks, offset, ratio, topk, pool, budget):
    rng = np.random.default_rng(tokens * 7 + blocks)
    scores = np.round(rng.standard_normal((tokens, blocks)) * 4).astype(np.float32)      # quantised: ties in both stages
    if tokens == 1:
        scores = np.array([[4, 0, 3, 3]], np.float32)                                    # model/indexer_test.go:351-365
    want = oracle.select_blocks_hierarchical(scores, offset, ratio, topk, pool, budget)
    got = bk.select_blocks_hierarchical(scores, offset, ratio, topk, pool, budget)
    for g, w in zip(got, want):
        assert np.array_equal(g, w)
    if tokens == 1:
        assert got[2][0].tolist() == [0, 1] and got[0][0].tolist() == [0]
    # the candidate list is optional output: without it the selection is the same
    from gonano_b200._lib import ptr, check
    sel2 = np.full((tokens, topk), -1, np.int32); cnt2 = np.zeros(tokens, np.int32)
    check(bk.lib.gn_select_blocks_hierarchical(ptr(scores), tokens, blocks, offset, ratio, topk, pool, budget, ptr(sel2), ptr(cnt2), None, None))
    assert np.array_equal(sel2, got[0]) and np.array_equal(cnt2, got[1])
    groups = max(1, -(-budget // pool))
    assert got[2].shape[1] == groups * pool and np.all(got[3] <= groups * pool)          # model/indexer_test.go:212-244
    allowed = np.minimum((offset + np.arange(tokens)) // ratio, blocks)
    assert np.all((got[2] < allowed[:, None]) | (got[2] == -1))
    # a later layer that re-selects inside the published candidates finds the same blocks (model/indexer_test.go:183-210)
    want_p = oracle.select_blocks_within_pool(scores, offset, ratio, topk, got[2], got[3])
    got_p = bk.select_blocks_within_pool(scores, offset, ratio, topk, got[2], got[3])
    assert np.array_equal(got_p[0], want_p[0]) and np.array_equal(got_p[1], want_p[1])
    assert np.array_equal(got_p[0], got[0]) and np.array_equal(got_p[1], got[1])
    # candidates published for an earlier position: entries at or beyond the allowed range are dropped
    late = np.roll(got[2], 3, axis=0); late_c = np.roll(got[3], 3)
    want_l = oracle.select_blocks_within_pool(scores, offset, ratio, topk, late, late_c)
    got_l = bk.select_blocks_within_pool(scores, offset, ratio, topk, late, late_c)
    assert np.array_equal(got_l[0], want_l[0]) and np.array_equal(got_l[1], want_l[1])


def test_hierarchical_selection_unbounded_equals_flat(bk):
    rng = np.random.default_rng(5)
    scores = rng.standard_normal((64, 40)).astype(np.float32)                            # no ties (model/indexer_test.go:327-349)
    flat, flat_c = bk.select_blocks(scores, 0, 2, 2)
    for pool in (1, 2, 3):
        sel, cnt, _, _ = bk.select_blocks_hierarchical(scores, 0, 2, 2, pool, 1000)
        assert np.array_equal(sel, flat) and np.array_equal(cnt, flat_c)


# the score part of SparseIndexer.Backward (model/indexer.go:107-151)
@pytest.mark.parametrize("rows,blocks,heads,dim", [(5, 3, 2, 2), (70, 33, 4, 32), (130, 64, 3, 100), (16, 300, 8, 64), (300, 545, 2, 64), (64, 200, 1, 128),
                                                   (257, 70, 3, 7)])   # from 64 x 64 on: the tiled kernels
def test_indexer_scores_backward(oracle, bk, rows, blocks, heads, dim):
    rng = np.random.default_rng(rows + dim)
    q = rng.standard_normal((rows, heads, dim)).astype(np.float32); k = rng.standard_normal((blocks, heads, dim)).astype(np.float32)
    w = rng.standard_normal(heads).astype(np.float32); gs = rng.standard_normal((rows, blocks)).astype(np.float32)
    seed = rng.standard_normal(heads).astype(np.float32)
    want = oracle.indexer_scores_backward(gs, q, k, w, seed)
    got = bk.indexer_scores_backward(gs, q, k, w, seed)
    scale = np.sqrt(dim)
    for g, x in zip(got, want):
        close(g, x, 1e-4, 1e-5 * scale * np.sqrt(max(rows, blocks)))


# the indexer's distillation: target from the main attention logits and the score gradient, free and restricted to a
# published candidate list (model/compress_attention.go:120-196, 203-231, 266-303)
@pytest.mark.parametrize("B,Hq,Hkv,T,D,ratio", [(1, 2, 1, 9, 8, 2), (2, 6, 2, 70, 128, 4), (1, 8, 1, 130, 64, 4), (2, 8, 2, 300, 128, 4), (1, 3, 1, 530, 40, 8)])   # the last two: tiled target
def test_indexer_distillation(oracle, bk, B, Hq, Hkv, T, D, ratio):
    rng = np.random.default_rng(T + Hq)
    blocks = (T + ratio - 1) // ratio
    q = (rng.standard_normal((B, Hq, T, D)) * 0.4).astype(np.float32); kc = (rng.standard_normal((B, Hkv, blocks, D)) * 0.4).astype(np.float32)
    want_t = oracle.indexer_distillation_target(q, kc, ratio)
    got_t = bk.indexer_distillation_target(q, kc, ratio)
    close(got_t, want_t, 1e-5, 1e-6)
    full = np.minimum(np.arange(T) // ratio, blocks) > 0
    assert np.allclose(got_t[:, full].sum(axis=-1), 1.0, atol=1e-5) and np.all(got_t[:, ~full] == 0)
    scores = (rng.standard_normal((B * Hkv, T, blocks)) * 2).astype(np.float32)
    want_g = oracle.indexer_distillation_grad(scores, want_t, ratio, 0.25)
    got_g = bk.indexer_distillation_grad(scores, want_t, ratio, 0.25)
    close(got_g, want_g, 1e-5, 1e-6)
    assert np.allclose(got_g.sum(axis=-1), 0.0, atol=1e-5)                               # softmax and target both sum to one
    # restricted to the candidates a two-level selection published; some rows get an empty list
    cand = np.zeros((B * Hkv, T, 8), np.int32); cc = np.zeros((B * Hkv, T), np.int32)
    for i in range(B * Hkv):
        _, _, cand[i], cc[i] = oracle.select_blocks_hierarchical(scores[i], 0, ratio, 2, 4, 8)
    cc[:, T // 2] = 0
    want_r = oracle.indexer_distillation_grad(scores, want_t, ratio, 0.25, cand.reshape(-1, 8), cc.reshape(-1))
    got_r = bk.indexer_distillation_grad(scores, want_t, ratio, 0.25, cand.reshape(-1, 8), cc.reshape(-1))
    close(got_r, want_r, 1e-5, 1e-6)
    assert np.all(got_r[:, T // 2] == 0)


def _csa_layer_step(ops, x, q, k, v, wc, bias, wq, wk, hw, sel, cnt, cand, ccnt, ratio, window, loss_weight, dout):
    """Training forward and backward of one sparse compressed attention layer that owns its compressor and indexer
    (model/train.go:99-169, 227-262, 289-301), from the blocks: the selection is an input (both arms get the same one);
    the indexer is trained by distillation toward the main attention logits, its key gradient joins the compressed keys'
    gradient before the compressor's backward, its hidden-state gradient joins the layer input's."""
    be = ops["be"]
    B, Hq, T, D = q.shape; Hkv = k.shape[1]; hr = Hq // Hkv; d = x.shape[-1]
    blocks = (T + ratio - 1) // ratio
    heads = hw.shape[0]; hd = wq.shape[0]; idim = hd // heads
    kc = np.zeros((B, Hkv, blocks, D), np.float32); vc = np.zeros_like(kc)
    for b in range(B):
        for h in range(Hkv):
            kc[b, h] = ops["comp"](x[b:b + 1], k[b, h][None], wc, bias, ratio)[0][0]
            vc[b, h] = ops["comp"](x[b:b + 1], v[b, h][None], wc, bias, ratio)[0][0]
    og, lg = ops["sparse"](q, kc, vc, sel, cnt)
    ol = np.zeros_like(q); ll = np.zeros((B, Hq, T), np.float32)
    for b in range(B):
        for h in range(Hq):
            o, l = be.attention_forward(q[b, h], k[b, h // hr], v[b, h // hr], T, T, D, 0, window)
            ol[b, h] = np.asarray(o).reshape(T, D); ll[b, h] = np.asarray(l).reshape(T)
    out, lse = ops["merge"](og.reshape(-1, D), lg.reshape(-1), ol.reshape(-1, D), ll.reshape(-1))
    out = np.asarray(out).reshape(B, Hq, T, D); lse = np.asarray(lse).reshape(B, Hq, T)
    rc = np.sum(dout.astype(np.float64) * out.astype(np.float64), axis=-1).astype(np.float32)
    dq, dkc, dvc = ops["sparse_bwd"](q, kc, vc, dout, lse, sel, cnt, rc)
    # the indexer: scores per (sequence, kv head), distillation gradient, backward through the scores and the two projections
    target = ops["target"](q, kc, ratio)
    dx = np.zeros_like(x); dwq = np.zeros_like(wq); dwk = np.zeros_like(wk); dhw = np.zeros_like(hw)
    for b in range(B):
        iq = np.asarray(be.matmul_transposed(x[b], wq, T, hd, d)).reshape(T, hd)
        for h in range(Hkv):
            i = b * Hkv + h
            ik = np.asarray(be.matmul_transposed(kc[b, h], wk, blocks, hd, D)).reshape(blocks, hd)
            scores = np.asarray(be.indexer_scores(iq, ik, hw, T, blocks, heads, idim)).reshape(1, T, blocks)
            gs = ops["dgrad"](scores, target[i:i + 1], ratio, loss_weight, cand[i], ccnt[i])[0]
            giq, gik, dhw = ops["idx_bwd"](gs, iq.reshape(T, heads, idim), ik.reshape(blocks, heads, idim), hw, dhw)
            giq = giq.reshape(T, hd); gik = gik.reshape(blocks, hd)
            dx[b] += np.asarray(be.matmul(giq, wq, T, d, hd)).reshape(T, d)
            dwq += np.asarray(be.matmul(np.ascontiguousarray(giq.T), x[b], hd, d, T)).reshape(hd, d)
            dkc[b, h] += np.asarray(be.matmul(gik, wk, blocks, D, hd)).reshape(blocks, D)
            dwk += np.asarray(be.matmul(np.ascontiguousarray(gik.T), kc[b, h], hd, D, blocks)).reshape(hd, D)
    dk = np.zeros_like(k); dv = np.zeros_like(v)
    for b in range(B):
        for h in range(Hq):
            g = ops["attn_bwd"](q[b, h], k[b, h // hr], v[b, h // hr], out[b, h], dout[b, h], lse[b, h], T, T, D, 0, window, rc[b, h],
                                dq[b, h].ravel(), dk[b, h // hr].ravel(), dv[b, h // hr].ravel())
            dq[b, h] = g[0].reshape(T, D); dk[b, h // hr] = g[1].reshape(T, D); dv[b, h // hr] = g[2].reshape(T, D)
    dwc = np.zeros_like(wc); db = np.zeros_like(bias)
    for b in range(B):
        for h in range(Hkv):
            for val, gc, gval in ((k, dkc, dk), (v, dvc, dv)):
                gh, gv_, gw, gb = ops["comp_bwd"](x[b:b + 1], val[b, h][None], wc, bias, ratio, gc[b, h][None])
                dx[b] += gh[0]; gval[b, h] += gv_[0]; dwc += gw; db += gb
    return out, (dq, dk, dv, dx, dwc, db, dwq, dwk, dhw)


def test_sparse_compressed_layer_training_step(oracle, bk):
    rng = np.random.default_rng(41)
    B, Hq, Hkv, T, D, d, ratio, window, topk, heads, idim, pool, budget = 2, 4, 2, 53, 64, 48, 4, 5, 3, 2, 16, 2, 6
    blocks = (T + ratio - 1) // ratio
    x = rng.standard_normal((B, T, d)).astype(np.float32)
    q = (rng.standard_normal((B, Hq, T, D)) * 0.4).astype(np.float32)
    k = (rng.standard_normal((B, Hkv, T, D)) * 0.4).astype(np.float32); v = rng.standard_normal((B, Hkv, T, D)).astype(np.float32)
    wc = (rng.standard_normal((D, d)) * 0.2).astype(np.float32); bias = (rng.standard_normal((ratio, D)) * 0.3).astype(np.float32)
    wq = (rng.standard_normal((heads * idim, d)) * 0.2).astype(np.float32); wk = (rng.standard_normal((heads * idim, D)) * 0.3).astype(np.float32)
    hw = np.array([0.7, 1.3], np.float32)
    dout = rng.standard_normal((B, Hq, T, D)).astype(np.float32)
    ref = oracle.Backend(0)
    # the selection and the candidates of the two-level selector, from the oracle's own index scores, for both arms
    cap = 6
    sel = np.zeros((B * Hkv, T, topk), np.int32); cnt = np.zeros((B * Hkv, T), np.int32)
    cand = np.zeros((B * Hkv, T, cap), np.int32); ccnt = np.zeros((B * Hkv, T), np.int32)
    for b in range(B):
        iq = ref.matmul_transposed(x[b], wq, T, heads * idim, d)
        for h in range(Hkv):
            kc = oracle.compressor_forward(x[b:b + 1], k[b, h][None], wc, bias, ratio)[0][0]
            ik = ref.matmul_transposed(kc, wk, blocks, heads * idim, D)
            scores = np.asarray(ref.indexer_scores(iq, ik, hw, T, blocks, heads, idim)).reshape(T, blocks)
            i = b * Hkv + h
            sel[i], cnt[i], cand[i], ccnt[i] = oracle.select_blocks_hierarchical(scores, 0, ratio, topk, pool, budget)
    sel = np.maximum(sel, 0)

    def ref_attn_bwd(q_, k_, v_, out_, dout_, lse_, ql, kl, hdim, off, win, rc_, dq_, dk_, dv_):
        return ref.attention_backward(q_, k_, v_, dout_, lse_, ql, kl, hdim, off, win, row_correction=rc_, dq=dq_, dk=dk_, dv=dv_)

    def dev_attn_bwd(q_, k_, v_, out_, dout_, lse_, ql, kl, hdim, off, win, rc_, dq_, dk_, dv_):
        return bk.attention_backward(q_, k_, v_, out_, dout_, lse_, ql, kl, hdim, off, win, row_correction=rc_, dq=dq_, dk=dk_, dv=dv_)

    want_o, want = _csa_layer_step(dict(be=ref, comp=oracle.compressor_forward, comp_bwd=oracle.compressor_backward, sparse=oracle.compressed_attention_sparse_forward,
                                        sparse_bwd=oracle.compressed_attention_sparse_backward, merge=oracle.merge_branches, target=oracle.indexer_distillation_target,
                                        dgrad=oracle.indexer_distillation_grad, idx_bwd=oracle.indexer_scores_backward, attn_bwd=ref_attn_bwd),
                                   x, q, k, v, wc, bias, wq, wk, hw, sel, cnt, cand, ccnt, ratio, window, 0.1, dout)
    got_o, got = _csa_layer_step(dict(be=bk, comp=bk.compressor_forward, comp_bwd=bk.compressor_backward, sparse=bk.compressed_attention_sparse_forward,
                                      sparse_bwd=bk.compressed_attention_sparse_backward, merge=bk.attention_merge, target=bk.indexer_distillation_target,
                                      dgrad=bk.indexer_distillation_grad, idx_bwd=bk.indexer_scores_backward, attn_bwd=dev_attn_bwd),
                                 x, q, k, v, wc, bias, wq, wk, hw, sel, cnt, cand, ccnt, ratio, window, 0.1, dout)
    close(got_o, want_o, 1e-4, 1e-5)
    names = ("dq", "dk", "dv", "dx", "dwc", "dbias", "dwq", "dwk", "dhw")
    for name, g, w in zip(names, got, want):
        scale = float(np.max(np.abs(w))) if w.size else 1.0
        err = float(np.max(np.abs(np.asarray(g, np.float64) - np.asarray(w, np.float64))))
        assert err <= 3e-4 * max(scale, 1.0) + 3e-5, (name, err, scale)


# the dense global branch of the cached inference path (model/compress_attention.go:962-1003): one decode step and a
# continuation of several tokens over cached blocks; at offset 0 it is the training form
@pytest.mark.parametrize("B,Hq,Hkv,T,D,ratio,blocks,offset", [(4, 8, 1, 1, 128, 4, 51, 203), (2, 6, 2, 7, 64, 4, 10, 30), (1, 2, 2, 5, 32, 8, 3, 100),
                                                              (2, 4, 2, 1, 128, 4, 10, 3), (2, 8, 1, 140, 128, 4, 200, 700), (1, 4, 2, 130, 128, 4, 70, 150),   # these two: tensor-core path
                                                              (4, 8, 1, 1, 128, 4, 300, 1000), (3, 6, 2, 1, 128, 4, 100, 37), (2, 4, 4, 1, 128, 2, 80, 1),
                                                              (8, 8, 1, 1, 128, 4, 2176, 8700)])   # one token over a long cache: the split-context decode kernel
def test_compressed_attention_forward_cached(oracle, bk, B, Hq, Hkv, T, D, ratio, blocks, offset):
    rng = np.random.default_rng(offset + T)
    q = (rng.standard_normal((B, Hq, T, D)) * 0.4).astype(np.float32)
    kc = (rng.standard_normal((B, Hkv, blocks, D)) * 0.4).astype(np.float32); vc = rng.standard_normal((B, Hkv, blocks, D)).astype(np.float32)
    want, want_l = oracle.compressed_attention_forward_at(q, kc, vc, ratio, offset)
    got, got_l = bk.compressed_attention_forward(q, kc, vc, ratio, offset)
    close(got, want, 1e-4, 1e-5); close(got_l, want_l, 1e-4, 1e-5)
    if offset < ratio:
        assert np.all(got[:, :, :ratio - offset] == 0)
    # engine == recompute (inference/inference_test.go:306-440 checks the cached path against a full forward): the last
    # rows of a full-sequence pass equal the cached continuation when the cache holds every block those rows may see
    if (offset + T + ratio - 1) // ratio <= blocks:
        full_T = offset + T
        fq = (rng.standard_normal((B, Hq, full_T, D)) * 0.4).astype(np.float32); fq[:, :, offset:] = q
        nb = (full_T + ratio - 1) // ratio
        fk = np.zeros((B, Hkv, nb, D), np.float32); fv = np.zeros_like(fk)
        m = min(nb, blocks); fk[:, :, :m] = kc[:, :, :m]; fv[:, :, :m] = vc[:, :, :m]
        whole, whole_l = bk.compressed_attention_forward(fq, fk, fv, ratio)
        close(whole[:, :, offset:], got, 1e-4, 1e-5); close(whole_l[:, :, offset:], got_l, 1e-4, 1e-5)   # the two passes may run on different kernels


def test_heavily_compressed_layer_incremental_equals_full(oracle, bk):
    """The cached inference path of one heavily-compressed layer, from the blocks: after a prefill every new token compresses
    the block it completes (compressTail, model/compress_attention.go:848-873: the compressor over that block's rows alone),
    attends to the cached compressed blocks at its position and to the raw keys inside the window, and merges the two.  Each
    row must equal the row of a full-sequence pass (the reference holds its engine to a naive recompute the same way,
    inference/inference_test.go:306-440)."""
    rng = np.random.default_rng(51)
    B, Hq, Hkv, T, D, d, ratio, window, T0 = 2, 4, 2, 41, 128, 64, 4, 6, 18
    hr = Hq // Hkv
    x = rng.standard_normal((B, T, d)).astype(np.float32)
    q = (rng.standard_normal((B, Hq, T, D)) * 0.4).astype(np.float32)
    k = (rng.standard_normal((B, Hkv, T, D)) * 0.4).astype(np.float32); v = rng.standard_normal((B, Hkv, T, D)).astype(np.float32)
    wc = (rng.standard_normal((D, d)) * 0.2).astype(np.float32); bias = (rng.standard_normal((ratio, D)) * 0.3).astype(np.float32)
    ref = oracle.Backend(0)

    def attn_fwd(q_, k_, v_, out_, dout_, lse_, *a, **kw):
        raise AssertionError("forward only")

    want, want_l = _hca_layer((oracle.compressor_forward, None, oracle.compressed_attention_forward, None, oracle.merge_branches, ref.attention_forward, attn_fwd),
                              x, q, k, v, wc, bias, ratio, window)
    full, full_l = _hca_layer((bk.compressor_forward, None, bk.compressed_attention_forward, None, bk.attention_merge, bk.attention_forward, attn_fwd),
                              x, q, k, v, wc, bias, ratio, window)
    close(full, want, 1e-4, 1e-5); close(full_l, want_l, 1e-4, 1e-5)

    cap = T // ratio
    kc = np.zeros((B, Hkv, cap, D), np.float32); vc = np.zeros_like(kc)
    have = 0

    def compress_completed(tokens):
        nonlocal have
        while (have + 1) * ratio <= tokens:
            rows = slice(have * ratio, (have + 1) * ratio)
            for b in range(B):
                for h in range(Hkv):
                    kc[b, h, have] = bk.compressor_forward(x[b:b + 1, rows], k[b, h, rows][None], wc, bias, ratio)[0][0, 0]
                    vc[b, h, have] = bk.compressor_forward(x[b:b + 1, rows], v[b, h, rows][None], wc, bias, ratio)[0][0, 0]
            have += 1

    compress_completed(T0)                                     # the prefill's completed blocks
    for p in range(T0, T):
        compress_completed(p + 1)                              # token p may complete a block; it never attends to it
        og, lg = bk.compressed_attention_forward(q[:, :, p:p + 1], kc[:, :, :have], vc[:, :, :have], ratio, offset=p)
        ol = np.zeros((B, Hq, 1, D), np.float32); ll = np.zeros((B, Hq, 1), np.float32)
        for b in range(B):
            for h in range(Hq):
                o, l = bk.attention_forward(q[b, h, p:p + 1], k[b, h // hr, :p + 1], v[b, h // hr, :p + 1], 1, p + 1, D, p, window)
                ol[b, h, 0] = np.asarray(o).reshape(D); ll[b, h, 0] = np.asarray(l).reshape(())
        out, lse = bk.attention_merge(og.reshape(-1, D), lg.reshape(-1), ol.reshape(-1, D), ll.reshape(-1))
        close(np.asarray(out).reshape(B, Hq, D), full[:, :, p], 2e-5, 2e-6)
        close(np.asarray(lse).reshape(B, Hq), full_l[:, :, p], 2e-5, 2e-6)


# the local sliding-window branch for every (batch, query head), head-major (model/compress_attention.go:488-541)
@pytest.mark.parametrize("B,Hq,Hkv,T,D,window,corr", [(2, 4, 2, 45, 64, 6, True), (2, 8, 1, 300, 128, 64, True), (1, 6, 2, 200, 128, 512, False),
                                                      (1, 2, 2, 37, 128, 5, False), (1, 3, 1, 20, 16, -1, True)])
def test_attention_windowed(oracle, bk, B, Hq, Hkv, T, D, window, corr):
    rng = np.random.default_rng(T + D + window)
    hr = Hq // Hkv
    q = (rng.standard_normal((B, Hq, T, D)) * 0.4).astype(np.float32)
    k = (rng.standard_normal((B, Hkv, T, D)) * 0.4).astype(np.float32); v = rng.standard_normal((B, Hkv, T, D)).astype(np.float32)
    dout = rng.standard_normal((B, Hq, T, D)).astype(np.float32)
    ref = oracle.Backend(0)
    want = np.zeros_like(q); want_l = np.zeros((B, Hq, T), np.float32)
    for b in range(B):
        for h in range(Hq):
            o, l = ref.attention_forward(q[b, h], k[b, h // hr], v[b, h // hr], T, T, D, 0, window)
            want[b, h] = np.asarray(o).reshape(T, D); want_l[b, h] = np.asarray(l).reshape(T)
    got, got_l = bk.attention_windowed_forward(q, k, v, 0, window)
    close(got, want, 1e-4, 1e-5); close(got_l, want_l, 1e-4, 1e-5)
    # backward with the forward's own statistics, or as one branch of a merged softmax: a larger log-sum-exp and a given row correction
    lse = want_l; rc = None
    if corr:
        lse = (want_l + np.abs(rng.standard_normal(want_l.shape)).astype(np.float32)).astype(np.float32)
        rc = rng.standard_normal((B, Hq, T)).astype(np.float32)
    wq = np.zeros_like(q); wk = np.zeros_like(k); wv = np.zeros_like(v)
    for b in range(B):
        for h in range(Hq):
            g = ref.attention_backward(q[b, h], k[b, h // hr], v[b, h // hr], dout[b, h], lse[b, h], T, T, D, 0, window,
                                       row_correction=None if rc is None else rc[b, h], dq=wq[b, h].ravel(), dk=wk[b, h // hr].ravel(), dv=wv[b, h // hr].ravel())
            wq[b, h] = g[0].reshape(T, D); wk[b, h // hr] = g[1].reshape(T, D); wv[b, h // hr] = g[2].reshape(T, D)
    seed = [rng.standard_normal(x.shape).astype(np.float32) for x in (q, k, v)]
    gq, gk, gv = bk.attention_windowed_backward(q, k, v, want, dout, lse, 0, window, rc, *seed)
    for g, s0, w in zip((gq, gk, gv), seed, (wq, wk, wv)):
        close(g, s0 + w, 2e-4, 2e-5 * max(1.0, float(np.max(np.abs(w)))))


# compressForward / compressBackward over every kv head at once (model/compress_attention.go:562-622, 1182-1209) against the
# oracle's compressor applied head by head to keys and values, as the reference does
@pytest.mark.parametrize("B,Hkv,T,d,D,ratio", [(2, 2, 37, 48, 32, 4), (1, 1, 130, 96, 128, 8), (3, 4, 16, 24, 16, 1)])
def test_compress_heads(oracle, bk, B, Hkv, T, d, D, ratio):
    rng = np.random.default_rng(B * 10 + T)
    blocks = (T + ratio - 1) // ratio
    x = rng.standard_normal((B, T, d)).astype(np.float32)
    k = rng.standard_normal((B, Hkv, T, D)).astype(np.float32); v = rng.standard_normal((B, Hkv, T, D)).astype(np.float32)
    w = (rng.standard_normal((D, d)) * 0.3).astype(np.float32); bias = (rng.standard_normal((ratio, D)) * 0.5).astype(np.float32)
    gkc = rng.standard_normal((B, Hkv, blocks, D)).astype(np.float32); gvc = rng.standard_normal((B, Hkv, blocks, D)).astype(np.float32)
    want_kc = np.zeros((B, Hkv, blocks, D), np.float32); want_vc = np.zeros_like(want_kc)
    want = [np.zeros_like(x), np.zeros_like(k), np.zeros_like(v), np.zeros_like(w), np.zeros_like(bias)]
    for b in range(B):
        for h in range(Hkv):
            for val, comp, gc, gval in ((k, want_kc, gkc, want[1]), (v, want_vc, gvc, want[2])):
                comp[b, h], prob = (a[0] for a in oracle.compressor_forward(x[b:b + 1], val[b, h][None], w, bias, ratio))
                gh, gv_, gw, gb = oracle.compressor_backward(x[b:b + 1], val[b, h][None], w, bias, ratio, gc[b, h][None])
                want[0][b] += gh[0]; gval[b, h] = gv_[0]; want[3] += gw; want[4] += gb
    kc, vc, prob = bk.compress_forward(x, k, v, w, bias, ratio)
    close(kc, want_kc, 1e-5, 1e-6); close(vc, want_vc, 1e-5, 1e-6)
    got = bk.compress_backward(x, k, v, w, prob, kc, vc, gkc, gvc, ratio)
    for g, t_ in zip(got, want):
        close(g, t_, 2e-4, 2e-5 * max(1.0, float(np.max(np.abs(t_)))))


# Backend.IndexerScores at sizes that take the tiled kernel (64 x 64 scores per CTA): ragged edges, several heads, dims that are not
# a multiple of the 32-dimension step
@pytest.mark.parametrize("rows,blocks,heads,dim", [(64, 64, 1, 64), (130, 77, 3, 24), (300, 545, 2, 100), (70, 200, 4, 7)])
def test_indexer_scores_tiled(oracle, bk, rows, blocks, heads, dim):
    rng = np.random.default_rng(rows + blocks)
    q = rng.standard_normal((rows, heads, dim)).astype(np.float32); k = rng.standard_normal((blocks, heads, dim)).astype(np.float32)
    w = rng.standard_normal(heads).astype(np.float32)
    want = np.asarray(oracle.Backend(0).indexer_scores(q, k, w, rows, blocks, heads, dim)).reshape(rows, blocks)
    got = np.asarray(bk.indexer_scores(q, k, w, rows, blocks, heads, dim)).reshape(rows, blocks)
    close(got, want, 1e-5, 1e-5 * np.sqrt(dim))


def test_merged_branches_equal_concatenated_attention_forward_and_backward(bk):
    """The reference's numerical contract of the merge (model/swa_test.go:14-113) on the device."""
    from test_oracle_golden import _merge_contract
    bwd = lambda q, k, v, o, dout, lse, ql, kl, hd, off, win, rc: bk.attention_backward(q, k, v, o, dout, lse, ql, kl, hd, off, win, row_correction=rc)
    _merge_contract(bk.attention_forward, bwd, bk.attention_merge, np.random.default_rng(7))
