"""``CudaBackend``: the host-side mirror of the reference's ``kernels.Backend``
(kernels/backend.go:285-297) over the C-ABI's Tier A.  Method names are the Go
method names in snake case; arguments keep the Go order and meaning, slices
are numpy float32 / int32 arrays.  Like the Go contract the methods write into
a destination the caller sized; for convenience they also return it.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import GnAttentionParams, check, ptr


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


class CudaBackend:
    """Selected the way ``tensors.UseKernelBackend(cuda.New())`` selects a backend in the reference."""

    def __init__(self):
        self.lib = _lib.load()

    # ---------------------------------------------------------- Elementwise
    def _binary(self, fn, left, right):
        left, right = _f32(left), _f32(right)
        dst = np.empty_like(left)
        check(fn(ptr(dst), ptr(left), ptr(right), left.size))
        return dst

    def _unary(self, fn, src):
        src = _f32(src)
        dst = np.empty_like(src)
        check(fn(ptr(dst), ptr(src), src.size))
        return dst

    def add(self, left, right): return self._binary(self.lib.gn_add, left, right)
    def subtract(self, left, right): return self._binary(self.lib.gn_subtract, left, right)
    def multiply(self, left, right): return self._binary(self.lib.gn_multiply, left, right)
    def divide(self, left, right): return self._binary(self.lib.gn_divide, left, right)
    def negate(self, src): return self._unary(self.lib.gn_negate, src)
    def abs(self, src): return self._unary(self.lib.gn_abs, src)
    def square(self, src): return self._unary(self.lib.gn_square, src)
    def relu_squared(self, src): return self._unary(self.lib.gn_relu_squared, src)
    def exp(self, src): return self._unary(self.lib.gn_exp, src)
    def sigmoid(self, src): return self._unary(self.lib.gn_sigmoid, src)
    def tanh(self, src): return self._unary(self.lib.gn_tanh, src)
    def rsqrt(self, src): return self._unary(self.lib.gn_rsqrt, src)

    def scale(self, src, factor):
        src = _f32(src); dst = np.empty_like(src)
        check(self.lib.gn_scale(ptr(dst), ptr(src), factor, src.size)); return dst

    def add_scaled(self, base, scaled, factor):
        base, scaled = _f32(base), _f32(scaled); dst = np.empty_like(base)
        check(self.lib.gn_add_scaled(ptr(dst), ptr(base), ptr(scaled), factor, base.size)); return dst

    def swiglu(self, gate, up, clamp):
        gate, up = _f32(gate), _f32(up); dst = np.empty_like(gate)
        check(self.lib.gn_swiglu(ptr(dst), ptr(gate), ptr(up), clamp, gate.size)); return dst

    def swiglu_backward(self, gate, up, out_grad, clamp):
        gate, up, out_grad = _f32(gate), _f32(up), _f32(out_grad)
        gg, ug = np.empty_like(gate), np.empty_like(gate)
        check(self.lib.gn_swiglu_backward(ptr(gg), ptr(ug), ptr(gate), ptr(up), ptr(out_grad), clamp, gate.size)); return gg, ug

    # ----------------------------------------------------------- Reductions
    def sum(self, values):
        values = _f32(values); out = C.c_float()
        check(self.lib.gn_sum(ptr(values), values.size, C.byref(out))); return out.value

    def max(self, values):
        values = _f32(values); out = C.c_float()
        check(self.lib.gn_max(ptr(values), values.size, C.byref(out))); return out.value

    def argmax(self, values):
        values = _f32(values); out = C.c_int64()
        check(self.lib.gn_argmax(ptr(values), values.size, C.byref(out))); return out.value

    # -------------------------------------------------------- LinearAlgebra
    def matmul(self, left, right, rows, cols, inner):
        left, right = _f32(left), _f32(right); dst = np.empty(rows * cols, np.float32)
        check(self.lib.gn_matmul(ptr(dst), ptr(left), ptr(right), rows, cols, inner)); return dst

    def matmul_transposed(self, left, right, rows, cols, inner):
        left, right = _f32(left), _f32(right); dst = np.empty(rows * cols, np.float32)
        check(self.lib.gn_matmul_transposed(ptr(dst), ptr(left), ptr(right), rows, cols, inner)); return dst

    def dot_product(self, left, right):
        left, right = _f32(left), _f32(right); out = C.c_float()
        check(self.lib.gn_dot_product(ptr(left), ptr(right), min(left.size, right.size), C.byref(out))); return out.value

    # -------------------------------------------------------------- Indexer
    def indexer_scores(self, query, key, weight, rows, blocks, heads, dim):
        query, key, weight = _f32(query), _f32(key), _f32(weight); dst = np.empty(rows * blocks, np.float32)
        check(self.lib.gn_indexer_scores(ptr(dst), ptr(query), ptr(key), ptr(weight), rows, blocks, heads, dim)); return dst

    def indexer_scores_backward(self, grad_scores, query, key, weight, grad_weight=None):
        """Score part of SparseIndexer.Backward (model/indexer.go:107-151): grad_query, grad_key (fresh), grad_weight (accumulated)."""
        gs, q, k, w = _f32(grad_scores), _f32(query), _f32(key), _f32(weight)
        rows, heads, dim = q.shape; blocks = k.shape[0]
        gq = np.zeros_like(q); gk = np.zeros_like(k); gw = np.zeros(heads, np.float32) if grad_weight is None else _f32(grad_weight).copy()
        check(self.lib.gn_indexer_scores_backward(ptr(gs), ptr(q), ptr(k), ptr(w), rows, blocks, heads, dim, ptr(gq), ptr(gk), ptr(gw)))
        return gq, gk, gw

    def indexer_distillation_target(self, q, kc, ratio):
        """distillationTarget (model/compress_attention.go:155-196): [B * Hkv, T, blocks]."""
        q, kc = _f32(q), _f32(kc)
        B, Hq, T, D = q.shape; Hkv, blocks = kc.shape[1], kc.shape[2]
        target = np.zeros((B * Hkv, T, blocks), np.float32)
        check(self.lib.gn_indexer_distillation_target(ptr(q), ptr(kc), B, Hq, Hkv, T, D, blocks, ratio, ptr(target)))
        return target

    def indexer_distillation_grad(self, scores, target, ratio, weight, candidates=None, candidate_counts=None):
        """(masked softmax of the scores - target) * weight (model/compress_attention.go:120-151, 203-231, 266-303); scores [n, T, blocks]."""
        scores, target = _f32(scores), _f32(target)
        n, T, blocks = scores.shape
        grad = np.zeros_like(scores)
        cand = _i32(candidates) if candidates is not None else None; cc = _i32(candidate_counts) if candidates is not None else None
        check(self.lib.gn_indexer_distillation_grad(ptr(scores), ptr(target), ptr(cand) if cand is not None else None, ptr(cc) if cand is not None else None,
                                                    0 if cand is None else cand.shape[-1], n * T, blocks, T, ratio, weight, ptr(grad)))
        return grad

    def indexer_block_max(self, scores, rows, blocks, group_size):
        scores = _f32(scores); g = max(group_size, 1)
        dst = np.empty(rows * ((blocks + g - 1) // g), np.float32)
        check(self.lib.gn_indexer_block_max(ptr(dst), ptr(scores), rows, blocks, group_size)); return dst

    # ------------------------------------------------------------------ compressed attention blocks
    def compressor_forward(self, hidden, value, weight, bias, ratio):
        """ChannelCompressor.Forward (model/compress.go:93-177) -> compressed [B, blocks, C], probabilities [B, blocks, ratio, C]."""
        hidden, value, weight, bias = _f32(hidden), _f32(value), _f32(weight), _f32(bias)
        B, T, d = hidden.shape; ch = value.shape[2]; blocks = (T + ratio - 1) // ratio
        out = np.zeros((B, blocks, ch), np.float32); prob = np.zeros((B, blocks, ratio, ch), np.float32)
        check(self.lib.gn_compressor_forward(ptr(hidden), ptr(value), ptr(weight), ptr(bias), B, T, d, ch, ratio, ptr(out), ptr(prob)))
        return out, prob

    def compressor_backward(self, hidden, value, weight, bias, ratio, grad_compressed, grad_weight=None, grad_bias=None):
        """ChannelCompressor.Backward (model/compress.go:182-237): returns grad_hidden, grad_value, grad_weight, grad_bias
        (the last two accumulate into the arrays given, zeros otherwise)."""
        hidden, value, weight, bias, grad_compressed = _f32(hidden), _f32(value), _f32(weight), _f32(bias), _f32(grad_compressed)
        B, T, d = hidden.shape; ch = value.shape[2]
        comp, prob = self.compressor_forward(hidden, value, weight, bias, ratio)
        gh = np.zeros_like(hidden); gv = np.zeros_like(value)
        gw = np.zeros_like(weight) if grad_weight is None else _f32(grad_weight).copy()
        gb = np.zeros_like(bias) if grad_bias is None else _f32(grad_bias).copy()
        check(self.lib.gn_compressor_backward(ptr(hidden), ptr(value), ptr(weight), ptr(prob), ptr(comp), ptr(grad_compressed), B, T, d, ch, ratio,
                                              ptr(gh), ptr(gv), ptr(gw), ptr(gb)))
        return gh, gv, gw, gb

    def compress_forward(self, hidden, key, value, weight, bias, ratio):
        """compressForward (model/compress_attention.go:562-622): key / value [B,Hkv,T,D] -> key_c, value_c [B,Hkv,blocks,D], probabilities [B,blocks,ratio,D]."""
        hidden, key, value, weight, bias = _f32(hidden), _f32(key), _f32(value), _f32(weight), _f32(bias)
        B, T, d = hidden.shape; H, D = key.shape[1], key.shape[3]
        blocks = (T + ratio - 1) // ratio
        kc = np.zeros((B, H, blocks, D), np.float32); vc = np.zeros_like(kc); prob = np.zeros((B, blocks, ratio, D), np.float32)
        check(self.lib.gn_compress_forward(ptr(hidden), ptr(key), ptr(value), ptr(weight), ptr(bias), B, H, T, d, D, ratio, ptr(kc), ptr(vc), ptr(prob)))
        return kc, vc, prob

    def compress_backward(self, hidden, key, value, weight, prob, kc, vc, gkc, gvc, ratio, grad_weight=None, grad_bias=None):
        """compressBackward (model/compress_attention.go:1182-1209): grad_hidden, grad_key, grad_value, grad_weight, grad_bias."""
        hidden, key, value, weight, prob, kc, vc, gkc, gvc = (_f32(x) for x in (hidden, key, value, weight, prob, kc, vc, gkc, gvc))
        B, T, d = hidden.shape; H, D = key.shape[1], key.shape[3]
        gh = np.zeros_like(hidden); gk = np.zeros_like(key); gv = np.zeros_like(value)
        gw = np.zeros_like(weight) if grad_weight is None else _f32(grad_weight).copy()
        gb = np.zeros((ratio, D), np.float32) if grad_bias is None else _f32(grad_bias).copy()
        check(self.lib.gn_compress_backward(ptr(hidden), ptr(key), ptr(value), ptr(weight), ptr(prob), ptr(kc), ptr(vc), ptr(gkc), ptr(gvc), B, H, T, d, D, ratio,
                                            ptr(gh), ptr(gk), ptr(gv), ptr(gw), ptr(gb)))
        return gh, gk, gv, gw, gb

    def compressed_attention_forward(self, q, kc, vc, ratio, offset=0):
        """compressedAttentionForward (model/compress_attention.go:624-673): q [B,Hq,T,D], kc / vc [B,Hkv,blocks,D]; with offset > 0 the
        T tokens stand at positions offset .. over the cached blocks (forwardCompressed, :962-1003)."""
        q, kc, vc = _f32(q), _f32(kc), _f32(vc)
        B, Hq, T, D = q.shape; Hkv, blocks = kc.shape[1], kc.shape[2]
        out = np.zeros_like(q); lse = np.zeros((B, Hq, T), np.float32)
        check(self.lib.gn_compressed_attention_forward_at(ptr(q), ptr(kc), ptr(vc), B, Hq, Hkv, T, D, blocks, ratio, offset, ptr(out), ptr(lse)))
        return out, lse

    def compressed_attention_backward(self, q, kc, vc, dout, lse, ratio, row_correction=None, dq=None, dkc=None, dvc=None):
        """compressedAttentionBackward (model/compress_attention.go:735-781): dq, dkc, dvc (accumulated into the arrays given)."""
        q, kc, vc, dout, lse = _f32(q), _f32(kc), _f32(vc), _f32(dout), _f32(lse)
        B, Hq, T, D = q.shape; Hkv, blocks = kc.shape[1], kc.shape[2]
        rc = _f32(row_correction) if row_correction is not None else None
        gq = np.zeros_like(q) if dq is None else _f32(dq).copy(); gk = np.zeros_like(kc) if dkc is None else _f32(dkc).copy()
        gv = np.zeros_like(vc) if dvc is None else _f32(dvc).copy()
        check(self.lib.gn_compressed_attention_backward(ptr(q), ptr(kc), ptr(vc), ptr(dout), ptr(lse), ptr(rc) if rc is not None else None, B, Hq, Hkv, T, D,
                                                        blocks, ratio, ptr(gq), ptr(gk), ptr(gv)))
        return gq, gk, gv

    def compressed_attention_sparse_backward(self, q, kc, vc, dout, lse, selection, counts, row_correction=None, dq=None, dkc=None, dvc=None):
        """compressedAttentionBackwardSparse (model/compress_attention.go:376-433): dq, dkc, dvc (accumulated into the arrays given)."""
        q, kc, vc, dout, lse = _f32(q), _f32(kc), _f32(vc), _f32(dout), _f32(lse); selection, counts = _i32(selection), _i32(counts)
        B, Hq, T, D = q.shape; Hkv, blocks = kc.shape[1], kc.shape[2]; topk = selection.shape[-1]
        rc = _f32(row_correction) if row_correction is not None else None
        gq = np.zeros_like(q) if dq is None else _f32(dq).copy(); gk = np.zeros_like(kc) if dkc is None else _f32(dkc).copy()
        gv = np.zeros_like(vc) if dvc is None else _f32(dvc).copy()
        check(self.lib.gn_compressed_attention_sparse_backward(ptr(q), ptr(kc), ptr(vc), ptr(dout), ptr(lse), ptr(rc) if rc is not None else None, ptr(selection),
                                                               ptr(counts), B, Hq, Hkv, T, D, blocks, topk, ptr(gq), ptr(gk), ptr(gv)))
        return gq, gk, gv

    def compressed_attention_sparse_forward(self, q, kc, vc, selection, counts):
        """compressedAttentionForwardSparse (model/compress_attention.go:321-374): selection [B*Hkv, T, topk], counts [B*Hkv, T]."""
        q, kc, vc = _f32(q), _f32(kc), _f32(vc); selection, counts = _i32(selection), _i32(counts)
        B, Hq, T, D = q.shape; Hkv, blocks = kc.shape[1], kc.shape[2]; topk = selection.shape[-1]
        out = np.zeros_like(q); lse = np.zeros((B, Hq, T), np.float32)
        check(self.lib.gn_compressed_attention_sparse_forward(ptr(q), ptr(kc), ptr(vc), ptr(selection), ptr(counts), B, Hq, Hkv, T, D, blocks, topk, ptr(out), ptr(lse)))
        return out, lse

    def attention_merge(self, oa, la, ob, lb):
        """mergeAttentionBranches (model/compress_attention.go:440-466)."""
        oa, la, ob, lb = _f32(oa), _f32(la), _f32(ob), _f32(lb)
        out = np.zeros_like(oa); lse = np.zeros_like(la)
        check(self.lib.gn_attention_merge(ptr(oa), ptr(la), ptr(ob), ptr(lb), la.size, oa.shape[-1], ptr(out), ptr(lse)))
        return out, lse

    def select_blocks(self, scores, offset, ratio, topk):
        """SelectBlocks (model/indexer.go:186-206): selection [tokens, topk] (-1 padded), counts [tokens]."""
        scores = _f32(scores); tokens, blocks = scores.shape
        sel = np.full((tokens, max(topk, 0)), -1, np.int32); cnt = np.zeros(tokens, np.int32)
        check(self.lib.gn_select_blocks(ptr(scores), tokens, blocks, offset, ratio, topk, ptr(sel) if topk > 0 else None, ptr(cnt)))
        return sel, cnt

    def select_blocks_hierarchical(self, scores, offset, ratio, topk, pool, budget):
        """selectRowBlockMax per token (model/indexer.go:442-513): selection, counts, candidates [tokens, cap] (-1 padded), candidate counts."""
        scores = _f32(scores); tokens, blocks = scores.shape
        cap = self.lib.gn_hierarchical_cap(pool, budget)
        sel = np.full((tokens, topk), -1, np.int32); cnt = np.zeros(tokens, np.int32)
        cand = np.full((tokens, cap), -1, np.int32); ccnt = np.zeros(tokens, np.int32)
        check(self.lib.gn_select_blocks_hierarchical(ptr(scores), tokens, blocks, offset, ratio, topk, pool, budget, ptr(sel), ptr(cnt), ptr(cand), ptr(ccnt)))
        return sel, cnt, cand, ccnt

    def select_blocks_within_pool(self, scores, offset, ratio, topk, candidates, candidate_counts):
        """selectWithinPool over a score matrix (model/indexer.go:547-613)."""
        scores = _f32(scores); tokens, blocks = scores.shape
        candidates, candidate_counts = _i32(candidates), _i32(candidate_counts)
        sel = np.full((tokens, topk), -1, np.int32); cnt = np.zeros(tokens, np.int32)
        check(self.lib.gn_select_blocks_within_pool(ptr(scores), tokens, blocks, offset, ratio, topk, ptr(candidates), ptr(candidate_counts), candidates.shape[1],
                                                    ptr(sel), ptr(cnt)))
        return sel, cnt

    # ------------------------------------------------------------------ MoE
    def topk_indices(self, scores, rows, count, k):
        scores = _f32(scores); dst = np.zeros(rows * k, np.int32)
        check(self.lib.gn_topk_indices(ptr(dst), ptr(scores), rows, count, k)); return dst

    def moe_gate_topk(self, logits, bias, rows, experts, k):
        logits, bias = _f32(logits), _f32(bias)
        probs = np.empty(rows * experts, np.float32); sel = np.zeros(rows * k, np.int32); w = np.zeros(rows * k, np.float32)
        check(self.lib.gn_moe_gate_topk(ptr(logits), ptr(bias), ptr(probs), ptr(sel), ptr(w), rows, experts, k)); return probs, sel, w

    def grouped_matmul_transposed(self, inp, weight, token_counts, experts, cols, inner):
        inp, weight, token_counts = _f32(inp), _f32(weight), _i32(token_counts)
        dst = np.zeros(int(token_counts.sum()) * cols, np.float32)
        check(self.lib.gn_grouped_matmul_transposed(ptr(dst), ptr(inp), ptr(weight), ptr(token_counts), experts, cols, inner)); return dst

    # ----------------------------------------------------------------- Rows
    def softmax_last_dim(self, src, rows, cols):
        src = _f32(src); dst = np.empty(rows * cols, np.float32)
        check(self.lib.gn_softmax_last_dim(ptr(dst), ptr(src), rows, cols)); return dst

    def rmsnorm_last_dim(self, src, rows, cols, epsilon):
        src = _f32(src); dst = np.empty(rows * cols, np.float32)
        check(self.lib.gn_rmsnorm_last_dim(ptr(dst), ptr(src), rows, cols, epsilon)); return dst

    # ------------------------------------------------------------ Attention
    @staticmethod
    def _params(q, k, v, ql, kl, hd, offset, window, seg):
        p = GnAttentionParams()
        p.query, p.key, p.value = q.ctypes.data, k.ctypes.data, v.ctypes.data
        p.query_len, p.key_len, p.head_dim, p.position_offset, p.window = ql, kl, hd, offset, window
        p.segment_ids = seg.ctypes.data if seg is not None else None
        return p

    def attention_forward(self, q, k, v, ql, kl, hd, offset, window, segments=None):
        q, k, v = _f32(q), _f32(k), _f32(v); seg = _i32(segments) if segments is not None else None
        out = np.empty(ql * hd, np.float32); lse = np.empty(ql, np.float32)
        p = self._params(q, k, v, ql, kl, hd, offset, window, seg)
        check(self.lib.gn_attention_forward(C.byref(p), ptr(out), ptr(lse))); return out, lse

    def attention_windowed_forward(self, q, k, v, offset, window):
        """attentionForwardWindowed (model/compress_attention.go:488-507): q [B,Hq,T,D], k / v [B,Hkv,T,D] -> out, lse [B,Hq,T]."""
        q, k, v = _f32(q), _f32(k), _f32(v)
        B, Hq, T, D = q.shape; Hkv = k.shape[1]
        out = np.zeros_like(q); lse = np.zeros((B, Hq, T), np.float32)
        check(self.lib.gn_attention_windowed_forward(ptr(q), ptr(k), ptr(v), B, Hq, Hkv, T, D, offset, window, ptr(out), ptr(lse)))
        return out, lse

    def attention_windowed_backward(self, q, k, v, out, dout, lse, offset, window, row_correction=None, dq=None, dk=None, dv=None):
        """attentionBackwardWindowed (model/compress_attention.go:509-541): dq, dk, dv (accumulated into the arrays given)."""
        q, k, v, dout, lse = _f32(q), _f32(k), _f32(v), _f32(dout), _f32(lse)
        B, Hq, T, D = q.shape; Hkv = k.shape[1]
        o = _f32(out) if out is not None else None; rc = _f32(row_correction) if row_correction is not None else None
        gq = np.zeros_like(q) if dq is None else _f32(dq).copy(); gk = np.zeros_like(k) if dk is None else _f32(dk).copy()
        gv = np.zeros_like(v) if dv is None else _f32(dv).copy()
        check(self.lib.gn_attention_windowed_backward(ptr(q), ptr(k), ptr(v), ptr(o) if o is not None else None, ptr(dout), ptr(lse),
                                                      ptr(rc) if rc is not None else None, B, Hq, Hkv, T, D, offset, window, ptr(gq), ptr(gk), ptr(gv)))
        return gq, gk, gv

    def attention_forward_split(self, q, k, v, ql, kl, hd, offset, window, key_start, key_end, segments=None):
        q, k, v = _f32(q), _f32(k), _f32(v); seg = _i32(segments) if segments is not None else None
        acc = np.empty(ql * hd, np.float32); mx = np.empty(ql, np.float32); sm = np.empty(ql, np.float32)
        p = self._params(q, k, v, ql, kl, hd, offset, window, seg)
        check(self.lib.gn_attention_forward_split(C.byref(p), key_start, key_end, ptr(acc), ptr(mx), ptr(sm))); return acc, mx, sm

    def attention_combine(self, accs, maxima, sums, ql, hd):
        acc = _f32(np.stack(accs)); mx = _f32(np.stack(maxima)); sm = _f32(np.stack(sums))
        out = np.empty(ql * hd, np.float32); lse = np.empty(ql, np.float32)
        check(self.lib.gn_attention_combine(ptr(acc), ptr(mx), ptr(sm), len(accs), ql, hd, ptr(out), ptr(lse))); return out, lse

    def attention_backward(self, q, k, v, output, out_grad, lse, ql, kl, hd, offset, window, row_correction=None, segments=None,
                           dq=None, dk=None, dv=None):
        q, k, v, output, out_grad, lse = _f32(q), _f32(k), _f32(v), _f32(output), _f32(out_grad), _f32(lse)
        seg = _i32(segments) if segments is not None else None
        rc = _f32(row_correction) if row_correction is not None else None
        dq = np.zeros(ql * hd, np.float32) if dq is None else _f32(dq).copy()
        dk = np.zeros(kl * hd, np.float32) if dk is None else _f32(dk).copy()
        dv = np.zeros(kl * hd, np.float32) if dv is None else _f32(dv).copy()
        p = self._params(q, k, v, ql, kl, hd, offset, window, seg)
        check(self.lib.gn_attention_backward(C.byref(p), ptr(output), ptr(out_grad), ptr(lse), ptr(rc), ptr(dq), ptr(dk), ptr(dv)))
        return dq, dk, dv


# -------------------------------------------------------------------------
# Stand-alone kernels of the RL step
# -------------------------------------------------------------------------
def sample_next_token(logits, temperature, top_k, uniforms=None, seeds=None, group=1, step=0):
    """inference.SampleNextToken (inference/sampler.go:16-25) for a [rows, vocab] logit matrix."""
    lib = _lib.load()
    logits = _f32(logits); rows, vocab = logits.shape
    out = np.empty(rows, np.int32)
    u = _f32(uniforms) if uniforms is not None else None
    s = np.ascontiguousarray(seeds, dtype=np.uint64) if seeds is not None else None
    check(lib.gn_sample_next_token(ptr(logits), rows, vocab, ptr(u), ptr(s), group, step, temperature, top_k, ptr(out)))
    return out


def group_advantage(rewards, group, mode=0):
    """Group-relative advantages (cmd/chat_rl/main.go:137-154); mode 1 divides by the group std."""
    lib = _lib.load()
    rewards = _f32(rewards); adv = np.empty_like(rewards)
    check(lib.gn_group_advantage(ptr(rewards), rewards.size // group, group, mode, ptr(adv)))
    return adv


def pg_loss_backward(logits, targets, advantages, seq_len, norm, softcap=0.0, want_grad=True, in_place=False):
    """Per-token nll, policy-gradient loss and dlogits at given logits (trainer/rl.go:23-56)."""
    lib = _lib.load()
    logits = _f32(logits); targets = _i32(targets); advantages = _f32(advantages)
    rows, vocab = logits.shape
    nll = np.empty(rows, np.float32)
    grad = logits if in_place else (np.empty((rows, vocab), np.float32) if want_grad else None)
    loss = C.c_double()
    check(lib.gn_pg_loss_backward(ptr(logits), ptr(targets), ptr(advantages), rows, vocab, seq_len, norm, softcap, ptr(nll), ptr(grad),
                                  C.byref(loss)))
    return loss.value, nll, grad


def distillation_loss_backward(student, teacher, temperature=1.0, mask=None, scale=1.0, want_grad=True):
    """tensors.DistillationLossPerPosition / DistillationGrad / DistillationLoss (tensors/loss.go:84-213):
    per-position losses, the valid count, the mean loss over the valid positions and the gradient at the student."""
    lib = _lib.load()
    student, teacher = _f32(student), _f32(teacher)
    rows, vocab = student.shape
    mk = _i32(mask) if mask is not None else None
    losses = np.zeros(rows, np.float32)
    grad = np.zeros((rows, vocab), np.float32) if want_grad else None
    total, valid = C.c_double(), C.c_int64()
    check(lib.gn_distillation_loss_backward(ptr(student), ptr(teacher), ptr(mk), rows, vocab, temperature, scale, ptr(losses), ptr(grad),
                                            C.byref(total), C.byref(valid)))
    mean = total.value / valid.value if valid.value else 0.0
    return losses, valid.value, mean, grad


# -------------------------------------------------------------------------
# Optimizer updates of one tensor (optimizer/optimizer.go, muon.go, sinkhorn.go); arrays are updated in place
# -------------------------------------------------------------------------
def adamw_step(param, grad, exp_avg, exp_avg_sq, step, lr, beta1, beta2, eps, weight_decay=0.0):
    lib = _lib.load()
    g = _f32(grad).copy()
    check(lib.gn_adamw_step(ptr(param), ptr(g), ptr(exp_avg), ptr(exp_avg_sq), param.size, step, lr, beta1, beta2, eps, weight_decay))


def muon_step(param, grad, mom, second_mom, rows, cols, lr, momentum=0.95, ns_steps=5, beta2=0.9, weight_decay=0.0):
    lib = _lib.load()
    g = _f32(grad).copy()
    check(lib.gn_muon_step(ptr(param), ptr(g), ptr(mom), ptr(second_mom), rows, cols, lr, momentum, ns_steps, beta2, weight_decay))


def sinkhorn_step(param, grad, mom, rows, cols, lr, momentum=0.95, gamma=0.18, steps=11, tau=1e-3, eps=1e-20):
    lib = _lib.load()
    g = _f32(grad).copy()
    check(lib.gn_sinkhorn_step(ptr(param), ptr(g), ptr(mom), rows, cols, lr, momentum, gamma, steps, tau, eps))
