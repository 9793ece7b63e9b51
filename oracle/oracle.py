"""ctypes binding of the CPU oracle (``oracle/gn_oracle.cpp``).

TEST INFRASTRUCTURE ONLY: imported by tests, by the smoke check and by the
benchmark's CPU-baseline leg, never by the product package.

``mode`` selects the flavour everywhere: 0 = restatement of the reference's
``kernels/scalar`` backend (float64 accumulation; the parity oracle), 1 =
restatement of the structure of ``kernels/simd`` (float32 lanes, polynomial
exp; the timed CPU baseline).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_BUILD = _HERE / "_build"

f32p = C.POINTER(C.c_float)
i32p = C.POINTER(C.c_int32)
u64p = C.POINTER(C.c_uint64)


def build(force: bool = False) -> None:
    """Compile the oracle with the committed Makefile (g++, OpenMP)."""
    if force:
        subprocess.run(["make", "-C", str(_HERE), "clean"], check=True, capture_output=True)
    subprocess.run(["make", "-C", str(_HERE)], check=True, capture_output=True)


def _has_avx512() -> bool:
    try:
        with open("/proc/cpuinfo") as handle:
            for line in handle:
                if line.startswith("flags"):
                    flags = set(line.split(":", 1)[1].split())
                    return {"avx512f", "avx512bw", "avx512dq", "avx512vl", "avx512cd"} <= flags
    except OSError:
        pass
    return False


def isa() -> str:
    return "avx512" if _has_avx512() else "avx2"


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    name = "libgnoracle_v4.so" if _has_avx512() else "libgnoracle_v3.so"
    path = _BUILD / name
    if not path.exists():
        build()
    _lib = C.CDLL(str(path))
    _declare(_lib)
    return _lib


class OrConfig(C.Structure):
    _fields_ = [
        ("sequence_len", C.c_int32), ("vocab_size", C.c_int32), ("n_layer", C.c_int32), ("n_head", C.c_int32),
        ("n_kv_head", C.c_int32), ("embed_dim", C.c_int32), ("rotary_dims", C.c_int32), ("window_pattern", C.c_char * 16),
        ("n_experts", C.c_int32), ("experts_per_token", C.c_int32), ("expert_hidden", C.c_int32), ("shared_hidden", C.c_int32),
        ("moe_clamp", C.c_float), ("moe_scale", C.c_float), ("mla_latent", C.c_int32), ("mla_rotary_dims", C.c_int32),
    ]


def _declare(l: C.CDLL) -> None:
    l.or_num_threads.restype = C.c_int
    l.or_sum.restype = C.c_float
    l.or_max.restype = C.c_float
    l.or_dot.restype = C.c_float
    l.or_argmax.restype = C.c_int64
    l.or_kth_largest.restype = C.c_float
    l.or_sampler_uniform.restype = C.c_float
    l.or_sampler_uniform.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32]
    l.or_reward_uniform.restype = C.c_float
    l.or_reward_uniform.argtypes = [C.c_uint64, C.c_uint32]
    l.or_cross_entropy_per_position.restype = C.c_int64
    l.or_model_create.restype = C.c_void_p
    l.or_model_param_name.restype = C.c_char_p
    l.or_model_param_numel.restype = C.c_int64
    l.or_model_param_data.restype = f32p
    l.or_model_param_grad.restype = f32p
    l.or_cache_create.restype = C.c_void_p
    l.or_policy_gradient_step.restype = C.c_float
    l.or_pg_loss_backward.restype = C.c_double


def _f(a):
    return a.ctypes.data_as(f32p)


def _i(a):
    return a.ctypes.data_as(i32p)


def f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


def num_threads() -> int:
    return int(lib().or_num_threads())


def set_threads(n: int) -> None:
    lib().or_set_threads(C.c_int(n))


# --------------------------------------------------------------------------
# kerneltest fixtures (kernels/kerneltest/compare.go:12-51)
# --------------------------------------------------------------------------
def kt_data(count: int) -> np.ndarray:
    idx = np.arange(count)
    return ((idx % 7).astype(np.float32) - np.float32(3.5) + np.float32(0.1) * (idx % 3).astype(np.float32)).astype(np.float32)


def kt_data_b(count: int) -> np.ndarray:
    idx = np.arange(count)
    return ((idx % 5).astype(np.float32) + np.float32(0.5)).astype(np.float32)


def kt_close(got, want, rel, floor) -> np.ndarray:
    got = np.asarray(got, dtype=np.float32)
    want = np.asarray(want, dtype=np.float32)
    diff = np.abs(got - want)
    scale = np.maximum(np.abs(want), 1.0)
    return diff <= floor + rel * scale


# --------------------------------------------------------------------------
# Backend (kernels/backend.go).  Names follow the Go methods in snake case.
# --------------------------------------------------------------------------
class Backend:
    def __init__(self, mode: int = 0):
        self.mode = mode
        self.l = lib()

    def _binary(self, fn, a, b):
        a, b = f32(a), f32(b)
        d = np.empty_like(a)
        fn(self.mode, _f(d), _f(a), _f(b), C.c_int64(a.size))
        return d

    def _unary(self, fn, a):
        a = f32(a)
        d = np.empty_like(a)
        fn(self.mode, _f(d), _f(a), C.c_int64(a.size))
        return d

    def add(self, a, b): return self._binary(self.l.or_add, a, b)
    def subtract(self, a, b): return self._binary(self.l.or_subtract, a, b)
    def multiply(self, a, b): return self._binary(self.l.or_multiply, a, b)
    def divide(self, a, b): return self._binary(self.l.or_divide, a, b)
    def negate(self, a): return self._unary(self.l.or_negate, a)
    def abs(self, a): return self._unary(self.l.or_abs, a)
    def square(self, a): return self._unary(self.l.or_square, a)
    def relu_squared(self, a): return self._unary(self.l.or_relu_squared, a)
    def exp(self, a): return self._unary(self.l.or_exp, a)
    def sigmoid(self, a): return self._unary(self.l.or_sigmoid, a)
    def tanh(self, a): return self._unary(self.l.or_tanh, a)
    def rsqrt(self, a): return self._unary(self.l.or_rsqrt, a)

    def scale(self, a, factor):
        a = f32(a); d = np.empty_like(a)
        self.l.or_scale(self.mode, _f(d), _f(a), C.c_float(factor), C.c_int64(a.size)); return d

    def add_scaled(self, base, scaled, factor):
        base, scaled = f32(base), f32(scaled); d = np.empty_like(base)
        self.l.or_add_scaled(self.mode, _f(d), _f(base), _f(scaled), C.c_float(factor), C.c_int64(base.size)); return d

    def swiglu(self, gate, up, clamp):
        gate, up = f32(gate), f32(up); d = np.empty_like(gate)
        self.l.or_swiglu(self.mode, _f(d), _f(gate), _f(up), C.c_float(clamp), C.c_int64(gate.size)); return d

    def swiglu_backward(self, gate, up, out_grad, clamp):
        gate, up, out_grad = f32(gate), f32(up), f32(out_grad)
        gg, ug = np.empty_like(gate), np.empty_like(gate)
        self.l.or_swiglu_backward(self.mode, _f(gg), _f(ug), _f(gate), _f(up), _f(out_grad), C.c_float(clamp), C.c_int64(gate.size))
        return gg, ug

    def sum(self, v): v = f32(v); return float(self.l.or_sum(self.mode, _f(v), C.c_int64(v.size)))
    def max(self, v): v = f32(v); return float(self.l.or_max(self.mode, _f(v), C.c_int64(v.size)))
    def argmax(self, v): v = f32(v); return int(self.l.or_argmax(self.mode, _f(v), C.c_int64(v.size)))

    def dot_product(self, a, b):
        a, b = f32(a), f32(b)
        return float(self.l.or_dot(self.mode, _f(a), _f(b), C.c_int64(min(a.size, b.size))))

    def matmul(self, left, right, rows, cols, inner):
        left, right = f32(left), f32(right); d = np.empty(rows * cols, np.float32)
        self.l.or_matmul(self.mode, _f(d), _f(left), _f(right), rows, cols, inner); return d

    def matmul_transposed(self, left, right, rows, cols, inner):
        left, right = f32(left), f32(right); d = np.empty(rows * cols, np.float32)
        self.l.or_matmul_transposed(self.mode, _f(d), _f(left), _f(right), rows, cols, inner); return d

    def softmax_last_dim(self, src, rows, cols):
        src = f32(src); d = np.empty(rows * cols, np.float32)
        self.l.or_softmax_lastdim(self.mode, _f(d), _f(src), C.c_int64(rows), cols); return d

    def rmsnorm_last_dim(self, src, rows, cols, eps):
        src = f32(src); d = np.empty(rows * cols, np.float32)
        self.l.or_rmsnorm_lastdim(self.mode, _f(d), _f(src), C.c_int64(rows), cols, C.c_float(eps)); return d

    def topk_indices(self, scores, rows, count, k):
        scores = f32(scores); d = np.zeros(rows * k, np.int32)
        self.l.or_topk_indices(self.mode, _i(d), _f(scores), rows, count, k); return d

    def moe_gate_topk(self, logits, bias, rows, experts, k):
        logits, bias = f32(logits), f32(bias)
        probs = np.empty(rows * experts, np.float32); sel = np.zeros(rows * k, np.int32); w = np.zeros(rows * k, np.float32)
        self.l.or_moe_gate_topk(self.mode, _f(logits), _f(bias), _f(probs), _i(sel), _f(w), rows, experts, k)
        return probs, sel, w

    def grouped_matmul_transposed(self, inp, weight, counts, experts, cols, inner):
        inp, weight, counts = f32(inp), f32(weight), i32(counts)
        d = np.zeros(int(counts.sum()) * cols, np.float32)
        self.l.or_grouped_matmul_transposed(self.mode, _f(d), _f(inp), _f(weight), _i(counts), experts, cols, inner); return d

    def indexer_scores(self, q, k, w, rows, blocks, heads, dim):
        q, k, w = f32(q), f32(k), f32(w); d = np.empty(rows * blocks, np.float32)
        self.l.or_indexer_scores(self.mode, _f(d), _f(q), _f(k), _f(w), rows, blocks, heads, dim); return d

    def indexer_block_max(self, scores, rows, blocks, group):
        scores = f32(scores); groups = (blocks + max(group, 1) - 1) // max(group, 1)
        d = np.empty(rows * groups, np.float32)
        self.l.or_indexer_block_max(self.mode, _f(d), _f(scores), rows, blocks, group); return d

    def attention_forward(self, q, k, v, ql, kl, hd, offset, window, segments=None):
        q, k, v = f32(q), f32(k), f32(v)
        out = np.empty(ql * hd, np.float32); lse = np.empty(ql, np.float32)
        seg = i32(segments) if segments is not None else None
        self.l.or_attention_forward(self.mode, _f(q), _f(k), _f(v), ql, kl, hd, offset, window,
                                    _i(seg) if seg is not None else None, 0 if seg is None else seg.size, _f(out), _f(lse))
        return out, lse

    def attention_forward_split(self, q, k, v, ql, kl, hd, offset, window, kstart, kend, segments=None):
        q, k, v = f32(q), f32(k), f32(v)
        acc = np.empty(ql * hd, np.float32); mx = np.empty(ql, np.float32); sm = np.empty(ql, np.float32)
        seg = i32(segments) if segments is not None else None
        self.l.or_attention_forward_split(self.mode, _f(q), _f(k), _f(v), ql, kl, hd, offset, window, kstart, kend,
                                          _i(seg) if seg is not None else None, 0 if seg is None else seg.size, _f(acc), _f(mx), _f(sm))
        return acc, mx, sm

    def attention_combine(self, accs, mxs, sms, ql, hd):
        acc = f32(np.stack(accs)); mx = f32(np.stack(mxs)); sm = f32(np.stack(sms))
        out = np.empty(ql * hd, np.float32); lse = np.empty(ql, np.float32)
        self.l.or_attention_combine(self.mode, _f(acc), _f(mx), _f(sm), len(accs), ql, hd, _f(out), _f(lse))
        return out, lse

    def attention_backward(self, q, k, v, dout, lse, ql, kl, hd, offset, window, row_correction=None, segments=None,
                           dq=None, dk=None, dv=None):
        q, k, v, dout, lse = f32(q), f32(k), f32(v), f32(dout), f32(lse)
        dq = np.zeros(ql * hd, np.float32) if dq is None else f32(dq).copy()
        dk = np.zeros(kl * hd, np.float32) if dk is None else f32(dk).copy()
        dv = np.zeros(kl * hd, np.float32) if dv is None else f32(dv).copy()
        rc = f32(row_correction) if row_correction is not None else None
        seg = i32(segments) if segments is not None else None
        self.l.or_attention_backward(self.mode, _f(q), _f(k), _f(v), _f(dout), _f(lse), _f(rc) if rc is not None else None,
                                     ql, kl, hd, offset, window, _i(seg) if seg is not None else None,
                                     0 if seg is None else seg.size, _f(dq), _f(dk), _f(dv))
        return dq, dk, dv


# --------------------------------------------------------------------------
# tensors-level functions
# --------------------------------------------------------------------------
def cross_entropy_per_position(logits, targets, ignore=-1, mode=0):
    logits = f32(logits); targets = i32(targets)
    rows, vocab = logits.shape
    losses = np.empty(rows, np.float32)
    valid = lib().or_cross_entropy_per_position(mode, _f(logits), _i(targets), C.c_int64(rows), vocab, ignore, _f(losses))
    return losses, int(valid)


def cross_entropy_grad(logits, targets, ignore=-1, scale=1.0, mode=0):
    logits = f32(logits); targets = i32(targets)
    rows, vocab = logits.shape
    grad = np.empty((rows, vocab), np.float32)
    lib().or_cross_entropy_grad(mode, _f(logits), _i(targets), C.c_int64(rows), vocab, ignore, C.c_float(scale), _f(grad))
    return grad


def distillation(student, teacher, temperature=1.0, mask=None, scale=1.0, want_grad=True):
    """tensors.DistillationLossPerPosition / DistillationGrad (tensors/loss.go:84-213): losses [rows], valid count, gradient."""
    student, teacher = f32(student), f32(teacher)
    rows, vocab = student.shape
    losses = np.zeros(rows, np.float32)
    grad = np.zeros((rows, vocab), np.float32) if want_grad else None
    mk = i32(mask) if mask is not None else None
    l = lib(); l.or_distillation.restype = C.c_int64
    valid = l.or_distillation(_f(student), _f(teacher), C.c_int64(rows), vocab, C.c_float(temperature), _i(mk) if mk is not None else None,
                              C.c_float(scale), _f(losses), _f(grad) if want_grad else None)
    return losses, int(valid), grad


def softcap(x, cap=15.0):
    x = f32(x); d = np.empty_like(x); lib().or_softcap(_f(d), _f(x), C.c_float(cap), C.c_int64(x.size)); return d


def softcap_backward(out, gout, cap=15.0):
    out, gout = f32(out), f32(gout); d = np.empty_like(out)
    lib().or_softcap_backward(_f(d), _f(out), _f(gout), C.c_float(cap), C.c_int64(out.size)); return d


def relu_squared_backward(inp, gout):
    inp, gout = f32(inp), f32(gout); d = np.empty_like(inp)
    lib().or_relu_squared_backward(_f(d), _f(inp), _f(gout), C.c_int64(inp.size)); return d


def rmsnorm_backward(inp, gout, eps=1e-6):
    inp, gout = f32(inp), f32(gout); d = np.empty_like(inp)
    rows, cols = inp.reshape(-1, inp.shape[-1]).shape
    lib().or_rmsnorm_backward(_f(d), _f(inp), _f(gout), C.c_int64(rows), cols, C.c_float(eps)); return d


def sigmoid_backward(out, gout):
    out, gout = f32(out), f32(gout); d = np.empty_like(out)
    lib().or_sigmoid_backward(_f(d), _f(out), _f(gout), C.c_int64(out.size)); return d


def sample_next_token(logits, temperature, top_k, uniforms=None, seeds=None, group=1, step=0):
    logits = f32(logits)
    rows, vocab = logits.shape
    out = np.empty(rows, np.int32)
    u = f32(uniforms) if uniforms is not None else None
    s = np.ascontiguousarray(seeds, dtype=np.uint64) if seeds is not None else None
    lib().or_sample_next_token(_f(logits), rows, vocab, _f(u) if u is not None else None,
                               s.ctypes.data_as(u64p) if s is not None else None, group, C.c_uint32(step),
                               C.c_float(temperature), top_k, _i(out))
    return out


def kth_largest(values, rank):
    values = f32(values)
    return float(lib().or_kth_largest(_f(values), values.size, rank))


def sampler_uniform(seed, step, row, col):
    return float(lib().or_sampler_uniform(seed, step, row, col))


def reward_uniform(seed, rollout):
    return float(lib().or_reward_uniform(seed, rollout))


def philox(c, k):
    out = (C.c_uint32 * 4)()
    lib().or_philox(C.c_uint32(c[0]), C.c_uint32(c[1]), C.c_uint32(c[2]), C.c_uint32(c[3]), C.c_uint32(k[0]), C.c_uint32(k[1]), out)
    return [int(x) for x in out]


def rotary_tables(x, cos, sin, B, T, H, D, offset):
    x = f32(x).copy(); cos, sin = f32(cos), f32(sin)
    half = cos.shape[-1]
    lib().or_rotary_tables(_f(x), _f(cos), _f(sin), half, B, T, H, D, offset)
    return x


def advantage(rewards, group, mode=0):
    rewards = f32(rewards); adv = np.empty_like(rewards)
    lib().or_advantage(_f(rewards), rewards.size // group, group, mode, _f(adv)); return adv


def build_batch(tokens, lengths, prompt_lengths, pad_token):
    tokens = i32(tokens); lengths = i32(lengths); prompt_lengths = i32(prompt_lengths)
    n, stride = tokens.shape
    max_len = int(lengths.max())
    inputs = np.empty((n, max_len - 1), np.int32); targets = np.empty((n, max_len - 1), np.int32)
    got = lib().or_build_batch(_i(tokens), _i(lengths), _i(prompt_lengths), n, stride, pad_token, _i(inputs), _i(targets))
    assert got == max_len
    return inputs, targets, max_len


def pg_loss_backward(logits, targets, adv, seq_len, norm, mode=0, want_grad=True):
    logits = f32(logits); targets = i32(targets); adv = f32(adv)
    rows, vocab = logits.shape
    nll = np.empty(rows, np.float32)
    grad = np.empty((rows, vocab), np.float32) if want_grad else None
    loss = lib().or_pg_loss_backward(mode, _f(logits), _i(targets), _f(adv), C.c_int64(rows), vocab, seq_len, C.c_float(norm),
                                     _f(nll), _f(grad) if want_grad else None)
    return float(loss), nll, grad


# --------------------------------------------------------------------------
# Optimizer (optimizer/optimizer.go, muon.go, sinkhorn.go): in-place updates of float32 arrays
# --------------------------------------------------------------------------
def adamw_step(param, grad, exp_avg, exp_avg_sq, step, lr, beta1, beta2, eps, weight_decay=0.0):
    lib().or_adamw_step(_f(param), _f(f32(grad)), _f(exp_avg), _f(exp_avg_sq), C.c_int64(param.size), step, C.c_float(lr), C.c_float(beta1),
                        C.c_float(beta2), C.c_float(eps), C.c_float(weight_decay))


def muon_step(param, grad, mom, second_mom, rows, cols, lr, momentum=0.95, ns_steps=5, beta2=0.9, weight_decay=0.0, mode=0):
    lib().or_muon_step(mode, _f(param), _f(f32(grad)), _f(mom), _f(second_mom), rows, cols, C.c_float(lr), C.c_float(momentum), ns_steps,
                       C.c_float(beta2), C.c_float(weight_decay))


def sinkhorn_step(param, grad, mom, rows, cols, lr, momentum=0.95, gamma=0.18, steps=11, tau=1e-3, eps=1e-20):
    lib().or_sinkhorn_step(_f(param), _f(f32(grad)), _f(mom), rows, cols, C.c_float(lr), C.c_float(momentum), C.c_float(gamma), steps,
                           C.c_float(tau), C.c_float(eps))


class Optimizer:
    """chat_rl's MuonAdamW over a dense-preset Model (model/optimizer.go:20-165, cmd/chat_rl/main.go:68-72)."""

    def __init__(self, model, unembedding_lr=0.004, embedding_lr=0.2, matrix_lr=0.02, weight_decay=0.0, scalar_lr=0.5, lr_mult=0.05):
        self.l = lib(); self.model = model
        self.l.or_optimizer_create.restype = C.c_void_p
        self.h = C.c_void_p(self.l.or_optimizer_create(model.h, C.c_float(unembedding_lr), C.c_float(embedding_lr), C.c_float(matrix_lr),
                                                       C.c_float(weight_decay), C.c_float(scalar_lr), C.c_float(lr_mult)))

    def step(self):
        """optimizer.Step() followed by ZeroGrad() (trainer/rl.go:65-66)."""
        self.l.or_optimizer_step(self.h)

    def __del__(self):
        try:
            self.l.or_optimizer_destroy(self.h)
        except Exception:
            pass


# --------------------------------------------------------------------------
# Model
# --------------------------------------------------------------------------
class Model:
    def __init__(self, sequence_len, vocab_size, n_layer, n_head, n_kv_head, embed_dim, rotary_dims=0, window_pattern="L", mode=0,
                 n_experts=0, experts_per_token=0, expert_hidden=0, shared_hidden=0, moe_clamp=0.0, moe_scale=0.0, mla_latent=0,
                 mla_rotary_dims=0):
        self.l = lib()
        self.cfg = OrConfig(sequence_len, vocab_size, n_layer, n_head, n_kv_head, embed_dim, rotary_dims, window_pattern.encode(),
                            n_experts, experts_per_token, expert_hidden, shared_hidden, moe_clamp, moe_scale, mla_latent, mla_rotary_dims)
        self.h = C.c_void_p(self.l.or_model_create(C.byref(self.cfg), mode))
        self.vocab = vocab_size
        self.names = [self.l.or_model_param_name(self.h, i).decode() for i in range(self.l.or_model_param_count(self.h))]

    def __del__(self):
        try:
            self.l.or_model_destroy(self.h)
        except Exception:
            pass

    def shape(self, name):
        r, c = C.c_int(), C.c_int()
        self.l.or_model_param_shape(self.h, name.encode(), C.byref(r), C.byref(c))
        return r.value, c.value

    def param(self, name) -> np.ndarray:
        n = self.l.or_model_param_numel(self.h, name.encode())
        return np.ctypeslib.as_array(self.l.or_model_param_data(self.h, name.encode()), shape=(n,))

    def grad(self, name) -> np.ndarray:
        n = self.l.or_model_param_numel(self.h, name.encode())
        return np.ctypeslib.as_array(self.l.or_model_param_grad(self.h, name.encode()), shape=(n,))

    def zero_grad(self):
        self.l.or_model_zero_grad(self.h)

    def window_sizes(self):
        out = np.zeros(self.cfg.n_layer, np.int32); self.l.or_model_window_sizes(self.h, _i(out)); return out

    def padded_vocab(self):
        return int(self.l.or_model_padded_vocab(self.h))

    def forward(self, ids):
        ids = i32(ids); B, T = ids.shape
        logits = np.empty((B, T, self.vocab), np.float32)
        self.l.or_model_forward(self.h, _i(ids), B, T, _f(logits)); return logits

    def forward_unabsorbed(self, ids):
        """MLA models: logits through the un-absorbed (training) attention construction."""
        ids = i32(ids); B, T = ids.shape
        logits = np.empty((B, T, self.vocab), np.float32)
        self.l.or_model_forward_unabsorbed(self.h, _i(ids), B, T, _f(logits)); return logits

    def moe_forward(self, layer, flat):
        """Routed-expert contribution of one layer for [rows, d] normalised activations -> (output, selected ids)."""
        flat = f32(flat); rows, d = flat.shape
        k = min(self.cfg.experts_per_token or 2, self.cfg.n_experts)
        out = np.empty((rows, d), np.float32); sel = np.empty((rows, k), np.int32)
        self.l.or_model_moe_forward(self.h, layer, _f(flat), C.c_int64(rows), _f(out), _i(sel)); return out, sel

    def train_forward(self, ids):
        ids = i32(ids); B, T = ids.shape
        logits = np.empty((B * T, self.vocab), np.float32)
        self.l.or_train_forward(self.h, _i(ids), B, T, _f(logits)); return logits

    def cache(self, batch, max_seq):
        return Cache(self, batch, max_seq)

    def forward_cached(self, cache, ids):
        ids = i32(ids); B, T = ids.shape
        logits = np.empty((B, T, self.vocab), np.float32)
        self.l.or_model_forward_cached(self.h, cache.h, _i(ids), B, T, _f(logits)); return logits

    def generate(self, prompt, group, max_tokens, temperature, top_k, seed, want_logits=False):
        prompt = i32(prompt)
        toks = np.zeros((group, max_tokens), np.int32); lens = np.zeros(group, np.int32)
        sl = np.zeros((max_tokens, group, self.vocab), np.float32) if want_logits else None
        steps = self.l.or_generate(self.h, _i(prompt), prompt.size, group, max_tokens, C.c_float(temperature), top_k,
                                   C.c_uint64(seed), _i(toks), _i(lens), _f(sl) if want_logits else None)
        return toks, lens, int(steps), sl

    def generate_ex(self, prompt, group, max_tokens, temperature, top_k, seed, thinking=False, thinking_budget=0, forced=None):
        """The engine with its forced-token queue and thinking budget (inference/engine.go:256-314): ``forced`` is a list of
        token lists, one per row, queued before the first step.  Returns tokens, lengths, masks, steps."""
        prompt = i32(prompt)
        toks = np.zeros((group, max_tokens), np.int32); lens = np.zeros(group, np.int32); masks = np.zeros((group, max_tokens), np.int32)
        stride = max([len(f) for f in forced] + [1]) if forced else 1
        fb = np.zeros((group, stride), np.int32); fc = np.zeros(group, np.int32)
        if forced:
            for g, f in enumerate(forced):
                fb[g, :len(f)] = f; fc[g] = len(f)
        steps = self.l.or_generate_ex(self.h, _i(prompt), prompt.size, group, max_tokens, C.c_float(temperature), top_k, C.c_uint64(seed),
                                      int(bool(thinking)), int(thinking_budget), _i(fb), stride, _i(fc), _i(toks), _i(lens), _i(masks))
        return toks, lens, masks, int(steps)

    def policy_gradient_step(self, inputs, targets, adv, norm, taps=False):
        inputs, targets, adv = i32(inputs), i32(targets), f32(adv)
        B, T = inputs.shape
        nll = np.empty(B * T, np.float32) if taps else None
        dl = np.empty((B * T, self.vocab), np.float32) if taps else None
        lg = np.empty((B * T, self.vocab), np.float32) if taps else None
        loss = self.l.or_policy_gradient_step(self.h, _i(inputs), _i(targets), _f(adv), B, T, C.c_float(norm),
                                              _f(nll) if taps else None, _f(dl) if taps else None, _f(lg) if taps else None)
        return float(loss), nll, dl, lg


class Cache:
    def __init__(self, model: Model, batch, max_seq):
        self.model = model
        self.h = C.c_void_p(model.l.or_cache_create(model.h, batch, max_seq))

    def __del__(self):
        try:
            self.model.l.or_cache_destroy(self.h)
        except Exception:
            pass

    def position(self):
        return int(self.model.l.or_cache_position(self.h))

    def replicate_from(self, src: "Cache"):
        self.model.l.or_cache_replicate(self.model.h, self.h, src.h)

# ---------------------------------------------------------------------------------------------- compressed attention blocks
def compressor_forward(hidden, value, weight, bias, ratio, mode=0):
    """ChannelCompressor.Forward (model/compress.go:93-177): hidden [B,T,d], value [B,T,C], weight [C,d], bias [ratio,C]
    -> compressed [B, blocks, C], probabilities [B, blocks, ratio, C]."""
    hidden, value, weight, bias = f32(hidden), f32(value), f32(weight), f32(bias)
    B, T, d = hidden.shape; C_ = value.shape[2]; blocks = (T + ratio - 1) // ratio
    out = np.zeros((B, blocks, C_), np.float32); prob = np.zeros((B, blocks, ratio, C_), np.float32)
    lib().or_compressor_forward(mode, _f(hidden), _f(value), _f(weight), _f(bias), B, T, d, C_, ratio, _f(out), _f(prob))
    return out, prob


def compressor_backward(hidden, value, weight, bias, ratio, grad_compressed, mode=0):
    """ChannelCompressor.Backward (model/compress.go:182-237): gradients of hidden, value, logit weight and bias."""
    hidden, value, weight, bias, grad_compressed = f32(hidden), f32(value), f32(weight), f32(bias), f32(grad_compressed)
    B, T, d = hidden.shape; C_ = value.shape[2]
    comp, prob = compressor_forward(hidden, value, weight, bias, ratio, mode)
    gh = np.zeros_like(hidden); gv = np.zeros_like(value); gw = np.zeros_like(weight); gb = np.zeros_like(bias)
    lib().or_compressor_backward(mode, _f(hidden), _f(value), _f(weight), _f(prob), _f(comp), _f(grad_compressed), B, T, d, C_, ratio,
                                 _f(gh), _f(gv), _f(gw), _f(gb))
    return gh, gv, gw, gb


def compressed_attention_forward(q, kc, vc, ratio, mode=0):
    """compressedAttentionForward (model/compress_attention.go:624-673): q [B,Hq,T,D], kc/vc [B,Hkv,blocks,D]."""
    q, kc, vc = f32(q), f32(kc), f32(vc)
    B, Hq, T, D = q.shape; Hkv, blocks = kc.shape[1], kc.shape[2]
    out = np.zeros_like(q); lse = np.zeros((B, Hq, T), np.float32)
    lib().or_compressed_attention_forward(mode, _f(q), _f(kc), _f(vc), B, Hq, Hkv, T, D, blocks, ratio, _f(out), _f(lse))
    return out, lse


def compressed_attention_sparse_forward(q, kc, vc, selection, counts, mode=0):
    """compressedAttentionForwardSparse (model/compress_attention.go:321-374): selection [B*Hkv, T, topk], counts [B*Hkv, T]."""
    q, kc, vc = f32(q), f32(kc), f32(vc); selection, counts = i32(selection), i32(counts)
    B, Hq, T, D = q.shape; Hkv, blocks = kc.shape[1], kc.shape[2]; topk = selection.shape[-1]
    out = np.zeros_like(q); lse = np.zeros((B, Hq, T), np.float32)
    lib().or_compressed_attention_sparse_forward(mode, _f(q), _f(kc), _f(vc), _i(selection), _i(counts), B, Hq, Hkv, T, D, blocks, topk, _f(out), _f(lse))
    return out, lse


def compressed_attention_sparse_backward(q, kc, vc, dout, lse, selection, counts, row_correction=None, mode=0):
    """compressedAttentionBackwardSparse (model/compress_attention.go:376-433): returns dq, dkc, dvc (from zero)."""
    q, kc, vc, dout, lse = f32(q), f32(kc), f32(vc), f32(dout), f32(lse); selection, counts = i32(selection), i32(counts)
    B, Hq, T, D = q.shape; Hkv, blocks = kc.shape[1], kc.shape[2]; topk = selection.shape[-1]
    rc = f32(row_correction) if row_correction is not None else None
    dq = np.zeros_like(q); dk = np.zeros_like(kc); dv = np.zeros_like(vc)
    lib().or_compressed_attention_sparse_backward(mode, _f(q), _f(kc), _f(vc), _f(dout), _f(lse), _f(rc) if rc is not None else None, _i(selection), _i(counts),
                                                  B, Hq, Hkv, T, D, blocks, topk, _f(dq), _f(dk), _f(dv))
    return dq, dk, dv


def compressed_attention_backward(q, kc, vc, dout, lse, ratio, row_correction=None, mode=0):
    """compressedAttentionBackward (model/compress_attention.go:735-781): returns dq, dkc, dvc (from zero)."""
    q, kc, vc, dout, lse = f32(q), f32(kc), f32(vc), f32(dout), f32(lse)
    B, Hq, T, D = q.shape; Hkv, blocks = kc.shape[1], kc.shape[2]
    rc = f32(row_correction) if row_correction is not None else None
    dq = np.zeros_like(q); dk = np.zeros_like(kc); dv = np.zeros_like(vc)
    lib().or_compressed_attention_backward(mode, _f(q), _f(kc), _f(vc), _f(dout), _f(lse), _f(rc) if rc is not None else None, B, Hq, Hkv, T, D, blocks, ratio,
                                           _f(dq), _f(dk), _f(dv))
    return dq, dk, dv


def merge_branches(oa, la, ob, lb):
    """mergeAttentionBranches (model/compress_attention.go:440-466)."""
    oa, la, ob, lb = f32(oa), f32(la), f32(ob), f32(lb)
    D = oa.shape[-1]; rows = la.size
    out = np.zeros_like(oa); lse = np.zeros_like(la)
    lib().or_merge_branches(_f(oa), _f(la), _f(ob), _f(lb), C.c_int64(rows), D, _f(out), _f(lse))
    return out, lse


def select_blocks(scores, offset, ratio, topk):
    """SelectBlocks (model/indexer.go:186-206): selection [tokens, topk] (-1 padded) and counts."""
    scores = f32(scores); tokens, blocks = scores.shape
    sel = np.full((tokens, max(topk, 0)), -1, np.int32); cnt = np.zeros(tokens, np.int32)
    lib().or_select_blocks(_f(scores), tokens, blocks, offset, ratio, topk, _i(sel), _i(cnt))
    return sel, cnt


def select_blocks_hierarchical(scores, offset, ratio, topk, pool, budget):
    """selectRowBlockMax per token (model/indexer.go:442-513): selection [tokens, topk], counts, candidates [tokens, cap], candidate counts."""
    scores = f32(scores); tokens, blocks = scores.shape
    cap = lib().or_hierarchical_cap(pool, budget)
    sel = np.full((tokens, max(topk, 0)), -1, np.int32); cnt = np.zeros(tokens, np.int32)
    cand = np.full((tokens, cap), -1, np.int32); ccnt = np.zeros(tokens, np.int32)
    lib().or_select_blocks_hierarchical(_f(scores), tokens, blocks, offset, ratio, topk, pool, budget, _i(sel), _i(cnt), _i(cand), _i(ccnt))
    return sel, cnt, cand, ccnt


def select_blocks_within_pool(scores, offset, ratio, topk, candidates, candidate_counts):
    """selectWithinPool over a score matrix (model/indexer.go:547-613)."""
    scores = f32(scores); tokens, blocks = scores.shape
    candidates, candidate_counts = i32(candidates), i32(candidate_counts)
    sel = np.full((tokens, max(topk, 0)), -1, np.int32); cnt = np.zeros(tokens, np.int32)
    lib().or_select_blocks_within_pool(_f(scores), tokens, blocks, offset, ratio, topk, _i(candidates), _i(candidate_counts), candidates.shape[1], _i(sel), _i(cnt))
    return sel, cnt


def indexer_scores_backward(grad_scores, query, key, weight, grad_weight=None):
    """Score part of SparseIndexer.Backward (model/indexer.go:107-151): grad_query, grad_key (fresh), grad_weight (accumulated)."""
    gs, q, k, w = f32(grad_scores), f32(query), f32(key), f32(weight)
    rows, heads, dim = q.shape; blocks = k.shape[0]
    gq = np.zeros_like(q); gk = np.zeros_like(k); gw = np.zeros(heads, np.float32) if grad_weight is None else f32(grad_weight).copy()
    lib().or_indexer_scores_backward(_f(gs), _f(q), _f(k), _f(w), rows, blocks, heads, dim, _f(gq), _f(gk), _f(gw))
    return gq, gk, gw


def indexer_distillation_target(q, kc, ratio):
    """distillationTarget (model/compress_attention.go:155-196): [B * Hkv, T, blocks]."""
    q, kc = f32(q), f32(kc)
    B, Hq, T, D = q.shape; Hkv, blocks = kc.shape[1], kc.shape[2]
    target = np.zeros((B * Hkv, T, blocks), np.float32)
    lib().or_indexer_distillation_target(_f(q), _f(kc), B, Hq, Hkv, T, D, blocks, ratio, _f(target))
    return target


def indexer_distillation_grad(scores, target, ratio, weight, candidates=None, candidate_counts=None):
    """(masked softmax of the scores - target) * weight (model/compress_attention.go:120-151, 203-231, 266-303); scores [n, T, blocks]."""
    scores, target = f32(scores), f32(target)
    n, T, blocks = scores.shape
    grad = np.zeros_like(scores)
    cand = i32(candidates) if candidates is not None else None; cc = i32(candidate_counts) if candidates is not None else None
    lib().or_indexer_distillation_grad(_f(scores), _f(target), _i(cand) if cand is not None else None, _i(cc) if cand is not None else None,
                                       0 if cand is None else cand.shape[-1], C.c_int64(n * T), blocks, T, ratio, C.c_float(weight), _f(grad))
    return grad


def compressed_attention_forward_at(q, kc, vc, ratio, offset, mode=0):
    """The dense global branch of the cached inference path (model/compress_attention.go:962-1003): T tokens at positions offset .. ."""
    q, kc, vc = f32(q), f32(kc), f32(vc)
    B, Hq, T, D = q.shape; Hkv, blocks = kc.shape[1], kc.shape[2]
    out = np.zeros_like(q); lse = np.zeros((B, Hq, T), np.float32)
    lib().or_compressed_attention_forward_at(mode, _f(q), _f(kc), _f(vc), B, Hq, Hkv, T, D, blocks, ratio, offset, _f(out), _f(lse))
    return out, lse
