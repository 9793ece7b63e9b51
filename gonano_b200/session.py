"""Resident session over the C-ABI's Tier B: the host-side mirror of the
reference's ``model.Transformer``, ``inference.Engine`` and ``trainer`` calls
that make up one RL step (cmd/chat_rl/main.go:87-184).

The arithmetic all happens in the CUDA library; this module only moves ids and
scalars across the boundary and assembles the padded batch the way
``cmd/chat_rl`` does.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib
from ._lib import GnConfig, GnGenerateOptions, GnOptimizerConfig, check, ptr

SPECIAL_TOKENS = 11  # tokenizer/special.go:19-31


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class Context:
    """One CUDA device + stream.  ``stream`` may be a raw ``cudaStream_t`` (int), e.g. torch's current stream."""

    def __init__(self, device: int = 0, stream: int | None = None):
        self.lib = _lib.load()
        self.h = C.c_void_p()
        check(self.lib.gn_ctx_create(device, C.c_void_p(stream) if stream else None, C.byref(self.h)))
        self.device = device

    def sync(self):
        check(self.lib.gn_ctx_sync(self.h))

    def launch_count(self) -> int:
        out = C.c_int64()
        check(self.lib.gn_ctx_launch_count(self.h, C.byref(out)))
        return out.value

    def set_gemm(self, kind: int):
        check(self.lib.gn_ctx_set_gemm(self.h, kind))

    def set_option(self, name: str, value: int):
        """Tuning / test switches of include/gonano_cuda.h (gn_ctx_set_option)."""
        check(self.lib.gn_ctx_set_option(self.h, name.encode(), int(value)))

    def profile_kernel(self, kernel: str, dims, iters: int = 10) -> float:
        """Mean milliseconds per launch of one hot kernel on synthetic device data (CUDA events)."""
        arr = (C.c_int64 * len(dims))(*[int(x) for x in dims])
        out = C.c_float()
        check(self.lib.gn_profile_kernel(self.h, kernel.encode(), arr, len(dims), iters, C.byref(out)))
        return out.value

    # ---- data-parallel exchange inside the library (NCCL; one process per GPU)
    @staticmethod
    def comm_unique_id() -> bytes:
        """Rank 0 creates the id and hands these bytes to the other ranks (by any transport)."""
        lib = _lib.load()
        buf = C.create_string_buffer(128)
        check(lib.gn_comm_unique_id(buf))
        return buf.raw

    def comm_init(self, unique_id: bytes, rank: int, world: int):
        """Collective: returns when every rank has joined."""
        check(self.lib.gn_ctx_comm_init(self.h, C.c_char_p(unique_id), rank, world))
        self.rank, self.world = rank, world

    def allreduce_max(self, value: int) -> int:
        v = C.c_int64(int(value))
        check(self.lib.gn_ctx_allreduce_max_i64(self.h, C.byref(v)))
        return int(v.value)

    def close(self):
        if self.h:
            self.lib.gn_ctx_destroy(self.h)
            self.h = C.c_void_p()


class Model:
    """``model.Transformer`` resident on the device: the dense preset (inference and training) and the latent preset
    (absorbed MLA + DeepSeekMoE, inference)."""

    def __init__(self, ctx: Context, sequence_len, vocab_size, n_layer, n_head, n_kv_head, embed_dim, rotary_dims=0, window_pattern="L",
                 n_experts=0, experts_per_token=0, expert_hidden=0, shared_hidden=0, moe_clamp=0.0, moe_scale=0.0, mla_latent=0,
                 mla_rotary_dims=0):
        self.ctx = ctx
        self.lib = ctx.lib
        self.cfg = GnConfig(sequence_len, vocab_size, n_layer, n_head, n_kv_head, embed_dim, rotary_dims, window_pattern.encode(),
                            n_experts, experts_per_token, expert_hidden, shared_hidden, moe_clamp, moe_scale, mla_latent, mla_rotary_dims)
        self.vocab = vocab_size
        self.h = C.c_void_p()
        check(self.lib.gn_model_create(ctx.h, C.byref(self.cfg), C.byref(self.h)))
        n = C.c_int()
        check(self.lib.gn_model_param_count(self.h, C.byref(n)))
        self.names, self._shape = [], {}
        for i in range(n.value):
            name, rows, cols = C.c_char_p(), C.c_int(), C.c_int()
            check(self.lib.gn_model_param_info(self.h, i, C.byref(name), C.byref(rows), C.byref(cols)))
            self.names.append(name.value.decode())
            self._shape[self.names[-1]] = (rows.value, cols.value)

    def close(self):
        if self.h:
            self.lib.gn_model_destroy(self.h)
            self.h = C.c_void_p()

    def shape(self, name):
        return self._shape[name]

    def upload(self, name, values):
        values = _f32(values).reshape(-1)
        check(self.lib.gn_model_upload(self.h, name.encode(), ptr(values), values.size))

    def download(self, name) -> np.ndarray:
        rows, cols = self._shape[name]
        out = np.empty(rows * cols, np.float32)
        check(self.lib.gn_model_download(self.h, name.encode(), ptr(out), out.size))
        return out

    def grad(self, name) -> np.ndarray:
        rows, cols = self._shape[name]
        out = np.empty(rows * cols, np.float32)
        check(self.lib.gn_model_download_grad(self.h, name.encode(), ptr(out), out.size))
        return out

    def zero_grad(self):
        check(self.lib.gn_model_zero_grad(self.h))

    def upload_grad(self, name, values):
        values = _f32(values)
        check(self.lib.gn_model_upload_grad(self.h, name.encode(), ptr(values), values.size))

    def grad_buffer(self):
        """(device address, float count) of the flat gradient buffer that a data-parallel all-reduce sums."""
        p, n = C.c_void_p(), C.c_int64()
        check(self.lib.gn_model_grad_buffer(self.h, C.byref(p), C.byref(n)))
        return p.value, n.value

    def param_buffer(self):
        p, n = C.c_void_p(), C.c_int64()
        check(self.lib.gn_model_param_buffer(self.h, C.byref(p), C.byref(n)))
        return p.value, n.value

    def checksum(self):
        ps, gs = C.c_double(), C.c_double()
        check(self.lib.gn_model_checksum(self.h, C.byref(ps), C.byref(gs)))
        return ps.value, gs.value

    def phase_ms(self, phase: str) -> float:
        out = C.c_float()
        check(self.lib.gn_model_phase_ms(self.h, phase.encode(), C.byref(out)))
        return out.value

    # ---- Transformer.Forward without a cache (model/transformer.go:211-342)
    def forward(self, ids) -> np.ndarray:
        ids = _i32(ids); B, T = ids.shape
        logits = np.empty((B, T, self.vocab), np.float32)
        check(self.lib.gn_model_forward(self.h, ptr(ids), B, T, ptr(logits)))
        return logits

    # ---- Engine.GenerateBatchWith for many prompts (inference/engine.go:336-369)
    def _options(self, rows, thinking, thinking_budget, forced):
        """inference.GenerateOptions plus tokens queued per row before the first step (what a handled tool call queues)."""
        if not thinking and not thinking_budget and not forced:
            return None, ()
        opt = GnGenerateOptions(int(bool(thinking)), int(thinking_budget), None, 0, None)
        keep = ()
        if forced:
            assert len(forced) == rows
            stride = max(max(len(f) for f in forced), 1)
            buf = np.zeros((rows, stride), np.int32); counts = np.zeros(rows, np.int32)
            for r, f in enumerate(forced):
                buf[r, :len(f)] = f; counts[r] = len(f)
            opt.forced = buf.ctypes.data; opt.forced_stride = stride; opt.forced_counts = counts.ctypes.data
            keep = (buf, counts)
        return opt, keep

    def generate_batch(self, prompts, group, max_tokens, temperature, top_k, seeds, want_logits=False, thinking=False, thinking_budget=0,
                       forced=None, want_masks=False):
        prompts = _i32(prompts); P, plen = prompts.shape
        seeds = np.ascontiguousarray(seeds, dtype=np.uint64)
        assert seeds.size == P
        rows = P * group
        tokens = np.zeros((rows, max_tokens), np.int32); lengths = np.zeros(rows, np.int32)
        masks = np.zeros((rows, max_tokens), np.int32) if want_masks else None
        step_logits = np.zeros((max_tokens, rows, self.vocab), np.float32) if want_logits else None
        steps = C.c_int()
        opt, keep = self._options(rows, thinking, thinking_budget, forced)
        check(self.lib.gn_generate_batch_ex(self.h, ptr(prompts), P, plen, group, max_tokens, temperature, top_k, ptr(seeds),
                                            C.byref(opt) if opt is not None else None, ptr(tokens), ptr(lengths), ptr(masks), ptr(step_logits),
                                            C.byref(steps)))
        del keep
        if want_masks:
            return tokens, lengths, steps.value, step_logits, masks
        return tokens, lengths, steps.value, step_logits

    # ---- the same engine one step at a time (tool calls on the host, ensembles)
    def rollout_begin(self, prompts, group, max_tokens, seeds, thinking=False, thinking_budget=0, forced=None):
        prompts = _i32(prompts); P, plen = prompts.shape
        seeds = np.ascontiguousarray(seeds, dtype=np.uint64)
        self._ro = (P * group, max_tokens)
        opt, keep = self._options(P * group, thinking, thinking_budget, forced)
        check(self.lib.gn_rollout_begin(self.h, ptr(prompts), P, plen, group, max_tokens, ptr(seeds), C.byref(opt) if opt is not None else None))
        del keep

    def rollout_logits(self):
        """(device address, logit rows, row divisor) of the current logits [logit_rows, vocab]."""
        p, n, div = C.c_void_p(), C.c_int(), C.c_int()
        check(self.lib.gn_rollout_logits(self.h, C.byref(p), C.byref(n), C.byref(div)))
        return p.value, n.value, div.value

    def rollout_sample(self, temperature, top_k, logits_device=None):
        rows = self._ro[0]
        column = np.zeros(rows, np.int32); mask = np.zeros(rows, np.int32); done = C.c_int()
        check(self.lib.gn_rollout_sample(self.h, C.c_void_p(logits_device) if logits_device else None, temperature, top_k, ptr(column), ptr(mask),
                                         C.byref(done)))
        return column, mask, bool(done.value)

    def rollout_force(self, row, tokens):
        tokens = _i32(tokens)
        check(self.lib.gn_rollout_force(self.h, int(row), ptr(tokens), tokens.size))

    def rollout_forward(self, column=None):
        check(self.lib.gn_rollout_forward(self.h, ptr(_i32(column)) if column is not None else None))

    def rollout_end(self):
        rows, max_tokens = self._ro
        tokens = np.zeros((rows, max_tokens), np.int32); lengths = np.zeros(rows, np.int32); masks = np.zeros((rows, max_tokens), np.int32)
        check(self.lib.gn_rollout_end(self.h, ptr(tokens), ptr(lengths), ptr(masks)))
        return tokens, lengths, masks

    # ---- trainer.PolicyGradientStep (trainer/rl.go:14-60)
    def optimizer_init(self, unembedding_lr=0.004, embedding_lr=0.2, matrix_lr=0.02, weight_decay=0.0, scalar_lr=0.5, lr_mult=0.05):
        """chat_rl's MuonAdamW (model.SetupOptimizer(0.004, 0.2, 0.02, 0.0, 0.5, true), every LR x 0.05; cmd/chat_rl/main.go:68-72)."""
        cfg = GnOptimizerConfig(unembedding_lr, embedding_lr, matrix_lr, weight_decay, scalar_lr, lr_mult)
        check(self.lib.gn_model_optimizer_init(self.h, C.byref(cfg)))

    def optimizer_step(self):
        """optimizer.Step() then ZeroGrad() (trainer/rl.go:65-66)."""
        check(self.lib.gn_model_optimizer_step(self.h))

    def optimizer_step_shard(self, shard, shard_count):
        """Data parallel: update only this shard's tensors and stage them in the gradient buffer for one more SUM all-reduce."""
        check(self.lib.gn_model_optimizer_step_shard(self.h, shard, shard_count))

    def optimizer_finish(self):
        check(self.lib.gn_model_optimizer_finish(self.h))

    def grad_allreduce(self):
        """SUM of the flat gradient buffer over the ranks of the context's communicator."""
        check(self.lib.gn_model_grad_allreduce(self.h))

    def optimizer_exchange(self):
        """After optimizer_step_shard on every rank: broadcast each tensor from its owner, then ZeroGrad."""
        check(self.lib.gn_model_optimizer_exchange(self.h))

    def policy_gradient_step(self, inputs, targets, advantages, norm, rows_per_pass=0, taps=False):
        inputs, targets, advantages = _i32(inputs), _i32(targets), _f32(advantages)
        B, T = inputs.shape
        loss = C.c_float()
        nll = np.empty(B * T, np.float32) if taps else None
        dl = np.empty((B * T, self.vocab), np.float32) if taps else None
        lg = np.empty((B * T, self.vocab), np.float32) if taps else None
        check(self.lib.gn_policy_gradient_step(self.h, ptr(inputs), ptr(targets), ptr(advantages), B, T, norm, rows_per_pass, C.byref(loss),
                                               ptr(nll), ptr(dl), ptr(lg)))
        return loss.value, nll, dl, lg


# -------------------------------------------------------------------------
# Batch assembly of cmd/chat_rl (host side, integer work)
# -------------------------------------------------------------------------
def build_batch(prompts, group, tokens, lengths, pad_token, max_len=None):
    """Pads every rollout (prompt + kept tokens) to the longest one with ``pad_token``
    (= <|assistant_end|>), shifts inputs/targets by one and masks targets whose index is
    below the prompt length (cmd/chat_rl/main.go:156-182).  Returns inputs, targets
    ([rows, max_len-1] int32) and max_len.  Pad positions are NOT masked, as in the reference.
    """
    prompts = _i32(prompts); tokens = _i32(tokens); lengths = _i32(lengths)
    P, plen = prompts.shape
    rows = P * group
    local = plen + int(lengths.max())
    max_len = local if max_len is None else max(int(max_len), local)   # data parallel: every rank pads to the global length
    padded = np.full((rows, max_len), pad_token, np.int32)
    padded[:, :plen] = np.repeat(prompts, group, axis=0)
    for r in range(rows):
        padded[r, plen:plen + lengths[r]] = tokens[r, :lengths[r]]
    inputs = np.ascontiguousarray(padded[:, :-1])
    targets = np.ascontiguousarray(padded[:, 1:]).copy()
    targets[:, :plen] = -1          # target index < prompt length (also hides the first sampled token)
    return inputs, targets, max_len


@dataclass
class RLStepResult:
    loss: float
    rollout_tokens: int
    rows: int
    max_len: int
    steps: int
    tokens: np.ndarray
    lengths: np.ndarray
    advantages: np.ndarray


def rl_step(model: Model, prompts, group, max_tokens, temperature, top_k, seeds, reward_fn, advantage_mode=0, rows_per_pass=0,
            norm=None, all_reduce=None, max_len_fn=None, optimizer=False, shard=None, data_parallel=False) -> RLStepResult:
    """One RL step the way cmd/chat_rl runs it (main.go:87-184):
    rollout -> rewards -> group-relative advantages -> padded batch -> PolicyGradientStep
    -> gradient all-reduce (``all_reduce(model)``, when data parallel) -> optimizer step and
    ZeroGrad when ``optimizer`` (trainer/rl.go:62-67; needs ``model.optimizer_init()``; ``shard=(rank, world)``
    splits the optimizer's tensors over the ranks).  ``reward_fn(tokens,
    lengths)`` returns one reward per rollout.  ``norm`` defaults to the padded length
    (main.go:183).  ``max_len_fn(local_max_len)`` returns the length every rank pads to.
    ``data_parallel=True`` uses the communicator of the model's context (``Context.comm_init``) for all three
    exchanges: the padded length, the gradient all-reduce and the sharded optimizer's broadcasts."""
    from .backend import group_advantage
    if data_parallel:
        ctx = model.ctx
        max_len_fn = ctx.allreduce_max
        all_reduce = lambda m: m.grad_allreduce()
        shard = (getattr(ctx, "rank", 0), getattr(ctx, "world", 1))
    prompts = _i32(prompts)
    tokens, lengths, steps, _ = model.generate_batch(prompts, group, max_tokens, temperature, top_k, seeds)
    rewards = _f32(reward_fn(tokens, lengths))
    adv = group_advantage(rewards, group, advantage_mode)
    pad = model.vocab - 7  # <|assistant_end|>
    local_max = prompts.shape[1] + int(lengths.max())
    inputs, targets, max_len = build_batch(prompts, group, tokens, lengths, pad, max_len_fn(local_max) if max_len_fn else None)
    model.zero_grad()
    loss, _, _, _ = model.policy_gradient_step(inputs, targets, adv, float(max_len) if norm is None else norm, rows_per_pass)
    if all_reduce is not None:
        all_reduce(model)
    if optimizer:
        if data_parallel and shard[1] > 1:
            # each rank updates the tensors it owns; every tensor is then broadcast from its owner
            model.optimizer_step_shard(shard[0], shard[1])
            model.optimizer_exchange()
        elif shard is not None and all_reduce is not None and shard[1] > 1:
            # each rank updates the tensors it owns; a second all-reduce of the same buffer distributes them (exactly)
            model.optimizer_step_shard(shard[0], shard[1])
            all_reduce(model)
            model.optimizer_finish()
        else:
            model.optimizer_step()
    return RLStepResult(loss, int(lengths.sum()), len(lengths), max_len, steps, tokens, lengths, adv)
