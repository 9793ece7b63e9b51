"""Data-parallel plumbing for the RL step: rollout prompts are sharded across ranks (one
process per GPU, a full policy replica each) and the flat gradient buffer is summed with one
all-reduce.  The reference is a single-process program (optimizer/optimizer.go:5-7); the
nearest thing it has is gradient accumulation into ``Tensor.Grad`` (tensors/tensor.go:189-194),
which is why the exchange is a plain SUM: the 1/norm factor is already inside dlogits
(trainer/rl.go:41) and ``norm`` is a global constant every rank agrees on.

``torch.distributed`` (NCCL over NVLink on GPUs, gloo on CPU in tests) is the transport.
"""
from __future__ import annotations

import os

import numpy as np


def shard_range(n_items: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous block of items for ``rank``; blocks differ by at most one item."""
    base, extra = divmod(n_items, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def env_rank_world() -> tuple[int, int, int]:
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


class _DeviceArray:
    """Exposes a raw device address to torch through the CUDA array interface."""

    def __init__(self, address: int, count: int):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (address, False), "version": 2}


def device_tensor(address: int, count: int, device: int):
    import torch
    return torch.as_tensor(_DeviceArray(address, count), device=f"cuda:{device}")


def all_reduce_sum(tensor):
    """SUM all-reduce of a torch tensor over the default process group (no-op when not initialised)."""
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(tensor, op=dist.ReduceOp.SUM)
    return tensor


class GradAllReduce:
    """Callable handed to ``session.rl_step``: sums the model's flat gradient buffer over ranks.

    The buffer is wrapped once as a torch tensor that aliases the library's device memory; the
    collective is issued on ``stream`` (the stream the model's context runs on), so it is
    ordered after the backward kernels without a host synchronisation."""

    def __init__(self, model, device: int, stream):
        import torch
        self.torch = torch
        address, count = model.grad_buffer()
        self.tensor = device_tensor(address, count, device)
        self.stream = stream
        self.bytes = count * 4
        self._pending = []   # (start, end) events of the calls since the last last_ms()

    def __call__(self, model=None):
        start, end = self.torch.cuda.Event(enable_timing=True), self.torch.cuda.Event(enable_timing=True)
        with self.torch.cuda.stream(self.stream):
            start.record(self.stream)
            all_reduce_sum(self.tensor)
            end.record(self.stream)
        self._pending.append((start, end))

    def last_ms(self) -> float:
        """Device time of the all-reduces issued since the previous call of this method (each includes waiting
        for the slowest rank); a step with a sharded optimizer issues two."""
        total = 0.0
        for start, end in self._pending:
            end.synchronize()
            total += float(start.elapsed_time(end))
        self._pending = []
        return total


def global_max_len(local_max_len: int) -> int:
    """Every rank must pad to, and normalise by, the same length (cmd/chat_rl/main.go:156-183)."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return local_max_len
    device = "cuda" if dist.get_backend() == "nccl" else "cpu"
    t = torch.tensor([local_max_len], dtype=torch.int64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return int(t.item())
