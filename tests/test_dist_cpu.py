"""The data-parallel path on CPU: two gloo ranks shard the prompts, run the policy-gradient step on
their shard (the oracle stands in for the device here) and all-reduce the flat gradient; the sum
must equal the single-process gradient over the whole batch, with the global padded length and norm."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_shard_range_covers_everything():
    from gonano_b200.dist import shard_range
    for n in [1, 7, 64, 65]:
        for world in [1, 2, 3, 8]:
            spans = [shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close(); return port


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), OMP_NUM_THREADS="2")
    import torch
    import torch.distributed as dist
    from gonano_b200 import dist as gdist, synthetic
    from gonano_b200.session import build_batch
    from oracle import oracle
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = synthetic.dense_config("tiny")
    V, G, P, plen, maxtok = cfg["vocab_size"], 2, 4, 3, 5
    model = oracle.Model(**cfg)
    for name, value in synthetic.fill_weights(model.names, model.shape, 1, std=0.1):
        model.param(name)[:] = value
    rng = np.random.default_rng(0)                       # every rank builds the same global problem
    prompts = rng.integers(0, V - 11, (P, plen), dtype=np.int32)
    tokens = rng.integers(0, V - 11, (P * G, maxtok), dtype=np.int32)
    lengths = np.array([5, 2, 3, 3, 1, 4, 2, 2], np.int32)      # the longest rollout lives on rank 0 only
    adv = rng.standard_normal(P * G).astype(np.float32)
    lo, hi = gdist.shard_range(P, rank, world)
    local_max = plen + int(lengths[lo * G:hi * G].max())
    max_len = gdist.global_max_len(local_max)
    inputs, targets, got_len = build_batch(prompts[lo:hi], G, tokens[lo * G:hi * G], lengths[lo * G:hi * G], V - 7, max_len)
    assert got_len == max_len == plen + 5
    model.zero_grad()
    loss, _, _, _ = model.policy_gradient_step(inputs, targets, adv[lo * G:hi * G], float(max_len))
    flat = torch.from_numpy(np.concatenate([model.grad(n) for n in model.names]).copy())
    gdist.all_reduce_sum(flat)
    lt = torch.tensor([loss], dtype=torch.float64)
    gdist.all_reduce_sum(lt)
    if rank == 0:
        np.save(os.path.join(out_dir, "grad.npy"), flat.numpy())
        np.save(os.path.join(out_dir, "loss.npy"), lt.numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_rank_gradient_equals_single_process(tmp_path, oracle):
    import torch.multiprocessing as mp
    from gonano_b200 import synthetic
    from gonano_b200.session import build_batch
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    got = np.load(tmp_path / "grad.npy"); got_loss = float(np.load(tmp_path / "loss.npy")[0])
    cfg = synthetic.dense_config("tiny")
    V, G, P, plen, maxtok = cfg["vocab_size"], 2, 4, 3, 5
    model = oracle.Model(**cfg)
    for name, value in synthetic.fill_weights(model.names, model.shape, 1, std=0.1):
        model.param(name)[:] = value
    rng = np.random.default_rng(0)
    prompts = rng.integers(0, V - 11, (P, plen), dtype=np.int32)
    tokens = rng.integers(0, V - 11, (P * G, maxtok), dtype=np.int32)
    lengths = np.array([5, 2, 3, 3, 1, 4, 2, 2], np.int32)
    adv = rng.standard_normal(P * G).astype(np.float32)
    inputs, targets, max_len = build_batch(prompts, G, tokens, lengths, V - 7)
    model.zero_grad()
    want_loss, _, _, _ = model.policy_gradient_step(inputs, targets, adv, float(max_len))
    want = np.concatenate([model.grad(n) for n in model.names])
    assert abs(got_loss - want_loss) <= 1e-6 * max(abs(want_loss), 1e-3)
    assert np.max(np.abs(got - want)) <= 1e-6 * np.max(np.abs(want))
