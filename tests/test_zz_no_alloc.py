"""The allocation-free loss entry point against the ordinary one.

gn_pg_loss_backward_static is for embedders that may not allocate device memory (they own the
whole GPU through their own arena, or cannot accept cudaMalloc's device-wide synchronisation in
their loop).  It must give what gn_pg_loss_backward gives - same kernel, scratch in a fixed
array - on consecutive calls that share that array, and refuse batches beyond its fixed limit.
This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _case(rng, rows, vocab, seq):
    z = rng.standard_normal((rows, vocab)).astype(np.float32) * np.float32(3)
    logits = (np.float32(15) * np.tanh(z / np.float32(15))).astype(np.float32)
    targets = rng.integers(0, vocab, rows).astype(np.int32)
    targets[rng.random(rows) < 0.4] = -1
    adv = rng.standard_normal((rows + seq - 1) // seq).astype(np.float32)
    return logits, targets, adv


def test_static_loss_matches_allocating_entry_point_twice():
    import torch
    from gonano_b200 import _lib
    from gonano_b200.backend import pg_loss_backward
    lib = _lib.load()
    rng = np.random.default_rng(11)
    dev = torch.device("cuda:0")
    # two calls in a row: the second is smaller and different, so anything left in the shared
    # array by the first one would show
    for rows, vocab, seq, softcap in [(96, 32768, 8, 15.0), (40, 8192, 5, 0.0)]:
        logits, targets, adv = _case(rng, rows, vocab, seq)
        norm = float(max(1, int((targets != -1).sum())))
        want_loss, want_nll, want_grad = pg_loss_backward(logits, targets, adv, seq, norm, softcap=softcap)
        d_logits = torch.from_numpy(logits).to(dev); d_targets = torch.from_numpy(targets).to(dev); d_adv = torch.from_numpy(adv).to(dev)
        d_nll = torch.full((rows,), 7.0, device=dev); d_grad = torch.full((rows, vocab), 7.0, device=dev)
        torch.cuda.synchronize()
        loss = C.c_double(-1.0)
        status = lib.gn_pg_loss_backward_static(d_logits.data_ptr(), d_targets.data_ptr(), d_adv.data_ptr(), rows, vocab, seq, norm, softcap,
                                                d_nll.data_ptr(), d_grad.data_ptr(), C.cast(C.byref(loss), C.c_void_p), None)
        assert status == 0, lib.gn_last_error()
        # same kernel, same order of operations: the tolerance is the loss tests' 1e-4 bar, the expectation is equality
        assert abs(loss.value - want_loss) <= 1e-4 * max(abs(want_loss), 1e-3)
        assert loss.value == want_loss
        assert np.array_equal(d_nll.cpu().numpy(), want_nll)
        assert np.array_equal(d_grad.cpu().numpy(), want_grad)


def test_static_loss_limits_are_enforced():
    import torch
    from gonano_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda:0")
    t = torch.zeros(16, device=dev)
    ti = torch.zeros(16, dtype=torch.int32, device=dev)
    loss = C.c_double()
    max_rows = lib.gn_static_loss_max_rows()      # the limit of the library that is loaded, not a copy of it
    assert max_rows >= 1024
    status = lib.gn_pg_loss_backward_static(t.data_ptr(), ti.data_ptr(), t.data_ptr(), max_rows + 1, 4, 1, 1.0, 0.0, None, None,
                                            C.cast(C.byref(loss), C.c_void_p), None)
    assert status != 0 and b"exceed" in lib.gn_last_error()
    host = np.zeros(16, np.float32)
    status = lib.gn_pg_loss_backward_static(host.ctypes.data, ti.data_ptr(), t.data_ptr(), 4, 4, 1, 1.0, 0.0, None, None,
                                            C.cast(C.byref(loss), C.c_void_p), None)
    assert status != 0 and b"device memory" in lib.gn_last_error()
    # a target beyond the vocabulary is never dereferenced: the call reports it instead
    logits = torch.zeros(4, 8, device=dev)
    bad = torch.tensor([1, 8, -1, 2], dtype=torch.int32, device=dev)
    adv = torch.ones(4, device=dev)
    status = lib.gn_pg_loss_backward_static(logits.data_ptr(), bad.data_ptr(), adv.data_ptr(), 4, 8, 1, 1.0, 0.0, None, None,
                                            C.cast(C.byref(loss), C.c_void_p), None)
    assert status == 1 and b"targets outside" in lib.gn_last_error()
