"""The C-ABI library loads and exports every symbol the header declares (no GPU needed),
fails loudly without a device, and the host-side batch assembly matches the oracle."""
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from gonano_b200 import build, _lib
    build.build()
    return _lib.load()


def declared_symbols():
    text = (ROOT / "include" / "gonano_cuda.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gn_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(lib):
    from gonano_b200 import _lib
    names = declared_symbols()
    assert len(names) > 50
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/gonano_cuda.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), set(names) ^ set(_lib.SIGNATURES)


def test_version_and_device_count(lib):
    assert b"sm_100a" in lib.gn_version()
    assert lib.gn_device_count() >= 0


def test_no_device_fails_loudly(lib):
    """Without a CUDA device a compute call returns an error status, never a CPU result."""
    if lib.gn_device_count() > 0:
        pytest.skip("a CUDA device is present")
    from gonano_b200 import backend, session
    from gonano_b200._lib import GonanoError
    with pytest.raises(GonanoError):
        backend.CudaBackend().add([1, 2], [3, 4])
    with pytest.raises(GonanoError):
        session.Context(0)


def test_invalid_arguments_are_rejected(lib):
    import ctypes as C
    out = C.c_float()
    assert lib.gn_sum(None, 0, C.byref(out)) == 0 and out.value == 0.0   # empty slice sums to 0
    assert lib.gn_max(None, 0, C.byref(out)) == 0 and out.value == 0.0   # kernels/scalar/reduce.go:13-15
    assert lib.gn_group_advantage(None, 1, 4, 0, None) != 0
    assert b"advantage" in lib.gn_last_error()


def test_compressed_attention_entry_points_check_their_arguments(lib):
    """The entry points of the compressed attention layers refuse missing arrays before they touch a device, name themselves
    in the error text, and treat empty inputs as nothing to do."""
    import ctypes as C
    buf = (C.c_float * 64)()
    ibuf = (C.c_int32 * 16)()
    p = C.cast(buf, C.c_void_p); ip = C.cast(ibuf, C.c_void_p)
    assert lib.gn_compressed_attention_forward(None, p, p, 1, 1, 1, 4, 8, 2, 2, p, None) != 0 and b"compressed_attention_forward" in lib.gn_last_error()
    assert lib.gn_compressed_attention_backward(p, p, p, None, p, None, 1, 1, 1, 4, 8, 2, 2, p, p, p) != 0 and b"compressed_attention_backward" in lib.gn_last_error()
    assert lib.gn_compressed_attention_sparse_forward(p, p, p, None, ip, 1, 1, 1, 4, 8, 2, 2, p, None) != 0
    assert lib.gn_compressed_attention_sparse_backward(p, p, p, p, p, None, ip, ip, 1, 1, 1, 4, 8, 2, 0, p, p, p) != 0     # topk 0
    assert lib.gn_attention_merge(p, p, p, None, 4, 8, p, None) != 0 and b"attention_merge" in lib.gn_last_error()
    assert lib.gn_select_blocks_hierarchical(p, 4, 4, 0, 0, 2, 2, 4, ip, ip, None, None) != 0                             # ratio 0
    assert lib.gn_select_blocks_within_pool(p, 4, 4, 0, 2, 2, None, ip, 4, ip, ip) != 0
    assert lib.gn_indexer_distillation_grad(p, None, None, None, 0, 4, 4, 2, 2, 1.0, p) != 0
    assert lib.gn_attention_windowed_forward(p, p, p, 1, 3, 2, 4, 8, 0, 2, p, None) != 0                                   # 3 query heads on 2 kv heads
    assert lib.gn_compress_forward(p, p, p, p, None, 1, 1, 4, 4, 8, 2, p, p, None) != 0 and b"compress_forward" in lib.gn_last_error()
    # nothing to do: no device is needed
    assert lib.gn_compressed_attention_forward(None, None, None, 0, 1, 1, 4, 8, 2, 2, None, None) == 0
    assert lib.gn_attention_merge(None, None, None, None, 0, 8, None, None) == 0
    assert lib.gn_select_blocks_hierarchical(None, 0, 4, 0, 2, 2, 2, 4, None, None, None, None) == 0
    assert lib.gn_hierarchical_cap(8, 512) == 512 and lib.gn_hierarchical_cap(8, 0) == 8 and lib.gn_hierarchical_cap(0, 3) == 3


def test_build_batch_matches_oracle(oracle):
    from gonano_b200 import session
    rng = np.random.default_rng(0)
    P, G, plen, maxtok, V = 3, 4, 5, 7, 100
    prompts = rng.integers(0, V - 11, (P, plen), dtype=np.int32)
    lengths = rng.integers(0, maxtok + 1, P * G).astype(np.int32)
    lengths[0] = maxtok
    tokens = rng.integers(0, V - 11, (P * G, maxtok), dtype=np.int32)
    inputs, targets, max_len = session.build_batch(prompts, G, tokens, lengths, V - 7)
    full = np.zeros((P * G, plen + maxtok), np.int32)
    full[:, :plen] = np.repeat(prompts, G, axis=0)
    for r in range(P * G):
        full[r, plen:plen + lengths[r]] = tokens[r, :lengths[r]]
    want_in, want_tg, want_len = oracle.build_batch(full, lengths + plen, np.full(P * G, plen), V - 7)
    assert max_len == want_len
    assert np.array_equal(inputs, want_in) and np.array_equal(targets, want_tg)
