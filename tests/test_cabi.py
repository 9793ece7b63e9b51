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
