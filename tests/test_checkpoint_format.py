"""The `.gn` checkpoint container (model/checkpoint/checkpoint.go:20-123): byte layout, round trip, config mapping."""
import json
import struct

import numpy as np
import pytest

from gonano_b200 import checkpoint, synthetic


def test_byte_layout(tmp_path):
    p = tmp_path / "m.gn"
    params = {"b.weight": np.arange(6, dtype=np.float32).reshape(2, 3), "a": np.array([1.5], np.float32)}
    checkpoint.write_gn(p, {"step": 7, "model_config": {"n_layer": 1}}, params)
    data = p.read_bytes()
    assert data[:8] == b"GONANO\x00\x01"                              # checkpoint.go:20
    (n,) = struct.unpack_from("<I", data, 8)                           # checkpoint.go:64-66
    meta = json.loads(data[12:12 + n])
    assert meta["step"] == 7 and meta["params"] == [{"name": "a", "shape": [1]}, {"name": "b.weight", "shape": [2, 3]}]   # sorted, checkpoint.go:41-48
    body = data[12 + n:]
    assert body == np.array([1.5, 0, 1, 2, 3, 4, 5], "<f4").tobytes()  # little-endian float32, in that order
    meta2, back = checkpoint.read_gn(p)
    assert meta2 == meta and set(back) == {"a", "b.weight"}
    assert np.array_equal(back["b.weight"], params["b.weight"]) and back["b.weight"].shape == (2, 3)


def test_rejects_bad_files(tmp_path):
    p = tmp_path / "bad.gn"
    p.write_bytes(b"NOTGONANO")
    with pytest.raises(ValueError, match="invalid magic"):
        checkpoint.read_gn(p)
    p.write_bytes(b"GONANO\x00\x01" + struct.pack("<I", 1000) + b"{}")
    with pytest.raises(ValueError, match="truncated metadata"):
        checkpoint.read_gn(p)
    blob = json.dumps({"params": [{"name": "w", "shape": [4]}]}).encode()
    p.write_bytes(b"GONANO\x00\x01" + struct.pack("<I", len(blob)) + blob + b"\x00" * 8)
    with pytest.raises(ValueError, match="truncated params"):
        checkpoint.read_gn(p)


def test_config_mapping_round_trip():
    for cfg in (synthetic.dense_config("d12"), synthetic.latent_config("c3")):
        meta = checkpoint.meta_from_config(cfg, step=3)
        assert meta["model_config"]["n_embd"] == cfg["embed_dim"] and "embed_dim" not in meta["model_config"]
        back = checkpoint.config_from_meta(meta)
        for key, value in cfg.items():
            assert back.get(key, 0) == value or (value in (0, 0.0) and key not in back), key


def test_unsupported_architecture_is_refused():
    meta = checkpoint.meta_from_config(synthetic.dense_config("c1"))
    meta["model_config"]["compression_ratio"] = 4
    with pytest.raises(ValueError, match="compression_ratio"):
        checkpoint.config_from_meta(meta)
    meta = checkpoint.meta_from_config(synthetic.dense_config("c1"))
    meta["model_config"]["head_wise_muon"] = True       # optimizer-only: the forward pass does not depend on it
    checkpoint.config_from_meta(meta)


def test_reference_shapes():
    cfg = synthetic.latent_config("latent-tiny")
    assert checkpoint.reference_shape("resid_lambdas", 1, 2, cfg) == (2,)
    assert checkpoint.reference_shape("transformer.h.0.moe.router_bias", 1, 4, cfg) == (4,)
    assert checkpoint.reference_shape("transformer.h.0.moe.experts.gate.weight", 4 * 32, 64, cfg) == (4, 32, 64)   # [E, Hidden, Dim]
    assert checkpoint.reference_shape("transformer.h.0.moe.experts.down.weight", 4 * 64, 32, cfg) == (4, 64, 32)   # [E, Dim, Hidden]
    assert checkpoint.reference_shape("lm_head.weight", 128, 64, cfg) == (128, 64)


def test_oracle_model_through_a_file(oracle, tmp_path):
    """Parameters written from one model and read into another give the same logits."""
    cfg = synthetic.dense_config("tiny")
    a = oracle.Model(**cfg)
    for name, value in synthetic.fill_weights(a.names, a.shape, 9, std=0.1):
        a.param(name)[:] = value
    params = {n: a.param(n).reshape(checkpoint.reference_shape(n, *a.shape(n), cfg)) for n in a.names}
    checkpoint.write_gn(tmp_path / "t.gn", checkpoint.meta_from_config(cfg, 1), params)
    meta, back = checkpoint.read_gn(tmp_path / "t.gn")
    b = oracle.Model(**checkpoint.config_from_meta(meta))
    for n in b.names:
        b.param(n)[:] = back[n].ravel()
    ids = np.array([[1, 2, 3, 4, 5]], np.int32)
    assert np.array_equal(a.forward(ids), b.forward(ids))


@pytest.mark.gpu
def test_device_model_save_and_load(tmp_path):
    from gonano_b200.session import Context, Model
    cfg = synthetic.latent_config("latent-tiny")
    ctx = Context(0)
    m = Model(ctx, **cfg)
    for name, value in synthetic.fill_weights(m.names, m.shape, 6, std=0.1):
        m.upload(name, value)
    checkpoint.save_model(m, cfg, tmp_path / "dev.gn", step=12)
    m2, meta = checkpoint.load_model(ctx, tmp_path / "dev.gn")
    assert meta["step"] == 12 and sorted(m2.names) == sorted(m.names)
    ids = np.array([[3, 1, 4, 1, 5, 9, 2, 6]], np.int32)
    assert np.array_equal(m.forward(ids), m2.forward(ids))
    m.close(); m2.close(); ctx.close()
