"""The KV-cache wire format (model/kvcache_codec.go): byte layout by hand, round trips, refusals."""
import struct

import numpy as np
import pytest

from gonano_b200 import kvcodec


def small_cache(latent=False):
    rng = np.random.default_rng(0)
    c = kvcodec.KVCache(batch=2, max_seq=5, layers=2, kv_heads=2, head_dim=3, position=3)
    c.keys[:] = rng.standard_normal(c.keys.shape).astype(np.float32)
    c.values[:] = rng.standard_normal(c.values.shape).astype(np.float32)
    c.previous_embedding = rng.standard_normal((2, 4)).astype(np.float32)
    if latent:
        c.latent = rng.standard_normal((2, 2, 5, 6)).astype(np.float32)
        c.rope_key = rng.standard_normal((2, 2, 5, 4)).astype(np.float32)
    return c


def test_byte_layout_follows_the_go_writer():
    c = small_cache()
    data = kvcodec.marshal(c)
    assert data[:8] == b"GONAKV\x00\x01"                                   # kvcache_codec.go:12-13
    header = struct.unpack_from("<IIIIIiIIIIIII", data, 8)                 # :42-54, little-endian (:303-316)
    assert header == (2, 5, 2, 2, 3, 3, 0, 0, 0, 0, 0, 0, 0)
    (flags,) = struct.unpack_from("<I", data, 8 + 13 * 4)
    assert flags == kvcodec.FLAG_PREVIOUS_EMBEDDING                         # :56-73
    off = 8 + 14 * 4
    # only the used prefix, key rows then value rows per (layer, row * heads + head)  (:76-86)
    first_keys = np.frombuffer(data, "<f4", 9, off)
    assert np.array_equal(first_keys, c.keys[0, 0, :3].reshape(-1))
    first_values = np.frombuffer(data, "<f4", 9, off + 36)
    assert np.array_equal(first_values, c.values[0, 0, :3].reshape(-1))
    raw = 2 * 4 * 2 * 9 * 4
    (channels,) = struct.unpack_from("<I", data, off + raw)                # :150-154
    assert channels == 4
    assert len(data) == off + raw + 4 + 2 * 4 * 4


@pytest.mark.parametrize("latent", [False, True])
def test_round_trip(latent):
    c = small_cache(latent)
    back = kvcodec.unmarshal(kvcodec.marshal(c))
    assert (back.batch, back.max_seq, back.layers, back.kv_heads, back.head_dim, back.position) == (2, 5, 2, 2, 3, 3)
    assert np.array_equal(back.keys[:, :, :3], c.keys[:, :, :3]) and not np.any(back.keys[:, :, 3:])      # unused tail is not stored
    assert np.array_equal(back.values[:, :, :3], c.values[:, :, :3])
    assert np.array_equal(back.previous_embedding, c.previous_embedding)
    if latent:
        assert np.array_equal(back.latent[:, :, :3], c.latent[:, :, :3]) and np.array_equal(back.rope_key[:, :, :3], c.rope_key[:, :, :3])
    else:
        assert back.latent is None


def test_stripped_snapshot_omits_the_raw_rows():
    c = small_cache()
    c.raw_stripped = True
    data = kvcodec.marshal(c)
    assert len(data) == 8 + 14 * 4 + 4 + 2 * 4 * 4
    back = kvcodec.unmarshal(data)
    assert back.raw_stripped and not np.any(back.keys)


def test_invalid_inputs_are_refused():
    good = kvcodec.marshal(small_cache())
    with pytest.raises(kvcodec.InvalidKVCache):
        kvcodec.unmarshal(b"NOTAKV\x00\x01" + good[8:])
    with pytest.raises(kvcodec.InvalidKVCache):
        kvcodec.unmarshal(good[:-3])
    bad = bytearray(good); struct.pack_into("<i", bad, 8 + 5 * 4, 9)          # sequence length beyond the cache
    with pytest.raises(kvcodec.InvalidKVCache):
        kvcodec.unmarshal(bytes(bad))
    bad = bytearray(good); struct.pack_into("<I", bad, 8 + 13 * 4, kvcodec.FLAG_COMPRESSION)
    with pytest.raises(kvcodec.InvalidKVCache):
        kvcodec.unmarshal(bytes(bad))


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["dense", "latent"])
def test_device_cache_round_trip(kind):
    """A rollout's cache leaves the device, goes through the wire format and comes back into a second model's cache
    unchanged; its keys are the ones a fresh forward of the same tokens produces."""
    from gonano_b200 import synthetic
    from gonano_b200.session import Context, Model
    cfg = synthetic.dense_config("h128") if kind == "dense" else synthetic.latent_config("latent-small")
    ctx = Context(0)
    a, b = Model(ctx, **cfg), Model(ctx, **cfg)
    for n, v in synthetic.fill_weights(a.names, a.shape, 1, std=0.05):
        a.upload(n, v); b.upload(n, v)
    prompts = synthetic.prompts(2, 20, cfg["vocab_size"], seed=2)
    a.generate_batch(prompts, 2, 6, 0.0, 0, np.array([1, 2], np.uint64))
    image = kvcodec.export_cache(a)
    assert image.batch == 4 and image.position >= 20 and image.max_seq == 26
    data = kvcodec.marshal(image)
    back = kvcodec.unmarshal(data)
    kvcodec.import_cache(b, back)
    again = kvcodec.export_cache(b)
    assert kvcodec.marshal(again) == data
    if kind == "dense":   # rows of one group share their prompt's keys (model/kvcache.go:383-448)
        assert np.array_equal(image.keys[:, 0, :20], image.keys[:, 1, :20]) and np.any(image.keys[:, 0, :20])
    else:
        assert np.array_equal(image.latent[:, 0, :20], image.latent[:, 1, :20]) and np.any(image.latent[:, 0, :20])
    a.close(); b.close(); ctx.close()
