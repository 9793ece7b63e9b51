"""The KV-cache wire format of the reference (model/kvcache_codec.go:12-330), for the cache forms the RL step uses:
the plain per-head key/value cache and the latent-attention cache, each with the previous-embedding row of the smear.

Layout (all little-endian): the 8-byte magic ``GONAKV\\0\\1``; thirteen 32-bit fields (batch, maximum sequence
length, layers, kv heads, head_dim, sequence length (signed), compression ratio, compressed max blocks, compressed
embedding dim, compressed kv width, indexer key width, latent width, rotary key width); a 32-bit flag word; then,
unless the snapshot is stripped, for every layer and every (row, kv head) the used prefix of the key rows followed
by the value rows; for a latent cache, for every layer and row the latent rows then the rotary key rows; finally
the channel count and the rows of the previous embedding.  Compressed / indexer sections (the flash preset) are not
produced and are refused on input.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field

import numpy as np

MAGIC = b"GONAKV\x00\x01"
FLAG_COMPRESSION, FLAG_INDEXER, FLAG_PREVIOUS_EMBEDDING, FLAG_RAW_STRIPPED, FLAG_MLA = 1, 2, 4, 8, 16


class InvalidKVCache(ValueError):
    """model.ErrInvalidKVCache."""


@dataclass
class KVCache:
    """Host image of a ``model.KVBuffer`` (model/kvcache.go:10-51) without compression state.

    ``keys`` / ``values``: [layers, batch * kv_heads, max_seq, head_dim] (index = row * kv_heads + head);
    ``latent``: [layers, batch, max_seq, latent_width] and ``rope_key``: [layers, batch, max_seq, rope_width] or None;
    ``previous_embedding``: [batch, channels] or None."""
    batch: int
    max_seq: int
    layers: int
    kv_heads: int
    head_dim: int
    position: int = 0
    keys: np.ndarray = None
    values: np.ndarray = None
    latent: np.ndarray | None = None
    rope_key: np.ndarray | None = None
    previous_embedding: np.ndarray | None = None
    raw_stripped: bool = False

    def __post_init__(self):
        shape = (self.layers, self.batch * self.kv_heads, self.max_seq, self.head_dim)
        if self.keys is None:
            self.keys = np.zeros(shape, np.float32)
        if self.values is None:
            self.values = np.zeros(shape, np.float32)


def marshal(cache: KVCache) -> bytes:
    """KVBuffer.MarshalBinary (model/kvcache_codec.go:40-158)."""
    out = bytearray(MAGIC)
    lat_w = 0 if cache.latent is None else cache.latent.shape[-1]
    rope_w = 0 if cache.rope_key is None else cache.rope_key.shape[-1]
    out += struct.pack("<IIIIIiIIIIIII", cache.batch, cache.max_seq, cache.layers, cache.kv_heads, cache.head_dim, cache.position,
                       0, 0, 0, 0, 0, lat_w, rope_w)
    flags = 0
    if cache.latent is not None:
        flags |= FLAG_MLA
    if cache.previous_embedding is not None:
        flags |= FLAG_PREVIOUS_EMBEDDING
    if cache.raw_stripped:
        flags |= FLAG_RAW_STRIPPED
    out += struct.pack("<I", flags)
    pos = cache.position
    if not cache.raw_stripped:
        for layer in range(cache.layers):
            for index in range(cache.batch * cache.kv_heads):
                out += np.ascontiguousarray(cache.keys[layer, index, :pos], "<f4").tobytes()
                out += np.ascontiguousarray(cache.values[layer, index, :pos], "<f4").tobytes()
    if cache.latent is not None:
        for layer in range(cache.layers):
            for row in range(cache.batch):
                out += np.ascontiguousarray(cache.latent[layer, row, :pos], "<f4").tobytes()
                out += np.ascontiguousarray(cache.rope_key[layer, row, :pos], "<f4").tobytes()
    if cache.previous_embedding is not None:
        prev = np.ascontiguousarray(cache.previous_embedding, "<f4").reshape(cache.batch, -1)
        out += struct.pack("<I", prev.shape[1])
        out += prev.tobytes()
    return bytes(out)


def unmarshal(data: bytes) -> KVCache:
    """UnmarshalKVBuffer (model/kvcache_codec.go:160-300)."""
    if len(data) < len(MAGIC) or data[:len(MAGIC)] != MAGIC:
        raise InvalidKVCache("bad magic")
    off = len(MAGIC)

    def take(fmt):
        nonlocal off
        size = struct.calcsize(fmt)
        if off + size > len(data):
            raise InvalidKVCache("truncated")
        values = struct.unpack_from(fmt, data, off)
        off += size
        return values

    batch, max_seq, layers, kv_heads, head_dim, position, ratio, _blocks, _cdim, _ckv, _idx, lat_w, rope_w = take("<IIIIIiIIIIIII")
    (flags,) = take("<I")
    if batch <= 0 or layers <= 0 or kv_heads <= 0 or head_dim <= 0 or max_seq <= 0:
        raise InvalidKVCache("non-positive geometry")
    if position < 0 or position > max_seq:
        raise InvalidKVCache("sequence length outside the cache")
    if flags & (FLAG_COMPRESSION | FLAG_INDEXER):
        raise InvalidKVCache("compressed / indexer sections are not supported by this reader")
    cache = KVCache(batch, max_seq, layers, kv_heads, head_dim, position, raw_stripped=bool(flags & FLAG_RAW_STRIPPED))

    def floats(count):
        nonlocal off
        if off + 4 * count > len(data):
            raise InvalidKVCache("truncated")
        values = np.frombuffer(data, "<f4", count, off).astype(np.float32)
        off += 4 * count
        return values

    if not cache.raw_stripped:
        for layer in range(layers):
            for index in range(batch * kv_heads):
                cache.keys[layer, index, :position] = floats(position * head_dim).reshape(position, head_dim)
                cache.values[layer, index, :position] = floats(position * head_dim).reshape(position, head_dim)
    if flags & FLAG_MLA:
        cache.latent = np.zeros((layers, batch, max_seq, lat_w), np.float32)
        cache.rope_key = np.zeros((layers, batch, max_seq, rope_w), np.float32)
        for layer in range(layers):
            for row in range(batch):
                cache.latent[layer, row, :position] = floats(position * lat_w).reshape(position, lat_w)
                cache.rope_key[layer, row, :position] = floats(position * rope_w).reshape(position, rope_w)
    if flags & FLAG_PREVIOUS_EMBEDDING:
        (channels,) = take("<I")
        if channels <= 0:
            raise InvalidKVCache("previous embedding without channels")
        cache.previous_embedding = floats(batch * channels).reshape(batch, channels)
    return cache


# ---------------------------------------------------------------------------------------------------------------
# Device <-> host image
# ---------------------------------------------------------------------------------------------------------------
def export_cache(model, rows=None) -> KVCache:
    """The session's KV cache (all rows, or the given ones) as a host image ready for ``marshal``."""
    import ctypes as C
    from ._lib import check, ptr
    lib = model.lib
    nrows, max_seq, position = C.c_int(), C.c_int(), C.c_int()
    check(lib.gn_model_kv_info(model.h, C.byref(nrows), C.byref(max_seq), C.byref(position)))
    rows = list(range(nrows.value)) if rows is None else list(rows)
    cfg = model.cfg
    L, Hkv, D, pos = cfg.n_layer, cfg.n_kv_head, cfg.embed_dim // cfg.n_head, position.value
    cache = KVCache(len(rows), max_seq.value, L, Hkv, D, pos)
    latent = cfg.mla_latent > 0
    if latent:
        lat_w = cfg.mla_latent
        rope = cfg.mla_rotary_dims if cfg.mla_rotary_dims > 0 else min(D // 2, 64) // 2 * 2
        cache.latent = np.zeros((L, len(rows), max_seq.value, lat_w), np.float32)
        cache.rope_key = np.zeros((L, len(rows), max_seq.value, Hkv * rope), np.float32)
    for layer in range(L):
        for i, row in enumerate(rows):
            if latent:
                buf = np.empty(pos * cache.latent.shape[-1], np.float32)
                check(lib.gn_model_kv_read(model.h, layer, 2, row, 0, pos, ptr(buf), buf.size))
                cache.latent[layer, i, :pos] = buf.reshape(pos, -1)
                buf = np.empty(pos * cache.rope_key.shape[-1], np.float32)
                check(lib.gn_model_kv_read(model.h, layer, 3, row, 0, pos, ptr(buf), buf.size))
                cache.rope_key[layer, i, :pos] = buf.reshape(pos, -1)
                continue
            for head in range(Hkv):
                for kind, dst in ((0, cache.keys), (1, cache.values)):
                    buf = np.empty(pos * D, np.float32)
                    check(lib.gn_model_kv_read(model.h, layer, kind, row, head, pos, ptr(buf), buf.size))
                    dst[layer, i * Hkv + head, :pos] = buf.reshape(pos, D)
    prev = np.empty((len(rows), cfg.embed_dim), np.float32)
    for i, row in enumerate(rows):
        buf = np.empty(cfg.embed_dim, np.float32)
        check(lib.gn_model_kv_read(model.h, 0, 4, row, 0, 0, ptr(buf), buf.size))
        prev[i] = buf
    cache.previous_embedding = prev
    return cache


def import_cache(model, cache: KVCache) -> None:
    """Sizes the session's KV cache for ``cache`` and writes it to the device."""
    from ._lib import check, ptr
    lib = model.lib
    check(lib.gn_model_kv_alloc(model.h, cache.batch, cache.max_seq, cache.position))
    pos, Hkv = cache.position, cache.kv_heads
    for layer in range(cache.layers):
        for row in range(cache.batch):
            if cache.latent is not None:
                buf = np.ascontiguousarray(cache.latent[layer, row, :pos], np.float32).reshape(-1)
                check(lib.gn_model_kv_write(model.h, layer, 2, row, 0, pos, ptr(buf), buf.size))
                buf = np.ascontiguousarray(cache.rope_key[layer, row, :pos], np.float32).reshape(-1)
                check(lib.gn_model_kv_write(model.h, layer, 3, row, 0, pos, ptr(buf), buf.size))
                continue
            for head in range(Hkv):
                for kind, src in ((0, cache.keys), (1, cache.values)):
                    buf = np.ascontiguousarray(src[layer, row * Hkv + head, :pos], np.float32).reshape(-1)
                    check(lib.gn_model_kv_write(model.h, layer, kind, row, head, pos, ptr(buf), buf.size))
    if cache.previous_embedding is not None:
        for row in range(cache.batch):
            buf = np.ascontiguousarray(cache.previous_embedding[row], np.float32)
            check(lib.gn_model_kv_write(model.h, 0, 4, row, 0, 0, ptr(buf), buf.size))
