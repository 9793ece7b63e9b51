"""gonano's `.gn` checkpoint format (model/checkpoint/checkpoint.go:20-123), read and written on the host so that a
checkpoint of the Go tools loads into the resident CUDA model and the result of an RL run can be handed back:

    "GONANO\\x00\\x01" | uint32 LE length of the metadata | JSON metadata | float32 LE blobs, one per parameter,
    in the order of metadata["params"] (sorted names when written by checkpoint.Save)

The metadata is the reference's `Meta` (`step`, `model_config`, `params` = [{name, shape}], optional `val_bpb`,
`user_config`, `loop_state`, `dataloader_state`).  `model_config` uses the JSON names of model.Config
(model/config.go:9-124).
"""
from __future__ import annotations

import json
import struct

import numpy as np

MAGIC = b"GONANO\x00\x01"

# model.Config JSON name -> keyword of session.Model / oracle.Model
_CONFIG_KEYS = {
    "sequence_len": "sequence_len", "vocab_size": "vocab_size", "n_layer": "n_layer", "n_head": "n_head", "n_kv_head": "n_kv_head",
    "n_embd": "embed_dim", "window_pattern": "window_pattern", "rotary_dims": "rotary_dims", "mla_latent": "mla_latent",
    "mla_rotary_dims": "mla_rotary_dims", "num_experts": "n_experts", "num_experts_per_token": "experts_per_token",
    "expert_hidden_dim": "expert_hidden", "shared_expert_hidden_dim": "shared_hidden", "moe_clamp": "moe_clamp", "moe_scale": "moe_scale",
}
# features of model.Config this library does not implement: a checkpoint that uses one must not load silently
_UNSUPPORTED = ("compression_ratio", "sparse_top_k", "ced", "query_compression_dim", "kv_latent_dim", "reuse_pattern", "swa_window")
# training-only or optimizer-only fields that do not change the forward pass
_IGNORED = ("indexer_dim", "indexer_heads", "indexer_loss_weight", "indexer_pool", "indexer_candidates", "head_wise_muon", "router_bias_update",
            "moe_balance_weight")


def read_gn(path):
    """checkpoint.Load (checkpoint.go:87-123): returns (metadata dict, {name: float32 array shaped as in the file})."""
    with open(path, "rb") as f:
        data = f.read()
    if len(data) < len(MAGIC) + 4 or data[:len(MAGIC)] != MAGIC:
        raise ValueError(f"checkpoint: invalid magic in {path}")
    pos = len(MAGIC)
    (meta_len,) = struct.unpack_from("<I", data, pos)
    pos += 4
    if pos + meta_len > len(data):
        raise ValueError(f"checkpoint: truncated metadata in {path}")
    meta = json.loads(data[pos:pos + meta_len].decode("utf-8"))
    pos += meta_len
    params = {}
    for pm in meta.get("params", []):
        shape = tuple(int(x) for x in pm["shape"])
        n = int(np.prod(shape, dtype=np.int64)) if shape else 1
        if pos + 4 * n > len(data):
            raise ValueError(f"checkpoint: truncated params in {path}")
        params[pm["name"]] = np.frombuffer(data, dtype="<f4", count=n, offset=pos).astype(np.float32).reshape(shape)
        pos += 4 * n
    return meta, params


def write_gn(path, meta, params):
    """checkpoint.Save (checkpoint.go:40-85): parameters in sorted-name order, metadata["params"] rewritten to match."""
    names = sorted(params)
    meta = dict(meta)
    meta["params"] = [{"name": n, "shape": [int(x) for x in np.asarray(params[n]).shape]} for n in names]
    blob = json.dumps(meta, separators=(",", ":")).encode("utf-8")
    with open(path, "wb") as f:
        f.write(MAGIC)
        f.write(struct.pack("<I", len(blob)))
        f.write(blob)
        for n in names:
            f.write(np.ascontiguousarray(params[n], dtype="<f4").tobytes())


def config_from_meta(meta) -> dict:
    """model_config of a checkpoint -> keyword arguments of session.Model; refuses architectures outside this library."""
    mc = dict(meta["model_config"])
    for key in _UNSUPPORTED:
        value = mc.get(key)
        if value not in (None, 0, "", False) and not (key == "compression_ratio" and value == 1):
            raise ValueError(f"checkpoint uses model_config.{key} = {value!r}, which this library does not implement")
    out = {}
    for key, value in mc.items():
        if key in _CONFIG_KEYS:
            out[_CONFIG_KEYS[key]] = value
        elif key not in _UNSUPPORTED and key not in _IGNORED:
            raise ValueError(f"checkpoint has an unknown model_config field {key!r}")
    out.setdefault("window_pattern", "L")
    return out


def meta_from_config(cfg: dict, step: int = 0) -> dict:
    """The inverse of config_from_meta for the fields this library knows (zero / empty values omitted, like omitempty)."""
    inverse = {v: k for k, v in _CONFIG_KEYS.items()}
    always = ("sequence_len", "vocab_size", "n_layer", "n_head", "n_kv_head", "n_embd", "window_pattern")
    mc = {}
    for key, value in cfg.items():
        name = inverse[key]
        if name in always or value not in (0, 0.0, "", None):
            mc[name] = value
    return {"step": int(step), "model_config": mc, "params": []}


def reference_shape(name: str, rows: int, cols: int, cfg: dict):
    """Shape of the reference tensor that the library holds as [rows, cols] (model/transformer.go:49-83, model/moe.go:63-69)."""
    if name in ("resid_lambdas", "x0_lambdas", "smear_lambda", "backout_lambda") or name.endswith(".moe.router_bias"):
        return (rows * cols,)
    if ".moe.experts." in name:
        experts = cfg["n_experts"]
        return (experts, rows // experts, cols)
    return (rows, cols)


def load_model(ctx, path):
    """checkpoint.Load + checkpoint.LoadModel (checkpoint.go:146-157): a resident Model with the file's parameters.
    Parameters the model does not have are ignored, as LoadModel does; a size mismatch is an error."""
    from .session import Model
    meta, params = read_gn(path)
    cfg = config_from_meta(meta)
    model = Model(ctx, **cfg)
    for name, value in params.items():
        if name in model.names:
            rows, cols = model.shape(name)
            if value.size != rows * cols:
                raise ValueError(f"checkpoint tensor {name} has {value.size} elements, the model expects {rows * cols}")
            model.upload(name, value.ravel())
    return model, meta


def save_model(model, cfg: dict, path, step: int = 0, extra_meta: dict | None = None):
    """Writes the resident model's parameters as a `.gn` file the Go tools can load."""
    meta = meta_from_config(cfg, step)
    if extra_meta:
        meta.update(extra_meta)
    params = {}
    for name in model.names:
        rows, cols = model.shape(name)
        params[name] = model.download(name).reshape(reference_shape(name, rows, cols, cfg))
    write_gn(path, meta, params)
