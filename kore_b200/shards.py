"""Per-layer safetensors shards: the on-disk side of loading a layer-by-layer model.

Mirrors ``crates/kore-serve/src/layered/sharder.rs``: a one-time offline step reads every
``*.safetensors`` file of a model directory (sorted, ``:161-180``), assigns each tensor to a layer
key by its name (``classify_tensor``, ``:94-138``: embedding, ``{layer_prefix}.{i}``, final norm,
lm_head, otherwise the first two name segments) and writes one ``{key with '.' -> '_'}.safetensors``
file per key (``shard_model``, ``:20-89``).  The reference's layered engine then loads one shard at a
time (f32 ``Linear`` layers); here a shard's projection weights go to ``BitLinear.new`` /
``QuatLinear.new``, i.e. they are quantised and packed on the GPU and the forward is the CUDA path.

The safetensors container itself is restated here (8-byte little-endian header length, JSON header
``{name: {dtype, shape, data_offsets}}``, raw little-endian data) so that the library needs no extra
package; the tests cross-check it against the ``safetensors`` package where that is installed.
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np

_DTYPES = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "I64": np.int64, "I32": np.int32, "I16": np.int16,
           "I8": np.int8, "U8": np.uint8, "BOOL": np.bool_}
_NAMES = {np.dtype(v): k for k, v in _DTYPES.items()}


@dataclass
class LayeredConfig:
    """The naming part of ``layered/config.rs:44-92`` (LLaMA / HuggingFace convention by default)."""

    num_layers: int
    embed_name: str = "model.embed_tokens"
    layer_prefix: str = "model.layers"
    norm_name: str = "model.norm"
    lm_head_name: str = "lm_head"

    def layer_names(self) -> List[str]:
        """embedding, every transformer block, final norm, lm_head (``config.rs:146-155``)"""
        return [self.embed_name] + [f"{self.layer_prefix}.{i}" for i in range(self.num_layers)] + [self.norm_name, self.lm_head_name]


def classify_tensor(tensor_name: str, config: LayeredConfig) -> str:
    """Layer key of a tensor name (``sharder.rs:94-138``), checked in the reference's order."""
    if tensor_name.startswith(config.embed_name):
        return config.embed_name
    for i in range(config.num_layers):
        if tensor_name.startswith(f"{config.layer_prefix}.{i}."):
            return f"{config.layer_prefix}.{i}"
    if tensor_name.startswith(config.norm_name):
        return config.norm_name
    if tensor_name.startswith(config.lm_head_name):
        return config.lm_head_name
    parts = tensor_name.split(".", 2)
    if len(parts) >= 2:
        return f"{parts[0]}.{parts[1]}"
    names = config.layer_names()
    return names[0] if names else "unknown"


# ---- safetensors container -----------------------------------------------------------------
def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    """name -> array (a copy) for every tensor of one file; bf16 tensors are rejected."""
    with open(path, "rb") as fh:
        raw = fh.read()
    if len(raw) < 8:
        raise ValueError(f"failed to parse {path}: shorter than the 8-byte header length")
    (hlen,) = struct.unpack("<Q", raw[:8])
    if 8 + hlen > len(raw):
        raise ValueError(f"failed to parse {path}: header length {hlen} exceeds the file")
    header = json.loads(raw[8:8 + hlen].decode("utf-8"))
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        if meta["dtype"] not in _DTYPES:
            raise ValueError(f"failed to parse {path}: unsupported dtype {meta['dtype']} of {name}")
        b0, b1 = meta["data_offsets"]
        arr = np.frombuffer(raw, dtype=np.dtype(_DTYPES[meta["dtype"]]).newbyteorder("<"), count=(b1 - b0) // np.dtype(_DTYPES[meta["dtype"]]).itemsize,
                            offset=8 + hlen + b0)
        out[name] = arr.reshape(meta["shape"]).copy()
    return out


def write_safetensors(path: str, tensors: Dict[str, np.ndarray]) -> None:
    """One file holding `tensors`; names sorted, data packed back to back, header padded with spaces to a
    multiple of 8 bytes (what the reference's serializer emits for ``write_shard_file``, ``sharder.rs:141-159``)."""
    header, blobs, off = {}, [], 0
    for name in sorted(tensors):
        a = np.ascontiguousarray(tensors[name])
        if a.dtype not in _NAMES:
            raise ValueError(f"invalid tensor {name}: unsupported dtype {a.dtype}")
        b = a.astype(a.dtype.newbyteorder("<"), copy=False).tobytes()
        header[name] = {"dtype": _NAMES[a.dtype], "shape": list(a.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(hj)))
        fh.write(hj)
        for b in blobs:
            fh.write(b)


def find_safetensors_files(model_dir: str) -> List[str]:
    """every ``*.safetensors`` of the directory, sorted (``sharder.rs:161-180``)"""
    try:
        names = os.listdir(model_dir)
    except OSError as exc:
        raise ValueError(f"cannot read directory {model_dir}: {exc}") from exc
    return sorted(os.path.join(model_dir, n) for n in names if n.endswith(".safetensors"))


def shard_model(model_dir: str, output_dir: str, config: LayeredConfig) -> int:
    """Regroup a model directory into one safetensors file per layer key; returns the number of files
    written (``sharder.rs:20-89``)."""
    os.makedirs(output_dir, exist_ok=True)
    files = find_safetensors_files(model_dir)
    if not files:
        raise ValueError(f"no .safetensors files found in {model_dir}")
    groups: Dict[str, Dict[str, np.ndarray]] = {}
    for path in files:
        for name, arr in read_safetensors(path).items():
            groups.setdefault(classify_tensor(name, config), {})[name] = arr
    for key, tensors in groups.items():
        write_safetensors(os.path.join(output_dir, key.replace(".", "_") + ".safetensors"), tensors)
    return len(groups)


def shard_path(output_dir: str, layer_key: str) -> str:
    return os.path.join(output_dir, layer_key.replace(".", "_") + ".safetensors")


# ---- shard -> device-resident quantized layers ---------------------------------------------
PROJECTIONS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


def load_layer(output_dir: str, layer_key: str, *, kind: str = "ternary", quantiser: str = "absmean", threshold: float = 0.3,
               device: int = 0, projections=PROJECTIONS) -> Tuple[Dict[str, object], Dict[str, np.ndarray]]:
    """Loads one shard: every 2-D ``{prefix}.weight`` whose last name segment before ``.weight`` is one of
    `projections` becomes a ``BitLinear`` (kind "ternary") or ``QuatLinear`` (kind "quaternary") — quantised and
    packed on the GPU, with ``{prefix}.bias`` if the shard holds one — and everything else (norm weights,
    embeddings, lm_head, ...) is returned as arrays.  Returns (layers by prefix, other tensors by name)."""
    from . import nn

    tensors = read_safetensors(shard_path(output_dir, layer_key))
    layers, used = {}, set()
    for name, arr in tensors.items():
        if not name.endswith(".weight") or arr.ndim != 2:
            continue
        prefix = name[: -len(".weight")]
        if prefix.rsplit(".", 1)[-1] not in projections:
            continue
        bias = tensors.get(prefix + ".bias")
        w = np.ascontiguousarray(arr, dtype=np.float32)
        b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        if kind == "ternary":
            layers[prefix] = nn.BitLinear.new(w, b, threshold, quantiser=quantiser, device=device)
        else:
            layers[prefix] = nn.QuatLinear.new(w, b, device=device)
        used.add(name)
        if bias is not None:
            used.add(prefix + ".bias")
    return layers, {n: a for n, a in tensors.items() if n not in used}
