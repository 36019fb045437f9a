"""`.koref` model container: reader, builder and the hand-over of its ternary / quaternary
tensors to device-resident layers.

Mirrors ``crates/kore-edge/src/format.rs``: 4 magic bytes ``KORF``, version u32 LE (1),
header size u32 LE, header JSON, zero padding to the next 64-byte boundary, weight blob
(``format.rs:1-27,145-191,194-224``).  Every tensor starts on a 64-byte boundary inside
the blob (``format.rs:316-335``); the header indexes tensors by name with ``dtype``
(``"f32" | "f16" | "ternary" | "quaternary" | "i8" | "u8"``), ``shape``, ``offset`` and
``nbytes`` (``format.rs:32-96``).  A quantized weight ``name`` of shape ``[out, in]`` holds
the wire-format rows (base-243, ``ceil(in/5)`` bytes per row; or 2-bit, ``ceil(in/4)``) and
its per-row scales live in the f32 tensor ``"{name}.scales"`` (``format.rs:245-248``,
use in ``crates/kore-edge/src/runtime.rs:339-384``).

``KorefModel.linear(name)`` uploads such a tensor once (the base-243 -> 2-bit repack runs on
the GPU) and returns a ``BitLinear`` / ``QuatLinear`` whose forward is the CUDA path.
"""
from __future__ import annotations

import json
import struct
from typing import Dict, List, Optional

import numpy as np

MAGIC = b"KORF"
VERSION = 1
BLOB_ALIGNMENT = 64
DTYPES = ("f32", "f16", "ternary", "quaternary", "i8", "u8")


class FormatError(Exception):
    """Errors of ``format.rs:252-272`` with the reference's wording."""

    def __init__(self, kind: str, detail: str = ""):
        self.kind = kind
        text = {
            "TooSmall": "file too small for .koref format",
            "BadMagic": "invalid magic bytes (expected KORF)",
            "UnsupportedVersion": f"unsupported version: {detail}",
            "InvalidHeader": f"invalid header: {detail}",
            "IoError": f"I/O error: {detail}",
        }[kind]
        super().__init__(text)


def align_up(n: int, align: int) -> int:
    return (n + align - 1) & ~(align - 1)


def storage_bytes(dtype: str, n: int) -> int:
    """bytes needed to store n elements (``format.rs:42-51``)"""
    if dtype == "f32":
        return n * 4
    if dtype == "f16":
        return n * 2
    if dtype in ("i8", "u8"):
        return n
    if dtype == "ternary":
        return -(-n // 5)
    if dtype == "quaternary":
        return -(-n // 4)
    raise ValueError(f"unknown dtype {dtype!r}")


HEADER_FIELDS = ("model_type", "vocab_size", "d_model", "n_heads", "n_kv_heads", "n_layers", "d_ff", "max_seq_len",
                 "norm_eps", "rope_base", "tensors", "ops")


class KorefModel:
    """header (dict with the fields of ``KorefHeader``) + weight blob"""

    def __init__(self, header: dict, weights: bytes):
        self.header = header
        self.weights = weights

    # ---- parsing ---------------------------------------------------------------------------
    @classmethod
    def from_bytes(cls, data: bytes) -> "KorefModel":
        if len(data) < 12:
            raise FormatError("TooSmall")
        if data[0:4] != MAGIC:
            raise FormatError("BadMagic")
        version, header_size = struct.unpack_from("<II", data, 4)
        if version != VERSION:
            raise FormatError("UnsupportedVersion", str(version))
        if len(data) < 12 + header_size:
            raise FormatError("TooSmall")
        try:
            text = bytes(data[12:12 + header_size]).decode("utf-8")
        except UnicodeDecodeError:
            raise FormatError("InvalidHeader", "not valid UTF-8")
        try:
            header = json.loads(text)
        except json.JSONDecodeError as exc:
            raise FormatError("InvalidHeader", str(exc))
        if not isinstance(header, dict):
            raise FormatError("InvalidHeader", "expected a JSON object")
        for field in HEADER_FIELDS:
            if field not in header:
                raise FormatError("InvalidHeader", f"missing field `{field}`")
        for name, entry in header["tensors"].items():
            for field in ("dtype", "shape", "offset", "nbytes"):
                if field not in entry:
                    raise FormatError("InvalidHeader", f"tensor {name!r}: missing field `{field}`")
        blob_start = align_up(12 + header_size, BLOB_ALIGNMENT)
        if len(data) < blob_start:
            raise FormatError("TooSmall")
        return cls(header, bytes(data[blob_start:]))

    @classmethod
    def from_file(cls, path) -> "KorefModel":
        try:
            with open(path, "rb") as fh:
                return cls.from_bytes(fh.read())
        except OSError as exc:
            raise FormatError("IoError", str(exc))

    def to_bytes(self) -> bytes:
        header_bytes = json.dumps(self.header, separators=(",", ":")).encode("utf-8")
        blob_start = align_up(12 + len(header_bytes), BLOB_ALIGNMENT)
        return b"".join((MAGIC, struct.pack("<II", VERSION, len(header_bytes)), header_bytes,
                         bytes(blob_start - 12 - len(header_bytes)), self.weights))

    # ---- accessors (``format.rs:226-249``) -------------------------------------------------
    def tensor_data(self, name: str) -> Optional[bytes]:
        entry = self.header["tensors"].get(name)
        if entry is None or entry["offset"] + entry["nbytes"] > len(self.weights):
            return None
        return self.weights[entry["offset"]:entry["offset"] + entry["nbytes"]]

    def tensor_f32(self, name: str) -> Optional[np.ndarray]:
        entry = self.header["tensors"].get(name)
        if entry is None or entry["dtype"] != "f32":
            return None
        data = self.tensor_data(name)
        return None if data is None else np.frombuffer(data, dtype="<f4", count=len(data) // 4)

    def tensor_scales(self, name: str) -> Optional[np.ndarray]:
        return self.tensor_f32(f"{name}.scales")

    # ---- hand-over to the CUDA path ---------------------------------------------------------
    def linear(self, name: str, bias_name: Optional[str] = None, device: int = 0):
        """The quantized weight ``name`` ([out, in], dtype ternary or quaternary) as a
        device-resident layer.  Raises where the reference's ``project`` would silently leave
        the output zero (missing tensor, missing scales, unsupported dtype,
        ``runtime.rs:381-383``)."""
        from . import _cabi, nn

        entry = self.header["tensors"].get(name)
        if entry is None:
            raise _cabi.KoreError(_cabi.ERR_STORAGE, f"tensor {name!r} not found")
        if entry["dtype"] not in ("ternary", "quaternary"):
            raise _cabi.KoreError(_cabi.ERR_DTYPE, f"tensor {name!r} has dtype {entry['dtype']}, expected ternary or quaternary")
        if len(entry["shape"]) != 2:
            raise _cabi.KoreError(_cabi.ERR_SHAPE, f"tensor {name!r}: expected a 2-D weight, got shape {entry['shape']}")
        out_features, in_features = (int(v) for v in entry["shape"])
        data, scales = self.tensor_data(name), self.tensor_scales(name)
        if data is None:
            raise _cabi.KoreError(_cabi.ERR_STORAGE, f"tensor {name!r}: data outside the weight blob")
        if scales is None:
            raise _cabi.KoreError(_cabi.ERR_STORAGE, f"tensor '{name}.scales' not found")
        bias = None
        if bias_name is not None:
            bias = self.tensor_f32(bias_name)
            if bias is None:
                raise _cabi.KoreError(_cabi.ERR_STORAGE, f"tensor {bias_name!r} not found")
        cls = nn.BitLinear if entry["dtype"] == "ternary" else nn.QuatLinear
        return cls.from_packed(np.frombuffer(data, np.uint8), np.ascontiguousarray(scales, np.float32),
                               None if bias is None else np.ascontiguousarray(bias, np.float32), in_features,
                               out_features, device=device)


class KorefBuilder:
    """``format.rs:281-349``"""

    def __init__(self, model_type: str, vocab_size: int, d_model: int, n_heads: int, n_kv_heads: int, n_layers: int,
                 d_ff: int, max_seq_len: int, norm_eps: float, rope_base: float):
        self.header = {"model_type": model_type, "vocab_size": vocab_size, "d_model": d_model, "n_heads": n_heads,
                       "n_kv_heads": n_kv_heads, "n_layers": n_layers, "d_ff": d_ff, "max_seq_len": max_seq_len,
                       "norm_eps": float(np.float32(norm_eps)), "rope_base": float(np.float32(rope_base)),
                       "tensors": {}, "ops": []}
        self._buf = bytearray()

    def add_tensor(self, name: str, dtype: str, shape, data: bytes) -> None:
        if dtype not in DTYPES:
            raise ValueError(f"unknown dtype {dtype!r}")
        self._buf.extend(bytes(align_up(len(self._buf), BLOB_ALIGNMENT) - len(self._buf)))
        self.header["tensors"][name] = {"dtype": dtype, "shape": [int(v) for v in shape], "offset": len(self._buf),
                                        "nbytes": len(data)}
        self._buf.extend(data)

    def add_f32(self, name: str, shape, data) -> None:
        self.add_tensor(name, "f32", shape, np.ascontiguousarray(data, dtype="<f4").tobytes())

    def add_quantized(self, name: str, dtype: str, out_features: int, in_features: int, packed, scales) -> None:
        """a wire-format weight and its ``.scales`` sibling"""
        per_row = storage_bytes(dtype, in_features)
        packed = np.ascontiguousarray(packed, np.uint8).reshape(-1)
        if dtype not in ("ternary", "quaternary") or packed.size != out_features * per_row:
            raise ValueError(f"{name}: expected {out_features} rows of {per_row} bytes")
        self.add_tensor(name, dtype, (out_features, in_features), packed.tobytes())
        self.add_f32(f"{name}.scales", (out_features,), scales)

    def add_op(self, op: str, inputs: List[str], outputs: List[str], params: Optional[Dict[str, str]] = None) -> None:
        self.header["ops"].append({"op": op, "inputs": list(inputs), "outputs": list(outputs), "params": dict(params or {})})

    def build(self) -> KorefModel:
        return KorefModel(self.header, bytes(self._buf))
