"""Byte-level restatement of the `.koref` container (``crates/kore-edge/src/format.rs``).

TEST INFRASTRUCTURE ONLY.  Written directly from the layout, independent of the package's
reader: fixed 12-byte prefix (``KORF``, version 1, header length), header JSON, zeros up to
a multiple of 64, blob; tensors at 64-byte multiples inside the blob.  Pinned against the
reference's own unit tests for the format (``format.rs:355-436``): align_up(0,1,64,65),
storage sizes, the 2x2 f32 round trip, bad magic, too small.
"""
import json
import struct

import numpy as np


def round64(n):
    return ((n + 63) // 64) * 64


def write(config: dict, tensors: list, ops=()):
    """tensors: list of (name, dtype tag, shape, raw bytes) in blob order"""
    blob = bytearray()
    index = {}
    for name, dtype, shape, raw in tensors:
        blob += b"\0" * (round64(len(blob)) - len(blob))
        index[name] = {"dtype": dtype, "shape": list(shape), "offset": len(blob), "nbytes": len(raw)}
        blob += raw
    header = dict(config)
    header["tensors"] = index
    header["ops"] = list(ops)
    text = json.dumps(header).encode()
    out = b"KORF" + struct.pack("<I", 1) + struct.pack("<I", len(text)) + text
    out += b"\0" * (round64(len(out)) - len(out))
    return out + bytes(blob)


def read(data: bytes):
    """-> (header dict, {name: raw bytes}); raises ValueError(kind)"""
    if len(data) < 12:
        raise ValueError("TooSmall")
    if data[:4] != b"KORF":
        raise ValueError("BadMagic")
    (version,) = struct.unpack("<I", data[4:8])
    if version != 1:
        raise ValueError("UnsupportedVersion")
    (hlen,) = struct.unpack("<I", data[8:12])
    if len(data) < 12 + hlen:
        raise ValueError("TooSmall")
    header = json.loads(data[12:12 + hlen].decode())
    start = round64(12 + hlen)
    if len(data) < start:
        raise ValueError("TooSmall")
    blob = data[start:]
    out = {}
    for name, e in header["tensors"].items():
        out[name] = blob[e["offset"]:e["offset"] + e["nbytes"]]
    return header, out


CONFIG = dict(model_type="test", vocab_size=256, d_model=64, n_heads=4, n_kv_heads=4, n_layers=2, d_ff=128,
              max_seq_len=128, norm_eps=float(np.float32(1e-5)), rope_base=10000.0)
