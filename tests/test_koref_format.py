"""`.koref` container: the package's reader/builder against the byte-level restatement and the
reference's own format tests (crates/kore-edge/src/format.rs:355-436)."""
import numpy as np
import pytest

from kore_b200 import koref
from oracle import kbref, koref_ref
from tests import cases


def test_align_up_kats():  # format.rs:355-361
    assert [koref.align_up(v, 64) for v in (0, 1, 64, 65)] == [0, 64, 64, 128]
    assert [koref_ref.round64(v) for v in (0, 1, 64, 65)] == [0, 64, 64, 128]


def test_storage_bytes_kats():  # format.rs:363-369
    assert koref.storage_bytes("f32", 10) == 40
    assert koref.storage_bytes("f16", 10) == 20
    assert koref.storage_bytes("ternary", 5) == 1
    assert koref.storage_bytes("quaternary", 4) == 1
    assert koref.storage_bytes("ternary", 6) == 2 and koref.storage_bytes("quaternary", 5) == 2
    assert koref.storage_bytes("i8", 7) == 7 and koref.storage_bytes("u8", 7) == 7
    assert set(koref.DTYPES) == {"f32", "f16", "ternary", "quaternary", "i8", "u8"}  # format.rs:371-384


def test_roundtrip_reference_case():  # format.rs:386-406
    b = koref.KorefBuilder("test", 256, 64, 4, 4, 2, 128, 128, 1e-5, 10000.0)
    b.add_f32("embed.weight", (2, 2), [1.0, 2.0, 3.0, 4.0])
    loaded = koref.KorefModel.from_bytes(b.build().to_bytes())
    assert loaded.header["model_type"] == "test"
    assert loaded.header["vocab_size"] == 256 and loaded.header["d_model"] == 64
    assert "embed.weight" in loaded.header["tensors"]
    assert loaded.tensor_f32("embed.weight").tolist() == [1.0, 2.0, 3.0, 4.0]
    # the restatement reads the same bytes
    header, raw = koref_ref.read(b.build().to_bytes())
    assert np.frombuffer(raw["embed.weight"], "<f4").tolist() == [1.0, 2.0, 3.0, 4.0]
    assert header["tensors"]["embed.weight"] == {"dtype": "f32", "shape": [2, 2], "offset": 0, "nbytes": 16}


def test_errors():  # format.rs:408-436
    with pytest.raises(koref.FormatError) as e:
        koref.KorefModel.from_bytes(b"BADXxxxxxxxx")
    assert e.value.kind == "BadMagic" and str(e.value) == "invalid magic bytes (expected KORF)"
    with pytest.raises(koref.FormatError) as e:
        koref.KorefModel.from_bytes(b"KORF")
    assert e.value.kind == "TooSmall" and str(e.value) == "file too small for .koref format"
    with pytest.raises(koref.FormatError) as e:
        koref.KorefModel.from_bytes(b"KORF" + (2).to_bytes(4, "little") + (0).to_bytes(4, "little"))
    assert e.value.kind == "UnsupportedVersion" and str(e.value) == "unsupported version: 2"
    with pytest.raises(koref.FormatError) as e:
        koref.KorefModel.from_bytes(b"KORF" + (1).to_bytes(4, "little") + (100).to_bytes(4, "little") + b"{}")
    assert e.value.kind == "TooSmall"
    with pytest.raises(koref.FormatError) as e:
        koref.KorefModel.from_bytes(b"KORF" + (1).to_bytes(4, "little") + (2).to_bytes(4, "little") + b"{}" + bytes(64))
    assert e.value.kind == "InvalidHeader"
    with pytest.raises(koref.FormatError) as e:
        koref.KorefModel.from_bytes(b"KORF" + (1).to_bytes(4, "little") + (2).to_bytes(4, "little") + b"\xff\xfe" + bytes(64))
    assert str(e.value) == "invalid header: not valid UTF-8"
    with pytest.raises(koref.FormatError) as e:
        koref.KorefModel.from_file("/nonexistent/model.koref")
    assert e.value.kind == "IoError"


def _quantized_case(seed, m, k):
    w = cases.gaussian(seed, (m, k), 0.02)
    pt, st = kbref.pack_weights_ternary(w, m, k, 0.3)
    pq, sq = kbref.pack_weights_quaternary(w, m, k)
    return w, (pt, st), (pq, sq)


def test_cross_read_write_and_alignment():
    m, k = 9, 23  # ragged: 5 and 6 bytes per row
    _, (pt, st), (pq, sq) = _quantized_case(31, m, k)
    gamma = cases.gaussian(32, (k,), 1.0)
    # restatement writes, package reads
    data = koref_ref.write(koref_ref.CONFIG, [
        ("l0.w", "ternary", (m, k), pt.tobytes()), ("l0.w.scales", "f32", (m,), st.astype("<f4").tobytes()),
        ("l0.norm", "f32", (k,), gamma.astype("<f4").tobytes()),
        ("l1.w", "quaternary", (m, k), pq.tobytes()), ("l1.w.scales", "f32", (m,), sq.astype("<f4").tobytes())])
    mod = koref.KorefModel.from_bytes(data)
    assert mod.tensor_data("l0.w") == pt.tobytes() and mod.tensor_data("l1.w") == pq.tobytes()
    assert (mod.tensor_scales("l0.w") == st).all() and (mod.tensor_scales("l1.w") == sq).all()
    assert (mod.tensor_f32("l0.norm") == gamma).all()
    assert mod.tensor_f32("l0.w") is None and mod.tensor_data("missing") is None and mod.tensor_scales("l0.norm") is None
    assert all(e["offset"] % 64 == 0 for e in mod.header["tensors"].values())
    assert mod.header["tensors"]["l0.w"]["nbytes"] == m * koref.storage_bytes("ternary", k)
    # package writes, restatement reads; and the package's own bytes round-trip exactly
    b = koref.KorefBuilder(**{kk: koref_ref.CONFIG[kk] for kk in koref_ref.CONFIG})
    b.add_quantized("l0.w", "ternary", m, k, pt, st)
    b.add_f32("l0.norm", (k,), gamma)
    b.add_quantized("l1.w", "quaternary", m, k, pq, sq)
    b.add_op("Linear", ["x"], ["y"], {"weight": "l0.w"})
    out = b.build().to_bytes()
    header, raw = koref_ref.read(out)
    assert raw["l0.w"] == pt.tobytes() and raw["l1.w"] == pq.tobytes()
    assert np.frombuffer(raw["l1.w.scales"], "<f4").tolist() == sq.tolist()
    assert header["ops"] == [{"op": "Linear", "inputs": ["x"], "outputs": ["y"], "params": {"weight": "l0.w"}}]
    assert (len(out) - len(b.build().weights)) % 64 == 0
    assert koref.KorefModel.from_bytes(out).to_bytes() == out
    with pytest.raises(ValueError):
        b.add_quantized("bad", "ternary", m, k, pt[:-1], st)
    # a truncated blob makes the affected tensor unavailable, as in format.rs:228-231
    cut = koref.KorefModel.from_bytes(out[:-8])
    assert cut.tensor_data("l1.w.scales") is None and cut.tensor_data("l0.w") == pt.tobytes()


@pytest.mark.gpu
def test_koref_linear_on_gpu(tmp_path):
    """tensors of a .koref file become device-resident layers whose forward matches the restated
    W2A8 arithmetic exactly, and whose weights dequantise to what the reference decodes"""
    import torch

    m, k, n = 200, 333, 7
    _, (pt, st), (pq, sq) = _quantized_case(41, m, k)
    bias = cases.gaussian(42, (m,), 0.1)
    data = koref_ref.write(koref_ref.CONFIG, [
        ("a.w", "ternary", (m, k), pt.tobytes()), ("a.w.scales", "f32", (m,), st.astype("<f4").tobytes()),
        ("a.b", "f32", (m,), bias.astype("<f4").tobytes()),
        ("b.w", "quaternary", (m, k), pq.tobytes()), ("b.w.scales", "f32", (m,), sq.astype("<f4").tobytes()),
        ("c.w", "f32", (2, 2), np.zeros(4, "<f4").tobytes())])
    path = tmp_path / "model.koref"
    path.write_bytes(data)
    mod = koref.KorefModel.from_file(path)
    x = cases.gaussian(43, (n, k), 1.0)
    for name, kind, packed, scales, b_name, b in (("a.w", kbref.TERNARY, pt, st, "a.b", bias), ("b.w", kbref.QUATERNARY, pq, sq, None, None)):
        lay = mod.linear(name, bias_name=b_name)
        y = lay.forward(torch.from_numpy(x).cuda()).cpu().numpy()
        y_ref = kbref.q_forward(kind, packed, scales, b, m, k, x, threads=2)[0]
        assert (y == y_ref).all()
        assert (lay.dequantize_weights() == kbref.dequantize_weights(kind, packed, scales, m, k)).all()
        lay.close()
    from kore_b200 import KoreError
    for bad in ("c.w", "missing"):
        with pytest.raises(KoreError):
            mod.linear(bad)
