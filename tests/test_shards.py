"""Per-layer safetensors shards (crates/kore-serve/src/layered/sharder.rs): tensor classification against the
reference's own test cases, regrouping of a multi-file model directory, the container format against the
`safetensors` package, and (on a GPU) shard -> BitLinear / QuatLinear against the oracle."""
import os

import numpy as np
import pytest

from kore_b200 import shards
from tests import cases


def test_classify_tensor_reference_cases():
    # sharder.rs:186-224: LayeredConfig::llama(.., 32 layers, ..)
    cfg = shards.LayeredConfig(num_layers=32)
    assert shards.classify_tensor("model.embed_tokens.weight", cfg) == "model.embed_tokens"
    assert shards.classify_tensor("model.layers.5.self_attn.q_proj.weight", cfg) == "model.layers.5"
    assert shards.classify_tensor("model.layers.31.mlp.gate_proj.weight", cfg) == "model.layers.31"
    assert shards.classify_tensor("model.norm.weight", cfg) == "model.norm"
    assert shards.classify_tensor("lm_head.weight", cfg) == "lm_head"
    # fallbacks of :117-137: first two segments, else the first layer name
    assert shards.classify_tensor("vision.tower.blocks.0.w", cfg) == "vision.tower"
    assert shards.classify_tensor("loose", cfg) == "model.embed_tokens"
    # layer 3 must not swallow layer 31 (the prefix check includes the trailing dot, :103-106)
    assert shards.classify_tensor("model.layers.31.x", cfg) == "model.layers.31"
    assert cfg.layer_names()[:2] == ["model.embed_tokens", "model.layers.0"] and cfg.layer_names()[-2:] == ["model.norm", "lm_head"]
    assert len(cfg.layer_names()) == 35  # config.rs:146-155


def _toy_model(rng, layers=2, d=64, f=96, vocab=50):
    t = {"model.embed_tokens.weight": rng.standard_normal((vocab, d)).astype(np.float32),
         "model.norm.weight": np.ones(d, np.float32), "lm_head.weight": rng.standard_normal((vocab, d)).astype(np.float32)}
    for i in range(layers):
        p = f"model.layers.{i}"
        for name, shape in (("self_attn.q_proj", (d, d)), ("self_attn.k_proj", (d, d)), ("self_attn.v_proj", (d, d)),
                            ("self_attn.o_proj", (d, d)), ("mlp.gate_proj", (f, d)), ("mlp.up_proj", (f, d)), ("mlp.down_proj", (d, f))):
            t[f"{p}.{name}.weight"] = (rng.standard_normal(shape) * 0.02).astype(np.float32)
        t[f"{p}.mlp.down_proj.bias"] = (rng.standard_normal(d) * 0.1).astype(np.float32)
        t[f"{p}.input_layernorm.weight"] = np.ones(d, np.float32)
        t[f"{p}.post_attention_layernorm.weight"] = np.ones(d, np.float32)
    return t


def test_shard_model_regroups_a_multi_file_directory(tmp_path):
    rng = np.random.default_rng(0)
    model = _toy_model(rng)
    names = sorted(model)
    src, dst = tmp_path / "model", tmp_path / "shards"
    os.makedirs(src)
    # two model files, tensors split arbitrarily (a layer's tensors straddle the files)
    shards.write_safetensors(str(src / "model-00001-of-00002.safetensors"), {n: model[n] for n in names[::2]})
    shards.write_safetensors(str(src / "model-00002-of-00002.safetensors"), {n: model[n] for n in names[1::2]})
    (src / "config.json").write_text("{}")  # not a safetensors file: ignored
    cfg = shards.LayeredConfig(num_layers=2)
    assert shards.shard_model(str(src), str(dst), cfg) == 5  # embed, 2 layers, norm, lm_head
    assert sorted(os.listdir(dst)) == ["lm_head.safetensors", "model_embed_tokens.safetensors", "model_layers_0.safetensors",
                                       "model_layers_1.safetensors", "model_norm.safetensors"]
    back = shards.read_safetensors(shards.shard_path(str(dst), "model.layers.1"))
    assert sorted(back) == [n for n in names if n.startswith("model.layers.1.")]
    for n, a in back.items():
        assert a.dtype == model[n].dtype and (a == model[n]).all()
    os.makedirs(tmp_path / "empty")
    with pytest.raises(ValueError, match="no .safetensors files"):  # sharder.rs:29-34
        shards.shard_model(str(tmp_path / "empty"), str(tmp_path / "o2"), cfg)


def test_container_matches_the_safetensors_package(tmp_path):
    st = pytest.importorskip("safetensors.numpy")
    rng = np.random.default_rng(1)
    tensors = {"a.weight": rng.standard_normal((3, 5)).astype(np.float32), "b": np.arange(7, dtype=np.int64),
               "c.half": rng.standard_normal((2, 2)).astype(np.float16), "d": np.array([1, 0, 1], np.uint8)}
    ours, theirs = str(tmp_path / "ours.safetensors"), str(tmp_path / "theirs.safetensors")
    shards.write_safetensors(ours, tensors)
    st.save_file(tensors, theirs)
    for path_a, reader in ((ours, st.load_file), (theirs, shards.read_safetensors)):  # each side reads the other's file
        got = reader(path_a)
        assert sorted(got) == sorted(tensors)
        for n in tensors:
            assert got[n].dtype == tensors[n].dtype and got[n].shape == tensors[n].shape and (got[n] == tensors[n]).all()
    with pytest.raises(ValueError):
        (tmp_path / "bad.safetensors").write_bytes(b"\x01\x02")
        shards.read_safetensors(str(tmp_path / "bad.safetensors"))


@pytest.mark.gpu
def test_shard_to_quantized_layers_matches_the_oracle(tmp_path):
    import torch

    from oracle import kbref

    rng = np.random.default_rng(2)
    model = _toy_model(rng, layers=1)
    src, dst = tmp_path / "model", tmp_path / "shards"
    os.makedirs(src)
    shards.write_safetensors(str(src / "model.safetensors"), model)
    shards.shard_model(str(src), str(dst), shards.LayeredConfig(num_layers=1))
    x = cases.gaussian(3, (5, 64), 1.0)
    for kind, oracle_kind, quantiser in (("ternary", kbref.TERNARY, "absmean"), ("quaternary", kbref.QUATERNARY, "reference")):
        layers, rest = shards.load_layer(str(dst), "model.layers.0", kind=kind, quantiser=quantiser)
        assert sorted(rest) == ["model.layers.0.input_layernorm.weight", "model.layers.0.post_attention_layernorm.weight"]
        assert len(layers) == 7
        w = model["model.layers.0.self_attn.q_proj.weight"]
        packed, scales = cases.make_weights(oracle_kind, quantiser, w)
        lay = layers["model.layers.0.self_attn.q_proj"]
        assert (lay.packed_weights() == packed).all() and (lay.scales() == scales).all()
        y_ref = kbref.q_forward(oracle_kind, packed, scales, None, 64, 64, x)[0]
        assert (lay(torch.from_numpy(x).cuda()).cpu().numpy() == y_ref).all()
        # the projection with a bias keeps it
        xd = cases.gaussian(4, (2, 96), 1.0)
        wd, bd = model["model.layers.0.mlp.down_proj.weight"], model["model.layers.0.mlp.down_proj.bias"]
        pd, sd = cases.make_weights(oracle_kind, quantiser, wd)
        y_ref = kbref.q_forward(oracle_kind, pd, sd, bd, 64, 96, xd)[0]
        assert (layers["model.layers.0.mlp.down_proj"](xd) == y_ref).all()
        for lay in layers.values():
            lay.close()
