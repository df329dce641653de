"""Weights: container, named loading with one collected error, random-weights mode (no GPU)."""
import json
import os

import pytest
import torch

from ember_b200.model import CausalLM
from ember_b200.parts import Runtime
from ember_b200.weights import SafetensorsDir, SafetensorsError, WeightError, WeightStore, random_tensors, save_file
from tests.tiny_configs import TINY, tiny_config

CPU = Runtime(device=torch.device("cpu"), dtype=torch.float32)


def test_container_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int64).reshape(2, 3),
         "d": torch.randn(2, 2).to(torch.float16)}
    save_file(t, str(tmp_path / "model.safetensors"), metadata={"x": "y"})
    sd = SafetensorsDir(str(tmp_path))
    assert sorted(sd.names()) == ["a", "b", "c", "d"]
    for n in t:
        assert sd.dtype(n) == t[n].dtype and torch.equal(sd.get(n), t[n])


def test_container_rejects_bad_files(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="too small"):
        SafetensorsDir(str(tmp_path))
    p.write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsDir(str(tmp_path))
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}).encode()
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 12)
    with pytest.raises(SafetensorsError, match="12 bytes for shape"):
        SafetensorsDir(str(tmp_path))
    with pytest.raises(SafetensorsError, match="not found"):
        SafetensorsDir(str(tmp_path / "nowhere"))


def test_sharded_folder(tmp_path):
    save_file({"a": torch.ones(2)}, str(tmp_path / "one.safetensors"))
    save_file({"b": torch.zeros(3)}, str(tmp_path / "two.safetensors"))
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "one.safetensors", "b": "two.safetensors"}}))
    sd = SafetensorsDir(str(tmp_path))
    assert sorted(sd.names()) == ["a", "b"] and sd.get("b").shape == (3,)


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    spec = tiny_config("b").to_model_spec()
    tensors = dict(random_tensors(spec, seed=1))
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(5, 5, dtype=torch.bfloat16)
    tensors["model.layers.9.extra.weight"] = torch.zeros(1)
    with pytest.raises(WeightError) as ei:
        CausalLM(spec).load(WeightStore.from_tensors(tensors, "test"), CPU)
    e = ei.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.9.extra.weight"]
    assert [w[0] for w in e.wrong_shape] == ["model.layers.0.self_attn.q_proj.weight"]
    text = str(e)
    for needle in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "[5, 5], expected [192, 96]"):
        assert needle in text


def test_extra_tensors_alone_are_a_warning_unless_strict():
    """A folder that carries a tensor the model does not use loads, with a warning that names it (the reference
    never sees such tensors: it looks up by name); a strict store makes it the listed error."""
    from ember_b200.weights import UnexpectedTensorsWarning
    spec = tiny_config("a").to_model_spec()
    tensors = dict(random_tensors(spec, seed=4))
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    with pytest.warns(UnexpectedTensorsWarning, match="rotary_emb.inv_freq"):
        CausalLM(spec).load(WeightStore.from_tensors(tensors, "test"), CPU)
    with pytest.raises(WeightError) as ei:
        CausalLM(spec).load(WeightStore.from_tensors(tensors, "test", strict=True), CPU)
    assert ei.value.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"] and not ei.value.missing


def test_stored_precision_is_kept_and_tied_head_is_tolerated():
    spec = tiny_config("a").to_model_spec()           # tied
    tensors = dict(random_tensors(spec, seed=2))
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()
    tensors["model.layers.0.mlp.down_proj.weight"] = tensors["model.layers.0.mlp.down_proj.weight"].float()
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()   # repeated tied matrix: allowed
    serving = Runtime(device=torch.device("cpu"), dtype=torch.bfloat16)
    m = CausalLM(spec).load(WeightStore.from_tensors(tensors), serving)
    assert m.blocks[0].feed_forward.down.weight.dtype == torch.float32      # stored in 32-bit: stays so
    assert m.blocks[0].feed_forward.gate_up.weight.dtype == torch.bfloat16
    assert m.head.weight is m.embedding
    m32 = CausalLM(spec).load(WeightStore.from_tensors(tensors), CPU)
    assert m32.blocks[0].feed_forward.gate_up.weight.dtype == torch.float32  # the float32 path widens everything
    store = WeightStore.from_tensors({"t": torch.arange(4, dtype=torch.int64), "h": torch.ones(2, dtype=torch.float16)})
    assert store.take("t", (4,), integer=True).dtype == torch.int32
    assert store.take("h", (2,)).dtype == torch.bfloat16


def test_untied_head_absent_falls_back_to_embedding():
    spec = tiny_config("b").to_model_spec()
    tensors = dict(random_tensors(spec, seed=3))
    del tensors["lm_head.weight"]
    m = CausalLM(spec).load(WeightStore.from_tensors(tensors), CPU)
    assert m.head.weight is m.embedding


def test_random_mode_is_seeded_and_order_independent(tiny_model_dirs):
    spec = tiny_config("a").to_model_spec()
    a, b, c = dict(random_tensors(spec, 5)), dict(random_tensors(spec, 5)), dict(random_tensors(spec, 6))
    assert all(torch.equal(a[n], b[n]) for n in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    w = a["model.layers.0.mlp.gate_proj.weight"].float()
    assert abs(w.std().item() - 0.02) < 0.002
    n = a["model.layers.1.input_layernorm.weight"].float()
    assert abs(n.mean().item() - 1.0) < 0.03
    # the written folder holds config.json and model.safetensors with every declared tensor
    d = tiny_model_dirs["a"]
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    names = {x.name for x in CausalLM(spec).weight_decls()}
    assert set(SafetensorsDir(d).names()) == names
