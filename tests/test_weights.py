"""Weights: safetensors reading and writing, the one clear error, dtypes, and
the seeded random mode."""
import json
import struct

import pytest
import torch

import tiny
from alofa_b200.errors import AlofaError
from alofa_b200.models.qwen2 import NAME, build_spec
from alofa_b200.parts import expected_tensors
from alofa_b200.weights import SafeTensorFile, load_state, write_safetensors
from alofa_b200.weights.random_init import random_state, write_random_model


def test_round_trip_keeps_dtypes(tmp_path):
    tensors = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7), "table": torch.arange(6, dtype=torch.int64).view(2, 3)}
    write_safetensors(tmp_path / "x.safetensors", tensors, {"note": "test"})
    st = SafeTensorFile(tmp_path / "x.safetensors")
    assert set(st.names()) == set(tensors)
    for name, t in tensors.items():
        got = st.tensor(name)
        assert got.dtype == t.dtype and torch.equal(got, t)
    st.close()


def test_header_checks(tmp_path):
    path = tmp_path / "bad.safetensors"
    path.write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(AlofaError, match="header length"):
        SafeTensorFile(path)
    header = json.dumps({"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 12]}}).encode()
    path.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 12)
    with pytest.raises(AlofaError, match="does not match its shape"):
        SafeTensorFile(path)
    header = json.dumps({"w": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 16]}}).encode()
    path.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 8)
    with pytest.raises(AlofaError, match="outside the file"):
        SafeTensorFile(path)
    header = json.dumps({"w": {"dtype": "F64", "shape": [1], "data_offsets": [0, 8]}}).encode()
    path.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 8)
    with pytest.raises(AlofaError, match="F64"):
        SafeTensorFile(path)
    header = json.dumps({"__metadata__": {"format": "pt"}}).encode()
    path.write_bytes(struct.pack("<Q", len(header)) + header)
    with pytest.raises(AlofaError, match="no tensor"):
        SafeTensorFile(path)


def test_float16_is_refused_by_name(tmp_path):
    write_safetensors(tmp_path / "h.safetensors", {"half": torch.ones(2, dtype=torch.float16)})
    st = SafeTensorFile(tmp_path / "h.safetensors")
    with pytest.raises(AlofaError, match="half"):
        st.tensor("half")
    st.close()


def test_one_error_lists_missing_unexpected_and_wrong(tmp_path):
    cfg, seed = tiny.CONFIGS["B"]
    expected = expected_tensors(build_spec(cfg))
    state = random_state(expected, seed)
    del state["model.layers.1.mlp.up_proj.weight"]
    del state["model.norm.weight"]
    state["model.layers.9.extra.weight"] = torch.zeros(2)
    state["model.layers.0.self_attn.k_proj.bias"] = torch.zeros(7)
    folder = tmp_path / "m"
    folder.mkdir()
    write_safetensors(folder / "model.safetensors", state)
    with pytest.raises(AlofaError) as err:
        load_state(expected, folder, torch.bfloat16, "cpu")
    text = str(err.value)
    assert "missing tensors (2)" in text and "model.layers.1.mlp.up_proj.weight" in text and "model.norm.weight" in text
    assert "unexpected tensors (1)" in text and "model.layers.9.extra.weight" in text
    assert "wrong shapes (1)" in text and "k_proj.bias got=(7,) want=(32,)" in text


def test_dtypes_on_load(tmp_path):
    cfg, seed = tiny.CONFIGS["A"]
    expected = expected_tensors(build_spec(cfg))
    state = random_state(expected, seed, torch.bfloat16)
    name32 = "model.layers.0.input_layernorm.weight"
    state[name32] = state[name32].to(torch.float32)
    folder = tmp_path / "m"
    folder.mkdir()
    write_safetensors(folder / "model.safetensors", state)
    as16 = load_state(expected, folder, torch.bfloat16, "cpu")
    assert as16[name32].dtype == torch.float32  # stored in 32-bit, stays so
    assert as16["model.embed_tokens.weight"].dtype == torch.bfloat16
    as32 = load_state(expected, folder, torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in as32.values())
    assert torch.equal(as32["model.embed_tokens.weight"], state["model.embed_tokens.weight"].float())  # widening is exact


def test_tied_head_is_optional_untied_is_required(tmp_path):
    cfg_a, _ = tiny.CONFIGS["A"]
    cfg_b, _ = tiny.CONFIGS["B"]
    assert expected_tensors(build_spec(cfg_a))["lm_head.weight"].optional
    assert not expected_tensors(build_spec(cfg_b))["lm_head.weight"].optional


def test_random_mode_is_seeded(tmp_path):
    cfg, _ = tiny.CONFIGS["A"]
    a = write_random_model(tmp_path / "a", NAME, cfg, 7)
    b = write_random_model(tmp_path / "b", NAME, cfg, 7)
    c = write_random_model(tmp_path / "c", NAME, cfg, 8)
    assert (a / "model.safetensors").read_bytes() == (b / "model.safetensors").read_bytes()
    assert (a / "model.safetensors").read_bytes() != (c / "model.safetensors").read_bytes()
    st = SafeTensorFile(a / "model.safetensors")
    w = st.tensor("model.layers.0.mlp.down_proj.weight").float()
    n = st.tensor("model.norm.weight").float()
    assert abs(float(w.std()) - 0.02) < 0.003 and abs(float(n.mean()) - 1.0) < 0.01
    assert "lm_head.weight" not in st.names()  # tied
    st.close()
    assert json.loads((a / "config.json").read_text())["architectures"] == [NAME]


def shard_folder(tmp_path, state, pieces=3, name="m"):
    """Write ``state`` as ``pieces`` shard files plus the index."""
    folder = tmp_path / name
    folder.mkdir()
    names = list(state)
    weight_map = {}
    for i in range(pieces):
        part = {n: state[n] for n in names[i::pieces]}
        shard = f"model-{i + 1:05d}-of-{pieces:05d}.safetensors"
        write_safetensors(folder / shard, part)
        weight_map.update({n: shard for n in part})
    (folder / "model.safetensors.index.json").write_text(json.dumps({"metadata": {"total_size": 0}, "weight_map": weight_map}))
    return folder, weight_map


def test_sharded_checkpoint_loads_like_the_single_file(tmp_path):
    cfg, seed = tiny.CONFIGS["B"]
    expected = expected_tensors(build_spec(cfg))
    state = random_state(expected, seed)
    folder, _ = shard_folder(tmp_path, state)
    got = load_state(expected, folder, torch.bfloat16, "cpu")
    assert set(got) == set(state) and all(torch.equal(got[n], state[n]) for n in state)


def test_sharded_checkpoint_one_error_across_shards(tmp_path):
    cfg, seed = tiny.CONFIGS["B"]
    expected = expected_tensors(build_spec(cfg))
    state = random_state(expected, seed)
    del state["model.norm.weight"]
    state["model.layers.0.self_attn.k_proj.bias"] = torch.zeros(7)
    state["stray.weight"] = torch.zeros(2)
    folder, weight_map = shard_folder(tmp_path, state)
    # one tensor twice: a copy of it in another shard than the index says; and one the index misplaces
    twice = "model.layers.1.mlp.up_proj.weight"
    other = next(s for s in sorted(set(weight_map.values())) if s != weight_map[twice])
    st = SafeTensorFile(folder / other)
    part = {n: st.tensor(n).clone() for n in st.names()}
    st.close()
    part[twice] = state[twice]
    write_safetensors(folder / other, part)
    moved = "model.layers.2.input_layernorm.weight"
    weight_map[moved] = next(s for s in sorted(set(weight_map.values())) if s != weight_map[moved])
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    with pytest.raises(AlofaError) as err:
        load_state(expected, folder, torch.bfloat16, "cpu")
    text = str(err.value)
    assert "missing tensors" in text and "model.norm.weight" in text and moved in text
    assert "unexpected tensors (1)" in text and "stray.weight" in text
    assert "wrong shapes (1)" in text and "k_proj.bias got=(7,)" in text
    assert f"{twice} is held by 2 shards" in text and f"{moved} is not in" in text


def test_shard_index_refusals(tmp_path):
    cfg, seed = tiny.CONFIGS["A"]
    expected = expected_tensors(build_spec(cfg))
    state = random_state(expected, seed)
    folder, weight_map = shard_folder(tmp_path, state, pieces=2)
    (folder / sorted(set(weight_map.values()))[1]).unlink()
    with pytest.raises(AlofaError, match="shard named by the index is missing"):
        load_state(expected, folder, torch.bfloat16, "cpu")
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "../elsewhere.safetensors"}}))
    with pytest.raises(AlofaError, match="outside the model folder"):
        load_state(expected, folder, torch.bfloat16, "cpu")
    (folder / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}}))
    with pytest.raises(AlofaError, match="no weight_map"):
        load_state(expected, folder, torch.bfloat16, "cpu")
    with pytest.raises(AlofaError, match="no model.safetensors"):
        load_state(expected, tmp_path, torch.bfloat16, "cpu")
