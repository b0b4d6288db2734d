"""Configuration: the strict reader, Qwen2's keys and checks, the registry."""
import json

import pytest

from alofa_b200.config import EngineConfig, get_architecture, known_architectures, read_model_config
from alofa_b200.errors import AlofaError
from alofa_b200.models.qwen2 import NAME, Qwen2Config, build_spec, to_json

BASE = {
    "architectures": ["Qwen2ForCausalLM"], "hidden_size": 96, "intermediate_size": 320, "max_position_embeddings": 256,
    "num_attention_heads": 3, "num_hidden_layers": 3, "num_key_value_heads": 1, "rms_norm_eps": 1e-05, "rope_theta": 1000000.0,
    "tie_word_embeddings": False, "vocab_size": 379, "hidden_act": "silu", "use_sliding_window": False, "sliding_window": 32768,
    "max_window_layers": 21, "torch_dtype": "bfloat16",
}


def write(tmp_path, obj=None, text=None):
    (tmp_path / "config.json").write_text(text if text is not None else json.dumps(obj))
    return tmp_path


def test_reads_every_size_from_the_file(tmp_path):
    arch, cfg = read_model_config(write(tmp_path, BASE))
    assert arch.name == NAME
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads) == (3, 96, 3, 1)
    assert cfg.head_dim == 32  # derived: hidden // heads
    assert (cfg.intermediate_size, cfg.vocab_size, cfg.max_position_embeddings) == (320, 379, 256)
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 1e6 and cfg.tie_word_embeddings is False
    assert cfg.window_of_layer(2) is None


def test_head_dim_key_wins_and_is_checked(tmp_path):
    arch, cfg = read_model_config(write(tmp_path, {**BASE, "head_dim": 32}))
    assert cfg.head_dim == 32
    with pytest.raises(AlofaError, match="head_dim"):
        read_model_config(write(tmp_path, {**BASE, "head_dim": 48}))


def test_sliding_window_keys(tmp_path):
    _, cfg = read_model_config(write(tmp_path, {**BASE, "use_sliding_window": True, "sliding_window": 24, "max_window_layers": 1}))
    assert [cfg.window_of_layer(i) for i in range(3)] == [None, 24, 24]
    spec = build_spec(cfg)
    windows = [layer.block.params["mixer"].params["window"] for layer in spec.layers]
    assert windows == [None, 24, 24]


@pytest.mark.parametrize(
    "change, word",
    [
        ({"num_key_value_heads": 2}, "num_key_value_heads"),
        ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
        ({"vocab_size": 0}, "vocab_size"),
        ({"hidden_act": "gelu"}, "hidden_act"),
        ({"num_hidden_layers": "3"}, "integer"),
        ({"tie_word_embeddings": 1}, "true or false"),
        ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ],
)
def test_bad_values_are_named(tmp_path, change, word):
    with pytest.raises(AlofaError, match=word):
        read_model_config(write(tmp_path, {**BASE, **change}))


def test_missing_key_is_named(tmp_path):
    obj = dict(BASE)
    del obj["rope_theta"]
    with pytest.raises(AlofaError, match="rope_theta"):
        read_model_config(write(tmp_path, obj))


def test_duplicate_key_is_refused(tmp_path):
    text = json.dumps(BASE)[:-1] + ', "hidden_size": 64}'
    with pytest.raises(AlofaError, match="repeats a key"):
        read_model_config(write(tmp_path, text=text))


def test_unknown_architecture_lists_the_known(tmp_path):
    with pytest.raises(AlofaError) as err:
        read_model_config(write(tmp_path, {**BASE, "architectures": ["NopeForCausalLM"]}))
    assert "NopeForCausalLM" in str(err.value) and NAME in str(err.value)
    assert NAME in known_architectures()
    with pytest.raises(AlofaError, match="architectures"):
        read_model_config(write(tmp_path, {k: v for k, v in BASE.items() if k != "architectures"}))


def test_json_round_trip(tmp_path):
    cfg = Qwen2Config(2, 64, 4, 2, 16, 128, 256, 1e-6, 1e4, True, 128)
    arch = get_architecture(NAME)
    again = arch.read_config(json.loads(json.dumps(to_json(cfg))), "memory")
    assert again == cfg


def test_spec_is_data(tmp_path):
    cfg = Qwen2Config(2, 64, 4, 2, 16, 128, 256, 1e-6, 1e4, True, 128)
    spec = build_spec(cfg)
    assert [(e.layer, e.cache) for e in spec.run] == [(0, 0), (1, 1)]
    mixer = spec.layers[1].block.params["mixer"]
    assert mixer.kind == "gqa_attention" and mixer.prefix == "model.layers.1.self_attn."
    assert mixer.params["num_heads"] == 4 and mixer.params["num_kv_heads"] == 2 and mixer.params["head_dim"] == 16
    assert mixer.params["position"].params["theta"] == 1e4
    assert spec.head.params["tied_to"] == "model.embed_tokens.weight"


def test_engine_config_checks():
    EngineConfig().validate()
    for bad in ({"dtype": "float16"}, {"block_size": 24}, {"max_batch": 0}, {"watermark_permille": 1001}, {"token_budget": -1}, {"token_budget": 0}):
        with pytest.raises(AlofaError):
            EngineConfig(**bad).validate()
