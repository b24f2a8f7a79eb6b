"""Configuration and registry (no GPU)."""
import copy

import pytest

from crucible_b200.config import (ConfigError, known_architectures, parse_config, shape, SHAPES,
                                  Architecture, register_architecture)
from helpers import TINY


def test_reference_spelling_is_parsed_into_layers():
    cfg = parse_config(TINY["tiny-a"]["config"])
    assert cfg.architecture == "CrucibleGPT"
    assert (cfg.vocab_size, cfg.hidden_size, cfg.max_context, cfg.n_layers) == (256, 64, 512, 2)
    m = cfg.layers[0].mixer
    assert (m.kind, m.n_heads, m.n_kv_heads, m.head_dim, m.window) == ("attention", 4, 2, 16, None)
    assert m.softmax_scale == pytest.approx(0.25)
    assert (m.position.kind, m.position.theta, m.position.rotary_dim) == ("rope", 10000.0, 16)
    assert cfg.layers[0].feed_forward.kind == "swiglu"
    assert cfg.layers[0].feed_forward.intermediate == 176
    assert cfg.layers[0].mixer_norm.eps == 1e-5 and cfg.final_norm.kind == "rmsnorm"
    assert cfg.tie_word_embeddings is True
    assert [e.layer for e in cfg.run_order] == [0, 1]


def test_hugging_face_spelling_gives_the_same_kind_of_model():
    cfg = parse_config(TINY["tiny-b"]["config"])
    assert cfg.architecture == "LlamaForCausalLM"
    m = cfg.layers[2].mixer
    assert (m.n_heads, m.n_kv_heads, m.head_dim) == (3, 1, 32)
    assert cfg.layers[0].mixer_norm.eps == 1e-6 and m.position.theta == 500000.0
    assert cfg.tie_word_embeddings is False
    assert cfg.tensor_names["layer.mixer.q"].format(layer=1) == "model.layers.1.self_attn.q_proj.weight"


def test_defaults_of_the_reference_spelling():
    raw = {"vocab_size": 100, "n_layer": 1, "n_head": 6, "n_kv_head": 3, "n_embd": 384,
           "block_size": 64, "attention": "gqa", "pos_encoding": "rope", "activation": "swiglu",
           "norm": "rmsnorm", "norm_placement": "pre"}
    cfg = parse_config(raw)          # no name: the reference exporter's keys identify it
    assert cfg.architecture == "CrucibleGPT"
    assert cfg.layers[0].mixer.head_dim == 64                    # n_embd / n_head
    assert cfg.layers[0].feed_forward.intermediate == 1024       # 64 * ceil((8 * 384 / 3) / 64)
    assert cfg.layers[0].mixer_norm.eps == 1e-6                  # the reference's constant
    assert cfg.layers[0].mixer.position.theta == 10000.0
    assert cfg.tie_word_embeddings is True


@pytest.mark.parametrize("key,value,needle", [
    ("n_head", 5, "n_kv_head"), ("vocab_size", 0, "vocab_size"), ("n_layer", -1, "n_layer"),
    ("rope_theta", "big", "rope_theta"), ("rms_norm_eps", 0, "rms_norm_eps"),
    ("tie_word_embeddings", "yes", "tie_word_embeddings"), ("pos_encoding", "alibi", "pos_encoding"),
    ("activation", "gelu", "activation"), ("norm", "layernorm", "norm"),
    ("norm_placement", "post", "norm_placement"), ("bias", True, "bias"), ("head_dim", 15, "head_dim"),
])
def test_errors_name_the_key(key, value, needle):
    raw = copy.deepcopy(TINY["tiny-a"]["config"])
    raw[key] = value
    with pytest.raises(ConfigError) as e:
        parse_config(raw)
    assert needle in str(e.value)


def test_missing_key_is_named():
    raw = copy.deepcopy(TINY["tiny-b"]["config"])
    del raw["rms_norm_eps"]
    with pytest.raises(ConfigError, match="rms_norm_eps"):
        parse_config(raw)


def test_unknown_architecture_lists_the_known_ones():
    with pytest.raises(ConfigError) as e:
        parse_config({"architectures": ["MambaForCausalLM"]})
    assert "CrucibleGPT" in str(e.value) and "LlamaForCausalLM" in str(e.value)
    with pytest.raises(ConfigError):
        parse_config({"hello": 1})
    assert set(known_architectures()) >= {"CrucibleGPT", "LlamaForCausalLM"}


def test_llama_refuses_what_it_does_not_run():
    raw = copy.deepcopy(TINY["tiny-b"]["config"])
    raw["rope_scaling"] = {"type": "linear", "factor": 2}
    with pytest.raises(ConfigError, match="rope_scaling"):
        parse_config(raw)


def test_named_shapes_all_parse():
    for name in SHAPES:
        cfg = parse_config(shape(name))
        assert cfg.n_layers > 0
    big = parse_config(shape("120m"))
    assert (big.hidden_size, big.vocab_size, big.layers[0].mixer.n_kv_heads) == (768, 50304, 4)


def test_registering_twice_is_refused():
    with pytest.raises(ValueError):
        register_architecture(Architecture("CrucibleGPT", lambda r: None, lambda c: {}))
