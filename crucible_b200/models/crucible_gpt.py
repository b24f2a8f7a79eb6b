"""The Llama-style dense decoder, in its two config.json spellings.

`CrucibleGPT` reads the keys the reference exporter writes (`export.py:89-97`,
parsed by `engine/src/config.rs:13-38`) and the reference's tensor names
(`engine/src/model.rs:62-100`).  `LlamaForCausalLM` reads the Hugging Face
spelling of the same network (`scripts/export_hf.py:83-103`) with the names of
`scripts/export_hf.py:38-51`.  Both produce the same kind of `ModelConfig`:
identical layers of pre-RMSNorm, grouped-query attention with half-split RoPE
and a SwiGLU feed-forward, run once each in order.

Like the reference's GPU loader (`engine/src/gpu_model.rs:506-520`) anything
other than rope / rmsnorm / pre / swiglu is refused, loudly.
"""
from __future__ import annotations

import math
from typing import Any, Mapping

from ..config.model_config import (ConfigError, FeedForwardSpec, KeyReader, MixerSpec,
                                   ModelConfig, NormSpec, PositionSpec, RunEntry, pre_norm_layer)
from ..config.registry import Architecture, register_architecture

# The reference fixes the RMSNorm epsilon in code (`model.py:108`,
# `engine/src/model.rs:20`); a config.json in its spelling that does not carry
# `rms_norm_eps` therefore means this value.
REFERENCE_RMS_EPS = 1e-6


def _dense_decoder(*, architecture: str, raw: Mapping[str, Any], vocab: int, hidden: int,
                   n_layer: int, n_head: int, n_kv_head: int, head_dim: int,
                   intermediate: int, max_context: int, theta: float, eps: float,
                   tie: bool, names: Mapping[str, str]) -> ModelConfig:
    if n_head % n_kv_head != 0:
        raise ConfigError(f"n_head ({n_head}) is not divisible by n_kv_head ({n_kv_head})")
    if head_dim % 2 != 0:
        raise ConfigError(f"head_dim ({head_dim}) must be even for the rotary pairing")
    position = PositionSpec(kind="rope", rotary_dim=head_dim, theta=theta,
                            max_positions=max_context)
    mixer = MixerSpec(kind="attention", width=hidden, n_heads=n_head, n_kv_heads=n_kv_head,
                      head_dim=head_dim, softmax_scale=1.0 / math.sqrt(head_dim),
                      window=None, position=position)
    norm = NormSpec(kind="rmsnorm", width=hidden, eps=eps)
    ffn = FeedForwardSpec(kind="swiglu", width=hidden, intermediate=intermediate)
    layer = pre_norm_layer(mixer, norm, ffn, norm)
    return ModelConfig(
        architecture=architecture, vocab_size=vocab, hidden_size=hidden,
        max_context=max_context, tie_word_embeddings=tie,
        layers=tuple(layer for _ in range(n_layer)),
        run_order=tuple(RunEntry(layer=i) for i in range(n_layer)),
        final_norm=norm, tensor_names=dict(names), raw=dict(raw))


# ---------------------------------------------------------------------------
# The reference's own spelling
# ---------------------------------------------------------------------------

CRUCIBLE_NAMES = {
    "embedding.table": "tok_emb.weight",
    "head.weight": "lm_head.weight",
    "final_norm.gain": "final_norm.weight",
    "layer.mixer_norm.gain": "blocks.{layer}.attn_norm.weight",
    "layer.mixer.q": "blocks.{layer}.attn.q_proj.weight",
    "layer.mixer.k": "blocks.{layer}.attn.k_proj.weight",
    "layer.mixer.v": "blocks.{layer}.attn.v_proj.weight",
    "layer.mixer.o": "blocks.{layer}.attn.o_proj.weight",
    "layer.feed_forward_norm.gain": "blocks.{layer}.mlp_norm.weight",
    "layer.feed_forward.gate": "blocks.{layer}.mlp.gate_proj.weight",
    "layer.feed_forward.up": "blocks.{layer}.mlp.up_proj.weight",
    "layer.feed_forward.down": "blocks.{layer}.mlp.down_proj.weight",
}


def _parse_crucible(raw: Mapping[str, Any]) -> ModelConfig:
    r = KeyReader(raw)
    # The four architecture switches are required keys in the reference
    # (`engine/src/config.rs:21-25`); only one value of each runs on the GPU.
    r.choice("pos_encoding", ("rope",), default="rope")
    r.choice("activation", ("swiglu",), default="swiglu")
    r.choice("norm", ("rmsnorm",), default="rmsnorm")
    r.choice("norm_placement", ("pre",), default="pre")
    if r.boolean("bias", False):
        raise ConfigError("config.json: 'bias': true is not supported (the reference's "
                          "engine never reads biases either)")
    hidden = r.integer("n_embd")
    n_head = r.integer("n_head")
    n_kv_head = r.integer("n_kv_head")
    if r.has("head_dim"):
        head_dim = r.integer("head_dim")
    else:
        if hidden % n_head != 0:
            raise ConfigError(f"n_embd ({hidden}) is not divisible by n_head ({n_head})")
        head_dim = hidden // n_head          # engine/src/config.rs:93-95
    if r.has("intermediate_size"):
        intermediate = r.integer("intermediate_size")
    else:
        # model.py:228-229: 2/3 of 4d, rounded up to a multiple of 64.
        intermediate = 64 * ((int(2 * (4 * hidden) / 3) + 63) // 64)
    return _dense_decoder(
        architecture="CrucibleGPT", raw=raw, vocab=r.integer("vocab_size"), hidden=hidden,
        n_layer=r.integer("n_layer"), n_head=n_head, n_kv_head=n_kv_head, head_dim=head_dim,
        intermediate=intermediate, max_context=r.integer("block_size"),
        theta=r.number("rope_theta", 10000.0),            # engine/src/config.rs:40-42
        eps=r.number("rms_norm_eps", REFERENCE_RMS_EPS),
        tie=r.boolean("tie_word_embeddings", True),        # engine/src/config.rs:44-46
        names=CRUCIBLE_NAMES)


def _describe_crucible(cfg: ModelConfig) -> dict:
    layer = cfg.layers[0]
    m = layer.mixer
    label = "mha" if m.n_kv_heads == m.n_heads else ("mqa" if m.n_kv_heads == 1 else "gqa")
    return {
        "architectures": ["CrucibleGPT"],
        "vocab_size": cfg.vocab_size, "n_layer": cfg.n_layers, "n_head": m.n_heads,
        "n_kv_head": m.n_kv_heads, "n_embd": cfg.hidden_size, "head_dim": m.head_dim,
        "intermediate_size": layer.feed_forward.intermediate,
        "block_size": cfg.max_context, "dropout": 0.0, "bias": False,
        "attention": label, "pos_encoding": "rope", "activation": "swiglu",
        "norm": "rmsnorm", "norm_placement": "pre",
        "rope_theta": m.position.theta, "rms_norm_eps": layer.mixer_norm.eps,
        "tie_word_embeddings": cfg.tie_word_embeddings,
    }


# ---------------------------------------------------------------------------
# The Hugging Face spelling of the same network
# ---------------------------------------------------------------------------

LLAMA_NAMES = {
    "embedding.table": "model.embed_tokens.weight",
    "head.weight": "lm_head.weight",
    "final_norm.gain": "model.norm.weight",
    "layer.mixer_norm.gain": "model.layers.{layer}.input_layernorm.weight",
    "layer.mixer.q": "model.layers.{layer}.self_attn.q_proj.weight",
    "layer.mixer.k": "model.layers.{layer}.self_attn.k_proj.weight",
    "layer.mixer.v": "model.layers.{layer}.self_attn.v_proj.weight",
    "layer.mixer.o": "model.layers.{layer}.self_attn.o_proj.weight",
    "layer.feed_forward_norm.gain": "model.layers.{layer}.post_attention_layernorm.weight",
    "layer.feed_forward.gate": "model.layers.{layer}.mlp.gate_proj.weight",
    "layer.feed_forward.up": "model.layers.{layer}.mlp.up_proj.weight",
    "layer.feed_forward.down": "model.layers.{layer}.mlp.down_proj.weight",
}


def _parse_llama(raw: Mapping[str, Any]) -> ModelConfig:
    r = KeyReader(raw)
    if raw.get("rope_scaling") not in (None, {}):
        raise ConfigError("config.json: 'rope_scaling' is not supported (plain RoPE only)")
    if r.boolean("attention_bias", False) or r.boolean("mlp_bias", False):
        raise ConfigError("config.json: projection biases are not supported")
    r.choice("hidden_act", ("silu",), default="silu")
    hidden = r.integer("hidden_size")
    n_head = r.integer("num_attention_heads")
    n_kv_head = r.integer("num_key_value_heads", n_head)
    if r.has("head_dim"):
        head_dim = r.integer("head_dim")
    else:
        if hidden % n_head != 0:
            raise ConfigError(f"hidden_size ({hidden}) is not divisible by "
                              f"num_attention_heads ({n_head})")
        head_dim = hidden // n_head
    return _dense_decoder(
        architecture="LlamaForCausalLM", raw=raw, vocab=r.integer("vocab_size"),
        hidden=hidden, n_layer=r.integer("num_hidden_layers"), n_head=n_head,
        n_kv_head=n_kv_head, head_dim=head_dim,
        intermediate=r.integer("intermediate_size"),
        max_context=r.integer("max_position_embeddings"),
        theta=r.number("rope_theta", 10000.0), eps=r.number("rms_norm_eps"),
        tie=r.boolean("tie_word_embeddings", False), names=LLAMA_NAMES)


def _describe_llama(cfg: ModelConfig) -> dict:
    layer = cfg.layers[0]
    m = layer.mixer
    return {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
        "num_hidden_layers": cfg.n_layers, "num_attention_heads": m.n_heads,
        "num_key_value_heads": m.n_kv_heads, "head_dim": m.head_dim,
        "intermediate_size": layer.feed_forward.intermediate,
        "max_position_embeddings": cfg.max_context, "hidden_act": "silu",
        "rope_theta": m.position.theta, "rms_norm_eps": layer.mixer_norm.eps,
        "tie_word_embeddings": cfg.tie_word_embeddings,
        "attention_bias": False, "mlp_bias": False,
    }


register_architecture(Architecture("CrucibleGPT", _parse_crucible, _describe_crucible))
register_architecture(Architecture("LlamaForCausalLM", _parse_llama, _describe_llama))
