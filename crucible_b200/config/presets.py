"""Named shapes, as config.json dictionaries.

These are data for the benchmark, the command line and the tests, not defaults
of the engine: every one goes through the same `parse_config` as a model
folder's config.json does.  The 120m entry is the reference's `PRESETS["120m"]`
(`model.py:387-391`) with the benchmark's KV-head count, context and epsilon.
"""
from __future__ import annotations


def _crucible(vocab, layers, heads, kv_heads, width, head_dim, inter, ctx, theta, eps, tie):
    label = "mha" if kv_heads == heads else ("mqa" if kv_heads == 1 else "gqa")
    return {
        "architectures": ["CrucibleGPT"], "vocab_size": vocab, "n_layer": layers,
        "n_head": heads, "n_kv_head": kv_heads, "n_embd": width, "head_dim": head_dim,
        "intermediate_size": inter, "block_size": ctx, "dropout": 0.0, "bias": False,
        "attention": label, "pos_encoding": "rope", "activation": "swiglu",
        "norm": "rmsnorm", "norm_placement": "pre", "rope_theta": theta,
        "rms_norm_eps": eps, "tie_word_embeddings": tie,
    }


def _llama(vocab, layers, heads, kv_heads, width, head_dim, inter, ctx, theta, eps, tie):
    return {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": vocab,
        "hidden_size": width, "num_hidden_layers": layers, "num_attention_heads": heads,
        "num_key_value_heads": kv_heads, "head_dim": head_dim, "intermediate_size": inter,
        "max_position_embeddings": ctx, "hidden_act": "silu", "rope_theta": theta,
        "rms_norm_eps": eps, "tie_word_embeddings": tie,
    }


SHAPES = {
    "tiny-a": _crucible(256, 2, 4, 2, 64, 16, 176, 128, 10000.0, 1e-5, True),
    "tiny-b": _crucible(509, 3, 3, 1, 96, 32, 320, 192, 500000.0, 1e-6, False),
    "120m": _crucible(50304, 12, 12, 4, 768, 64, 2048, 4096, 10000.0, 1e-5, True),
    "llama-1b": _llama(128256, 16, 32, 8, 2048, 64, 8192, 8192, 500000.0, 1e-5, True),
    "llama-8b": _llama(128256, 32, 32, 8, 4096, 128, 14336, 8192, 500000.0, 1e-5, False),
}


def shape(name: str) -> dict:
    try:
        return dict(SHAPES[name])
    except KeyError:
        raise KeyError(f"unknown shape {name!r}; known: {sorted(SHAPES)}") from None
