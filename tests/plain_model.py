"""A plain, slow implementation of the Llama-style decoder, for comparison only.

Whole sequences, no cache, no batching, one function per part, on the CPU in
float64 (or float32 on request).  It shares no code with the engine: it reads
config.json and model.safetensors with its own few lines (through the
`safetensors` package) and is written from the reference's formulas; each
function cites the lines it follows.  `tests/golden/` pins it once against the
reference's own PyTorch model.

Also here: the plain sampler (greedy, top-k, temperature, xorshift64* generator)
written from `engine/src/sampling.rs`.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import torch


# ---------------------------------------------------------------------------
# reading a model folder (own reader; not the engine's)
# ---------------------------------------------------------------------------

def read_folder(model_dir: str, dtype=torch.float64):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    from safetensors import safe_open
    weights = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(dtype)
    return normalise_config(cfg), weights


def normalise_config(cfg: dict) -> dict:
    """One flat dict of the sizes the formulas need, from either spelling of
    config.json (reference spelling: `export.py:89-97`; Hugging Face spelling:
    `scripts/export_hf.py:83-103`)."""
    if "n_embd" in cfg:
        d = cfg["n_embd"]
        heads = cfg["n_head"]
        out = dict(vocab=cfg["vocab_size"], layers=cfg["n_layer"], heads=heads,
                   kv_heads=cfg["n_kv_head"], width=d,
                   head_dim=cfg.get("head_dim", d // heads),           # config.rs:93-95
                   inter=cfg.get("intermediate_size",
                                 64 * ((int(2 * (4 * d) / 3) + 63) // 64)),   # model.py:228-229
                   theta=cfg.get("rope_theta", 10000.0),               # config.rs:40-42
                   eps=cfg.get("rms_norm_eps", 1e-6),                  # model.py:108
                   tie=cfg.get("tie_word_embeddings", True),           # config.rs:44-46
                   ctx=cfg["block_size"], names="crucible")
    else:
        d = cfg["hidden_size"]
        heads = cfg["num_attention_heads"]
        out = dict(vocab=cfg["vocab_size"], layers=cfg["num_hidden_layers"], heads=heads,
                   kv_heads=cfg.get("num_key_value_heads", heads), width=d,
                   head_dim=cfg.get("head_dim", d // heads), inter=cfg["intermediate_size"],
                   theta=cfg.get("rope_theta", 10000.0), eps=cfg["rms_norm_eps"],
                   tie=cfg.get("tie_word_embeddings", False),
                   ctx=cfg["max_position_embeddings"], names="llama")
    return out


def tensor_name(cfg: dict, what: str, layer: Optional[int] = None) -> str:
    """Checkpoint names: `engine/src/model.rs:62-100` (reference spelling) and
    `scripts/export_hf.py:38-51` (Hugging Face spelling)."""
    crucible = {"embed": "tok_emb.weight", "head": "lm_head.weight",
                "final_norm": "final_norm.weight",
                "attn_norm": "blocks.{l}.attn_norm.weight", "q": "blocks.{l}.attn.q_proj.weight",
                "k": "blocks.{l}.attn.k_proj.weight", "v": "blocks.{l}.attn.v_proj.weight",
                "o": "blocks.{l}.attn.o_proj.weight", "mlp_norm": "blocks.{l}.mlp_norm.weight",
                "gate": "blocks.{l}.mlp.gate_proj.weight", "up": "blocks.{l}.mlp.up_proj.weight",
                "down": "blocks.{l}.mlp.down_proj.weight"}
    llama = {"embed": "model.embed_tokens.weight", "head": "lm_head.weight",
             "final_norm": "model.norm.weight",
             "attn_norm": "model.layers.{l}.input_layernorm.weight",
             "q": "model.layers.{l}.self_attn.q_proj.weight",
             "k": "model.layers.{l}.self_attn.k_proj.weight",
             "v": "model.layers.{l}.self_attn.v_proj.weight",
             "o": "model.layers.{l}.self_attn.o_proj.weight",
             "mlp_norm": "model.layers.{l}.post_attention_layernorm.weight",
             "gate": "model.layers.{l}.mlp.gate_proj.weight",
             "up": "model.layers.{l}.mlp.up_proj.weight",
             "down": "model.layers.{l}.mlp.down_proj.weight"}
    table = crucible if cfg["names"] == "crucible" else llama
    return table[what].format(l=layer)


# ---------------------------------------------------------------------------
# one function per part
# ---------------------------------------------------------------------------

def plain_embedding(table: torch.Tensor, tokens: Sequence[int]) -> torch.Tensor:
    """x[t] = table[token[t]]; no scaling, nothing added (`model.py:347`)."""
    return table[torch.tensor(list(tokens), dtype=torch.long)]


def plain_rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps), then * gain (`model.py:113-118`)."""
    ms = x.pow(2).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(ms + eps) * gain


def plain_rope_tables(head_dim: int, n_pos: int, theta: float, dtype=torch.float64):
    """inv_freq_i = theta^(-2i/hd); angle = pos * inv_freq (`model.py:131-136`;
    the engine computes them in f64, `engine/src/ops.rs:101-115`)."""
    i = torch.arange(0, head_dim, 2, dtype=torch.float64)
    inv_freq = 1.0 / (theta ** (i / head_dim))
    ang = torch.outer(torch.arange(n_pos, dtype=torch.float64), inv_freq)
    return ang.cos().to(dtype), ang.sin().to(dtype)


def plain_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
               positions: Optional[Sequence[int]] = None) -> torch.Tensor:
    """x: [T, heads, hd].  Half-split pairing: (x1, x2) = halves of the head;
    out = [x1 cos - x2 sin, x1 sin + x2 cos] (`model.py:139-145`)."""
    t = x.shape[0]
    pos = torch.arange(t) if positions is None else torch.tensor(list(positions))
    c = cos[pos].unsqueeze(1)
    s = sin[pos].unsqueeze(1)
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1)


def plain_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                    window: Optional[int] = None) -> torch.Tensor:
    """q: [T, Hq, hd], k, v: [T, Hkv, hd], all of one sequence from position 0.
    Query head h reads KV head h // n_rep (`engine/src/model.rs:211-215`); keys
    0..t only; s = q.k / sqrt(hd); softmax; weighted sum of v
    (`engine/src/model.rs:190-250`, `model.py:205-211`)."""
    t, hq, hd = q.shape
    n_rep = hq // k.shape[1]
    out = torch.zeros_like(q)
    scale = 1.0 / math.sqrt(hd)
    for h in range(hq):
        kh, vh = k[:, h // n_rep], v[:, h // n_rep]
        scores = (q[:, h] @ kh.T) * scale                      # [T, T]
        i = torch.arange(t).unsqueeze(1)
        j = torch.arange(t).unsqueeze(0)
        banned = j > i
        if window is not None:
            banned = banned | (j < i - window + 1)
        scores = scores.masked_fill(banned, float("-inf"))
        m = scores.max(dim=-1, keepdim=True).values
        e = torch.exp(scores - m)
        out[:, h] = (e @ vh) / e.sum(dim=-1, keepdim=True)
    return out


def plain_swiglu(n: torch.Tensor, gate: torch.Tensor, up: torch.Tensor,
                 down: torch.Tensor) -> torch.Tensor:
    """(silu(n Wg^T) * (n Wu^T)) Wd^T, silu(g) = g / (1 + exp(-g))
    (`model.py:240-241`, `engine/src/model.rs:254-273`)."""
    g = n @ gate.T
    u = n @ up.T
    return ((g / (1.0 + torch.exp(-g))) * u) @ down.T


def plain_block(x, cfg, w, layer, cos, sin):
    """x + attn(norm(x)); then x + mlp(norm(x)) (`model.py:262-264`)."""
    t = x.shape[0]
    hq, hkv, hd = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    n = plain_rmsnorm(x, w[tensor_name(cfg, "attn_norm", layer)], cfg["eps"])
    q = (n @ w[tensor_name(cfg, "q", layer)].T).view(t, hq, hd)
    k = (n @ w[tensor_name(cfg, "k", layer)].T).view(t, hkv, hd)
    v = (n @ w[tensor_name(cfg, "v", layer)].T).view(t, hkv, hd)
    q, k = plain_rope(q, cos, sin), plain_rope(k, cos, sin)      # not v (model.py:196-197)
    a = plain_attention(q, k, v, cfg.get("window")).reshape(t, hq * hd)
    x = x + a @ w[tensor_name(cfg, "o", layer)].T
    n = plain_rmsnorm(x, w[tensor_name(cfg, "mlp_norm", layer)], cfg["eps"])
    return x + plain_swiglu(n, w[tensor_name(cfg, "gate", layer)],
                            w[tensor_name(cfg, "up", layer)], w[tensor_name(cfg, "down", layer)])


def plain_forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int],
                  rows: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Logits of one whole sequence: [T, vocab] at every position, or [len(rows), vocab]
    at the positions `rows` only (the layers still run the whole sequence; only the head's
    product is spared, which for a wide vocabulary is most of the work)
    (`model.py:342-365`; the head is the embedding when tied, `model.py:289`)."""
    dtype = w[tensor_name(cfg, "embed")].dtype
    cos, sin = plain_rope_tables(cfg["head_dim"], len(tokens), cfg["theta"], dtype)
    x = plain_embedding(w[tensor_name(cfg, "embed")], tokens)
    for layer in range(cfg["layers"]):
        x = plain_block(x, cfg, w, layer, cos, sin)
    if rows is not None:
        x = x[torch.tensor(list(rows), dtype=torch.long)]
    x = plain_rmsnorm(x, w[tensor_name(cfg, "final_norm")], cfg["eps"])
    head = w[tensor_name(cfg, "embed")] if cfg["tie"] else w[tensor_name(cfg, "head")]
    return x @ head.T


# ---------------------------------------------------------------------------
# the plain sampler (`engine/src/sampling.rs`)
# ---------------------------------------------------------------------------

class PlainRng:
    """xorshift64* (`sampling.rs:55-76`): state = seed | 1."""
    MASK = (1 << 64) - 1

    def __init__(self, seed: int):
        self.s = (seed | 1) & self.MASK

    def next_f32(self) -> float:
        s = self.s
        s ^= s >> 12
        s ^= (s << 25) & self.MASK
        s ^= s >> 27
        self.s = s
        return float(((s * 0x2545F4914F6CDD1D) & self.MASK) >> 40) / float(1 << 24)


def plain_argmax(logits: Sequence[float]) -> int:
    """Highest logit, lowest index on ties, NaN never displaces (`sampling.rs:141-149`)."""
    best = 0
    for i, x in enumerate(logits):
        if x > logits[best]:
            best = i
    return best


def plain_top_k(logits: Sequence[float], k: int):
    """k best in canonical order: logit descending (NaN last), id ascending
    (`sampling.rs:161-163`, `:209-235`); k clamps to [1, V]."""
    k = max(1, min(k, len(logits)))

    def key(item):
        i, v = item
        if v != v:
            return (1, 0.0, i)
        return (0, -v, i)
    return sorted(enumerate(logits), key=key)[:k]


def plain_sample(logits: Sequence[float], temperature: float, top_k: int, rng: PlainRng) -> int:
    """`sampling.rs:243-298`: greedy if temperature <= 0 (no randomness used);
    else weights exp((v - max)/T) as f32, summed and walked in f64."""
    import numpy as np
    if not temperature > 0.0:
        return plain_argmax(logits)
    cands = plain_top_k(logits, top_k)
    best = cands[0][0]
    vmax = -math.inf
    for _, v in cands:
        if v > vmax:
            vmax = v
    t32 = np.float32(temperature)
    weights = []
    total = 0.0
    for _, v in cands:
        with np.errstate(all="ignore"):
            wv = np.exp((np.float32(v) - np.float32(vmax)) / t32, dtype=np.float32)
        wv = float(wv) if np.isfinite(wv) else 0.0
        weights.append(wv)
        total += wv
    if not total > 0.0:
        return best
    threshold = float(np.float32(rng.next_f32())) * total
    acc = 0.0
    for (i, _), wv in zip(cands, weights):
        acc += wv
        if acc >= threshold:
            return i
    return cands[-1][0]


def plain_generate(cfg, w, prompt: Sequence[int], n_new: int, temperature: float = 0.0,
                   top_k: int = 40, seed: int = 1234) -> List[int]:
    """Recomputes the whole sequence for every new token (no cache)."""
    tokens = list(prompt)
    rng = PlainRng(seed)
    out = []
    for _ in range(n_new):
        logits = plain_forward(cfg, w, tokens)[-1].to(torch.float32).tolist()
        tok = plain_sample(logits, temperature, top_k, rng)
        out.append(tok)
        tokens.append(tok)
    return out
