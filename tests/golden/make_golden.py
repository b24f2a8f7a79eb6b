"""Pins the plain implementation (tests/plain_model.py) to the reference's own model.

Run once, by hand, where the reference checkout is present:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's `model.py` (PyTorch, CPU, float32), builds two tiny
models that differ in every size and option, and patches from the outside what
the reference fixes in code: the SwiGLU width (`model.py:228-229` derives it),
the RMSNorm epsilon (`model.py:108`), and the tied head (`model.py:289`).  It
lets the reference initialise its own weights, rounds them to bfloat16 so the
stored file is exact, and writes for each model a folder with config.json,
model.safetensors (reference tensor names), tokens.json and logits.npy: the
reference's float32 logits at every position.  tests/test_plain_model.py reads
these folders and compares; it does not import the reference.
"""
import json
import os
import sys

import numpy as np
import torch

CASES = {
    # name: (vocab, layers, heads, kv_heads, width, inter, ctx, theta, eps, tied, attention)
    "golden_a": dict(vocab=64, layers=2, heads=4, kv_heads=2, width=32, inter=48, ctx=32,
                     theta=10000.0, eps=1e-5, tied=True, attention="gqa", seed=11, n_tokens=24),
    "golden_b": dict(vocab=77, layers=3, heads=3, kv_heads=1, width=48, inter=80, ctx=40,
                     theta=500000.0, eps=1e-6, tied=False, attention="mqa", seed=12, n_tokens=29),
}


def main(reference_dir: str) -> None:
    sys.path.insert(0, reference_dir)
    from model import GPT, GPTConfig           # the reference's own code
    from safetensors.torch import save_file
    here = os.path.dirname(os.path.abspath(__file__))
    for name, c in CASES.items():
        torch.manual_seed(c["seed"])
        cfg = GPTConfig(vocab_size=c["vocab"], n_layer=c["layers"], n_head=c["heads"],
                        n_kv_head=c["kv_heads"], n_embd=c["width"], block_size=c["ctx"],
                        attention=c["attention"], rope_theta=c["theta"])
        model = GPT(cfg)
        for block in model.blocks:
            block.mlp.gate_proj = torch.nn.Linear(c["width"], c["inter"], bias=False)
            block.mlp.up_proj = torch.nn.Linear(c["width"], c["inter"], bias=False)
            block.mlp.down_proj = torch.nn.Linear(c["inter"], c["width"], bias=False)
            for lin in (block.mlp.gate_proj, block.mlp.up_proj, block.mlp.down_proj):
                torch.nn.init.normal_(lin.weight, mean=0.0, std=0.05)
            block.attn_norm.eps = c["eps"]
            block.mlp_norm.eps = c["eps"]
        model.final_norm.eps = c["eps"]
        if not c["tied"]:
            model.lm_head = torch.nn.Linear(c["width"], c["vocab"], bias=False)
            torch.nn.init.normal_(model.lm_head.weight, mean=0.0, std=0.05)
        with torch.no_grad():
            for p_name, p in model.named_parameters():
                if p_name.endswith("norm.weight"):
                    p.copy_(1.0 + 0.1 * torch.randn_like(p))     # gains that are not all 1
                else:
                    p.mul_(2.5)                                   # larger logits: stricter test
                p.copy_(p.to(torch.bfloat16).to(torch.float32))   # exact in bfloat16
        model.eval()
        tokens = torch.randint(0, c["vocab"], (c["n_tokens"],),
                               generator=torch.Generator().manual_seed(c["seed"] + 100))
        with torch.no_grad():
            logits, _ = model(tokens.view(1, -1), targets=tokens.view(1, -1))
        out = os.path.join(here, name)
        os.makedirs(out, exist_ok=True)
        state = {k: v.detach().to(torch.bfloat16).contiguous().clone()
                 for k, v in model.state_dict().items()
                 if not (c["tied"] and k == "lm_head.weight")}
        save_file(state, os.path.join(out, "model.safetensors"))
        config = {"vocab_size": c["vocab"], "n_layer": c["layers"], "n_head": c["heads"],
                  "n_kv_head": c["kv_heads"], "n_embd": c["width"], "block_size": c["ctx"],
                  "dropout": 0.0, "bias": False, "attention": c["attention"],
                  "pos_encoding": "rope", "activation": "swiglu", "norm": "rmsnorm",
                  "norm_placement": "pre", "rope_theta": c["theta"],
                  "head_dim": c["width"] // c["heads"], "intermediate_size": c["inter"],
                  "rms_norm_eps": c["eps"], "tie_word_embeddings": c["tied"],
                  "dtype": "bfloat16"}
        with open(os.path.join(out, "config.json"), "w") as f:
            json.dump(config, f, indent=2)
        with open(os.path.join(out, "tokens.json"), "w") as f:
            json.dump(tokens.tolist(), f)
        np.save(os.path.join(out, "logits.npy"), logits[0].to(torch.float32).numpy())
        print(name, "logits", tuple(logits[0].shape), "max |logit|",
              float(logits.abs().max()))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <checkout of the reference>")
    main(sys.argv[1])
