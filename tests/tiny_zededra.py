"""Tiny Zededra configurations and helpers for the tests.

Sizes are chosen so that nothing the engine could confuse is equal: heads, key and
value sizes differ between layers and between mixers, latent sizes include one that
is not a multiple of the attention kernels' head sizes (40) and the two sizes the
tensor-core kernels take (64, 128), experts are chosen two and three at a time, one
layer has no feed-forward, one mLSTM has more value columns than one CTA owns, and
the repeated run of layers starts after the first layer and runs three times.
"""

import json
from pathlib import Path

import torch
from safetensors.torch import save_file

from mini_llm_stack_b200.config import config_from_dict
from mini_llm_stack_b200.weights import random_tensors


def latent(heads, dim, vdim, kv_rank, q_rank, scale):
    return {"dim": dim, "heads": heads, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
            "vdim": vdim}


def mlstm(heads, dim, vdim, cap):
    return {"dim": dim, "gate_cap": cap, "heads": heads, "vdim": vdim}


def dense(ff, limit):
    return {"ff": ff, "kind": "dense", "limit": limit}


def moe(experts, top, ff, shared=None):
    out = {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": experts, "top": top}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


Z_MIXED = {
    "architecture": "Zededra", "vocab": 97, "width": 48, "norm": {"eps": 1e-5},
    "loop": {"start": 1, "stop": 4, "times": 3},
    "layers": [
        {"type": "latent_attention", "mixer": latent(3, 16, 24, 40, 24, 0.3), "mlp": dense(72, 1.0)},
        {"type": "mlstm", "mixer": mlstm(2, 24, 40, 8.0), "mlp": moe(5, 2, 32, shared=40)},
        {"type": "latent_attention", "mixer": latent(2, 32, 16, 64, 16, 0.2), "mlp": None},
        {"type": "mlstm", "mixer": mlstm(4, 8, 80, 15.0), "mlp": moe(3, 3, 24)},
        {"type": "latent_attention", "mixer": latent(5, 8, 8, 16, 32, 0.4), "mlp": dense(40, 2.5)},
    ],
}

# no repeated run, a width that is no multiple of eight, one expert a token
Z_PLAIN = {
    "architecture": "Zededra", "vocab": 53, "width": 36, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "mlstm", "mixer": mlstm(3, 12, 20, 10.0), "mlp": dense(44, 0.7)},
        {"type": "latent_attention", "mixer": latent(4, 12, 20, 24, 20, 0.25),
         "mlp": moe(4, 1, 28, shared=12)},
    ],
}

# latents of 64 and 128: bfloat16 runs go through the tcgen05 / TMA attention kernels
Z_WIDE = {
    "architecture": "Zededra", "vocab": 131, "width": 128, "norm": {"eps": 1e-6},
    "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [
        {"type": "latent_attention", "mixer": latent(4, 32, 48, 64, 96, 0.18), "mlp": dense(192, 1.5)},
        {"type": "latent_attention", "mixer": latent(7, 16, 16, 128, 64, 0.25),
         "mlp": moe(6, 2, 64, shared=64)},
        {"type": "mlstm", "mixer": mlstm(4, 32, 64, 12.0), "mlp": dense(160, 3.0)},
    ],
}


def one_layer(layer: dict, width: int = 40, vocab: int = 61, eps: float = 1e-5) -> dict:
    """A model of the embedding, one layer, the final norm and the tied head."""
    return {"architecture": "Zededra", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": [layer]}


def make_zededra(folder, raw: dict, seed: int, dtype: str = "bfloat16", std: float = 0.08,
                 norm_std: float = 0.1, patch=None):
    """Write a model folder; returns float64 weights as the file holds them.

    Matrices are drawn with a larger deviation than the engine's default so that every
    mechanism moves the logits; ``patch(weights)`` may change tensors before they are
    stored (in the stored dtype's rounding)."""
    cfg = config_from_dict(dict(raw, dtype=dtype))
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    g = torch.Generator().manual_seed(seed + 1000)
    w = {}
    for name, t in random_tensors(cfg, seed, norm_std, dtype="float32"):
        if t.dim() == 2:
            t = torch.randn(t.shape, generator=g) * std
        elif name.endswith(".b"):
            t = torch.randn(t.shape, generator=g)
        w[name] = t
    if patch:
        patch(w)
    store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    w = {n: t.to(store).contiguous() for n, t in w.items()}
    save_file(w, str(folder / "model.safetensors"))
    (folder / "config.json").write_text(json.dumps(cfg.to_dict(), indent=1))
    return {n: t.double() for n, t in w.items()}
