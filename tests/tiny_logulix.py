"""Tiny Logulix configurations and helpers for the tests.

Sizes are chosen so that nothing the engine could confuse is equal: heads, key and value
sizes differ between layers and mixers; key heads are fewer than, or as many as, query
heads; convolutions have two, three and four taps or none; windows are shorter than a
page, between pages, longer than the prompts, or absent; rotations cover a part of a head
or all of it, with and without scaled frequencies; the repeated run of layers starts after
the first layer or at it, runs two or three times, and a model has none; an attention
layer without a feed-forward is the last layer of one model.
"""

import json
from pathlib import Path

import torch
from safetensors.torch import save_file

from mini_llm_stack_b200.config import config_from_dict
from mini_llm_stack_b200.weights import random_tensors


def attention(heads, kv, dim, scale, conv=None, window=None, rot=None, softcap=None):
    m = {"dim": dim, "heads": heads, "kv_heads": kv, "scale": scale, "vdim": dim}
    if conv is not None:
        m["conv"] = conv
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = rot
    if softcap is not None:
        m["softcap"] = softcap
    return m


def rot(dims, base, factor=None):
    out = {"base": base, "dims": dims}
    if factor is not None:
        out["scaling"] = {"factor": factor}
    return out


def wkv(heads, dim, rank):
    return {"dim": dim, "heads": heads, "rank": rank}


def retention(heads, dim, vdim, decay, rot=None):
    m = {"decay": decay, "dim": dim, "heads": heads, "vdim": vdim}
    if rot is not None:
        m["rot"] = rot
    return m


def dense(ff):
    return {"ff": ff, "kind": "dense"}


L_MIXED = {
    "architecture": "Logulix", "vocab": 97, "width": 48, "norm": {"eps": 1e-5},
    "embedding": {"scale": 0.7}, "logit_scale": 1.3,
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        {"type": "attention", "mlp": dense(72),
         "mixer": attention(4, 2, 16, 0.3, conv=2, window=21, rot=rot(8, 500.0, 2.0), softcap=5.0)},
        {"type": "wkv", "mixer": wkv(3, 16, 5), "mlp": None},
        {"type": "retention", "mlp": dense(40),
         "mixer": retention(2, 24, 40, [0.9, 0.97], rot=rot(12, 1000.0))},
        {"type": "attention", "mlp": None,
         "mixer": attention(2, 1, 32, 0.2, conv=4, window=7)},
    ],
}

# no repeated run, no scales, a width that is no multiple of eight, full causal attention
L_PLAIN = {
    "architecture": "Logulix", "vocab": 53, "width": 36, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "wkv", "mixer": wkv(2, 20, 4), "mlp": dense(44)},
        {"type": "retention", "mixer": retention(3, 8, 24, [0.5, 0.99, 0.8]), "mlp": None},
        {"type": "attention", "mlp": dense(28),
         "mixer": attention(3, 3, 12, 0.25, rot=rot(12, 10000.0), softcap=8.0)},
    ],
}

# heads of 64 and 128: bfloat16 runs go through the tensor-core attention kernels where
# they take the options; the whole model is the repeated run
L_WIDE = {
    "architecture": "Logulix", "vocab": 131, "width": 128, "norm": {"eps": 1e-6},
    "embedding": {"scale": 1.5}, "logit_scale": 0.5,
    "loop": {"start": 0, "stop": 3, "times": 2},
    "layers": [
        {"type": "attention", "mlp": dense(192),
         "mixer": attention(4, 2, 64, 0.125, conv=3, window=70, rot=rot(64, 10000.0, 4.0),
                            softcap=20.0)},
        {"type": "wkv", "mixer": wkv(2, 64, 8), "mlp": None},
        {"type": "retention", "mlp": dense(160),
         "mixer": retention(2, 64, 128, [0.96875, 0.998], rot=rot(32, 1e6))},
    ],
}

# nothing is paged: only states of fixed size
L_STATES = {
    "architecture": "Logulix", "vocab": 61, "width": 40, "norm": {"eps": 1e-5},
    "logit_scale": 2.0, "loop": {"start": 0, "stop": 1, "times": 2},
    "layers": [
        {"type": "retention", "mixer": retention(2, 10, 6, [0.999, 0.9], rot=rot(10, 100.0)),
         "mlp": None},
        {"type": "wkv", "mixer": wkv(5, 8, 3), "mlp": dense(24)},
    ],
}


# an attention layer without a feed-forward right before the repeated run (its output bias
# still waits on the stream when the pass begins), one pass only, retention after the run
L_EDGE = {
    "architecture": "Logulix", "vocab": 71, "width": 32, "norm": {"eps": 1e-6},
    "embedding": {"scale": 2.0}, "loop": {"start": 1, "stop": 2, "times": 1},
    "layers": [
        {"type": "attention", "mlp": None,
         "mixer": attention(2, 2, 8, 0.35, conv=3, window=5, rot=rot(8, 40.0), softcap=4.0)},
        {"type": "wkv", "mixer": wkv(2, 16, 3), "mlp": None},
        {"type": "retention", "mixer": retention(4, 4, 12, [0.7, 0.8, 0.9, 0.95]), "mlp": dense(48)},
    ],
}


def one_layer(layer: dict, width: int = 40, vocab: int = 61, eps: float = 1e-5) -> dict:
    """A model of the embedding, one layer, the final norm and the head."""
    return {"architecture": "Logulix", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": [layer]}


def make_logulix(folder, raw: dict, seed: int, dtype: str = "bfloat16", std: float = 0.08,
                 norm_std: float = 0.1, patch=None):
    """Write a model folder; returns float64 weights as the file holds them.

    Matrices are drawn with a larger deviation than the engine's default so that every
    mechanism moves the logits; biases, mixing weights, bonuses and convolution taps get
    values of their own kind; ``patch(weights)`` may change tensors before they are stored
    (in the stored dtype's rounding)."""
    cfg = config_from_dict(dict(raw, dtype=dtype))
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    g = torch.Generator().manual_seed(seed + 1000)
    w = {}
    for name, t in random_tensors(cfg, seed, norm_std, dtype="float32"):
        if ".mu." in name:
            t = torch.rand(t.shape, generator=g)
        elif name.endswith(".conv"):
            t = torch.randn(t.shape, generator=g) * 0.6
        elif name.endswith(".w0"):
            t = torch.randn(t.shape, generator=g) * 0.5 - 1.0
        elif name.endswith(".mix.u") or name.endswith(".b"):
            t = torch.randn(t.shape, generator=g) * 0.5
        elif name.endswith(".w1") or name.endswith(".w2"):
            t = torch.randn(t.shape, generator=g) * 0.3
        elif t.dim() == 2:
            t = torch.randn(t.shape, generator=g) * std
        w[name] = t
    if patch:
        patch(w)
    store = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    w = {n: t.to(store).contiguous() for n, t in w.items()}
    save_file(w, str(folder / "model.safetensors"))
    (folder / "config.json").write_text(json.dumps(cfg.to_dict(), indent=1))
    return {n: t.double() for n, t in w.items()}
