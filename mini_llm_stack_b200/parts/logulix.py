"""Logulix: layers of wkv, retention or convolved-key attention mixers, some with an
ungated feed-forward, RMS norms, a scaled embedding, a run of layers that may be repeated
behind a projection of [stream; embedding], and an untied, scaled output head.

Tensor names: ``embed``, ``loop.in``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``final.norm``, ``head``.  A repeated layer keeps one set of weights and one
cache or state slot per pass; before every pass ``PassProjection`` rewrites the stream.
"""

from __future__ import annotations

from ..config.logulix_config import LogulixConfig, default_decay_rank
from ..config.registry import register_architecture
from .block import PreNormBlock
from .conv_attention import ConvKeyAttention
from .feedforward import SquaredReluFeedForward
from .linear_recurrence import RetentionMixer, WkvMixer
from .model import ComposedModel, LayerCall, OutputHead, PassProjection, TokenEmbedding
from .norm import RMSNorm
from .position import PartialRotary


def _rotary(rot, pairing: str):
    if rot is None:
        return None
    factor = (rot.get("scaling") or {}).get("factor", 1.0)
    return PartialRotary(rot["dims"], rot["base"], factor, pairing)


def _mixer(cfg: LogulixConfig, layer: dict):
    m, kind = layer["mixer"], layer["type"]
    if kind == "attention":
        return ConvKeyAttention(cfg.width, m["heads"], m["kv_heads"], m["dim"], m["scale"],
                                cfg.norm_eps, position=_rotary(m.get("rot"), "interleaved"),
                                taps=m.get("conv") or 0, softcap=m.get("softcap") or 0.0,
                                window=(m.get("mask") or {}).get("size"))
    if kind == "wkv":
        return WkvMixer(cfg.width, m["heads"], m["dim"],
                        m.get("rank") or default_decay_rank(cfg.width), cfg.norm_eps)
    return RetentionMixer(cfg.width, m["heads"], m["dim"], m["vdim"], m["decay"], cfg.norm_eps,
                          position=_rotary(m.get("rot"), "half"))


def build_logulix(cfg: LogulixConfig) -> ComposedModel:
    embedding = TokenEmbedding(cfg.vocab, cfg.width, tensor_name="", scale=cfg.embedding_scale)
    blocks = []
    for layer in cfg.layers:
        mlp = layer.get("mlp")
        ffn = SquaredReluFeedForward(cfg.width, mlp["ff"]) if mlp is not None else None
        blocks.append(PreNormBlock(
            RMSNorm(cfg.width, cfg.norm_eps, tensor_name=""), _mixer(cfg, layer),
            RMSNorm(cfg.width, cfg.norm_eps, tensor_name="") if ffn is not None else None, ffn,
            names=("norm1", "mix", "norm2", "mlp")))
    entries = []
    if cfg.loop is not None:
        entries.append(("loop", PassProjection(cfg.width, tensor_name="in")))
    calls = []
    for slot, (layer, number, first) in enumerate(cfg.layer_runs()):
        calls.append(LayerCall(layer, slot, True, entry=(0, number) if first else None))
    return ComposedModel(cfg, embedding, blocks, calls,
                         RMSNorm(cfg.width, cfg.norm_eps, tensor_name=""),
                         OutputHead(cfg.vocab, cfg.width, tied_to=None, tensor_name="",
                                    scale=cfg.logit_scale),
                         names=("embed", None, "final.norm", "head"),
                         block_prefix=lambda i: f"l{i}", entries=entries)


register_architecture("Logulix", LogulixConfig, build_logulix, aliases=("logulix",))
