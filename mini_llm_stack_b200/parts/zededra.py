"""Zededra: layers of latent attention or mLSTM mixers with dense or routed
feed-forwards, layer norms without bias, a run of layers that may be repeated, and an
output head tied to the embedding.

Tensor names: ``embed``, ``loop.step``, ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``.  A repeated layer keeps one set of
weights and one cache or state slot per pass; before every pass ``PassEntry`` adds the
pass's row of ``loop.step`` (and, from the second pass on, the embedding's output).
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.zededra_config import ZededraConfig
from .block import PreNormBlock
from .feedforward import ClampedGLUFeedForward, RoutedExperts, SwiGLUFeedForward
from .latent_attention import LatentAttention
from .mlstm import MLstmMixer
from .model import ComposedModel, LayerCall, OutputHead, PassEntry, TokenEmbedding
from .norm import LayerNorm


def _mixer(cfg: ZededraConfig, layer: dict):
    m = layer["mixer"]
    if layer["type"] == "latent_attention":
        return LatentAttention(cfg.width, m["heads"], m["dim"], m["vdim"], m["kv_rank"],
                               m["q_rank"], m["scale"], cfg.norm_eps)
    return MLstmMixer(cfg.width, m["heads"], m["dim"], m["vdim"], m["gate_cap"], cfg.norm_eps)


def _feedforward(cfg: ZededraConfig, mlp):
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return ClampedGLUFeedForward(cfg.width, mlp["ff"], mlp["limit"])
    shared = None
    if mlp.get("shared") is not None:
        shared = SwiGLUFeedForward(cfg.width, mlp["shared"]["ff"], names=("gate", "up", "down"))
    return RoutedExperts(cfg.width, mlp["router"]["experts"], mlp["router"]["top"],
                         mlp["expert"]["ff"], shared=shared, weigh="input", renormalise=False)


def build_zededra(cfg: ZededraConfig) -> ComposedModel:
    embedding = TokenEmbedding(cfg.vocab, cfg.width, tensor_name="")
    blocks = []
    for layer in cfg.layers:
        ffn = _feedforward(cfg, layer.get("mlp"))
        blocks.append(PreNormBlock(
            LayerNorm(cfg.width, cfg.norm_eps, tensor_name=""), _mixer(cfg, layer),
            LayerNorm(cfg.width, cfg.norm_eps, tensor_name="") if ffn is not None else None, ffn,
            names=("norm1", "mix", "norm2", "mlp")))
    entries = []
    if cfg.loop is not None:
        entries.append(("loop", PassEntry(cfg.width, cfg.loop["times"], tensor_name="step")))
    calls = []
    for slot, (layer, number, first) in enumerate(cfg.layer_runs()):
        calls.append(LayerCall(layer, slot, True, entry=(0, number) if first else None))
    return ComposedModel(cfg, embedding, blocks, calls,
                         LayerNorm(cfg.width, cfg.norm_eps, tensor_name=""),
                         OutputHead(cfg.vocab, cfg.width, tied_to=embedding),
                         names=("embed", None, "final.norm", None),
                         block_prefix=lambda i: f"l{i}", entries=entries)


register_architecture("Zededra", ZededraConfig, build_zededra, aliases=("zededra",))
