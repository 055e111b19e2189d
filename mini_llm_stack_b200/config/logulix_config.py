"""Typed configuration of the Logulix decoder, read from its config.json.

config.json: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``
(the embedding's rows are multiplied by it), ``logit_scale`` (the logits are), an
optional ``loop`` (``start``, ``stop``, ``times``: layers start .. stop-1 run ``times``
times in a row with the same weights) and ``layers``, a list in which every entry names
its mixer (``type``: ``attention``, ``wkv`` or ``retention``), the mixer's sizes and
constants (``mixer``) and its feed-forward (``mlp``: ``kind`` ``dense``, or null for
none).  Every size and constant of a model comes from there; what a mixer's entry does
not name (a convolution, a cap on the scores, a window, a rotation, a scaling of the
rotation's frequencies) the mixer does not have.  Positions are not bounded by the
design, so a sequence is as long as the engine lets it be (``max_seq_len``, an
engine-side bound that config.json may carry).
"""

from __future__ import annotations

from dataclasses import dataclass, replace

from .model_config import ConfigError, canonical_dtype_name
from .zededra_config import DEFAULT_MAX_SEQ_LEN, _keys, _need, _positive_int


def _positive(v, what):
    _need(isinstance(v, (int, float)) and not isinstance(v, bool) and v > 0,
          f"{what} must be positive, got {v!r}")
    return v


def _check_rot(rot, dim: int, what: str):
    if rot is None:
        return
    _keys(rot, {"base", "dims"}, what, optional={"scaling"})
    _positive(rot["base"], f"{what}.base")
    dims = _positive_int(rot["dims"], f"{what}.dims")
    _need(dims % 2 == 0 and dims <= dim,
          f"{what}.dims ({dims}) must be even and at most the head's size {dim}")
    if rot.get("scaling") is not None:
        _keys(rot["scaling"], {"factor"}, f"{what}.scaling")
        _positive(rot["scaling"]["factor"], f"{what}.scaling.factor")


def _check_attention(m, what):
    _keys(m, {"dim", "heads", "kv_heads", "scale"}, what,
          optional={"vdim", "conv", "mask", "rot", "softcap"})
    for k in ("dim", "heads", "kv_heads"):
        _positive_int(m[k], f"{what}.{k}")
    _need(m["heads"] % m["kv_heads"] == 0,
          f"{what}.heads ({m['heads']}) must be a multiple of kv_heads ({m['kv_heads']})")
    # the values are the keys, so a value is as long as a key
    _need(m.get("vdim", m["dim"]) == m["dim"],
          f"{what}.vdim must equal dim ({m['dim']}): the values are the keys")
    _positive(m["scale"], f"{what}.scale")
    if m.get("conv") is not None:
        _positive_int(m["conv"], f"{what}.conv")
    if m.get("softcap") is not None:
        _positive(m["softcap"], f"{what}.softcap")
    if m.get("mask") is not None:
        _keys(m["mask"], {"size"}, f"{what}.mask")
        _positive_int(m["mask"]["size"], f"{what}.mask.size")
    _check_rot(m.get("rot"), m["dim"], f"{what}.rot")


def _check_wkv(m, what):
    _keys(m, {"dim", "heads"}, what, optional={"rank"})
    _positive_int(m["dim"], f"{what}.dim")
    _positive_int(m["heads"], f"{what}.heads")
    if m.get("rank") is not None:
        _positive_int(m["rank"], f"{what}.rank")


def default_decay_rank(width: int) -> int:
    """Inner size of a wkv mixer's decay when neither config.json (``rank``) nor a weight
    file's shapes say it."""
    return max(4, width // 20)


def _check_retention(m, what):
    _keys(m, {"dim", "heads", "vdim", "decay"}, what, optional={"rot"})
    for k in ("dim", "heads", "vdim"):
        _positive_int(m[k], f"{what}.{k}")
    d = m["decay"]
    _need(isinstance(d, (list, tuple)) and len(d) == m["heads"]
          and all(isinstance(v, (int, float)) and not isinstance(v, bool) for v in d),
          f"{what}.decay must list one number a head ({m['heads']})")
    _check_rot(m.get("rot"), m["dim"], f"{what}.rot")


_MIXERS = {"attention": _check_attention, "wkv": _check_wkv, "retention": _check_retention}


def _check_mlp(mlp, what):
    if mlp is None:
        return
    _need(isinstance(mlp, dict) and "kind" in mlp, f"{what} needs a 'kind'")
    _need(mlp["kind"] == "dense", f"{what}.kind {mlp['kind']!r} is not known (dense)")
    _keys(mlp, {"kind", "ff"}, what)
    _positive_int(mlp["ff"], f"{what}.ff")


@dataclass(frozen=True)
class LogulixConfig:
    architecture: str = "Logulix"
    vocab: int = 256
    width: int = 64
    layers: tuple = ()
    loop: object = None            # None or {"start", "stop", "times"}
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    max_seq_len: int = DEFAULT_MAX_SEQ_LEN
    dtype: str = "bfloat16"

    # what the framework reads
    @property
    def vocab_size(self) -> int:
        return self.vocab

    def __post_init__(self):
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        _positive_int(self.max_seq_len, "max_seq_len")
        _positive(self.norm_eps, "norm.eps")
        _need(isinstance(self.embedding_scale, (int, float)), "embedding.scale must be a number")
        _need(isinstance(self.logit_scale, (int, float)), "logit_scale must be a number")
        canonical_dtype_name(self.dtype)
        _need(len(self.layers) > 0, "layers must name at least one layer")
        for i, layer in enumerate(self.layers):
            what = f"layers[{i}]"
            _keys(layer, {"type", "mixer"}, what, optional={"mlp"})
            _need(layer["type"] in _MIXERS,
                  f"{what}.type {layer['type']!r} is not known ({sorted(_MIXERS)})")
            _need(isinstance(layer["mixer"], dict), f"{what}.mixer must be an object")
            _MIXERS[layer["type"]](layer["mixer"], f"{what}.mixer")
            _check_mlp(layer.get("mlp"), f"{what}.mlp")
        if self.loop is not None:
            _keys(self.loop, {"start", "stop", "times"}, "loop")
            a, b, n = self.loop["start"], self.loop["stop"], self.loop["times"]
            _need(all(isinstance(v, int) and not isinstance(v, bool) for v in (a, b, n)),
                  "loop.start, loop.stop and loop.times must be integers")
            _need(0 <= a < b <= len(self.layers),
                  f"loop {a}..{b} is not a run of the {len(self.layers)} layers")
            _need(n >= 1, "loop.times must be at least 1")

    def layer_runs(self) -> list:
        """``[(layer, number of the pass or None, first layer of its pass)]`` in the
        order in which the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None, False) for i in range(n)]
        a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        runs = [(i, None, False) for i in range(a)]
        for t in range(times):
            runs += [(i, t, i == a) for i in range(a, b)]
        return runs + [(i, None, False) for i in range(b, n)]

    def with_tensor_shapes(self, shapes: dict) -> "LogulixConfig":
        """The sizes config.json leaves to the tensors, read off a weight file's shapes
        (tensor name -> shape): the inner size of a wkv mixer's decay is the first extent
        of ``l<i>.mix.w1`` (config.json may name it as the mixer's ``rank``)."""
        layers = []
        for i, layer in enumerate(self.layers):
            shape = shapes.get(f"l{i}.mix.w1")
            if layer["type"] == "wkv" and layer["mixer"].get("rank") is None and shape:
                layer = dict(layer, mixer=dict(layer["mixer"], rank=int(shape[0])))
            layers.append(layer)
        return replace(self, layers=tuple(layers))

    @classmethod
    def from_dict(cls, raw: dict) -> "LogulixConfig":
        known = {"architecture", "vocab", "width", "layers", "loop", "norm", "embedding",
                 "logit_scale", "max_seq_len", "dtype"}
        unknown = sorted(set(raw) - known)
        _need(not unknown, f"config.json has keys this architecture does not know: {unknown}")
        for req in ("vocab", "width", "layers", "norm"):
            _need(req in raw, f"config.json lacks the required key {req!r}")
        _keys(raw["norm"], {"eps"}, "norm")
        _need(isinstance(raw["layers"], list), "layers must be a list")
        emb = raw.get("embedding")
        if emb is not None:
            _keys(emb, {"scale"}, "embedding")
        return cls(architecture=raw.get("architecture", "Logulix"), vocab=raw["vocab"],
                   width=raw["width"], layers=tuple(raw["layers"]), loop=raw.get("loop"),
                   norm_eps=float(raw["norm"]["eps"]),
                   embedding_scale=float(emb["scale"]) if emb is not None else 1.0,
                   logit_scale=float(raw.get("logit_scale", 1.0)),
                   max_seq_len=raw.get("max_seq_len", DEFAULT_MAX_SEQ_LEN),
                   dtype=canonical_dtype_name(raw.get("dtype", "bfloat16")))

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture,
               "embedding": {"scale": self.embedding_scale},
               "layers": list(self.layers), "logit_scale": self.logit_scale}
        if self.loop is not None:
            out["loop"] = dict(self.loop)
        out.update({"norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width})
        if self.max_seq_len != DEFAULT_MAX_SEQ_LEN:
            out["max_seq_len"] = self.max_seq_len
        if self.dtype != "bfloat16":
            out["dtype"] = self.dtype
        return out


__all__ = ["LogulixConfig", "ConfigError"]
