"""Typed configuration of the Zededra decoder, read from its config.json.

config.json: ``architecture``, ``vocab``, ``width``, ``norm.eps``, an optional ``loop``
(``start``, ``stop``, ``times``: layers start .. stop-1 run ``times`` times in a row with
the same weights) and ``layers``, a list in which every entry names its mixer (``type``:
``latent_attention`` or ``mlstm``), the mixer's sizes and constants (``mixer``) and its
feed-forward (``mlp``: ``kind`` ``dense`` or ``moe``, or null for none).  Every size and
constant of a model comes from there.  The design has no positions, so a sequence is as
long as the engine lets it be (``max_seq_len``, an engine-side bound that config.json
may carry).
"""

from __future__ import annotations

from dataclasses import dataclass

from .model_config import ConfigError, canonical_dtype_name

_MIXER_KEYS = {
    "latent_attention": {"dim", "heads", "kv_rank", "q_rank", "scale", "vdim"},
    "mlstm": {"dim", "gate_cap", "heads", "vdim"},
}
_INT_KEYS = {"dim", "heads", "kv_rank", "q_rank", "vdim"}
DEFAULT_MAX_SEQ_LEN = 1 << 20


def _need(cond, msg):
    if not cond:
        raise ConfigError(msg)


def _positive_int(v, what):
    _need(isinstance(v, int) and not isinstance(v, bool) and v > 0,
          f"{what} must be a positive integer, got {v!r}")
    return v


def _keys(d, want: set, what: str, optional: set = frozenset()):
    _need(isinstance(d, dict), f"{what} must be an object, got {d!r}")
    missing, unknown = want - set(d), set(d) - want - optional
    _need(not missing, f"{what} lacks {sorted(missing)}")
    _need(not unknown, f"{what} has keys this architecture does not know: {sorted(unknown)}")


def _check_mlp(mlp, what):
    if mlp is None:
        return None
    _need(isinstance(mlp, dict) and "kind" in mlp, f"{what} needs a 'kind'")
    if mlp["kind"] == "dense":
        _keys(mlp, {"kind", "ff", "limit"}, what)
        _positive_int(mlp["ff"], f"{what}.ff")
        _need(isinstance(mlp["limit"], (int, float)) and mlp["limit"] > 0,
              f"{what}.limit must be positive")
    elif mlp["kind"] == "moe":
        _keys(mlp, {"kind", "expert", "router"}, what, optional={"shared"})
        _keys(mlp["expert"], {"ff"}, f"{what}.expert")
        _positive_int(mlp["expert"]["ff"], f"{what}.expert.ff")
        _keys(mlp["router"], {"experts", "top"}, f"{what}.router")
        n = _positive_int(mlp["router"]["experts"], f"{what}.router.experts")
        top = _positive_int(mlp["router"]["top"], f"{what}.router.top")
        _need(top <= n, f"{what}.router.top ({top}) exceeds the {n} experts")
        if mlp.get("shared") is not None:
            _keys(mlp["shared"], {"ff"}, f"{what}.shared")
            _positive_int(mlp["shared"]["ff"], f"{what}.shared.ff")
    else:
        raise ConfigError(f"{what}.kind {mlp['kind']!r} is not known (dense, moe)")
    return mlp


@dataclass(frozen=True)
class ZededraConfig:
    architecture: str = "Zededra"
    vocab: int = 256
    width: int = 64
    layers: tuple = ()
    loop: object = None            # None or {"start", "stop", "times"}
    norm_eps: float = 1e-6
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
        _need(self.norm_eps > 0, "norm.eps must be positive")
        canonical_dtype_name(self.dtype)
        _need(len(self.layers) > 0, "layers must name at least one layer")
        for i, layer in enumerate(self.layers):
            what = f"layers[{i}]"
            _keys(layer, {"type", "mixer"}, what, optional={"mlp"})
            _need(layer["type"] in _MIXER_KEYS,
                  f"{what}.type {layer['type']!r} is not known ({sorted(_MIXER_KEYS)})")
            _keys(layer["mixer"], _MIXER_KEYS[layer["type"]], f"{what}.mixer")
            for k, v in layer["mixer"].items():
                if k in _INT_KEYS:
                    _positive_int(v, f"{what}.mixer.{k}")
                else:
                    _need(isinstance(v, (int, float)) and v > 0,
                          f"{what}.mixer.{k} must be positive")
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

    @classmethod
    def from_dict(cls, raw: dict) -> "ZededraConfig":
        known = {"architecture", "vocab", "width", "layers", "loop", "norm", "max_seq_len",
                 "dtype"}
        unknown = sorted(set(raw) - known)
        _need(not unknown, f"config.json has keys this architecture does not know: {unknown}")
        for req in ("vocab", "width", "layers", "norm"):
            _need(req in raw, f"config.json lacks the required key {req!r}")
        _keys(raw["norm"], {"eps"}, "norm")
        _need(isinstance(raw["layers"], list), "layers must be a list")
        return cls(architecture=raw.get("architecture", "Zededra"), vocab=raw["vocab"],
                   width=raw["width"], layers=tuple(raw["layers"]), loop=raw.get("loop"),
                   norm_eps=float(raw["norm"]["eps"]),
                   max_seq_len=raw.get("max_seq_len", DEFAULT_MAX_SEQ_LEN),
                   dtype=canonical_dtype_name(raw.get("dtype", "bfloat16")))

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "layers": list(self.layers)}
        if self.loop is not None:
            out["loop"] = dict(self.loop)
        out.update({"norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width})
        if self.max_seq_len != DEFAULT_MAX_SEQ_LEN:
            out["max_seq_len"] = self.max_seq_len
        if self.dtype != "bfloat16":
            out["dtype"] = self.dtype
        return out
