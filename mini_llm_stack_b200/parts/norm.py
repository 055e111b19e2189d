"""Norms: RMS norm with a learned weight, and layer norm with a weight and no bias.

Reference formula (train/model.py:29-33): ``xf = x.float()``;
``y = xf * rsqrt(mean(xf**2, -1) + eps)``; ``out = (y * w.float()).to(x.dtype)``.
eps sits inside the square root, added to the mean; the weight multiplies after
the normalisation; no bias.  All of it runs in float32 with one rounding at the
end.  The residual stream's pending addend is added in the same pass.
"""

from __future__ import annotations

from .base import Norm, ResidualStream, TensorSpec


class RMSNorm(Norm):
    decode_capturable = prompt_capturable = True   # forward only launches kernels on the current stream

    def __init__(self, dim: int, eps: float, tensor_name: str = "weight"):
        """``tensor_name``: the local name of the weight ("" = the part's own prefix)."""
        self.dim = int(dim)
        self.eps = float(eps)
        self.tensor_name = tensor_name
        self.weight = None

    def tensor_specs(self) -> dict:
        return {self.tensor_name: TensorSpec((self.dim,), kind="vector", init="ones")}

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        self.weight = tensors[self.tensor_name].contiguous()

    def forward(self, stream: ResidualStream, rows=None, n_rows: int = 0):
        """Add the pending delta into the stream, return the normalised rows.

        With ``rows`` (int32 row indices) only those rows are read, summed and
        normalised: the output is [n_rows, dim] and the stream itself is left
        as it was.
        """
        rt = self.runtime
        more_rows, more_vec = stream.take_more()
        if more_rows is not None or more_vec is not None:
            # (also before picked rows: the addends go into every row of the stream)
            rt.ops.residual_add(stream.x, more_rows, more_vec)
        delta = stream.take_pending()
        if rows is None:
            t = stream.x.shape[0]
            h = rt.buffer("normed", (t, self.dim), rt.act_dtype)
            rt.ops.add_rmsnorm(stream.x, delta, self.weight, self.eps, h)
        else:
            h = rt.buffer("normed_rows", (n_rows, self.dim), rt.act_dtype)
            rt.ops.gather_add_rmsnorm(stream.x, delta, rows, n_rows, self.weight,
                                      self.eps, h)
        return h


class LayerNorm(Norm):
    """``(x - mean) / sqrt(var + eps) * w`` with the biased variance and no bias, in
    float32 with one rounding.  Adds the stream's pending delta and its other waiting
    addends (``ResidualStream.push_more``) in the same pass.  ``tensor_name`` is the
    local name of the weight ("" = the part's own prefix)."""

    decode_capturable = prompt_capturable = True

    def __init__(self, dim: int, eps: float, tensor_name: str = "weight"):
        self.dim, self.eps, self.tensor_name = int(dim), float(eps), tensor_name
        self.weight = None

    def tensor_specs(self) -> dict:
        return {self.tensor_name: TensorSpec((self.dim,), kind="vector", init="ones")}

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        self.weight = tensors[self.tensor_name].contiguous()
        runtime.ops.require_part("layernorm")

    def forward(self, stream: ResidualStream, rows=None, n_rows: int = 0):
        rt = self.runtime
        more_rows, more_vec = stream.take_more()
        delta = stream.take_pending()
        if rows is None:
            h = rt.buffer("normed", (stream.x.shape[0], self.dim), rt.act_dtype)
        else:
            h = rt.buffer("normed_rows", (n_rows, self.dim), rt.act_dtype)
        rt.ops.add_layernorm(stream.x, delta, self.weight, self.eps, h, rows=rows, n_rows=n_rows,
                             more_rows=more_rows, more_vec=more_vec)
        return h
