"""mLSTM mixer: a matrix memory per head with exponential gates and a stabiliser.

With H heads of query/key size e and value size f, per head and token (all of it
float32 but the projections):

    q = W_q h * e^-1/2,  k = W_k h,  v = W_v h
    i = cap * tanh((W_i h + b_i) / cap)                      log input gate
    g = logsigmoid(cap * tanh((W_f h + b_f) / cap))          log forget gate
    m' = max(g + m, i)                    m starts at 0
    C' = exp(g + m - m') C + exp(i - m') k v^T,   n' likewise with k alone
    o = C'^T q / (max(|n' . q|, exp(-m')) + 1e-6)
    out = W_o (unit_rms_per_head(o) * w_norm * sigmoid(W_g h))

C, n and m live in the request's state slot (``FixedState``, float32, zero when the
slot is claimed) and are carried from token to token and from step to step.  The
gate projections run as a true float32 product.
"""

from __future__ import annotations

import torch

from .base import CacheHandle, FixedState, Mixer, StepContext, TensorSpec


def state_columns(e: int, f: int, threads: int = 256, most_rows: int = 64) -> int:
    """Columns of a head's memory one CTA of the scan kernel owns (the kernel's own rule,
    restated so that the state's size is known without a device): at most 16, at most f,
    halved until a thread holds at most ``most_rows`` of the e rows."""
    fc = min(f, 16)
    while fc > 1 and -(-e // (threads // fc)) > most_rows:
        fc = (fc + 1) // 2
    return fc


class MLstmMixer(Mixer):
    decode_capturable = prompt_capturable = True   # forward only launches kernels on the current stream

    def __init__(self, d_model: int, n_heads: int, qk_dim: int, v_dim: int, gate_cap: float,
                 eps: float):
        self.d_model, self.n_heads = int(d_model), int(n_heads)
        self.qk_dim, self.v_dim = int(qk_dim), int(v_dim)
        self.gate_cap, self.eps = float(gate_cap), float(eps)

    def tensor_specs(self) -> dict:
        d, h, e, f = self.d_model, self.n_heads, self.qk_dim, self.v_dim
        return {
            "q": TensorSpec((h * e, d)),
            "k": TensorSpec((h * e, d)),
            "v": TensorSpec((h * f, d)),
            "g": TensorSpec((h * f, d)),
            "o": TensorSpec((d, h * f)),
            "norm": TensorSpec((h * f,), kind="vector", init="ones"),
            "i": TensorSpec((h, d)),
            "i.b": TensorSpec((h,), kind="vector", init="zeros"),
            "f": TensorSpec((h, d)),
            "f.b": TensorSpec((h,), kind="vector", init="zeros"),
        }

    def state_width(self) -> int:
        """Floats of one head's state: C [e, f], n [e] and one m per column group."""
        e, f = self.qk_dim, self.v_dim
        fc = state_columns(e, f)
        return e * f + e + -(-f // fc)

    def cache_spec(self):
        return FixedState((self.n_heads, self.state_width()), torch.float32)

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        ops = runtime.ops
        ops.require_part("mlstm")
        if ops.mlstm_state_width(self.qk_dim, self.v_dim) != self.state_width():
            raise RuntimeError("the scan kernel lays the mLSTM state out differently")
        self.w_qkvg = ops.prepare_weight(torch.cat(
            [tensors["q"], tensors["k"], tensors["v"], tensors["g"]], dim=0))
        self.w_gates = torch.cat([tensors["i"], tensors["f"]], dim=0).float().contiguous()
        self.b_i, self.b_f = tensors["i.b"].contiguous(), tensors["f.b"].contiguous()
        self.w_norm = tensors["norm"].contiguous()
        self.w_o = ops.prepare_weight(tensors["o"])

    def decode_graph_key(self, step: StepContext) -> tuple:
        return ("mlstm", self.n_heads, self.qk_dim, self.v_dim)

    def forward(self, h, step: StepContext, cache: CacheHandle):
        rt, ops = self.runtime, self.runtime.ops
        t = step.n_tokens
        nh, e, f = self.n_heads, self.qk_dim, self.v_dim
        qkvg = rt.buffer("mlstm_qkvg", (t, 2 * nh * e + 2 * nh * f), rt.act_dtype)
        ops.linear(h, self.w_qkvg, qkvg)
        gates = rt.buffer("mlstm_gates", (t, 2 * nh), torch.float32)
        ops.linear(h, self.w_gates, gates)
        num = rt.buffer("mlstm_num", (t, nh * f), torch.float32)
        den = rt.buffer("mlstm_den", (t, nh), torch.float32)
        ops.mlstm_scan(qkvg, (0, nh * e, 2 * nh * e), gates, self.b_i, self.b_f, self.gate_cap,
                       step, cache.state, nh, e, f, num, den)
        o = rt.buffer("attn_out", (t, nh * f), rt.act_dtype)
        ops.mlstm_finish(num, den, qkvg, 2 * nh * e + nh * f, self.w_norm, self.eps, o, nh, f)
        delta = rt.buffer("delta", (t, self.d_model), rt.act_dtype)
        return ops.linear_parts(o, self.w_o, delta)
