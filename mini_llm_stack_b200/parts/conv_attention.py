"""Grouped-query attention whose values are its keys, behind a short convolution.

With d = model width, H query heads and G key heads of size e (query head h reads key
head ``h // (H/G)``), per token:

    q = W_q h + b_q,  k = W_k h + b_k                    (float32 out of the product)
    q, k <- causal convolution over time on every channel (``taps`` taps, no bias)
    v = k                                                 (as the convolution leaves it)
    q <- rms_norm(q over all H*e entries) * g_q,  k likewise over its G*e entries
    q, k <- rotation of the first ``dims`` entries of every head (``PartialRotary``)
    score = (q . k) * scale;  score <- cap * tanh(score / cap)
    softmax over the keys j with 0 <= i - j < window;  out = W_o concat_h(P v) + b_o

Every option may be absent: no convolution (``taps`` 0), no cap, no window, no rotation.
The rotated keys and the values live in the paged cache (``PagedKV`` with the window),
the convolution's last ``taps - 1`` inputs of every request in its state slot
(``FixedState``): the mixer's cache is a ``PagedWithState``.
"""

from __future__ import annotations

import torch

from .attention import plan_paged_attention
from .base import (CacheHandle, FixedState, Mixer, PagedKV, PagedWithState, StepContext,
                   TensorSpec)


class ConvKeyAttention(Mixer):
    decode_capturable = prompt_capturable = True   # forward only launches kernels on the current stream

    def __init__(self, d_model: int, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                 eps: float, position=None, taps: int = 0, softcap: float = 0.0, window=None):
        if n_heads % n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        self.d_model, self.n_heads, self.n_kv_heads = int(d_model), int(n_heads), int(n_kv_heads)
        self.head_dim, self.scale, self.eps = int(head_dim), float(scale), float(eps)
        self.position, self.taps = position, int(taps)
        self.softcap, self.window = float(softcap or 0.0), window
        if position is not None and position.pairing != "interleaved":
            raise ValueError("this mixer's kernel rotates neighbouring entries")
        self.channels = (self.n_heads + self.n_kv_heads) * self.head_dim

    def tensor_specs(self) -> dict:
        d, cq, ck = self.d_model, self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        out = {
            "q": TensorSpec((cq, d)), "q.b": TensorSpec((cq,), kind="vector", init="zeros"),
            "k": TensorSpec((ck, d)), "k.b": TensorSpec((ck,), kind="vector", init="zeros"),
            "q.norm": TensorSpec((cq,), kind="vector", init="ones"),
            "k.norm": TensorSpec((ck,), kind="vector", init="ones"),
            "o": TensorSpec((d, cq)), "o.b": TensorSpec((d,), kind="vector", init="zeros"),
        }
        if self.taps:
            out["q.conv"] = TensorSpec((cq, self.taps))
            out["k.conv"] = TensorSpec((ck, self.taps))
        return out

    def cache_spec(self):
        paged = PagedKV(self.n_kv_heads, self.head_dim, self.window)
        if self.taps > 1:
            return PagedWithState(paged, FixedState(((self.taps - 1) * self.channels,),
                                                    torch.float32))
        return paged

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        ops = runtime.ops
        # one projection for q and k: rows [q heads | k heads]
        self.w_qk = ops.prepare_weight(torch.cat([tensors["q"], tensors["k"]], dim=0))
        self.b_qk = torch.cat([tensors["q.b"], tensors["k.b"]]).contiguous()
        self.conv = (torch.cat([tensors["q.conv"], tensors["k.conv"]], dim=0).contiguous()
                     if self.taps else None)
        self.g_q, self.g_k = tensors["q.norm"].contiguous(), tensors["k.norm"].contiguous()
        self.w_o = ops.prepare_weight(tensors["o"])
        self.b_o = tensors["o.b"].contiguous()
        if self.position is not None:
            self.position.bind({}, runtime)
        ops.require_part("shortconv")
        ops.require_part("layernorm")
        if ops.attention_tensor_cores(self.head_dim):
            ops.require_attention(self.head_dim, self.n_heads, self.n_kv_heads)
        self._facts = ops.attention_facts(self.head_dim)

    def plan(self, step: StepContext):
        return plan_paged_attention(step, self._facts, self.n_heads, self.n_kv_heads,
                                    self.head_dim)

    def decode_graph_key(self, step: StepContext) -> tuple:
        plan = self.plan(step)
        if plan is None:
            return ()
        return ("gqa", self.n_kv_heads, self.n_heads // self.n_kv_heads, self.head_dim,
                plan.n_split)

    def forward(self, h, step: StepContext, cache: CacheHandle):
        rt, ops = self.runtime, self.runtime.ops
        t, hd = step.n_tokens, self.head_dim
        proj = rt.buffer("qk_proj", (t, self.channels), torch.float32)
        # a step of one token a request: the product may stay in the parts it was cut into
        # along K (the kernel below adds them up), and that kernel moves the tail on itself
        single = step.max_q_len == 1
        src = ops.linear_parts(h, self.w_qk, proj) if single else None
        if src is None:
            ops.linear(h, self.w_qk, proj)
        # the attention kernels read a row of [q heads | k heads | v heads]; only q is there
        q_row = rt.buffer("qkv", (t, (self.n_heads + 2 * self.n_kv_heads) * hd), rt.act_dtype)
        pos = self.position
        ops.qk_conv_norm_rope_store(proj, self.b_qk, self.conv, self.taps, self.g_q, self.g_k,
                                    self.eps, cache.state, pos.freq if pos else None,
                                    pos.dims if pos else 0, q_row, cache, step, self.n_heads,
                                    self.n_kv_heads, hd,
                                    parts=src if (src is not None and src is not proj) else None,
                                    move_tail=single and cache.writes)
        if self.taps > 1 and cache.writes and not single:
            ops.tail_update(proj, 0, self.channels, self.b_qk, cache.state, self.taps - 1, step)
        o = rt.buffer("attn_out", (t, self.n_heads * hd), rt.act_dtype)
        ops.paged_attention(q_row, o, cache, step, self.n_heads, self.n_kv_heads, hd, self.scale,
                            self.window or 0, plan=self.plan(step), softcap=self.softcap)
        # the output bias goes to the stream beside the product (which may stay in its K-parts)
        delta = rt.buffer("delta_f32", (t, self.d_model), torch.float32)
        return ops.linear_parts(o, self.w_o, delta), self.b_o
