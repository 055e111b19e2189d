"""Causal attention whose keys and values are read off one cached latent a token.

With d = model width, H heads of query/key size e and value size f, a latent of
size r and a query latent of size rq (all float32 norms, eps inside the root):

    cq = unit_rms(W_dq h) * g_q            q_h = W_uq[h] cq
    c  = unit_rms(W_dkv h) * g_kv          k_h = W_uk[h] c,  v_h = W_uv[h] c
    score_ij = (q_hi . k_hj) * scale,  j <= i;  softmax;  out = W_o concat_h(sum_j p_ij v_hj)

No position enters.  Only c is cached, and neither keys nor values are ever rebuilt:
``q . (W_uk c) = (W_uk^T q) . c`` and ``sum_j p_j W_uv c_j = W_uv sum_j p_j c_j``, so the
query is taken into the latent space, the framework's paged attention kernels run
as multi-query attention with the latent pool as the one key and value head
(``PagedKV(1, r', shared_kv=True)``, r' = r rounded up to the kernels' head sizes,
the padding zero), and the result is taken out of the latent space again.
"""

from __future__ import annotations

import torch

from .attention import plan_paged_attention
from .base import CacheHandle, Mixer, PagedKV, StepContext, TensorSpec


class LatentAttention(Mixer):
    decode_capturable = prompt_capturable = True   # forward only launches kernels on the current stream

    PAD = 16          # the attention kernels take head sizes in steps of 16

    def __init__(self, d_model: int, n_heads: int, qk_dim: int, v_dim: int, kv_rank: int,
                 q_rank: int, scale: float, eps: float):
        self.d_model, self.n_heads = int(d_model), int(n_heads)
        self.qk_dim, self.v_dim = int(qk_dim), int(v_dim)
        self.kv_rank, self.q_rank = int(kv_rank), int(q_rank)
        self.scale, self.eps = float(scale), float(eps)
        self.pool_rank = max(self.PAD, -(-self.kv_rank // self.PAD) * self.PAD)

    def tensor_specs(self) -> dict:
        d, h = self.d_model, self.n_heads
        return {
            "dq": TensorSpec((self.q_rank, d)),
            "dq.norm": TensorSpec((self.q_rank,), kind="vector", init="ones"),
            "uq": TensorSpec((h * self.qk_dim, self.q_rank)),
            "dkv": TensorSpec((self.kv_rank, d)),
            "dkv.norm": TensorSpec((self.kv_rank,), kind="vector", init="ones"),
            "uk": TensorSpec((h * self.qk_dim, self.kv_rank)),
            "uv": TensorSpec((h * self.v_dim, self.kv_rank)),
            "o": TensorSpec((d, h * self.v_dim)),
        }

    def cache_spec(self):
        return PagedKV(1, self.pool_rank, None, shared_kv=True)

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        ops = runtime.ops
        h, e, f, r, rp = self.n_heads, self.qk_dim, self.v_dim, self.kv_rank, self.pool_rank
        self.w_down = ops.prepare_weight(torch.cat([tensors["dq"], tensors["dkv"]], dim=0))
        self.g_q = tensors["dq.norm"].contiguous()
        self.g_kv = tensors["dkv.norm"].contiguous()
        self.w_uq = ops.prepare_weight(tensors["uq"])
        uk = tensors["uk"].view(h, e, r)
        uv = tensors["uv"].view(h, f, r)
        # W_uk[h]^T as [H, r', e] and W_uv[h] as [H, f, r'], zero where the latent is padded
        self.w_into = torch.zeros((h, rp, e), dtype=uk.dtype, device=uk.device)
        self.w_into[:, :r] = uk.transpose(1, 2)
        self.w_out_of = torch.zeros((h, f, rp), dtype=uv.dtype, device=uv.device)
        self.w_out_of[:, :, :r] = uv
        self.w_o = ops.prepare_weight(tensors["o"])
        ops.require_part("latent")
        ops.require_attention(rp, h, 1)
        self._facts = ops.attention_facts(rp)

    def plan(self, step: StepContext):
        return plan_paged_attention(step, self._facts, self.n_heads, 1, self.pool_rank)

    def decode_graph_key(self, step: StepContext) -> tuple:
        plan = self.plan(step)
        if plan is None:
            return ()
        return ("latent", self.n_heads, self.pool_rank, plan.n_split)

    def forward(self, h, step: StepContext, cache: CacheHandle):
        rt, ops = self.runtime, self.runtime.ops
        t = step.n_tokens
        nh, e, f, rp = self.n_heads, self.qk_dim, self.v_dim, self.pool_rank
        down = rt.buffer("latent_down", (t, self.q_rank + self.kv_rank), torch.float32)
        ops.linear(h, self.w_down, down)
        cq = rt.buffer("latent_cq", (t, self.q_rank), rt.act_dtype)
        ops.latent_norm_store(down, self.q_rank, self.kv_rank, self.g_q, self.g_kv, self.eps,
                              cq, cache, step)
        q = rt.buffer("latent_q", (t, nh * e), rt.act_dtype)
        ops.linear(cq, self.w_uq, q)
        # the kernels read a row of [q heads | k heads | v heads]; only the q heads are there
        q_in = rt.buffer("latent_q_in", (t, (nh + 2) * rp), rt.act_dtype)
        ops.headwise_linear(q, e, self.w_into, q_in, rp, t)
        o_in = rt.buffer("latent_o_in", (t, nh * rp), rt.act_dtype)
        ops.paged_attention(q_in, o_in, cache, step, nh, 1, rp, self.scale, 0,
                            plan=self.plan(step))
        o = rt.buffer("attn_out", (t, nh * f), rt.act_dtype)
        ops.headwise_linear(o_in, rp, self.w_out_of, o, f, t)
        delta = rt.buffer("delta", (t, self.d_model), rt.act_dtype)
        return ops.linear_parts(o, self.w_o, delta)
