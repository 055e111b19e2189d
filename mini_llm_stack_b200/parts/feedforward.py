"""Feed-forwards: dense SwiGLU, a clamped gated unit, an ungated unit with the square of
relu, and routed experts.

Reference (train/model.py:127-135): ``w_down(silu(w_gate x) * (w_up x))`` with
``silu(z) = z * sigmoid(z)``, no biases.  Gate and up share one projection
here; ``silu(gate) * up`` is computed in float32, in the projection's own
epilogue where the tcgen05 kernel takes the sizes.
"""

from __future__ import annotations

import torch

from .base import FeedForward, StepContext, TensorSpec


class SwiGLUFeedForward(FeedForward):
    decode_capturable = prompt_capturable = True   # forward only launches kernels on the current stream

    def __init__(self, d_model: int, intermediate_size: int,
                 names=("w_gate.weight", "w_up.weight", "w_down.weight")):
        self.d_model, self.intermediate_size = int(d_model), int(intermediate_size)
        self.names = tuple(names)             # local names of the gate, up and down matrices
        self.w_gate_up = self.w_down = None

    def tensor_specs(self) -> dict:
        d, i = self.d_model, self.intermediate_size
        g, u, dn = self.names
        return {g: TensorSpec((i, d)), u: TensorSpec((i, d)), dn: TensorSpec((d, i))}

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        tensors = {"w_gate.weight": tensors[self.names[0]], "w_up.weight": tensors[self.names[1]],
                   "w_down.weight": tensors[self.names[2]]}
        parts = [tensors["w_gate.weight"], tensors["w_up.weight"]]
        if parts[0].dtype != parts[1].dtype:
            parts = [p.float() for p in parts]
        ops = runtime.ops
        # one kernel for projection and activation where the tensor-core kernel takes
        # the sizes: its weight holds gate and up rows interleaved in blocks of 16
        self.fused = (parts[0].dtype == torch.bfloat16
                      and ops.can_fuse_swiglu(self.d_model, self.intermediate_size))
        if self.fused:
            self.w_gate_up = ops.prepare_weight(ops.interleave_gate_up(parts[0], parts[1]))
        else:
            self.w_gate_up = ops.prepare_weight(torch.cat(parts, dim=0))
        self.w_down = ops.prepare_weight(tensors["w_down.weight"])

    def forward(self, h, step: StepContext):
        rt = self.runtime
        t = h.shape[0]
        i = self.intermediate_size
        act = rt.buffer("ffn_act", (t, i), rt.act_dtype)
        if self.fused:
            rt.ops.linear_swiglu(h, self.w_gate_up, act)
        else:
            gu = rt.buffer("gate_up", (t, 2 * i), rt.act_dtype)
            rt.ops.linear(h, self.w_gate_up, gu)
            rt.ops.swiglu(gu, act)
        delta = rt.buffer("delta", (t, self.d_model), rt.act_dtype)
        return rt.ops.linear_parts(act, self.w_down, delta)


class ClampedGLUFeedForward(FeedForward):
    """``W_down (g' * sigmoid(alpha * g') * (u' + 1))`` with ``g' = min(W_gate h, limit)``
    and ``u' = clamp(W_up h, -limit, limit)``; no biases.  The activation runs in
    float32, in the projection's own epilogue where the tcgen05 kernel takes the sizes
    (as ``SwiGLUFeedForward`` does), else on the projection's output."""

    decode_capturable = prompt_capturable = True

    def __init__(self, d_model: int, intermediate_size: int, limit: float, alpha: float = 1.702,
                 names=("gate", "up", "down")):
        self.d_model, self.intermediate_size = int(d_model), int(intermediate_size)
        self.limit, self.alpha = float(limit), float(alpha)
        self.names = tuple(names)

    def tensor_specs(self) -> dict:
        d, i = self.d_model, self.intermediate_size
        g, u, dn = self.names
        return {g: TensorSpec((i, d)), u: TensorSpec((i, d)), dn: TensorSpec((d, i))}

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        g, u, dn = self.names
        ops = runtime.ops
        self.fused = (tensors[g].dtype == torch.bfloat16 and tensors[u].dtype == torch.bfloat16
                      and ops.can_fuse_swiglu(self.d_model, self.intermediate_size))
        if self.fused:
            self.w_gate_up = ops.prepare_weight(ops.interleave_gate_up(tensors[g], tensors[u]))
        else:
            self.w_gate_up = ops.prepare_weight(torch.cat([tensors[g], tensors[u]], dim=0))
        self.w_down = ops.prepare_weight(tensors[dn])

    def forward(self, h, step: StepContext):
        rt = self.runtime
        t, i = h.shape[0], self.intermediate_size
        act = rt.buffer("ffn_act", (t, i), rt.act_dtype)
        if self.fused:
            rt.ops.linear_clamped_glu(h, self.w_gate_up, act, self.alpha, self.limit)
        else:
            gu = rt.buffer("gate_up", (t, 2 * i), rt.act_dtype)
            rt.ops.linear(h, self.w_gate_up, gu)
            rt.ops.clamped_glu(gu, act, self.alpha, self.limit)
        delta = rt.buffer("delta", (t, self.d_model), rt.act_dtype)
        return rt.ops.linear_parts(act, self.w_down, delta)


class SquaredReluFeedForward(FeedForward):
    """``W_down relu(W_up h)^2``: no gate, no biases.  The activation runs in float32, in
    the projection's own epilogue where the tcgen05 kernel takes the sizes (as
    ``SwiGLUFeedForward`` does), else on the projection's output."""

    decode_capturable = prompt_capturable = True

    def __init__(self, d_model: int, intermediate_size: int, names=("up", "down")):
        self.d_model, self.intermediate_size = int(d_model), int(intermediate_size)
        self.names = tuple(names)

    def tensor_specs(self) -> dict:
        d, i = self.d_model, self.intermediate_size
        return {self.names[0]: TensorSpec((i, d)), self.names[1]: TensorSpec((d, i))}

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        self.w_up = runtime.ops.prepare_weight(tensors[self.names[0]])
        self.w_down = runtime.ops.prepare_weight(tensors[self.names[1]])
        self.fused = (self.w_up.dtype == torch.bfloat16
                      and runtime.ops.can_fuse_activation(self.d_model))

    def forward(self, h, step: StepContext):
        rt = self.runtime
        t = h.shape[0]
        act = rt.buffer("ffn_act", (t, self.intermediate_size), rt.act_dtype)
        if self.fused:
            rt.ops.linear_relu_squared(h, self.w_up, act)
        else:
            rt.ops.linear(h, self.w_up, act)
            rt.ops.relu_squared(act, act)
        delta = rt.buffer("delta", (t, self.d_model), rt.act_dtype)
        return rt.ops.linear_parts(act, self.w_down, delta)


class RoutedExperts(FeedForward):
    """A mixture of small SwiGLU experts with a sigmoid router.

    Router logits ``z = W_r h`` and scores ``s = sigmoid(z)`` in float32; a token takes
    its ``top`` experts with the largest scores (lowest index on a tie) and weighs them
    by the scores themselves (``renormalise``: divided by their sum).  ``weigh`` says
    where a weight multiplies: "input" (the expert sees ``w * h``) or "output".  A
    ``shared`` feed-forward, if any, runs for every token and is added.  Tensors:
    ``router`` [E, d] and ``e<i>.gate / up / down`` for every expert; the shared
    part's under ``shared``."""

    decode_capturable = prompt_capturable = True   # routing, sorting and the products stay on the device

    def __init__(self, d_model: int, n_experts: int, top: int, expert_size: int, shared=None,
                 weigh: str = "input", renormalise: bool = False):
        if weigh not in ("input", "output"):
            raise ValueError(f"weigh must be 'input' or 'output', not {weigh!r}")
        if not 0 < int(top) <= int(n_experts):
            raise ValueError("top must lie in 1..n_experts")
        self.d_model, self.n_experts, self.top = int(d_model), int(n_experts), int(top)
        self.expert_size, self.shared = int(expert_size), shared
        self.weigh, self.renormalise = weigh, bool(renormalise)

    def tensor_specs(self) -> dict:
        d, f = self.d_model, self.expert_size
        out = {"router": TensorSpec((self.n_experts, d))}
        for i in range(self.n_experts):
            out[f"e{i}.gate"] = TensorSpec((f, d))
            out[f"e{i}.up"] = TensorSpec((f, d))
            out[f"e{i}.down"] = TensorSpec((d, f))
        if self.shared is not None:
            out.update({f"shared.{n}": s for n, s in self.shared.tensor_specs().items()})
        return out

    def bind(self, tensors: dict, runtime) -> None:
        self.runtime = runtime
        n = self.n_experts
        self.w_router = tensors["router"].float().contiguous()       # scores are float32
        self.w_gate_up = torch.stack([torch.cat([tensors[f"e{i}.gate"], tensors[f"e{i}.up"]], 0)
                                      for i in range(n)]).contiguous()
        self.w_down = torch.stack([tensors[f"e{i}.down"] for i in range(n)]).contiguous()
        if self.shared is not None:
            self.shared.bind({k[len("shared."):]: v for k, v in tensors.items()
                              if k.startswith("shared.")}, runtime)
        runtime.ops.require_part("experts")

    def _work(self, t: int) -> dict:
        rt, n_slots = self.runtime, t * self.top
        tiles = rt.ops.expert_max_tiles(n_slots, self.n_experts)
        i32 = torch.int32
        return {"idx": rt.buffer("route_idx", (n_slots,), i32),
                "weight": rt.buffer("route_weight", (n_slots,), torch.float32),
                "order": rt.buffer("route_order", (n_slots,), i32),
                "offsets": rt.buffer("route_offsets", (self.n_experts + 1,), i32),
                "cursor": rt.buffer("route_cursor", (self.n_experts,), i32),
                "tile_expert": rt.buffer("route_tile_expert", (tiles,), i32),
                "tile_row0": rt.buffer("route_tile_row0", (tiles,), i32),
                "max_tiles": tiles}

    def forward(self, h, step: StepContext):
        rt, ops = self.runtime, self.runtime.ops
        t = h.shape[0]
        logits = rt.buffer("route_logits", (t, self.n_experts), torch.float32)
        ops.linear(h, self.w_router, logits)
        work = self._work(t)
        ops.route(logits, self.top, self.renormalise, work)
        n_slots = t * self.top
        y = rt.buffer("expert_act", (n_slots, self.expert_size), rt.act_dtype)
        per_slot = rt.buffer("expert_out", (n_slots, self.d_model), torch.float32)
        ops.expert_glu(h, self.w_gate_up, y, work, self.top, self.weigh == "input")
        ops.expert_down(y, self.w_down, per_slot, work, self.top, self.weigh == "output")
        shared = None
        if self.shared is not None:
            shared = self.shared.forward(h, step)
            if not isinstance(shared, torch.Tensor):
                shared = shared.float()              # a product left as its K-parts
        delta = rt.buffer("routed_delta", (t, self.d_model), rt.act_dtype)
        ops.expert_combine(per_slot, self.top, shared, delta)
        return delta
