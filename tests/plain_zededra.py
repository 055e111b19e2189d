"""A plain, slow Zededra on whole sequences: one function per mechanism.

Written from the design's equations with torch tensor algebra only; it shares
no code with the engine.  Everything runs in the dtype of the weights it is
given (float64 for an oracle, float32 otherwise); ``tokens`` is one sequence.
``rnd`` (identity by default) is applied to every activation a 16-bit engine
would store (projections, mixer and feed-forward outputs, normed rows): with
``to_bf16`` the function shows how far rounding alone moves a result.

Notation: d = model width, H = heads, e = query/key size of a head, f = value
size of a head, r = latent size, eps = the model's norm epsilon.
"""

import torch


def ident(t):
    return t


def to_bf16(t):
    return t.to(torch.bfloat16).to(t.dtype)


# --------------------------------------------------------------------------- norms
def plain_layernorm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w with the biased variance, no bias."""
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def plain_unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


# --------------------------------------------------------------- latent attention
def plain_latent_attention(h, w, p, m, eps, rnd=ident):
    """Causal softmax attention whose keys and values are read off one shared
    latent a token: c = unit_rms(W_dkv h) * g_kv; k_h = W_uk[h] c; v_h = W_uv[h] c;
    queries through a latent of their own.  No positions enter."""
    S = h.shape[0]
    H, e, f = m["heads"], m["dim"], m["vdim"]
    cq = rnd(plain_unit_rms(h @ w[f"{p}.dq"].T, eps) * w[f"{p}.dq.norm"])
    q = rnd(cq @ w[f"{p}.uq"].T).view(S, H, e)
    c = rnd(plain_unit_rms(h @ w[f"{p}.dkv"].T, eps) * w[f"{p}.dkv.norm"])
    k = rnd(c @ w[f"{p}.uk"].T).view(S, H, e)
    v = rnd(c @ w[f"{p}.uv"].T).view(S, H, f)
    s = torch.einsum("ihe,jhe->hij", q, k) * m["scale"]
    hidden = torch.triu(torch.ones(S, S, dtype=torch.bool), diagonal=1)
    s = s.masked_fill(hidden, float("-inf"))
    a = torch.softmax(s, dim=-1)
    o = rnd(torch.einsum("hij,jhf->ihf", a, v).reshape(S, H * f))
    return rnd(o @ w[f"{p}.o"].T), c


# -------------------------------------------------------------------------- mLSTM
def plain_soft_cap(z, cap):
    return cap * torch.tanh(z / cap)


def plain_mlstm(h, w, p, m, eps, state=None, rnd=ident):
    """Matrix memory with exponential gates, token by token.

    log gates: i = softcap(W_i h + b_i), f = logsigmoid(softcap(W_f h + b_f));
    stabiliser mx (starts at 0): mx' = max(f + mx, i);
    C' = exp(f + mx - mx') C + exp(i - mx') k v^T, n' likewise with k;
    o = C'^T q / (max(|n' . q|, exp(-mx')) + 1e-6), q pre-scaled by e^(-1/2).
    Then per head unit-rms, the weight over all heads, the sigmoid gate, W_o.
    ``state`` = (C [H,e,f], n [H,e], mx [H]) carries over; returned as well."""
    S = h.shape[0]
    H, e, f = m["heads"], m["dim"], m["vdim"]
    cap = m["gate_cap"]
    q = rnd(h @ w[f"{p}.q"].T).view(S, H, e) * e ** -0.5
    k = rnd(h @ w[f"{p}.k"].T).view(S, H, e)
    v = rnd(h @ w[f"{p}.v"].T).view(S, H, f)
    ig = plain_soft_cap(h @ w[f"{p}.i"].T + w[f"{p}.i.b"], cap)
    fg = torch.nn.functional.logsigmoid(plain_soft_cap(h @ w[f"{p}.f"].T + w[f"{p}.f.b"], cap))
    if state is None:
        C = torch.zeros(H, e, f, dtype=h.dtype)
        n = torch.zeros(H, e, dtype=h.dtype)
        mx = torch.zeros(H, dtype=h.dtype)
    else:
        C, n, mx = state
    rows = []
    for t in range(S):
        new = torch.maximum(fg[t] + mx, ig[t])
        keep = torch.exp(fg[t] + mx - new)
        take = torch.exp(ig[t] - new)
        C = keep[:, None, None] * C + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        mx = new
        num = torch.einsum("hef,he->hf", C, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        rows.append(num / den[:, None])
    o = torch.stack(rows)                                   # [S, H, f]
    o = plain_unit_rms(o, eps).reshape(S, H * f) * w[f"{p}.norm"]
    o = rnd(o * torch.sigmoid(rnd(h @ w[f"{p}.g"].T)))
    return rnd(o @ w[f"{p}.o"].T), (C, n, mx)


# ------------------------------------------------------------------ feed-forwards
def plain_clamped_glu(h, w, p, limit, rnd=ident):
    """g = min(W_g h, L); u = clamp(W_u h, -L, L); W_d (g sigmoid(1.702 g) (u + 1))."""
    g = torch.clamp(rnd(h @ w[f"{p}.gate"].T), max=limit)
    u = torch.clamp(rnd(h @ w[f"{p}.up"].T), -limit, limit)
    return rnd(rnd(g * torch.sigmoid(1.702 * g) * (u + 1)) @ w[f"{p}.down"].T)


def plain_silu_glu(h, w, p, rnd=ident):
    g = h @ w[f"{p}.gate"].T
    return rnd(g * torch.sigmoid(g) * (h @ w[f"{p}.up"].T)) @ w[f"{p}.down"].T


def plain_route(h, w_router, top):
    """Sigmoid scores of a float32 router; the ``top`` largest (lowest index on
    ties) with their own scores as weights, not renormalised."""
    s = torch.sigmoid(h.float() @ w_router.float().T)
    order = torch.sort(s, dim=-1, descending=True, stable=True)
    return order.indices[:, :top], order.values[:, :top]


def plain_routed_experts(h, w, p, mlp, rnd=ident):
    """sum over the chosen experts of expert(weight * h), plus the shared expert."""
    top = mlp["router"]["top"]
    idx, val = plain_route(h, w[f"{p}.router"], top)
    out = torch.zeros(h.shape[0], w[f"{p}.e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(top):
            ex = int(idx[t, j])
            out[t] += plain_silu_glu((val[t, j].to(h.dtype) * h[t])[None], w, f"{p}.e{ex}", rnd)[0]
    if mlp.get("shared"):
        out = out + rnd(plain_silu_glu(h, w, f"{p}.shared", rnd))
    return rnd(out)


def plain_feedforward(h, w, p, mlp, rnd=ident):
    if mlp["kind"] == "dense":
        return plain_clamped_glu(h, w, p, mlp["limit"], rnd)
    return plain_routed_experts(h, w, p, mlp, rnd)


# -------------------------------------------------------------------------- model
def layer_runs(cfg):
    """[(layer index, number of the pass or None, first of its pass)] in running order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None, False) for i in range(a)]
    for t in range(times):
        runs += [(i, t, i == a) for i in range(a, b)]
    runs += [(i, None, False) for i in range(b, n)]
    return runs


def plain_zededra(w, cfg, tokens, trace=None, rnd=ident):
    """Logits [S, vocab] of one whole sequence; ``trace`` (a list) receives the
    residual stream after every layer run."""
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][torch.as_tensor(tokens)]
    x = x0
    for i, t, first in layer_runs(cfg):
        L = cfg["layers"][i]
        if first:
            if t > 0:
                x = x + x0
            x = x + w["loop.step"][t]
        h = rnd(plain_layernorm(x, w[f"l{i}.norm1"], eps))
        if L["type"] == "mlstm":
            y, _ = plain_mlstm(h, w, f"l{i}.mix", L["mixer"], eps, rnd=rnd)
        elif L["type"] == "latent_attention":
            y, _ = plain_latent_attention(h, w, f"l{i}.mix", L["mixer"], eps, rnd)
        else:
            raise ValueError(L["type"])
        x = x + y
        if L.get("mlp"):
            h = rnd(plain_layernorm(x, w[f"l{i}.norm2"], eps))
            x = x + plain_feedforward(h, w, f"l{i}.mlp", L["mlp"], rnd)
        if trace is not None:
            trace.append(x)
    return rnd(plain_layernorm(x, w["final.norm"], eps)) @ w["embed"].T
