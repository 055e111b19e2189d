"""A plain, slow Logulix on whole sequences: one function per mechanism.

Written from the design's equations with torch tensor algebra and explicit loops
over the tokens; it shares no code with the engine.  Everything runs in the dtype
of the weights it is given (float64 for an oracle); ``tokens`` is one sequence.
``rnd`` (identity by default) is applied to every activation a 16-bit engine would
store (projections, convolution outputs, mixer and feed-forward outputs, normed
rows): with ``to_bf16`` the function shows how far rounding alone moves a result.

Notation: d = model width, H = heads, G = key/value heads, e = query/key size of a
head, f = value size of a head, eps = the model's norm epsilon, p = position.
"""

import math

import torch


def ident(t):
    return t


def to_bf16(t):
    return t.to(torch.bfloat16).to(t.dtype)


# --------------------------------------------------------------------------- norms
def plain_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


# ------------------------------------------------------------------------ rotation
def plain_rotate(x, dims, base, factor, pairing, positions):
    """Rotate the first ``dims`` entries of every head of x [S, heads, e] by the
    angles p * base^(-2i/dims) / factor.  ``pairing`` "interleaved": entry 2i goes
    with 2i+1; "half": entry i goes with i + dims/2."""
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims) / factor
    ang = positions.to(x.dtype)[:, None] * freq[None, :]            # [S, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    if pairing == "interleaved":
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    else:
        a, b = x[..., :half], x[..., half:dims]
        out[..., :half] = a * c - b * s
        out[..., half:dims] = b * c + a * s
    return out


# -------------------------------------------------------------- short convolution
def plain_causal_conv(u, w):
    """y_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before the start.
    u [S, C], w [C, taps]."""
    S, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(S):
        for j in range(taps):
            src = t - taps + 1 + j
            if src >= 0:
                y[t] += w[:, j] * u[src]
    return y


# ----------------------------------------------------------------------- attention
def plain_window_attention(h, w, p, m, eps, rnd=ident):
    """Grouped-query softmax attention whose values are the keys: biased q and k
    projections, a short causal convolution on both, v = the convolved k; then an
    RMS norm over the whole q row and the whole k row, interleaved rotation, capped
    scores, a sliding window, and a biased output projection."""
    S = h.shape[0]
    H, G, e = m["heads"], m["kv_heads"], m["dim"]
    q = rnd(h @ w[f"{p}.q"].T + w[f"{p}.q.b"])
    k = rnd(h @ w[f"{p}.k"].T + w[f"{p}.k.b"])
    if m.get("conv"):
        q = rnd(plain_causal_conv(q, w[f"{p}.q.conv"]))
        k = rnd(plain_causal_conv(k, w[f"{p}.k.conv"]))
    v = k.view(S, G, e)
    q = plain_rms(q, eps) * w[f"{p}.q.norm"]
    k = plain_rms(k, eps) * w[f"{p}.k.norm"]
    q, k = q.view(S, H, e), k.view(S, G, e)
    pos = torch.arange(S)
    rot = m.get("rot")
    if rot:
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        q = plain_rotate(q, rot["dims"], rot["base"], factor, "interleaved", pos)
        k = plain_rotate(k, rot["dims"], rot["base"], factor, "interleaved", pos)
    q, k = rnd(q), rnd(k)
    out = torch.zeros(S, H, e, dtype=h.dtype)
    cap = m.get("softcap")
    win = (m.get("mask") or {}).get("size")
    for i in range(S):
        lo = 0 if win is None else max(0, i - win + 1)
        for hh in range(H):
            g = hh // (H // G)
            s = (k[lo:i + 1, g] @ q[i, hh]) * m["scale"]
            if cap:
                s = cap * torch.tanh(s / cap)
            a = torch.softmax(s, dim=0)
            out[i, hh] = a @ v[lo:i + 1, g]
    o = rnd(out.reshape(S, H * e))
    return rnd(o @ w[f"{p}.o"].T + w[f"{p}.o.b"])


# ------------------------------------------------------------------------------ wkv
def plain_wkv(h, w, p, m, eps, rnd=ident):
    """Time mixing with a matrix state per head and a data-dependent decay per key
    channel: the current token reads the state with a bonus u, then the state
    decays and takes the token in."""
    S, d = h.shape
    H, e = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros(1, d, dtype=h.dtype), h[:-1]], dim=0)

    def mix(s):
        return rnd(h + (prev - h) * w[f"{p}.mu.{s}"])

    r = rnd(mix("r") @ w[f"{p}.r"].T).view(S, H, e)
    k = rnd(mix("k") @ w[f"{p}.k"].T).view(S, H, e)
    v = rnd(mix("v") @ w[f"{p}.v"].T).view(S, H, e)
    gz = rnd(mix("g") @ w[f"{p}.g"].T)
    gate = gz * torch.sigmoid(gz)
    lo = torch.tanh(mix("w") @ w[f"{p}.w1"].T)
    decay = torch.exp(-torch.exp(lo @ w[f"{p}.w2"].T + w[f"{p}.w0"])).view(S, H, e)
    u = w[f"{p}.u"].view(H, e)
    state = torch.zeros(H, e, e, dtype=h.dtype)                  # [head, key, value]
    o = torch.zeros(S, H, e, dtype=h.dtype)
    for t in range(S):
        kv = k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hij,hi->hj", state + u[:, :, None] * kv, r[t])
        state = decay[t][:, :, None] * state + kv
    o = plain_rms(o, eps).reshape(S, H * e) * w[f"{p}.norm"] * gate
    return rnd(rnd(o) @ w[f"{p}.o"].T)


# ------------------------------------------------------------------------ retention
def plain_retention(h, w, p, m, eps, rnd=ident):
    """Linear attention with one fixed decay a head and no softmax: the state takes
    the token in first and is read afterwards."""
    S = h.shape[0]
    H, e, f = m["heads"], m["dim"], m["vdim"]
    q = rnd(h @ w[f"{p}.q"].T).view(S, H, e)
    k = rnd(h @ w[f"{p}.k"].T).view(S, H, e)
    v = rnd(h @ w[f"{p}.v"].T).view(S, H, f)
    gz = rnd(h @ w[f"{p}.g"].T)
    pos = torch.arange(S)
    rot = m.get("rot")
    if rot:
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        q = plain_rotate(q, rot["dims"], rot["base"], factor, "half", pos)
        k = plain_rotate(k, rot["dims"], rot["base"], factor, "half", pos)
    k = k * e ** -0.5
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    state = torch.zeros(H, e, f, dtype=h.dtype)
    o = torch.zeros(S, H, f, dtype=h.dtype)
    for t in range(S):
        state = decay[:, None, None] * state + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hij,hi->hj", state, q[t])
    o = plain_rms(o, eps).reshape(S, H * f) * (gz * torch.sigmoid(gz))
    return rnd(rnd(o) @ w[f"{p}.o"].T)


# --------------------------------------------------------------------- feed-forward
def plain_relu2_mlp(h, w, p, rnd=ident):
    """W_down relu(W_up h)^2."""
    a = torch.relu(h @ w[f"{p}.up"].T)
    return rnd(rnd(a * a) @ w[f"{p}.down"].T)


def plain_gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ---------------------------------------------------------------------------- model
MIXERS = {"attention": plain_window_attention, "wkv": plain_wkv, "retention": plain_retention}


def layer_runs(cfg):
    """[(layer, first of its pass)] in the order in which the layers run."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b = loop["start"], loop["stop"]
    runs = [(i, False) for i in range(a)]
    for _ in range(loop["times"]):
        runs += [(i, i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, n)]


def plain_forward(w, cfg, tokens, rnd=ident, layers_out=None):
    """Logits [S, vocab] of one sequence; ``layers_out`` (a list) receives the
    residual stream after every layer run."""
    eps = cfg["norm"]["eps"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x0 = w["embed"][ids] * cfg.get("embedding", {}).get("scale", 1.0)
    x = x0
    for i, first in layer_runs(cfg):
        layer, p = cfg["layers"][i], f"l{i}"
        if first:
            x = rnd(torch.cat([x, x0], dim=-1)) @ w["loop.in"].T
        h = rnd(plain_rms(x, eps) * w[f"{p}.norm1"])
        x = x + MIXERS[layer["type"]](h, w, f"{p}.mix", layer["mixer"], eps, rnd)
        if layer.get("mlp") is not None:
            h = rnd(plain_rms(x, eps) * w[f"{p}.norm2"])
            x = x + plain_relu2_mlp(h, w, f"{p}.mlp", rnd)
        if layers_out is not None:
            layers_out.append(x.clone())
    h = rnd(plain_rms(x, eps) * w["final.norm"])
    return (h @ w["head"].T) * cfg.get("logit_scale", 1.0)
