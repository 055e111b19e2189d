"""Logulix on the GPU against the plain implementation of ``plain_logulix``.

Kernels alone (through ``Ops``), every mechanism as a one-layer model, then whole models:
prompts whole, decoded token by token, in portions down to two tokens, unequal requests in
one batch, pages and state slots used again, long decoding through CUDA graphs, greedy
generation through ``LLM.generate`` and the trace program.  Where random weights would hide
a fault the weights are made to show it: the query and key norm weights are scaled up until
every softmax is nearly one key (any key the engine loses, far away, at a page's edge or at
the window's, then changes the logits), decays are moved near one so that the first tokens
of a sequence still matter hundreds of tokens later, and a window one token too long or too
short is shown to move the oracle far more than the engine is allowed to differ.
"""

import copy
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_logulix as PL
import tiny_logulix as L
from engine_helpers import Replayer, tokens_for

pytestmark = pytest.mark.gpu

# largest |engine - plain| as a fraction of the largest |logit|: float32 differs from the
# float64 oracle by the order of its sums; bfloat16 by the rounding of products and activations
TOL = {"float32": 5e-5, "bfloat16": 3e-2}
# A sharp softmax turns a small change of a score into another key, so a row may also be off
# by NOISE times what rounding does to that row of the oracle itself (the oracle run again
# with its activations rounded to the engine's format, against its exact run in float64).
NOISE = 6.0


def close(got, want, tol, what, slack=None):
    scale = want.abs().max().item()
    err = (got.double() - want.double()).abs().max(dim=1).values
    bound = tol * scale if slack is None else tol * scale + NOISE * slack
    bad = int((err > bound).sum())
    assert bad == 0, (
        f"{what}: {bad} rows of {len(err)} differ by more than {tol:.0e} * {scale:.3f} "
        f"(worst {err.max().item():.3e}); first wrong row {int((err > bound).nonzero()[0])}")


def sharp(factor):
    """Scale the query and key norm weights (the projections themselves are normalised
    away) so that softmax picks nearly one key."""
    def patch(w):
        for n in w:
            if n.endswith(".q.norm") or n.endswith(".k.norm"):
                w[n] *= factor
    return patch


def long_memory(w):
    """wkv decays near one: early tokens stay in the state."""
    for n in w:
        if n.endswith(".mix.w0"):
            w[n] = w[n] * 0.3 - 4.5


def both(*patches):
    def patch(w):
        for p in patches:
            p(w)
    return patch


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("logulix")
    out = {}
    for key, raw, patch in (("mixed", L.L_MIXED, None), ("plain", L.L_PLAIN, None),
                            ("wide", L.L_WIDE, None), ("states", L.L_STATES, long_memory),
                            ("edge", L.L_EDGE, None),
                            ("sharp", L.L_WIDE, both(sharp(4.0), long_memory))):
        for dtype in ("float32", "bfloat16"):
            folder = tmp / f"{key}_{dtype}"
            out[(key, dtype)] = (folder, raw, L.make_logulix(folder, raw, 11, dtype, patch=patch))
    return out


def oracle(w, raw, tokens):
    return PL.plain_forward(w, raw, tokens)


def check(got, w, raw, tokens, dtype, what):
    """The engine's rows against the oracle's, every row with its own slack."""
    want = oracle(w, raw, tokens)
    g = torch.Generator().manual_seed(0)
    if dtype == "float32":
        def rounded_to(t):
            return t.float().to(t.dtype)
        step = 2.0 ** -23
    else:
        rounded_to, step = PL.to_bf16, 2.0 ** -8

    def nudged(t):
        return rounded_to(t * (1 + (torch.rand(t.shape, generator=g, dtype=t.dtype) - 0.5) * step))

    slack = torch.zeros(len(tokens), dtype=want.dtype)
    for rnd in (rounded_to, nudged, nudged):
        rounded = PL.plain_forward(w, raw, tokens, rnd=rnd)
        slack = torch.maximum(slack, (rounded - want).abs().max(dim=1).values)
    close(got, want, TOL[dtype], what, slack=slack)


# ------------------------------------------------------------------ kernels alone
@pytest.fixture(scope="module")
def rt32():
    from mini_llm_stack_b200.ops.kernels import Runtime
    return Runtime("cuda:0", torch.float32)


class _Step:
    """The few arrays of a step the kernels under test read."""

    def __init__(self, q_lens, slots):
        cu = [0]
        for n in q_lens:
            cu.append(cu[-1] + n)
        self.n_tokens, self.n_requests = cu[-1], len(q_lens)
        self.cu_q = torch.tensor(cu, dtype=torch.int32, device="cuda")
        self.state_slot = torch.tensor(slots, dtype=torch.int32, device="cuda")
        self.req_of_token = torch.tensor([r for r, n in enumerate(q_lens) for _ in range(n)],
                                         dtype=torch.int32, device="cuda")


def plain_scan(a, k, v, state, decay_tok=None, decay_head=None, bonus=None, read_first=False):
    """One request, float64: a, k [n, H, e], v [n, H, f], state [H, e, f] (changed in place)."""
    out = torch.zeros(a.shape[0], a.shape[1], v.shape[2], dtype=torch.float64)
    for t in range(a.shape[0]):
        kv = k[t][:, :, None] * v[t][:, None, :]
        if read_first:
            out[t] = torch.einsum("hij,hi->hj", state + bonus[:, :, None] * kv, a[t])
            state[:] = decay_tok[t][:, :, None] * state + kv
        else:
            state[:] = decay_head[:, None, None] * state + kv
            out[t] = torch.einsum("hij,hi->hj", state, a[t])
    return out


@pytest.mark.parametrize("heads,e,f", [(2, 8, 16), (3, 20, 5), (1, 100, 37), (2, 64, 64),
                                       (1, 256, 24)])
@pytest.mark.parametrize("read_first", [True, False])
def test_scan_kernel_in_both_orders_over_two_steps(rt32, heads, e, f, read_first):
    """Two requests of unequal length in slots 2 and 0, walked in two steps: the second
    step continues from the state the first left; key sizes that are no multiple of the
    row groups, value sizes that are no multiple of a CTA's columns."""
    g = torch.Generator().manual_seed(e * 31 + f)
    lens = [(19, 3), (2, 33)]                                   # tokens of (request 0, 1) a step
    state = torch.zeros(3, heads * e * f + 7, device="cuda")    # a wider row than S alone
    ref = [torch.zeros(heads, e, f, dtype=torch.float64) for _ in range(2)]
    bonus = torch.randn(heads, e, generator=g)
    dh = torch.rand(heads, generator=g) * 0.2 + 0.8
    for q_lens in lens:
        step = _Step(q_lens, [2, 0])
        t = step.n_tokens
        a, k = torch.randn(t, heads * e, generator=g), torch.randn(t, heads * e, generator=g)
        v = torch.randn(t, 5 + heads * f, generator=g)          # values start at column 5
        dt = torch.rand(t, heads * e, generator=g) * 0.3 + 0.7
        out = torch.empty(t, heads * f, device="cuda")
        rt32.ops.linear_scan((a.cuda(), 0), (k.cuda(), 0), (v.cuda(), 5), state, step, heads, e, f,
                             out, decay_tok=dt.cuda() if read_first else None,
                             decay_head=None if read_first else dh.cuda(),
                             bonus=bonus.cuda() if read_first else None, read_first=read_first)
        at = 0
        for r, n in enumerate(q_lens):
            rows = slice(at, at + n)
            want = plain_scan(a[rows].double().view(n, heads, e), k[rows].double().view(n, heads, e),
                              v[rows, 5:].double().view(n, heads, f), ref[r],
                              dt[rows].double().view(n, heads, e), dh.double(), bonus.double(),
                              read_first)
            got = out[rows].cpu().double().view(n, heads, f)
            assert (got - want).abs().max().item() < 2e-5 * max(1.0, want.abs().max().item())
            at += n
    for r, slot in enumerate([2, 0]):
        got = state[slot, :heads * e * f].cpu().double().view(heads, e, f)
        assert (got - ref[r]).abs().max().item() < 2e-5 * max(1.0, ref[r].abs().max().item())
    assert state[1].abs().max().item() == 0 and state[:, heads * e * f:].abs().max().item() == 0


def test_scan_finish_kernel(rt32):
    g = torch.Generator().manual_seed(2)
    t, heads, f = 6, 3, 20
    o, w = torch.randn(t, heads * f, generator=g) * 4, torch.randn(heads * f, generator=g)
    gate = torch.randn(t, 11 + heads * f, generator=g)
    for weight in (w, None):
        out = torch.empty(t, heads * f, device="cuda")
        rt32.ops.scan_finish(o.cuda(), gate.cuda(), 11, None if weight is None else weight.cuda(),
                             1e-5, out, heads, f)
        z = gate[:, 11:].double()
        want = PL.plain_rms(o.double().view(t, heads, f), 1e-5).reshape(t, heads * f) \
            * (z * torch.sigmoid(z))
        if weight is not None:
            want = want * weight.double()
        assert torch.allclose(out.cpu().double(), want, atol=2e-6)


@pytest.mark.parametrize("dims", [0, 6, 16])
def test_rotate_rows_kernel_far_positions(rt32, dims):
    """Rotation of a part of every head, entry i with i + dims/2, at positions up to a
    million: the angle is formed in float64."""
    g = torch.Generator().manual_seed(4)
    t, heads, e = 5, 3, 16
    src = torch.randn(t, 2 * heads * e + 9, generator=g)
    pos = torch.tensor([0, 1, 777, 65537, 1000003], dtype=torch.int32)
    rotary = None
    if dims:
        from mini_llm_stack_b200.parts.position import PartialRotary
        rotary = PartialRotary(dims, 10000.0, 3.0, "half")
        rotary.bind({}, rt32)
    out = torch.empty(t, 2 * heads * e, device="cuda")
    rt32.ops.rotate_rows(src.cuda(), 0, heads * e, pos.cuda(), rotary.freq if dims else None, dims,
                         0.25, out, heads, e)
    q = src[:, :heads * e].double().view(t, heads, e)
    k = src[:, heads * e:2 * heads * e].double().view(t, heads, e)
    if dims:
        q = PL.plain_rotate(q, dims, 10000.0, 3.0, "half", pos)
        k = PL.plain_rotate(k, dims, 10000.0, 3.0, "half", pos)
    want = torch.cat([q.reshape(t, -1), k.reshape(t, -1) * 0.25], dim=1)
    assert torch.allclose(out.cpu().double(), want, atol=3e-6)


@pytest.mark.parametrize("n_tail", [1, 3])
def test_tail_update_and_token_shift_over_short_steps(rt32, n_tail):
    """Steps shorter than the tail shift it; the shift's previous row comes from the tail at
    a step's first token and from the step's own rows afterwards."""
    g = torch.Generator().manual_seed(n_tail)
    c, width = 13, 20
    tail = torch.zeros(4, 3 + n_tail * c, device="cuda")
    view = tail[:, 3:]
    history = {0: [torch.zeros(c)] * n_tail, 1: [torch.zeros(c)] * n_tail}
    bias = torch.randn(c, generator=g)
    for q_lens in ([1, 5], [2, 1], [1, 1], [7, 2]):
        step = _Step(q_lens, [3, 1])
        src = torch.randn(step.n_tokens, width, generator=g)
        if n_tail == 1:
            mu = torch.rand(3, c, generator=g)
            h = src[:, :c].contiguous()
            out = torch.empty(2, step.n_tokens, c, device="cuda")
            out32 = torch.empty(step.n_tokens, c, device="cuda")
            rt32.ops.token_shift_mix(h.cuda(), mu.cuda(), view, out, out32, step)
            at = 0
            for r, n in enumerate(q_lens):
                prev = torch.stack([history[r][-1]] + [h[at + i] for i in range(n - 1)])
                for s in range(3):
                    want = h[at:at + n] + (prev - h[at:at + n]) * mu[s]
                    got = (out[s] if s < 2 else out32)[at:at + n].cpu()
                    assert torch.allclose(got, want, atol=1e-6), (q_lens, r, s)
                at += n
            rt32.ops.tail_update(h.cuda(), 0, c, None, view, 1, step)
            rows = h
        else:
            rt32.ops.tail_update(src.cuda(), 4, c, bias.cuda(), view, n_tail, step)
            rows = src[:, 4:4 + c] + bias
        at = 0
        for r, n in enumerate(q_lens):
            history[r] = (history[r] + [rows[at + i] for i in range(n)])[-n_tail:]
            at += n
        for r, slot in enumerate([3, 1]):
            assert torch.allclose(view[slot].cpu().view(n_tail, c), torch.stack(history[r]),
                                  atol=1e-6)
    assert tail[:, :3].abs().max().item() == 0 and tail[[0, 2]].abs().max().item() == 0


def test_small_stream_kernels(rt32):
    """relu squared, the logits' scale, the scaled embedding, and [x + delta | x0]."""
    g = torch.Generator().manual_seed(8)
    z = torch.randn(7, 33, generator=g)
    for dt in (torch.float32, torch.bfloat16):
        zd = z.to(dt).cuda()
        out = torch.empty_like(zd)
        rt32.ops.relu_squared(zd, out)
        assert torch.allclose(out.float().cpu(), (z.to(dt).float().clamp(min=0) ** 2).to(dt).float())
    x = torch.randn(5, 12, generator=g).cuda()
    before = x.clone()
    rt32.ops.scale_(x, 0.3)
    assert torch.allclose(x, before * 0.3)
    table = torch.randn(9, 12, generator=g).cuda()
    ids = torch.tensor([3, 0, 8], dtype=torch.int32, device="cuda")
    e = torch.empty(3, 12, device="cuda")
    rt32.ops.embed(ids, table, e, 9, 0.25)
    assert torch.allclose(e, table[[3, 0, 8]] * 0.25)
    rt32.ops.require_part("layernorm")
    x, delta, x0 = (torch.randn(6, 10, generator=g).cuda() for _ in range(3))
    for d in (delta, None):
        xs = x.clone()
        out = torch.empty(6, 20, device="cuda")
        rt32.ops.settle_concat(xs, d, x0, out)
        want = x + (d if d is not None else 0)
        assert torch.allclose(xs, want) and torch.allclose(out, torch.cat([want, x0], dim=1))


def test_fused_relu_squared_product():
    """The up projection with the square of relu in its epilogue (bfloat16, tcgen05): few
    rows (weight-major, K cut in parts), a prompt's rows on one CTA and on pairs of CTAs."""
    from mini_llm_stack_b200.ops.kernels import Runtime
    ops = Runtime("cuda:0", torch.bfloat16).ops
    g = torch.Generator().manual_seed(3)
    d, inter = 256, 200
    w = (torch.randn(inter, d, generator=g) * 0.2).bfloat16().cuda()
    assert ops.can_fuse_activation(d)
    for m in (3, 40, 100, 300):
        a = torch.randn(m, d, generator=g).bfloat16().cuda()
        out = torch.empty(m, inter, dtype=torch.bfloat16, device="cuda")
        ops.linear_relu_squared(a, w, out)
        want = (a.double() @ w.double().T).clamp(min=0) ** 2
        assert (out.double() - want).abs().max().item() < 1e-2 * want.abs().max().item(), m
    ops.check_status()


def test_capped_scores_on_the_tensor_core_kernels_agree_with_the_plain_kernel(models, monkeypatch):
    """bfloat16, heads of 64, a cap, a window: prompts on the tcgen05 kernel and decoded
    tokens on the context-split kernel against the one-warp-per-row kernel."""
    folder, raw, w = models[("sharp", "bfloat16")]
    toks = {0: tokens_for(raw["vocab"], 300, 5), 1: tokens_for(raw["vocab"], 150, 6)}
    runs = {}
    for impl in ("auto", "simt"):
        monkeypatch.setenv("MLS_B200_ATTENTION", impl)
        rp = Replayer(folder, "bfloat16", num_blocks=40, max_requests=2)
        assert rp.model.runtime.ops.attention_impl == impl
        rp.step([(0, 260), (1, 3)], toks)
        for _ in range(40):
            rp.step([(0, 1), (1, 1)], toks)
        rp.step([(1, 107)], toks)
        runs[impl] = torch.cat([rp.logits(0), rp.logits(1)])
    # the kernels round their probabilities at different places, and the softmax is sharp:
    # single logits may differ by a few hundredths, the mean difference is far smaller
    scale = runs["simt"].abs().max().item()
    assert (runs["auto"] - runs["simt"]).abs().mean().item() < 3e-3 * scale
    assert (runs["auto"] - runs["simt"]).abs().max().item() < 1e-1 * scale
    for impl in runs:
        check(runs[impl][:300], w, raw, toks[0], "bfloat16", f"capped scores, {impl}")
        check(runs[impl][300:], w, raw, toks[1], "bfloat16", f"capped scores, {impl}")


# ------------------------------------------------------- mechanisms as one-layer models
ONE_LAYER = {
    "attention_all": {"type": "attention", "mlp": None,
                      "mixer": L.attention(4, 2, 16, 0.4, conv=3, window=19,
                                           rot=L.rot(10, 300.0, 2.5), softcap=6.0)},
    "attention_bare": {"type": "attention", "mixer": L.attention(2, 2, 24, 0.3), "mlp": None},
    "attention_conv4_window_of_a_page": {
        "type": "attention", "mlp": None,
        "mixer": L.attention(3, 1, 8, 0.5, conv=4, window=16, rot=L.rot(8, 50.0))},
    "attention_conv2_window1": {"type": "attention", "mlp": None,
                                "mixer": L.attention(2, 1, 16, 0.5, conv=2, window=1, softcap=2.0)},
    # more taps than the four-channel kernel unrolls, and a head size it does not take
    "attention_conv9_head_6": {"type": "attention", "mlp": None,
                               "mixer": L.attention(2, 2, 6, 0.5, conv=9, window=12,
                                                    rot=L.rot(4, 20.0))},
    "attention_conv9_head_16": {"type": "attention", "mlp": None,
                                "mixer": L.attention(2, 1, 16, 0.4, conv=9, rot=L.rot(16, 20.0))},
    "attention_conv1": {"type": "attention", "mlp": None,
                        "mixer": L.attention(1, 1, 32, 0.2, conv=1, window=40, softcap=50.0)},
    "attention_head_80": {"type": "attention", "mlp": None,
                          "mixer": L.attention(2, 1, 80, 0.1, conv=3, window=33,
                                               rot=L.rot(80, 10000.0), softcap=15.0)},
    "attention_head_128": {"type": "attention", "mlp": None,
                           "mixer": L.attention(2, 1, 128, 0.09, conv=2, window=50,
                                                rot=L.rot(64, 10000.0, 8.0), softcap=30.0)},
    "wkv": {"type": "wkv", "mixer": L.wkv(2, 12, 6), "mlp": None},
    "wkv_one_head_rank1": {"type": "wkv", "mixer": L.wkv(1, 40, 1), "mlp": None},
    "retention": {"type": "retention", "mlp": None,
                  "mixer": L.retention(2, 12, 20, [0.95, 0.999], rot=L.rot(8, 200.0, 1.5))},
    "retention_no_rotation": {"type": "retention", "mlp": None,
                              "mixer": L.retention(1, 6, 50, [1.0])},
    "relu2": {"type": "wkv", "mixer": L.wkv(1, 8, 2), "mlp": L.dense(56)},
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_one_mechanism_alone(tmp_path, name, dtype):
    raw = L.one_layer(ONE_LAYER[name])
    patch = long_memory if name.startswith("wkv") else sharp(3.0)
    w = L.make_logulix(tmp_path / name, raw, 5, dtype, std=0.15, patch=patch)
    toks = {0: tokens_for(raw["vocab"], 70, 3), 1: tokens_for(raw["vocab"], 45, 4)}
    rp = Replayer(tmp_path / name, dtype, num_blocks=8, max_requests=2)
    rp.step([(0, 70)], toks, end=[0])                       # whole
    rp.step([(1, 1)], toks)                                 # the first token alone
    rp.step([(1, 16)], toks)                                # portions, then token by token
    rp.step([(1, 2)], toks)
    for _ in range(26):
        rp.step([(1, 1)], toks)
    for i in toks:
        check(rp.logits(i), w, raw, toks[i], dtype, f"{name} {dtype} request {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [15, 16, 17, 40])
def test_a_window_one_token_off_would_show(tmp_path, window, dtype):
    """Sharp attention behind a window: the engine agrees with the oracle of that window,
    and the oracles of a window one token longer or shorter are far away, in a prompt and
    in decoded tokens, with windows that end at, before and behind a page's edge."""
    layer = {"type": "attention", "mlp": None,
             "mixer": L.attention(2, 1, 16, 1.0, conv=2, window=window, rot=L.rot(16, 100.0))}
    raw = L.one_layer(layer)
    w = L.make_logulix(tmp_path / "m", raw, 9, dtype, std=0.2, patch=sharp(2.0))
    n = 100
    toks = {0: tokens_for(raw["vocab"], n, 1), 1: tokens_for(raw["vocab"], n, 1)}
    rp = Replayer(tmp_path / "m", dtype, num_blocks=8, max_requests=1)
    rp.step([(0, n)], toks, end=[0])
    rp.step([(1, 37)], toks)
    for _ in range(n - 37):
        rp.step([(1, 1)], toks)
    want = oracle(w, raw, toks[0])
    for off in (-1, 1):
        wrong_raw = copy.deepcopy(raw)
        wrong_raw["layers"][0]["mixer"]["mask"]["size"] = window + off
        wrong = oracle(w, wrong_raw, toks[0])
        moved = (wrong - want).abs().max(dim=1).values[window:]
        for i in (0, 1):
            err = (rp.logits(i).double() - want).abs().max(dim=1).values[window:]
            if dtype == "float32":
                assert (moved > 20 * err).sum() >= 10, (window, off, i)
            else:
                assert (moved > 4 * err).sum() >= 3, (window, off, i)
    for i in (0, 1):
        check(rp.logits(i), w, raw, toks[i], dtype, f"window {window} {dtype} run {i}")


# ------------------------------------------------------------------- whole models
LENGTHS = {"mixed": [1, 2, 19, 150], "plain": [1, 33, 97], "wide": [3, 64, 260],
           "sharp": [5, 300], "states": [1, 2, 170], "edge": [1, 7, 60]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", sorted(LENGTHS))
def test_whole_prompts_and_decoding_agree_with_the_plain_model(models, key, dtype):
    folder, raw, w = models[(key, dtype)]
    rp = Replayer(folder, dtype, num_blocks=24, max_requests=2)
    for i, n in enumerate(LENGTHS[key]):
        toks = {i: tokens_for(raw["vocab"], n, 40 + i), ("d", i): tokens_for(raw["vocab"], n, 40 + i)}
        rp.step([(i, n)], toks, end=[i])
        check(rp.logits(i), w, raw, toks[i], dtype, f"{key} {dtype} whole prompt of {n}")
        # the same tokens: most at once, the last ones (up to 40, over page edges) one by one
        tail = min(40, n - 1)
        if tail:
            rp.step([(("d", i), n - tail)], toks)
            for _ in range(tail):
                rp.step([(("d", i), 1)], toks)
            rp.runner.release(("d", i))
            check(rp.logits(("d", i)), w, raw, toks[i], dtype, f"{key} {dtype} decoded tail of {n}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["mixed", "sharp", "states"])
def test_portions_of_every_size_do_not_change_the_logits(models, key, dtype):
    folder, raw, w = models[(key, dtype)]
    n = 231
    toks = {"r": tokens_for(raw["vocab"], n, 9), "w": tokens_for(raw["vocab"], n, 9)}
    rp = Replayer(folder, dtype, num_blocks=16, max_requests=1)
    fed = 0
    for size in [2, 3, 11, 16, 1, 1, 2, 47, 17, 64, 5, 2, 33]:      # cuts inside pages and at their edges
        rp.step([("r", size)], toks)
        fed += size
    while fed < n:
        rp.step([("r", 1)], toks)
        fed += 1
    rp.runner.release("r")
    check(rp.logits("r"), w, raw, toks["r"], dtype, f"{key} {dtype} portions")
    if dtype == "float32":
        rp.step([("w", n)], toks, end=["w"])
        assert torch.equal(rp.logits("r"), rp.logits("w")), "the cut changes float32 bits"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["mixed", "wide", "states"])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(models, key, dtype):
    """Five requests over three state slots and so few pages that a finished request's
    pages and slot go to the next one at once; every request must come out as alone."""
    folder, raw, w = models[(key, dtype)]
    lens = {0: 90, 1: 37, 2: 61, 3: 120, 4: 2}
    toks = {i: tokens_for(raw["vocab"], n, 70 + i) for i, n in lens.items()}
    rp = Replayer(folder, dtype, num_blocks=18, max_requests=3)
    rp.step([(0, 40), (1, 2)], toks)
    rp.step([(0, 1), (1, 35), (2, 30)], toks, end=[1])
    rp.step([(0, 17), (2, 1), (3, 50)], toks)                 # 3 takes the slot and pages of 1
    rp.step([(0, 32), (2, 30), (3, 2)], toks, end=[0, 2])
    rp.step([(3, 1), (4, 2)], toks, end=[4])                  # 4 starts from a slot 0 or 2 left
    rp.step([(3, 67)], toks, end=[3])
    assert rp.runner.cache.slots.num_free == 3
    for i in lens:
        check(rp.logits(i), w, raw, toks[i], dtype, f"{key} {dtype} request {i}")
    if dtype == "float32":
        # a token's logits do not depend on its batch: bit for bit the run of each alone
        for i in (1, 3):
            alone = Replayer(folder, dtype, num_blocks=18, max_requests=1)
            alone.step([(i, lens[i])], toks, end=[i])
            assert torch.equal(alone.logits(i), rp.logits(i)), f"request {i} depends on its batch"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_replays_graphs_and_keeps_the_state(models, dtype):
    """(A sequence's first token is ill-conditioned by design: with an empty state a head's
    output is ``(r . (u * k)) v``, and the head norm keeps only the sign of that number.  Where
    it is nearly zero, rounding decides the sign, and with decays near one the whole sequence
    follows.  The seeds give first tokens that are not such a case.)"""
    folder, raw, w = models[("sharp", dtype)]
    n = 190
    toks = {"a": tokens_for(raw["vocab"], n, 23), "b": tokens_for(raw["vocab"], n - 30, 24)}
    rp = Replayer(folder, dtype, num_blocks=32, max_requests=2)
    rp.step([("a", 10), ("b", 3)], toks)
    for _ in range(n - 30 - 3):                               # both decode, one token a step
        rp.step([("a", 1), ("b", 1)], toks)
    rp.runner.release("b")
    for _ in range(n - 10 - (n - 33)):
        rp.step([("a", 1)], toks)
    assert any(isinstance(v, tuple) for k, v in rp.runner._graphs.items() if k != "moved"), \
        "no decode step was replayed from a graph"
    for r in toks:
        check(rp.logits(r), w, raw, toks[r], dtype, f"long decoding {r} {dtype}")


def test_greedy_generation_through_the_scheduler(models):
    from mini_llm_stack_b200.engine.llm import LLM
    folder, raw, w = models[("mixed", "float32")]
    prompts = [tokens_for(raw["vocab"], n, 300 + n) for n in (3, 41, 18, 1)]
    # three at a time, portions of at most 16 tokens, so few pages that requests wait
    llm = LLM.from_folder(folder, dtype="float32", num_blocks=14, block_size=8, max_batch=3,
                          max_tokens_per_step=24, chunk_size=16)
    got = llm.generate(prompts, max_new_tokens=10)
    for p, g in zip(prompts, got):
        seq = list(p)
        for tok in g:
            row = oracle(w, raw, seq)[-1]
            assert row[tok] >= row.max() - 1e-4 * row.abs().max(), (len(p), len(seq), tok)
            seq.append(tok)
        assert len(g) == 10
    llm.engine.cache.check()
    assert llm.engine.cache.slots.num_free == 3


def test_trace_program_replays_a_folder(models, tmp_path):
    """``bin/trace_run`` picks the model class by config.json and reads the decay's inner
    size off the weight file; two requests, portions beside single tokens."""
    import shutil
    _, raw, w = models[("plain", "float32")]
    folder = tmp_path / "model"
    shutil.copytree(models[("plain", "float32")][0], folder)
    cfg = json.loads((Path(folder) / "config.json").read_text())
    for layer in cfg["layers"]:
        layer["mixer"].pop("rank", None)                      # the tensors' shapes say it
    (Path(folder) / "config.json").write_text(json.dumps(cfg))
    a, b = tokens_for(raw["vocab"], 50, 1), tokens_for(raw["vocab"], 9, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:48], "want": []},
                                     {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[48:49], "want": [0]},
                                     {"id": "b", "tokens": b[8:], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[49:], "want": [0]}], "end": ["a"]}]
    root = Path(__file__).resolve().parent.parent
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(folder),
                           "--dtype", "float32", "--out", str(out), "--max-tokens", "128"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", text=True,
                          capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [ln for ln in proc.stdout.splitlines() if ln.startswith("done")] == \
        [f"done {i}" for i in range(4)]
    la, lb = oracle(w, raw, a), oracle(w, raw, b)
    want = {0: la[[0, 29]], 1: lb[[7]], 2: torch.stack([la[48], lb[8]]), 3: la[[49]]}
    for i, rows in want.items():
        got = torch.frombuffer(bytearray((out / f"{i}.f32").read_bytes()), dtype=torch.float32)
        close(got.view(rows.shape), rows, TOL["float32"], f"trace step {i}")
