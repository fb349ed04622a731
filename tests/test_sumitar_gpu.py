"""Sumitar in the engine against the plain implementation (tests/plain/sumitar_plain.py): every mechanism alone, then whole
models under every way of cutting the work, long decoding, generation through the Python entry point, the trace program and
the command-line programs."""
import json
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

import sumitar_tiny as ST
import traces
from part_util import DEV, bind_random, feed, rel_err
from plain import sumitar_plain as SP
from replay_util import run_trace

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F64 = torch.float64
BOTH = [torch.float32, torch.bfloat16]


def tol_for(dtype):
    return 2e-4 if dtype in ("float32", torch.float32) else 6e-2


def tol_part(dtype, f32=3e-5, bf16=5e-2):
    return f32 if dtype == torch.float32 else bf16


# ---------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("rows,hidden", [(1, 40), (7, 96), (33, 1536), (5, 73), (3, 52)])
def test_the_tanh_norm_on_both_sides_of_a_float32_stream(dtype, rows, hidden):
    """h += N(y; after); out = N(h; before): with and without a pending branch, on chosen rows (the stream then stays as it
    is), as a fold without an output, and on its own."""
    from zedinfer_b200 import ops
    g = torch.Generator().manual_seed(rows * 1000 + hidden)
    h0 = torch.randn(rows, hidden, generator=g) * 3
    y = (torch.randn(rows, hidden, generator=g) * 2).to(dtype)
    post = (0.7, 1 + 0.2 * torch.randn(hidden, generator=g), 0.1 * torch.randn(hidden, generator=g))
    pre = (1.3, 1 + 0.2 * torch.randn(hidden, generator=g), 0.1 * torch.randn(hidden, generator=g))
    dev = lambda nm: (nm[0], nm[1].to(DEV), nm[2].to(DEV))
    norm = lambda v, nm: torch.tanh(nm[0] * v.double()) * nm[1].double() + nm[2].double()
    want_h = h0.double() + norm(y, post)
    tol = tol_part(dtype, 2e-6, 1e-2)
    # a pending branch folded, the next sublayer's input written
    h, out = h0.clone().to(DEV), torch.empty(rows, hidden, dtype=dtype, device=DEV)
    ops.tanh_norm_fold(h, y.to(DEV), dev(post), dev(pre), out)
    assert rel_err(h, want_h) < 2e-6 and rel_err(out, norm(want_h, pre)) < tol
    # nothing pending
    h, out = h0.clone().to(DEV), torch.empty(rows, hidden, dtype=dtype, device=DEV)
    ops.tanh_norm_fold(h, None, None, dev(pre), out)
    assert torch.equal(h.cpu(), h0) and rel_err(out, norm(h0, pre)) < tol
    # chosen rows: the stream is left alone
    idx = torch.tensor([rows - 1, 0, rows // 2], dtype=torch.int32)
    h, out = h0.clone().to(DEV), torch.empty(3, hidden, dtype=dtype, device=DEV)
    ops.tanh_norm_fold(h, y.to(DEV), dev(post), dev(pre), out, row_idx=idx.to(DEV))
    assert torch.equal(h.cpu(), h0) and rel_err(out, norm(want_h, pre)[idx.long()]) < tol
    # a fold alone
    h = h0.clone().to(DEV)
    ops.tanh_norm_fold(h, y.to(DEV), dev(post), None, None)
    assert rel_err(h, want_h) < 2e-6
    # two branches joined on the way: the same as joining them first (up to that step's rounding)
    y2 = (torch.randn(rows, hidden, generator=g) * 0.5).to(dtype)
    w1, w2, eps = 1 + 0.3 * torch.randn(hidden, generator=g), 1 + 0.3 * torch.randn(hidden, generator=g), 1e-5
    joined = 0.5 * (SP.rms_unit(y.double(), eps) * w1.double() + SP.rms_unit(y2.double(), eps) * w2.double())
    want_j = h0.double() + norm(joined, post)
    h, out = h0.clone().to(DEV), torch.empty(rows, hidden, dtype=dtype, device=DEV)
    ops.tanh_norm_fold(h, y.to(DEV), dev(post), dev(pre), out, join=(y2.to(DEV), w1.to(DEV), w2.to(DEV), eps))
    assert rel_err(h, want_j) < 2e-6 and rel_err(out, norm(want_j, pre)) < tol
    h, out = h0.clone().to(DEV), torch.empty(3, hidden, dtype=dtype, device=DEV)
    ops.tanh_norm_fold(h, y.to(DEV), dev(post), dev(pre), out, row_idx=idx.to(DEV), join=(y2.to(DEV), w1.to(DEV), w2.to(DEV), eps))
    assert torch.equal(h.cpu(), h0) and rel_err(out, norm(want_j, pre)[idx.long()]) < tol
    # the norm on its own, of rows of either type
    for x in (h0, y):
        out = torch.empty(rows, hidden, dtype=dtype, device=DEV)
        ops.tanh_norm(x.to(DEV), pre[0], pre[1].to(DEV), pre[2].to(DEV), out)
        assert rel_err(out, norm(x, pre)) < tol


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("rows,hidden,eps", [(1, 40, 1e-5), (9, 176, 1e-6), (4, 73, 1e-4), (2, 2048, 1e-5)])
def test_two_branches_joined_by_their_unit_rows(dtype, rows, hidden, eps):
    """(U(x) wx + U(z) wz) / 2; one input so small that the epsilon inside the root shows."""
    from zedinfer_b200 import ops
    g = torch.Generator().manual_seed(hidden)
    x = torch.randn(rows, hidden, generator=g).to(dtype)
    z = (torch.randn(rows, hidden, generator=g) * 2e-3).to(dtype)
    wx, wz = 1 + 0.3 * torch.randn(hidden, generator=g), 1 + 0.3 * torch.randn(hidden, generator=g)
    out = torch.empty(rows, hidden, dtype=dtype, device=DEV)
    ops.rms_pair_mean(x.to(DEV), z.to(DEV), wx.to(DEV), wz.to(DEV), eps, out)
    ref = 0.5 * (SP.rms_unit(x.double(), eps) * wx.double() + SP.rms_unit(z.double(), eps) * wz.double())
    assert rel_err(out, ref) < tol_part(dtype, 3e-6, 1e-2)
    # the premise: without the epsilon the small input would weigh as much as the other
    assert float((SP.rms_unit(z.double(), 0.0) - SP.rms_unit(z.double(), eps)).abs().max()) > 0.05


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("rows,width", [(1, 8), (6, 80), (3, 257), (2, 8960), (40, 36)])
def test_an_activation_of_normed_powers(dtype, rows, width):
    from zedinfer_b200 import ops
    g = torch.Generator().manual_seed(width)
    wide = (torch.randn(rows, width + 8, generator=g) * 1.5).to(dtype).to(DEV)
    z = wide[:, 3:3 + width] if dtype == torch.float32 else wide[:, 8:8 + width]           # rows may be strided
    coeffs, eps = (0.8, -0.4, 0.25, 0.1), 1e-5
    out = torch.empty(rows, width, dtype=dtype, device=DEV)
    ops.poly_norm(z, coeffs, eps, out)
    zd = z.double().cpu()
    ref = coeffs[0] * SP.rms_unit(zd, eps) + coeffs[1] * SP.rms_unit(zd ** 2, eps) + coeffs[2] * SP.rms_unit(zd ** 3, eps) + coeffs[3]
    assert rel_err(out, ref) < tol_part(dtype, 3e-6, 1e-2)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("rows,k", [(11, 200), (1, 52), (70, 1536), (9, 73)])
def test_a_gate_per_row(dtype, rows, k):
    from zedinfer_b200 import ops
    g = torch.Generator().manual_seed(3)
    x, w = torch.randn(rows, k, generator=g).to(dtype), (torch.randn(k, generator=g) * 0.1).to(dtype)
    out = torch.empty(rows, dtype=torch.float32, device=DEV)
    ops.row_gate(x.to(DEV), w.to(DEV), out)
    assert rel_err(out, SP.logistic(x.double() @ w.double())) < 3e-6


@pytest.mark.parametrize("experts,top", [(14, 2), (5, 5), (3, 1), (40, 6), (2, 2)])
def test_scores_over_all_experts_and_a_bias_on_the_choice_alone(experts, top):
    """The weights are the softmax over ALL experts at the chosen ones, not renormalised; the bias moves the choice and not
    the weights; the lowest index wins a tie.  From logits, and from the fused router."""
    from zedinfer_b200 import ops
    g = torch.Generator().manual_seed(experts)
    n, k = 37, 48
    x = torch.randn(n, k, generator=g)
    wr = torch.randn(experts, k, generator=g) * 0.3
    wr[1 % experts] = wr[0]                                          # experts 0 and 1 tie everywhere
    corr = torch.randn(experts, generator=g) * 0.2
    corr[1 % experts] = corr[0]
    z = x.double() @ wr.double().T
    s = torch.softmax(z, dim=-1)
    pick = s + corr.double()
    order = torch.stack([torch.tensor(sorted(range(experts), key=lambda e: (-float(pick[t, e]), e))[:top]) for t in range(n)])
    for fused in (False, True):
        idx = torch.empty(n, top, dtype=torch.int32, device=DEV)
        wts = torch.empty(n, top, dtype=torch.float32, device=DEV)
        if fused:
            ops.route(x.to(DEV), wr.to(DEV), None, top, idx, wts, score="softmax_all", choice_bias=corr.to(DEV))
        else:
            ops.route_topk(z.float().to(DEV), top, idx, wts, score="softmax_all", choice_bias=corr.to(DEV))
        assert torch.equal(idx.cpu().long(), order), fused
        assert rel_err(wts, torch.gather(s, 1, order)) < 1e-5
    # the bias alone decides among equal scores, and without it the choice is by score
    idx = torch.empty(n, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(n, top, dtype=torch.float32, device=DEV)
    ops.route_topk(z.float().to(DEV), top, idx, wts, score="softmax_all")
    plain_order = torch.stack([torch.tensor(sorted(range(experts), key=lambda e: (-float(s[t, e]), e))[:top]) for t in range(n)])
    assert torch.equal(idx.cpu().long(), plain_order)


@pytest.mark.parametrize("dtype", BOTH)
def test_pairs_of_experts_without_weights_get_no_row_and_return_the_input(dtype):
    from zedinfer_b200 import ops
    n, top, real, hidden = 9, 3, 4, 40
    g = torch.Generator().manual_seed(1)
    idx = torch.stack([torch.randperm(real + 2, generator=g)[:top] for _ in range(n)]).to(torch.int32)
    pairs = n * top
    offsets = torch.empty(real + 1, dtype=torch.int32, device=DEV)
    row_pair = torch.full((pairs,), -7, dtype=torch.int32, device=DEV)
    pair_row = torch.empty(pairs, dtype=torch.int32, device=DEV)
    ops.moe_group(idx.to(DEV), real, offsets, row_pair, pair_row)
    flat = idx.reshape(-1)
    placed = int((flat < real).sum())
    pr = pair_row.cpu()
    assert int(offsets[-1]) == placed and bool((pr[flat >= real] == -1).all()) and sorted(pr[flat < real].tolist()) == list(range(placed))
    for e in range(real):
        rows = row_pair.cpu()[int(offsets[e]):int(offsets[e + 1])]
        assert bool((flat[rows.long()] == e).all())
    y = torch.randn(pairs, hidden, generator=g).to(dtype)
    x = torch.randn(n, hidden, generator=g).to(dtype)
    shared = torch.randn(n, hidden, generator=g).to(dtype)
    wts, gate = torch.rand(n, top, generator=g), torch.rand(n, generator=g)
    out = torch.empty(n, hidden, dtype=dtype, device=DEV)
    ops.moe_combine(y.to(DEV), pair_row.view(n, top), wts.to(DEV), shared.to(DEV), out, x=x.to(DEV), shared_gate=gate.to(DEV))
    ref = gate.double()[:, None] * shared.double()
    for t in range(n):
        for j in range(top):
            r = int(pr[t * top + j])
            ref[t] += wts[t, j].double() * (y[r].double() if r >= 0 else x[t].double())
    assert rel_err(out, ref) < tol_part(dtype, 2e-6, 1e-2)


def plain_walk(rule, q, k, v, heads, kv, dim, vdim, s0=None, beta=None, g=None):
    """The recurrence token by token in float64 on what enters it: ``q, k [T, kv, dim]``, ``v [T, heads, vdim]``, decays ``g``
    ``[T, heads]`` (delta) or gates ``[T, heads, dim]`` (forget, where the key is 1 - gate)."""
    t = q.shape[0]
    o = torch.zeros(t, heads, vdim, dtype=F64)
    s_end = torch.zeros(heads, dim, vdim, dtype=F64)
    for a in range(heads):
        s = torch.zeros(dim, vdim, dtype=F64) if s0 is None else s0[a].clone()
        c = a // (heads // kv)
        for i in range(t):
            if rule == "delta":
                s = g[i, a] * s
                u = beta[i, a] * (v[i, a] - s.T @ k[i, c])
                s = s + torch.outer(k[i, c], u)
            else:
                s = g[i, a][:, None] * s + torch.outer(1.0 - g[i, a], v[i, a])
            o[i, a] = s.T @ q[i, c]
        s_end[a] = s
    return o, s_end


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("rule", ["delta", "forget"])
@pytest.mark.parametrize("heads,kv,dim,vdim", [(4, 2, 16, 24), (3, 1, 136, 12), (2, 2, 72, 8), (1, 1, 8, 136), (6, 3, 40, 20), (2, 1, 200, 17)])
def test_the_matrix_state_with_one_decay_per_head_and_with_a_forget_gate(dtype, rule, heads, kv, dim, vdim):
    """Three segments of unequal length (one of a single token, one that starts from a state the slot already holds, one
    without a slot) through the walk that makes its own inputs ready and through the one that finds them made ready in a
    workspace: both equal the plain walk, leave the same state behind, and equal each other bit by bit."""
    from zedinfer_b200 import ops
    if rule == "forget":
        kv = heads
    g0 = torch.Generator().manual_seed(dim * 7 + vdim)
    lens = [37, 1, 50]
    n = sum(lens)
    q = torch.randn(n, kv * dim, generator=g0).to(dtype)
    k = torch.randn(n, kv * dim, generator=g0).to(dtype)
    v = torch.randn(n, heads * vdim, generator=g0).to(dtype)
    b = torch.randn(n, heads, generator=g0).to(dtype)
    a_log = torch.linspace(-2.0, 0.5, heads)
    if rule == "delta":
        a = (torch.randn(n, heads, generator=g0) * 2).to(dtype)
        dt_bias = torch.randn(heads, generator=g0)
    else:
        a = (torch.randn(n, heads * dim, generator=g0) * 2).to(dtype)
        dt_bias = torch.rand(heads * dim, generator=g0) * 0.9                      # the gates' lower bounds
    entries = heads * vdim * dim + 11
    start = torch.randn(heads, vdim, dim, generator=g0) * 0.2
    bounds = torch.tensor([[0, 37], [37, 38], [38, 88]], dtype=torch.int32, device=DEV)
    slots = torch.tensor([2, -1, 0], dtype=torch.int32, device=DEV)
    qd, kd, vd = q.double().view(n, kv, dim), k.double().view(n, kv, dim), v.double().view(n, heads, vdim)
    if rule == "delta":
        qd = qd / torch.sqrt((qd * qd).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
        kd = kd / torch.sqrt((kd * kd).sum(-1, keepdim=True) + 1e-6)
        beta = SP.logistic(b.double())
        gd = torch.exp(-torch.exp(a_log.double())[None, :] * SP.softplus(a.double() + dt_bias.double()))
    else:
        qd = SP.silu(qd) * 0.5
        beta = None
        low = dt_bias.double().view(heads, dim)
        gd = low + (1.0 - low) * SP.logistic(a.double().view(n, heads, dim))
    refs, ends, at = [], [], 0
    for i, ln in enumerate(lens):
        s0 = start.double().transpose(1, 2) if i == 2 else None
        sl = slice(at, at + ln)
        o, e = plain_walk(rule, qd[sl], kd[sl], vd[sl], heads, kv, dim, vdim, s0, None if beta is None else beta[sl], gd[sl])
        refs.append(o.reshape(ln, heads * vdim))
        ends.append(e)
        at += ln
    ref = torch.cat(refs)
    results = []
    for with_work in (False, True):
        state = torch.full((3, entries), 7.0, device=DEV)
        state[0, :heads * vdim * dim] = start.reshape(-1).to(DEV)
        state[2, :heads * vdim * dim] = 0.0
        y = torch.empty(n, heads * vdim, dtype=torch.float32, device=DEV)
        work = torch.empty(ops.linear_state_work_floats(rule, n, heads, dim, vdim), dtype=torch.float32, device=DEV) if with_work else None
        if rule == "delta":
            ops.linear_state("delta", q.to(DEV), k.to(DEV), v.to(DEV), state, slots, bounds, y, 3, heads, kv, dim, vdim, a=a.to(DEV),
                             b=b.to(DEV), dt_bias=dt_bias.to(DEV), a_log=a_log.to(DEV), q_scale=dim ** -0.5, unit_eps=1e-6, work=work,
                             decay_per_head=True)
        else:
            ops.linear_state("forget", q.to(DEV), None, v.to(DEV), state, slots, bounds, y, 3, heads, heads, dim, vdim, a=a.to(DEV),
                             dt_bias=dt_bias.to(DEV), act_silu="q", q_scale=0.5, work=work)
        tol = tol_part(dtype, 2e-5, 2e-5)                  # the inputs are what they are in either type; the walk is float32
        assert rel_err(y, ref) < tol, with_work
        got_end = state[:, :heads * vdim * dim].view(3, heads, vdim, dim).transpose(2, 3).cpu()
        assert rel_err(got_end[2], ends[0]) < tol and rel_err(got_end[0], ends[2]) < tol
        assert bool((state[:, heads * vdim * dim:] == 7.0).all()) and bool((state[1] == 7.0).all())        # nothing else is touched
        results.append((y.clone(), state.clone()))
    assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("gate", ["silu", None, "sigmoid"])
@pytest.mark.parametrize("inner,groups,wlen", [(48, 4, 12), (96, 1, 96), (1200, 3, 400), (20, 20, 1)])
def test_unit_groups_times_weight_times_a_gate_of_three_kinds(dtype, gate, inner, groups, wlen):
    from zedinfer_b200 import ops
    g = torch.Generator().manual_seed(inner)
    n, eps = 5, 1e-5
    y = torch.randn(n, inner, generator=g) * 3
    z = torch.randn(n, inner, generator=g).to(dtype)
    w = (1 + 0.2 * torch.randn(wlen, generator=g)).to(dtype)
    out = torch.empty(n, inner, dtype=dtype, device=DEV)
    ops.group_rmsnorm_gate(y.to(DEV), z.to(DEV) if gate else None, w.to(DEV), groups, eps, out, gate=gate)
    ref = SP.rms_unit(y.double().view(n, groups, -1), eps).view(n, inner) * w.double().repeat(inner // wlen)
    if gate:
        ref = ref * (SP.silu(z.double()) if gate == "silu" else SP.logistic(z.double()))
    assert rel_err(out, ref) < tol_part(dtype, 3e-6, 1e-2)


# ---------------------------------------------------------------------------------------------
# mixers and feed-forwards alone
# ---------------------------------------------------------------------------------------------
SCHEDULE_ABC = [[("a", 6), ("b", 2)], [("b", 1), ("a", 1)], [("a", 1)], [("a", 2), ("b", 7), "end:b"], [("c", 3), ("a", 20)],
                [("c", 1), ("a", 1)], [("c", 8), ("a", 14)]]


def three_requests(hidden, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return {"a": torch.randn(45, hidden, generator=g).to(dtype), "b": torch.randn(10, hidden, generator=g).to(dtype),
            "c": torch.randn(12, hidden, generator=g).to(dtype)}


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("heads,kv,dim,vdim,taps", [(4, 2, 16, 24, 3), (3, 1, 136, 12, 2), (2, 2, 72, 8, 1), (6, 3, 40, 20, 4), (1, 1, 8, 70, 6)])
def test_delta_rule_with_a_decay_per_head_over_portions_and_slots_used_again(dtype, heads, kv, dim, vdim, taps):
    """Two requests in shared steps, cut down to single tokens, then a third in the slot the second gave back: it starts
    from zeros (state and the convolution's last inputs), not from what the slot last held."""
    from zedinfer_b200.cache import CacheManager
    from zedinfer_b200.parts import GatedDeltaMixer
    hidden, eps = 64, 1e-5
    mixer = GatedDeltaMixer(hidden, heads, kv, dim, vdim, taps, eps)
    assert mixer.tensor_specs()["dt_bias"].shape == (heads,) and mixer.tensor_specs()["a"].shape == (heads, hidden)
    over = {"A_log": torch.linspace(-3.0, 0.5, heads), "dt_bias": torch.linspace(-3.0, 1.0, heads), "norm": 1 + 0.1 * torch.randn(vdim)}
    t = bind_random(mixer, dtype, seed=dim, scale=0.3, overrides=over)
    cache = CacheManager([(0, mixer.cache_need())], 16, max_requests=2)
    cache.allocate_device(1, dtype, DEV)
    view = cache.view_for_call(0)
    assert view.kind == "state"
    xs = three_requests(hidden, dtype, 5)
    got, = feed([mixer], [view], cache, dtype, xs, SCHEDULE_ABC)
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": taps}
    for rid, x in xs.items():
        assert rel_err(got[rid], SP.gated_delta(x.double(), t, "", m, eps)) < tol_part(dtype), rid


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("heads,dim,vdim", [(3, 16, 24), (1, 40, 20), (4, 8, 136), (2, 136, 16), (5, 40, 64), (1, 256, 4)])
def test_forget_gate_mixer_over_portions_and_slots_used_again(dtype, heads, dim, vdim):
    from zedinfer_b200.cache import CacheManager
    from zedinfer_b200.parts import ForgetGateMixer
    hidden, eps = 64, 1e-5
    mixer = ForgetGateMixer(hidden, heads, dim, vdim, eps)
    over = {"lower": torch.rand(heads * dim) * 0.95, "norm": 1 + 0.1 * torch.randn(vdim), "f.b": torch.randn(heads * dim)}
    t = bind_random(mixer, dtype, seed=dim, scale=0.3, overrides=over)
    cache = CacheManager([(0, mixer.cache_need())], 16, max_requests=2)
    cache.allocate_device(1, dtype, DEV)
    view = cache.view_for_call(0)
    xs = three_requests(hidden, dtype, 6)
    got, = feed([mixer], [view], cache, dtype, xs, SCHEDULE_ABC)
    m = {"heads": heads, "dim": dim, "vdim": vdim}
    for rid, x in xs.items():
        assert rel_err(got[rid], SP.forget_gate_recurrence(x.double(), t, "", m, eps)) < tol_part(dtype), rid


def _left(hidden, heads, kv, dim, vdim, window, rot_dims, base, scale):
    from zedinfer_b200.config import PartSpec
    from zedinfer_b200.parts import AttentionMixer
    position = PartSpec("rope_span", {"head_dim": dim, "dims": rot_dims, "theta": base, "interleaved": False})
    return AttentionMixer(hidden, heads, kv, dim, position, qkv_bias=True, scale=scale, window=window, v_head_dim=vdim, head_scale="temp",
                          names={"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b"})


def _left_m(heads, kv, dim, vdim, window, rot_dims, base, scale):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "rot": {"dims": rot_dims, "base": base}, "scale": scale,
            "mask": {"size": window}}


SCHEDULE_AB = [[("a", 9), ("b", 2)], [("b", 1), ("a", 1)], [("a", 1)], [("a", 33), ("b", 15)], [("b", 1)], [("a", 2)], [("a", 15)]]


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("heads,kv,dim,vdim,window,rot_dims,base,page", [
    (4, 2, 32, 16, 13, 16, 5000.0, 4), (2, 1, 64, 64, 40, 64, 10000.0, 16), (4, 4, 128, 128, 21, 32, 300.0, 16), (3, 3, 24, 40, 3, 2, 77.0, 8),
    (8, 2, 64, 128, 29, 24, 2e5, 16), (1, 1, 8, 8, 1, 8, 10.0, 8)])
def test_windowed_attention_with_biases_and_a_number_per_head(dtype, heads, kv, dim, vdim, window, rot_dims, base, page):
    """Over portions and single tokens of two requests in shared steps; the heads' numbers differ widely, so one that is
    left out or given to the wrong head shows."""
    from zedinfer_b200.cache import CacheManager
    hidden = 80
    scale = 1.0 / dim                                          # scores of a few units however wide the head
    mixer = _left(hidden, heads, kv, dim, vdim, window, rot_dims, base, scale)
    t = bind_random(mixer, dtype, seed=dim + heads, scale=0.2, overrides={"temp": torch.linspace(0.3, 4.0, heads)})
    cache = CacheManager([(0, mixer.cache_need())], page, max_requests=2)
    cache.allocate_device(40, dtype, DEV)
    view = cache.view_for_call(0)
    g = torch.Generator().manual_seed(7)
    xs = {"a": torch.randn(61, hidden, generator=g).to(dtype), "b": torch.randn(19, hidden, generator=g).to(dtype)}
    got, = feed([mixer], [view], cache, dtype, xs, SCHEDULE_AB)
    m = _left_m(heads, kv, dim, vdim, window, rot_dims, base, scale)
    for rid, x in xs.items():
        ref = SP.window_attention(x.double(), t, "", m)
        assert rel_err(got[rid], ref) < tol_part(dtype, 2e-5, 3e-2), rid
        if heads > 1 and window > 1:
            flat = dict(t, temp=torch.ones(heads, dtype=F64))
            assert rel_err(SP.window_attention(x.double(), flat, "", m), ref) > 3 * tol_part(dtype, 2e-5, 3e-2)      # the premise


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("dim,vdim,window,page,rot_dims,base", [(32, 24, 150, 16, 16, 50.0), (64, 128, 97, 8, 32, 300.0), (128, 128, 256, 16, 64, 1000.0),
                                                              (16, 24, 580, 4, 16, 20.0), (64, 64, 80, 16, 24, 2e5)])
def test_one_key_answers_just_inside_the_window_and_none_just_outside(dtype, dim, vdim, window, page, rot_dims, base):
    """One head whose scores rest on the turned span alone, 600 tokens.  A query aligned with the key that is window - 1
    tokens back gets that key's value; one aligned with the key window tokens back does not (all its other scores are zero, it
    gets the mean of what it sees).  Asked from inside a prompt's portion and by tokens fed alone, across page borders; with a
    window of 580 a key 560 back answers among hundreds."""
    from zedinfer_b200.cache import CacheManager
    total = 600
    hidden = 2 * dim + vdim                                    # x = [query row | key row | value marks]
    half = rot_dims // 2
    scale = 200.0 / half                                       # an aligned pair scores 200 (the head's number is 1), its neighbours clearly less
    mixer = _left(hidden, 1, 1, dim, vdim, window, rot_dims, base, scale)
    wq, wk, wv = torch.zeros(dim, hidden), torch.zeros(dim, hidden), torch.zeros(vdim, hidden)
    wq[:, :dim] = torch.eye(dim)
    wk[:, dim:2 * dim] = torch.eye(dim)
    wv[:, 2 * dim:] = torch.eye(vdim)
    wo = torch.eye(hidden, vdim)
    tensors = {"q": wq, "k": wk, "v": wv, "o": wo, "q.b": torch.zeros(dim), "k.b": torch.zeros(dim), "v.b": torch.zeros(vdim), "temp": torch.ones(1)}
    mixer.bind({k: v.to(dtype).to(DEV) for k, v in tensors.items()})
    inside = {599: 599 - (window - 1), 450: max(450 - (window - 1), 1), 598: 598 - (window - 1)}
    outside = {597: 597 - window, 596: 596 - window} if window < 500 else {}
    asks = {**inside, **outside}
    raw = torch.zeros(dim, dtype=F64)
    raw[:half] = 1.0                                           # the first entry of every pair
    keys, queries = torch.zeros(total, dim, dtype=F64), torch.zeros(total, dim, dtype=F64)
    for p_query, j in asks.items():
        keys[j] = raw
        # turned by its own position P the query becomes the raw row turned by j, which is what the key at j becomes
        queries[p_query] = SP.turn_span(raw[None, None], torch.tensor([j - p_query]), rot_dims, base)[0, 0]
    marks = torch.randn(total, vdim, generator=torch.Generator().manual_seed(dim)).double()
    x = torch.cat([queries, keys, marks], dim=1).to(dtype)
    cache = CacheManager([(0, mixer.cache_need())], page, max_requests=1)
    cache.allocate_device(total // page + 2, dtype, DEV)
    view = cache.view_for_call(0)
    schedule = [[("r", 200)], [("r", 395)]] + [[("r", 1)]] * 5
    got, = feed([mixer], [view], cache, dtype, {"r": x}, schedule, table_width=160)
    got = got["r"]
    xd = x.double()
    ref = SP.window_attention(xd, {k: v.double() for k, v in tensors.items()}, "", _left_m(1, 1, dim, vdim, window, rot_dims, base, scale))
    tol = 1e-3 if dtype == torch.float32 else 3e-2
    assert rel_err(got[:, :vdim], ref[:, :vdim]) < tol
    vals = xd[:, 2 * dim:]
    for p_query, j in asks.items():
        if p_query in inside:
            assert rel_err(ref[p_query, :vdim], vals[j]) < 2e-2                 # the test's own premise: that key alone answers
            assert rel_err(got[p_query, :vdim], vals[j]) < 5e-2, (p_query, j)
        else:
            assert float((ref[p_query, :vdim] - vals[j]).abs().max()) > 0.5      # premise: it does not answer
            assert float((got[p_query, :vdim].double().cpu() - vals[j]).abs().max()) > 0.5, (p_query, j)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("hidden,ff", [(64, 80), (52, 36), (160, 224), (48, 8)])
def test_feed_forward_of_normed_powers(dtype, hidden, ff):
    from zedinfer_b200.parts import PolyNormMLP
    part = PolyNormMLP(hidden, ff, 1e-5)
    t = bind_random(part, dtype, seed=ff, scale=0.3, overrides={"act": torch.tensor([0.9, -0.5, 0.3, 0.2])})
    g = torch.Generator().manual_seed(2)
    for n in (3, 70):
        x = torch.randn(n, hidden, generator=g).to(dtype)
        ctx = _bare_context(n, dtype)
        got = part.forward(x.to(DEV), ctx)
        assert rel_err(got, SP.poly_norm_ff(x.double(), t, "", 1e-5)) < tol_part(dtype, 3e-5, 4e-2)


def _bare_context(n, dtype):
    from zedinfer_b200.parts import StepContext
    dev = torch.device(DEV)
    z = torch.zeros(n, dtype=torch.int32, device=dev)
    return StepContext(n_tokens=n, n_segments=1, dtype=dtype, device=dev, token_ids=z, positions=z, tok_seg=z, tables=[], slots=None,
                       seg_start_host=[0], seg_len_host=[n], seg_pos0_host=[0], slots_host=[-1])


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("experts,identity,top,ff,shared", [(10, 3, 2, 80, 112), (5, 1, 6, 24, 40), (3, 2, 1, 24, None), (1, 1, 2, 8, None), (4, 0, 3, 32, 16)])
@pytest.mark.parametrize("tokens", [5, 150])
def test_routed_feed_forward_with_experts_that_return_their_input(dtype, experts, identity, top, ff, shared, tokens):
    """Few tokens (the weight-streaming grouped product) and many (the tensor-core one in bfloat16).  In bfloat16 the part's
    own choice is given to the plain implementation: a close call that rounding turns is no fault of the products."""
    from zedinfer_b200.config import PartSpec
    from zedinfer_b200.parts import RoutedExperts
    hidden = 64
    part = RoutedExperts(hidden, ff, experts, top, limit=None, router_bias=False, score="softmax_all", choice_bias_name="correction",
                         identity=identity, shared=PartSpec("clamped_gated_mlp", {"hidden_size": hidden, "intermediate_size": shared, "limit": None})
                         if shared else None, shared_gate_name="sg" if shared else None)
    t = bind_random(part, dtype, seed=experts * 10 + top, scale=0.25, overrides={"correction": torch.randn(experts + identity) * 0.05})
    x = torch.randn(tokens, hidden, generator=torch.Generator().manual_seed(tokens)).to(dtype)
    got = part.forward(x.to(DEV), _bare_context(tokens, dtype))
    idx, wts = part.route(x.to(DEV))
    f = {"router": {"experts": experts, "identity": identity, "top": top}, "shared": {"ff": shared} if shared else None}
    xd = x.double()
    ref_idx, ref_w = SP.router_choice(xd, t, "", top)
    if dtype == torch.float32:
        assert torch.equal(idx.cpu().long(), ref_idx) and rel_err(wts, ref_w) < 1e-5
        ref = SP.routed_ff(xd, t, "", f)
    else:
        s = torch.softmax(xd @ t["router"].T, dim=-1)
        ref = torch.zeros_like(xd)
        for n in range(tokens):
            for j in range(top):
                e = int(idx[n, j])
                ref[n] += s[n, e] * (SP.gated_ff(xd[n:n + 1], t, f"e{e}.")[0] if e < experts else xd[n])
        if shared:
            ref = ref + SP.logistic(xd @ t["shared.sg"].T) * SP.gated_ff(xd, t, "shared.")
    assert rel_err(got, ref) < tol_part(dtype, 3e-5, 4e-2)


# ---------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """float32 runs take the configurations as they are; bfloat16 runs take them with every router choosing all of its
    outputs, since a choice that rounding turns moves every later token through the states."""
    root = tmp_path_factory.mktemp("sumitar_models")
    out = {name: ST.make_model_dir(root, name) for name in ST.CONFIGS}
    out.update({name + "_all": ST.make_model_dir(root, name, choose_all=True) for name in ST.CONFIGS})
    return out


def model_for(models, name, dtype):
    return models[name] if dtype == "float32" else models[name + "_all"]


def make_requests(cfg, lengths, seed):
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(cfg["vocab"]) for _ in range(n)] for i, n in enumerate(lengths)}


_plain_cache = {}


def expected_logits(model_dir, requests):
    if model_dir not in _plain_cache:
        _plain_cache[model_dir] = SP.read_model(model_dir, F64)
    cfg, w = _plain_cache[model_dir]
    return {rid: SP.forward(cfg, w, toks).float() for rid, toks in requests.items()}


def judge(got, exp, dtype):
    """float32: every position within the tolerance.  bfloat16: rounding errors have a tail, the same however the work is
    cut: at most 2 % of the positions may be beyond the tolerance, none beyond four times it."""
    tol = tol_for(dtype)
    errs = {key: float((row - exp[key[0]][key[1]]).abs().max()) / max(1.0, float(exp[key[0]].abs().max()))
            for key, row in got.items()}
    over = sorted((k for k, e in errs.items() if not e <= tol), key=lambda k: (str(k[0]), k[1]))
    allowed = 0 if dtype == "float32" else max(1, len(errs) // 50)
    assert len(over) <= allowed, f"{len(over)} of {len(errs)} positions beyond {tol}; first {over[0]} with {errs[over[0]]}"
    assert all(e <= 4 * tol for e in errs.values()), max(errs.values())


LENGTHS = {"A": [7, 13, 95, 45], "B": [1, 17, 120, 64], "C": [110, 5, 60], "D": [50, 2, 61], "E": [40, 3, 90], "F": [33, 1, 70]}
PAGES = {"A": 4, "B": 16, "C": 8, "D": 8, "E": 16, "F": 8}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
@pytest.mark.parametrize("family", ["whole", "tail", "chunks", "mixed"])
def test_cuts_match_plain(models, name, dtype, family):
    """Whole prompts; a tail decoded token by token; portions down to two tokens; mixed batches of unequal requests in a
    pool so small that pages and state slots are handed out again."""
    from zedinfer_b200.engine.core import EngineCore
    cfg, _ = ST.CONFIGS[name]
    requests = make_requests(cfg, LENGTHS[name] + ([64, 31, 77] if family == "mixed" else []), seed=5)
    if family == "tail":
        steps = traces.tail_decode(requests, tail=40)
    else:
        steps = {"whole": traces.whole, "chunks": traces.chunks, "mixed": traces.mixed}[family](requests)
    page = PAGES[name]
    need = traces.max_live_tokens(steps, round_to=page)
    folder = model_for(models, name, dtype)
    core = EngineCore(folder, dtype, page_size=page, num_pages=max(1, need // page), max_requests=4)
    got = run_trace(core, steps)
    core.check_kernels()
    judge(got, expected_logits(folder, requests), dtype)
    assert core.cache.num_live == 0 and all(g.pool.num_used == 0 for g in core.cache.groups)
    assert core.cache.slots.num_free_slots == core.cache.slots.num_slots


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("B", "bfloat16"), ("C", "bfloat16"), ("D", "bfloat16")])
def test_many_decoding_requests_with_and_without_graphs(models, name, dtype, graphs):
    """Steps as a scheduler makes them: up to 12 decoding requests beside one prompt portion, then decode-only steps whose
    number of rows falls to one; with graphs the decode-only steps replay captured buckets whose rows of padding hold no
    state slot."""
    from zedinfer_b200.engine.core import EngineCore
    cfg, _ = ST.CONFIGS[name]
    rng = random.Random(8)
    requests = make_requests(cfg, [rng.randint(40, 90) for _ in range(15)], seed=3)
    steps = traces.decode_heavy(requests, seed=4, max_live=12, tail=(8, 30), portion=32)
    need = traces.max_live_tokens(steps, round_to=16)
    folder = model_for(models, name, dtype)
    core = EngineCore(folder, dtype, page_size=16, num_pages=need // 16, max_requests=16, cuda_graphs=graphs)
    core.GPU_BOUND_RATIO = float("inf")
    assert core.capture_safe, core.capture_blockers
    got = run_trace(core, steps)
    core.check_kernels()
    judge(got, expected_logits(folder, requests), dtype)
    if graphs:
        assert core._decode_graphs
    assert core.cache.num_live == 0 and all(g.pool.num_used == 0 for g in core.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_the_first_tokens(models, dtype):
    """One token, two tokens, and a request decoded for 260 steps from a prompt of three: every window passes over decoded
    tokens many times, the matrix states and the convolution's last inputs go through hundreds of single-token steps."""
    from zedinfer_b200.engine.core import EngineCore
    cfg, _ = ST.CONFIGS["A"]
    requests = make_requests(cfg, [1, 2, 263], seed=9)
    steps = traces.tail_decode(requests, tail=260)
    folder = model_for(models, "A", dtype)
    core = EngineCore(folder, dtype, page_size=4, num_pages=80, max_requests=2)
    judge(run_trace(core, steps), expected_logits(folder, requests), dtype)


@pytest.mark.parametrize("name", ["A", "C", "D", "F"])
def test_float32_is_the_same_however_it_is_cut(models, name):
    """The same positions through four different schedules: the same bits (every float32 sum of the design has one order,
    which depends on constants alone; the recurrences run token by token whatever the portions)."""
    from zedinfer_b200.engine.core import EngineCore
    cfg, _ = ST.CONFIGS[name]
    requests = make_requests(cfg, [90, 41], seed=2)
    runs = []
    for steps in (traces.whole(requests), traces.tail_decode(requests, tail=20), traces.chunks(requests), traces.mixed(requests)):
        core = EngineCore(models[name], "float32", page_size=16, num_pages=40, max_requests=4)
        runs.append(run_trace(core, steps))
    for other in runs[1:]:
        assert all(torch.equal(other[k], runs[0][k]) for k in runs[0])


@pytest.mark.parametrize("name,graphs", [("A", False), ("A", True), ("B", True), ("C", False), ("D", True), ("F", True)])
def test_greedy_generation_equals_plain(models, name, graphs):
    """Through the Python entry point and its scheduler: prompts in portions of five, a pool of pages and three state
    slots that the requests fill again, greedy tokens equal to the plain implementation's."""
    from zedinfer_b200 import GenerationConfig, SchedulerConfig
    from zedinfer_b200.engine import InferenceEngine
    cfg, _ = ST.CONFIGS[name]
    rng = random.Random(4)
    prompts = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (9, 23, 1, 14, 6)]
    engine = InferenceEngine.create(models[name], SchedulerConfig(num_kv_pages=30, kv_block_size=4, max_batch_requests=3,
                                                                  max_prefill_tokens=5, cuda_graphs=graphs),
                                    dtype="float32")
    results = engine.generate_batch(prompts, GenerationConfig(max_new_tokens=20, ignore_eos=True))
    pcfg, w = SP.read_model(models[name], F64)
    for p, r in zip(prompts, results):
        assert r.finish_reason == "length"
        assert r.output_ids == SP.greedy(pcfg, w, p, 20)
    st = engine.cache_stats()
    assert st["live_requests"] == 0 and st["free_pages"] == st["pages_per_group"]


@pytest.mark.parametrize("name,dtype", [("B", "bfloat16"), ("B", "float32"), ("D", "float32"), ("E", "bfloat16")])
def test_trace_program_on_a_sumitar_folder(models, tmp_path, name, dtype):
    """The program on a folder with both kinds of layer, on one without a paged cache and on one without delta-rule layers."""
    cfg, _ = ST.CONFIGS[name]
    requests = make_requests(cfg, [70, 9, 33, 50, 21], seed=6)
    steps = traces.mixed(requests, seed=1)
    need = traces.max_live_tokens(steps, round_to=64)
    out = tmp_path / "out"
    folder = model_for(models, name, dtype)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                           "--out", str(out), "--max-tokens", str(need)],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    got, progress = {}, {}
    for st in steps:
        rows = np.fromfile(out / f"{st['step']}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        row = 0
        for e in st["entries"]:
            base = progress.get(e["id"], 0)
            for j in e["want"]:
                got[(e["id"], base + j)] = torch.from_numpy(rows[row].copy())
                row += 1
            progress[e["id"]] = base + len(e["tokens"])
        assert row == rows.shape[0]
    judge(got, expected_logits(folder, requests), dtype)


def test_command_line_programs_take_the_design(tmp_path, capsys):
    """From a bare config.json with weights drawn on the device: the bench program, continuous batching, and the
    consistency program, which returns 0 only if every float32 logit is the same bit pattern however the work is cut."""
    from zedinfer_b200.cli import batch_bench, bench, consistency
    path = tmp_path / "config.json"
    path.write_text(json.dumps(ST.SM_A))
    common = [str(path), "--random-weights", "7", "--kv-pages", "40", "--max-seq-len", "128"]
    assert bench.main(common + ["-p", "24", "-d", "5", "-r", "1"]) == 0
    out = capsys.readouterr().out
    assert "Prefill:" in out and "Decode :" in out
    assert batch_bench.main(common + ["-b", "5", "-p", "6", "--prefill-len-max", "40", "-d", "7", "-r", "1",
                                      "--warmup-rounds", "1", "--max-prefill-tokens", "16"]) == 0
    assert "5 requests, 35 tokens generated" in capsys.readouterr().out
    assert consistency.main([str(path), "--random-weights", "5", "--tokens", "120", "--requests", "5"]) == 0
    lines = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert all(l["values_not_bit_equal"] == 0 for l in lines if l["dtype"] == "float32")
