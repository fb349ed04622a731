"""Kevatar in the engine against the plain implementation (tests/plain/kevatar_plain.py): every mechanism alone, then
whole models under every way of cutting the work, long decoding, generation through the Python entry point, the trace
program and the command-line programs."""
import json
import math
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

import kevatar_tiny as KT
import traces
from plain import kevatar_plain as KP
from replay_util import run_trace

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F64 = torch.float64


def tol_for(dtype):
    return 2e-4 if dtype in ("float32", torch.float32) else 6e-2


def rel_err(got, ref):
    """Largest difference relative to the size of the reference (at least 1)."""
    return float((got.double().cpu() - ref.double()).abs().max()) / max(1.0, float(ref.abs().max()))


def step_context(cache, dtype, portions, table_width=64):
    """A step's context for ``portions = [(request id, tokens), ...]`` on ``cache`` (requests are opened as they appear)."""
    from zedinfer_b200.engine.core import PinnedStaging, StepEntry, build_step_context
    entries, rcs = [], []
    for rid, n in portions:
        rc = cache.get(rid) or cache.open(rid)
        cache.ensure(rc, rc.length + n)
        entries.append(StepEntry(rid, [0] * n, []))
        rcs.append(rc)
    ctx, _ = build_step_context(entries, rcs, cache, table_width, dtype, torch.device(DEV), 10, PinnedStaging())
    return ctx, entries, rcs


def feed(mixers, cache, view, dtype, xs, schedule, table_width=64):
    """Run ``mixers`` (the first owns the cache, the others read it with queries of their own) over the requests ``xs = {id:
    [T, hidden]}`` cut as ``schedule = [[(id, tokens), ...], ...]`` says (a step may hold portions of several requests;
    ``"end:<id>"`` closes one); returns one ``{id: [T, hidden]}`` per mixer."""
    mixers = mixers if isinstance(mixers, (list, tuple)) else [mixers]
    done = {rid: 0 for rid in xs}
    outs = [{rid: [] for rid in xs} for _ in mixers]
    for step in schedule:
        portions = [p for p in step if not isinstance(p, str)]
        if portions:
            ctx, entries, rcs = step_context(cache, dtype, portions, table_width)
            x = torch.cat([xs[rid][done[rid]:done[rid] + n] for rid, n in portions]).to(DEV)
            ys = [m.forward(x, ctx, view, owns_cache=(i == 0)).cpu() for i, m in enumerate(mixers)]
            at = 0
            for (rid, n), rc in zip(portions, rcs):
                for out, y in zip(outs, ys):
                    out[rid].append(y[at:at + n])
                at += n
                done[rid] += n
                cache.commit(rc, rc.length + n)
        for p in step:
            if isinstance(p, str):
                cache.close(cache.get(p[4:]))
    res = [{rid: torch.cat(v) for rid, v in out.items() if v} for out in outs]
    return res if len(res) > 1 else res[0]


def bind_random(part, dtype, seed, scale=0.3, overrides=None):
    """Random tensors for a part (its own names), bound on the device; returns them as float64 on the host."""
    g = torch.Generator().manual_seed(seed)
    t = {k: (torch.randn(v.shape, generator=g) * scale).to(dtype) for k, v in part.tensor_specs().items()}
    for k, v in (overrides or {}).items():
        t[k] = v.to(dtype)
    part.bind({k: v.to(DEV) for k, v in t.items()})
    return {k: v.double() for k, v in t.items()}


# ---------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------
def plain_walk(rule, q, k, v, heads, kv, dim, vdim, s0=None, beta=None, g=None, lam=None):
    """The recurrence token by token in float64: ``q, k [T, kv, dim]``, ``v [T, heads, vdim]`` as they enter it."""
    t = q.shape[0]
    o = torch.zeros(t, heads, vdim, dtype=F64)
    s_end = torch.zeros(heads, dim, vdim, dtype=F64)
    for a in range(heads):
        s = torch.zeros(dim, vdim, dtype=F64) if s0 is None else s0[a].clone()
        c = a // (heads // kv)
        for i in range(t):
            if rule == "delta":
                s = g[i, a][:, None] * s
                u = beta[i, a] * (v[i, a] - s.T @ k[i, c])
            else:
                s = lam[a] * s
                u = v[i, a]
            s = s + torch.outer(k[i, c], u)
            o[i, a] = s.T @ q[i, c]
        s_end[a] = s
    return o, s_end


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rule", ["delta", "decay"])
@pytest.mark.parametrize("heads,kv,dim,vdim", [(4, 2, 16, 24), (3, 1, 136, 12), (2, 2, 72, 8), (1, 1, 8, 136), (6, 3, 40, 20), (2, 1, 200, 17)])
def test_the_matrix_state_walks_token_by_token_in_either_form(dtype, rule, heads, kv, dim, vdim):
    """Three segments of unequal length (one of a single token, one that starts from a state the slot already holds, one
    without a slot) through the walk that makes its own inputs ready and through the one that finds them made ready in a
    workspace: both equal the plain walk, leave the same state behind, and equal each other bit by bit."""
    from zedinfer_b200 import ops
    if rule == "decay":
        kv = heads
    g0 = torch.Generator().manual_seed(dim * 7 + vdim)
    lens = [37, 1, 50]
    n = sum(lens)
    q = torch.randn(n, kv * dim, generator=g0).to(dtype)
    k = torch.randn(n, kv * dim, generator=g0).to(dtype)
    v = torch.randn(n, heads * vdim, generator=g0).to(dtype)
    a = (torch.randn(n, heads * dim, generator=g0) * 2).to(dtype)
    b = torch.randn(n, heads, generator=g0).to(dtype)
    dt_bias = torch.randn(heads * dim, generator=g0)
    a_log = torch.linspace(-2.0, 0.5, heads)
    lam = torch.linspace(0.5, 0.999, heads)
    entries = heads * vdim * dim + 11
    start = torch.randn(heads, vdim, dim, generator=g0) * 0.2
    bounds = torch.tensor([[0, 37], [37, 38], [38, 88]], dtype=torch.int32, device=DEV)
    slots = torch.tensor([2, -1, 0], dtype=torch.int32, device=DEV)
    # the plain walk on what enters the recurrence
    qd, kd, vd = q.double().view(n, kv, dim), k.double().view(n, kv, dim), v.double().view(n, heads, vdim)
    if rule == "delta":
        qd = qd / torch.sqrt((qd * qd).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
        kd = kd / torch.sqrt((kd * kd).sum(-1, keepdim=True) + 1e-6)
        beta = KP.logistic(b.double())
        gd = torch.exp(-torch.exp(a_log.double())[None, :, None] * KP.softplus(a.double().view(n, heads, dim) + dt_bias.double().view(heads, dim)))
    else:
        qd, kd, vd = KP.silu(qd), KP.silu(kd), KP.silu(vd)
        beta = gd = None
    refs, ends, at = [], [], 0
    for i, ln in enumerate(lens):
        s0 = start.double().transpose(1, 2) if i == 2 else None
        sl = slice(at, at + ln)
        o, e = plain_walk(rule, qd[sl], kd[sl], vd[sl], heads, kv, dim, vdim, s0, None if beta is None else beta[sl],
                          None if gd is None else gd[sl], lam.double())
        refs.append(o.reshape(ln, heads * vdim))
        ends.append(e)
        at += ln
    ref = torch.cat(refs)
    results = []
    for with_work in (False, True):
        state = torch.full((3, entries), 7.0, device=DEV)
        state[0, :heads * vdim * dim] = start.reshape(-1).to(DEV)
        state[2, :heads * vdim * dim] = 0.0
        y = torch.empty(n, heads * vdim, device=DEV)
        work = torch.empty(ops.linear_state_work_floats(rule, n, heads, dim, vdim), device=DEV) if with_work else None
        kw = dict(a=a.to(DEV), b=b.to(DEV), dt_bias=dt_bias.to(DEV), a_log=a_log.to(DEV), q_scale=dim ** -0.5) if rule == "delta" else \
            dict(decay=lam.to(DEV), act_silu=True)
        ops.linear_state(rule, q.to(DEV), k.to(DEV), v.to(DEV), state, slots, bounds, y, 3, heads, kv, dim, vdim, work=work, **kw)
        torch.cuda.synchronize()
        assert rel_err(y, ref) < 2e-5
        assert rel_err(state[2, :heads * vdim * dim].view(heads, vdim, dim).transpose(1, 2), ends[0]) < 2e-5
        assert rel_err(state[0, :heads * vdim * dim].view(heads, vdim, dim).transpose(1, 2), ends[2]) < 2e-5
        assert bool((state[1] == 7.0).all()) and bool((state[:, heads * vdim * dim:] == 7.0).all())     # nothing else is touched
        results.append((y.cpu(), state.cpu()))
    assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])
    # single tokens (no bounds): segment s is token s
    state = torch.zeros(n, entries, device=DEV)
    y1 = torch.empty(n, heads * vdim, device=DEV)
    ops.linear_state(rule, q.to(DEV), k.to(DEV), v.to(DEV), state, torch.arange(n, dtype=torch.int32, device=DEV), None, y1, n, heads, kv,
                     dim, vdim, **kw)
    first = torch.cat([plain_walk(rule, qd[i:i + 1], kd[i:i + 1], vd[i:i + 1], heads, kv, dim, vdim, None,
                                  None if beta is None else beta[i:i + 1], None if gd is None else gd[i:i + 1], lam.double())[0].reshape(1, -1)
                       for i in (0, 40, n - 1)])
    assert rel_err(y1[[0, 40, n - 1]], first) < 2e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inner,groups,wlen", [(48, 4, 12), (96, 1, 96), (1200, 3, 400), (20, 20, 1), (136, 1, 136)])
def test_unit_groups_times_weight_times_gate(dtype, inner, groups, wlen):
    from zedinfer_b200 import ops
    g = torch.Generator().manual_seed(inner)
    y = torch.randn(9, inner, generator=g) * 3
    z = torch.randn(9, inner + 8, generator=g).to(dtype)
    w = (1 + 0.2 * torch.randn(wlen, generator=g)).to(dtype)
    out = torch.empty(9, inner, dtype=dtype, device=DEV)
    ops.group_rmsnorm_gate(y.to(DEV), z.to(DEV)[:, 8:], w.to(DEV), groups, 1e-3, out)
    ref = KP.rms_unit(y.double().view(9, groups, -1), 1e-3).view(9, inner) * w.double().repeat(inner // wlen) * KP.logistic(z.double()[:, 8:])
    assert rel_err(out, ref) < (1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,hidden", [(1, 40), (7, 96), (33, 1536), (5, 73)])
def test_the_branch_norm_adds_into_a_float32_stream(dtype, rows, hidden):
    from zedinfer_b200 import ops
    g = torch.Generator().manual_seed(hidden)
    h = torch.randn(rows, hidden, generator=g) * 4
    y = (torch.randn(rows, hidden, generator=g) * 0.01).to(dtype)            # small: the eps inside the root matters
    w = (1 + 0.3 * torch.randn(hidden, generator=g)).to(dtype)
    hd, rounded = h.to(DEV), torch.empty(rows, hidden, dtype=dtype, device=DEV)
    ops.norm_add(hd, y.to(DEV), w.to(DEV), 1e-4, rounded)
    ref = h.double() + KP.rms_unit(y.double(), 1e-4) * w.double()
    assert hd.dtype == torch.float32 and rel_err(hd, ref) < 2e-6
    assert torch.equal(rounded.cpu(), hd.cpu().to(dtype))
    eps_free = h.double() + KP.rms_unit(y.double(), 0.0) * w.double()
    assert rel_err(hd, eps_free) > 1e-2                                           # the test's own premise


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,cols,col0", [(10, 50, 20), (3, 12, 9), (16, 16, 0), (33, 70, 37)])
def test_a_token_s_table_entry_gated_by_the_stream(dtype, width, cols, col0):
    from zedinfer_b200 import ops
    g = torch.Generator().manual_seed(width)
    t = (torch.randn(14, width + 8, generator=g) * 2).to(dtype)
    table = torch.randn(29, cols, generator=g).to(dtype)
    ids = torch.randint(0, 29, (14,), generator=g).int()
    out = torch.empty(14, width, dtype=dtype, device=DEV)
    ops.gelu_mul_rows(t.to(DEV)[:, 8:], table.to(DEV), col0, ids.to(DEV), out)
    ref = KP.gelu_tanh(t.double()[:, 8:]) * table.double()[ids.long(), col0:col0 + width]
    assert rel_err(out, ref) < (1e-5 if dtype == torch.float32 else 2e-2)


# ---------------------------------------------------------------------------------------------
# mixers alone
# ---------------------------------------------------------------------------------------------
def _attention(hidden, heads, kv, dim, vdim, window, rot, scale, softcap, eps, shared=False, cache_window="own"):
    from zedinfer_b200.config import PartSpec
    from zedinfer_b200.parts import AttentionMixer
    position = PartSpec("rope_span", {"head_dim": dim, "dims": rot["dims"] if rot else 0, "theta": rot["base"] if rot else 10000.0,
                                      "interleaved": True, "scaling": rot.get("scaling") if rot else None, "unit_rms_eps": eps})
    names = {"q": "q", "o": "o"} if shared else {"q": "q", "k": "k", "v": "v", "o": "o"}
    return AttentionMixer(hidden, heads, kv, dim, position, qkv_bias=False, scale=scale, softcap=softcap, window=window,
                          v_head_dim=vdim, shared_kv=shared, names=names, cache_window=cache_window)


SCHEDULE_AB = [[("a", 9), ("b", 2)], [("b", 1), ("a", 1)], [("a", 1)], [("a", 33), ("b", 15)], [("b", 1)], [("a", 2)], [("a", 15)]]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dim,vdim,window,reader_window,rot,softcap,page", [
    (4, 2, 32, 16, 13, 29, {"dims": 16, "base": 5000.0, "scaling": {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}}, 5.0, 4),
    (2, 1, 64, 64, 40, 7, {"dims": 64, "base": 10000.0, "scaling": None}, None, 16),
    (4, 4, 128, 128, 21, 21, {"dims": 32, "base": 300.0, "scaling": {"factor": 2.0, "original": 32, "fast": 8.0, "slow": 0.5}}, 20.0, 16),
    (3, 3, 24, 40, None, 3, {"dims": 2, "base": 77.0, "scaling": None}, 3.0, 8),
    (6, 2, 16, 8, 3, None, {"dims": 12, "base": 900.0, "scaling": {"factor": 16.0, "original": 4096, "fast": 2e5, "slow": 1e5}}, None, 8),
])
def test_windowed_attention_and_a_reader_of_its_cache(dtype, heads, kv, dim, vdim, window, reader_window, rot, softcap, page):
    """An attention layer and a second one that has queries of its own only and reads the first one's keys and values,
    each through its own window, over portions and single tokens of two requests in shared steps."""
    from zedinfer_b200.cache import CacheManager
    hidden, eps = 80, 1e-5
    keep = None if window is None or reader_window is None else max(window, reader_window)
    owner = _attention(hidden, heads, kv, dim, vdim, window, rot, 0.3, softcap, eps, cache_window=keep)
    reader = _attention(hidden, heads, kv, dim, vdim, reader_window, rot, 0.2, None if softcap is None else 2 * softcap, eps, shared=True)
    assert sorted(reader.tensor_specs()) == ["o", "q"]
    t = bind_random(owner, dtype, seed=dim + heads, scale=0.2)
    tr = bind_random(reader, dtype, seed=dim, scale=0.2)
    cache = CacheManager([(0, owner.cache_need())], page, max_requests=2)
    cache.allocate_device(40, dtype, DEV)
    view = cache.view_for_call(0)
    g = torch.Generator().manual_seed(7)
    xs = {"a": torch.randn(61, hidden, generator=g).to(dtype), "b": torch.randn(19, hidden, generator=g).to(dtype)}
    got_owner, got_reader = feed([owner, reader], cache, view, dtype, xs, SCHEDULE_AB)
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "rot": rot, "scale": 0.3, "softcap": softcap,
         "mask": None if window is None else {"size": window}}
    mr = dict(m, scale=0.2, softcap=None if softcap is None else 2 * softcap, mask=None if reader_window is None else {"size": reader_window})
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for rid, x in xs.items():
        pos = torch.arange(x.shape[0])
        k, v = KP.attention_keys_values(x.double(), pos, m, t, "", eps)
        assert rel_err(got_owner[rid], KP.attention_mixer(x.double(), pos, m, t, "", eps, k, v)) < tol, rid
        assert rel_err(got_reader[rid], KP.attention_mixer(x.double(), pos, mr, tr, "", eps, k, v)) < tol, rid


def _aligned(total, asks, rot, dim):
    """Key rows and query rows ``[total, dim]`` (zero almost everywhere) such that, after each is turned by its own position
    and made a unit head, the query at P of ``asks = {P: j}`` lies along the key at j, whose neighbours j - 1 and j + 1 carry
    the same row and so score a little less; every other key is zero and scores zero."""
    raw = torch.zeros(dim, dtype=F64)
    raw[0:rot["dims"]:2] = 1.0
    keys, queries = torch.zeros(total, dim, dtype=F64), torch.zeros(total, dim, dtype=F64)
    for p_query, j in asks.items():
        for d in (-1, 0, 1):
            if 0 <= j + d < total:
                keys[j + d] = raw
        queries[p_query] = KP.turn_pairs(raw[None, None], torch.tensor([j - p_query]), rot)[0, 0]
    return keys, queries


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim,window,page,rot", [
    (32, 150, 16, {"dims": 16, "base": 50.0, "scaling": None}),
    (64, 97, 8, {"dims": 32, "base": 300.0, "scaling": {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}}),
    (128, 256, 16, {"dims": 64, "base": 1000.0, "scaling": {"factor": 2.0, "original": 64, "fast": 16.0, "slow": 2.0}}),
    (16, None, 4, {"dims": 16, "base": 20.0, "scaling": None}),
])
def test_one_key_answers_just_inside_the_window_and_none_just_outside(dtype, dim, window, page, rot):
    """One head whose scores rest on the turned span alone, 600 tokens.  A query aligned with the key that is window - 1
    tokens back gets that key's value; one aligned with the key window tokens back gets the mean of the values it still sees
    (all its other scores are zero).  Asked from inside a prompt's portion and by tokens fed alone, across page borders; the
    reader of the cache looks less far than the owner keeps.  Without a window a key 560 tokens back answers."""
    from zedinfer_b200.cache import CacheManager
    total, vdim, eps = 600, 24, 1e-6
    reader_window = 11
    hidden = 2 * dim + vdim                                    # x = [query row | key row | value marks]
    scale = 300.0 / dim                                        # an aligned pair scores 300, its neighbours clearly less
    owner = _attention(hidden, 1, 1, dim, vdim, window, rot, scale, None, eps, cache_window=window)
    reader = _attention(hidden, 1, 1, dim, vdim, reader_window, rot, scale, None, eps, shared=True)
    wq, wk, wv = torch.zeros(dim, hidden), torch.zeros(dim, hidden), torch.zeros(vdim, hidden)
    wq[:, :dim] = torch.eye(dim)
    wk[:, dim:2 * dim] = torch.eye(dim)
    wv[:, 2 * dim:] = torch.eye(vdim)
    wo = torch.eye(hidden, vdim)
    owner.bind({k: v.to(dtype).to(DEV) for k, v in {"q": wq, "k": wk, "v": wv, "o": wo}.items()})
    reader.bind({k: v.to(dtype).to(DEV) for k, v in {"q": wq, "o": wo}.items()})
    w_eff = total if window is None else window
    inside = {599: 599 - (w_eff - 1) if window else 39, 450: 450 - (w_eff - 1) if window else 5, 598: 598 - (reader_window - 1)}
    outside = {597: 597 - w_eff, 430: 430 - w_eff, 596: 596 - reader_window} if window else {596: 596 - reader_window}
    asks = {**inside, **outside}
    keys, queries = _aligned(total, asks, rot, dim)
    marks = torch.randn(total, vdim, generator=torch.Generator().manual_seed(dim)).double()
    x = torch.cat([queries, keys, marks], dim=1).to(dtype)
    cache = CacheManager([(0, owner.cache_need())], page, max_requests=1)
    cache.allocate_device(total // page + 2, dtype, DEV)
    view = cache.view_for_call(0)
    schedule = [[("r", 200)], [("r", 395)]] + [[("r", 1)]] * 5
    got_owner, got_reader = feed([owner, reader], cache, view, dtype, {"r": x}, schedule, table_width=160)
    got_owner, got_reader = got_owner["r"], got_reader["r"]
    xd, pos = x.double(), torch.arange(total)
    m = {"heads": 1, "kv_heads": 1, "dim": dim, "vdim": vdim, "rot": rot, "scale": scale, "softcap": None,
         "mask": None if window is None else {"size": window}}
    t = {"q": wq.double(), "k": wk.double(), "v": wv.double(), "o": wo.double()}
    k, v = KP.attention_keys_values(xd, pos, m, t, "", eps)
    ref_owner = KP.attention_mixer(xd, pos, m, t, "", eps, k, v)
    ref_reader = KP.attention_mixer(xd, pos, dict(m, mask={"size": reader_window}), t, "", eps, k, v)
    tol = 1e-3 if dtype == torch.float32 else 3e-2
    assert rel_err(got_owner[:, :vdim], ref_owner[:, :vdim]) < tol and rel_err(got_reader[:, :vdim], ref_reader[:, :vdim]) < tol
    vals = xd[:, 2 * dim:]
    for p_query, j in asks.items():
        ours, ref = (got_reader, ref_reader) if p_query in (598, 596) else (got_owner, ref_owner)
        if p_query in inside:
            assert rel_err(ref[p_query, :vdim], vals[j]) < 1e-2                 # the test's own premise: that key alone answers
            assert rel_err(ours[p_query, :vdim], vals[j]) < 4e-2, (p_query, j)
        else:
            assert float((ref[p_query, :vdim] - vals[j]).abs().max()) > 0.5      # premise: it does not answer
            assert float((ours[p_query, :vdim].double().cpu() - vals[j]).abs().max()) > 0.5, (p_query, j)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dim,vdim,taps,decay_rank,gate_rank", [(4, 2, 16, 24, 3, 6, 14), (3, 1, 136, 12, 2, 4, 20), (2, 2, 72, 8, 1, 5, 3),
                                                                       (6, 3, 40, 20, 4, 16, 2), (1, 1, 8, 70, 4, 1, 1)])
def test_delta_rule_mixer_over_portions_and_slots_used_again(dtype, heads, kv, dim, vdim, taps, decay_rank, gate_rank):
    """Two requests in shared steps, cut down to single tokens, then a third in the slot the second gave back: it starts
    from zeros (state and the convolution's last inputs), not from what the slot last held."""
    from zedinfer_b200.cache import CacheManager
    from zedinfer_b200.parts import ChannelDeltaMixer
    hidden, eps = 64, 1e-5
    mixer = ChannelDeltaMixer(hidden, heads, kv, dim, vdim, taps, decay_rank, gate_rank, eps)
    over = {"A_log": torch.linspace(-3.0, 0.5, heads), "dt_bias": torch.linspace(-3.0, 1.0, heads * dim), "norm": 1 + 0.1 * torch.randn(vdim)}
    t = bind_random(mixer, dtype, seed=dim, scale=0.3, overrides=over)
    cache = CacheManager([(0, mixer.cache_need())], 16, max_requests=2)
    cache.allocate_device(1, dtype, DEV)
    view = cache.view_for_call(0)
    assert view.kind == "state"
    g = torch.Generator().manual_seed(5)
    xs = {"a": torch.randn(45, hidden, generator=g).to(dtype), "b": torch.randn(10, hidden, generator=g).to(dtype),
          "c": torch.randn(12, hidden, generator=g).to(dtype)}
    schedule = [[("a", 6), ("b", 2)], [("b", 1), ("a", 1)], [("a", 1)], [("a", 2), ("b", 7), "end:b"], [("c", 3), ("a", 20)],
                [("c", 1), ("a", 1)], [("c", 8), ("a", 14)]]
    got = feed(mixer, cache, view, dtype, xs, schedule)
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": taps}
    for rid, x in xs.items():
        assert rel_err(got[rid], KP.channel_delta_mixer(x.double(), m, t, "", eps)) < (3e-5 if dtype == torch.float32 else 5e-2), rid


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,vdim,decay", [(3, 16, 24, (0.5, 0.9, 0.99)), (1, 40, 20, (0.93,)), (4, 8, 136, (0.2, 0.7, 0.95, 0.9995)),
                                                  (2, 136, 16, (1.0, 0.999))])
def test_lightning_mixer_over_portions_and_slots_used_again(dtype, heads, dim, vdim, decay):
    from zedinfer_b200.cache import CacheManager
    from zedinfer_b200.parts import LightningMixer
    hidden, eps = 64, 1e-5
    mixer = LightningMixer(hidden, heads, dim, vdim, decay, eps)
    t = bind_random(mixer, dtype, seed=dim, scale=0.3, overrides={"norm": 1 + 0.1 * torch.randn(heads * vdim)})
    cache = CacheManager([(0, mixer.cache_need())], 16, max_requests=2)
    cache.allocate_device(1, dtype, DEV)
    view = cache.view_for_call(0)
    g = torch.Generator().manual_seed(6)
    xs = {"a": torch.randn(45, hidden, generator=g).to(dtype), "b": torch.randn(10, hidden, generator=g).to(dtype),
          "c": torch.randn(12, hidden, generator=g).to(dtype)}
    schedule = [[("a", 6), ("b", 2)], [("b", 1), ("a", 1)], [("a", 1)], [("a", 2), ("b", 7), "end:b"], [("c", 3), ("a", 20)],
                [("c", 1), ("a", 1)], [("c", 8), ("a", 14)]]
    got = feed(mixer, cache, view, dtype, xs, schedule)
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    for rid, x in xs.items():
        assert rel_err(got[rid], KP.lightning_mixer(x.double(), m, t, "", eps)) < (3e-5 if dtype == torch.float32 else 5e-2), rid


# ---------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("kevatar_models")
    return {name: KT.make_model_dir(root, name) for name in KT.CONFIGS}


def make_requests(cfg, lengths, seed):
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(cfg["vocab"]) for _ in range(n)] for i, n in enumerate(lengths)}


_plain_cache = {}


def expected_logits(model_dir, requests):
    if model_dir not in _plain_cache:
        _plain_cache[model_dir] = KP.read_model(model_dir, F64)
    cfg, w = _plain_cache[model_dir]
    return {rid: KP.forward(cfg, w, toks).float() for rid, toks in requests.items()}


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


def test_layers_that_read_another_layer_s_keys_hold_no_cache(models):
    """A reader has no cache of its own; its owner keeps as many keys as the reader that looks furthest back needs; a
    model of recurrent layers alone asks for no pages, one of attention alone for no state slot."""
    from zedinfer_b200.config.registry import load_model_config
    from zedinfer_b200.engine.model import Model
    _, _, spec = load_model_config(models["A"])
    assert [c.cache_of for c in spec.schedule] == [None, None, None, 1, 1]
    assert [k for k, _ in Model(spec).cache_needs()] == [0, 1, 2]
    assert spec.layers[1].mixer.params["cache_window"] == 29 and spec.layers[3].mixer.params["window"] == 29
    _, _, spec_c = load_model_config(models["C"])
    assert spec_c.layers[0].mixer.params["cache_window"] is None
    kinds = lambda s: sorted({type(need).__name__ for _, need in Model(s).cache_needs()})
    assert kinds(load_model_config(models["D"])[2]) == ["StateNeed"] and "StateNeed" not in kinds(load_model_config(models["E"])[2])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
@pytest.mark.parametrize("family", ["whole", "tail", "chunks", "mixed"])
def test_cuts_match_plain(models, name, dtype, family):
    """Whole prompts; a tail decoded token by token; portions down to two tokens; mixed batches of unequal requests in a
    pool so small that pages and state slots are handed out again."""
    from zedinfer_b200.engine.core import EngineCore
    cfg, _ = KT.CONFIGS[name]
    requests = make_requests(cfg, LENGTHS[name] + ([64, 31, 77] if family == "mixed" else []), seed=5)
    if family == "tail":
        steps = traces.tail_decode(requests, tail=40)
    else:
        steps = {"whole": traces.whole, "chunks": traces.chunks, "mixed": traces.mixed}[family](requests)
    page = PAGES[name]
    need = traces.max_live_tokens(steps, round_to=page)
    core = EngineCore(models[name], dtype, page_size=page, num_pages=max(1, need // page), max_requests=4)
    got = run_trace(core, steps)
    core.check_kernels()
    judge(got, expected_logits(models[name], requests), dtype)
    assert core.cache.num_live == 0 and all(g.pool.num_used == 0 for g in core.cache.groups)
    assert core.cache.slots.num_free_slots == core.cache.slots.num_slots


def test_low_ranks_come_from_the_tensors_where_the_configuration_is_silent(tmp_path):
    from zedinfer_b200.engine.core import EngineCore
    bare = KT.make_model_dir(tmp_path, "A", strip_ranks=True)
    cfg, _ = KT.CONFIGS["A"]
    requests = make_requests(cfg, [33], seed=1)
    core = EngineCore(bare, "float32", page_size=8, num_pages=8, max_requests=1)
    judge(run_trace(core, traces.whole(requests)), expected_logits(KT.make_model_dir(tmp_path, "A"), requests), "float32")


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("B", "bfloat16"), ("C", "bfloat16"), ("D", "bfloat16")])
def test_many_decoding_requests_with_and_without_graphs(models, name, dtype, graphs):
    """Steps as a scheduler makes them: up to 12 decoding requests beside one prompt portion, then decode-only steps whose
    number of rows falls to one; with graphs the decode-only steps replay captured buckets whose rows of padding hold no
    state slot."""
    from zedinfer_b200.engine.core import EngineCore
    cfg, _ = KT.CONFIGS[name]
    rng = random.Random(8)
    requests = make_requests(cfg, [rng.randint(40, 90) for _ in range(15)], seed=3)
    steps = traces.decode_heavy(requests, seed=4, max_live=12, tail=(8, 30), portion=32)
    need = traces.max_live_tokens(steps, round_to=16)
    core = EngineCore(models[name], dtype, page_size=16, num_pages=need // 16, max_requests=16, cuda_graphs=graphs)
    core.GPU_BOUND_RATIO = float("inf")
    assert core.capture_safe, core.capture_blockers
    got = run_trace(core, steps)
    core.check_kernels()
    judge(got, expected_logits(models[name], requests), dtype)
    if graphs:
        assert core._decode_graphs
    assert core.cache.num_live == 0 and all(g.pool.num_used == 0 for g in core.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_the_first_tokens(models, dtype):
    """One token, two tokens, and a request decoded for 260 steps from a prompt of three: every window passes over decoded
    tokens many times, the matrix states and the convolution's last inputs go through hundreds of single-token steps."""
    from zedinfer_b200.engine.core import EngineCore
    cfg, _ = KT.CONFIGS["A"]
    requests = make_requests(cfg, [1, 2, 263], seed=9)
    steps = traces.tail_decode(requests, tail=260)
    core = EngineCore(models["A"], dtype, page_size=4, num_pages=80, max_requests=2)
    judge(run_trace(core, steps), expected_logits(models["A"], requests), dtype)


@pytest.mark.parametrize("name", ["A", "C", "D", "F"])
def test_float32_is_the_same_however_it_is_cut(models, name):
    """The same positions through four different schedules: the same bits (every float32 sum of the design has one order,
    which depends on constants alone; the recurrences run token by token whatever the portions)."""
    from zedinfer_b200.engine.core import EngineCore
    cfg, _ = KT.CONFIGS[name]
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
    cfg, _ = KT.CONFIGS[name]
    rng = random.Random(4)
    prompts = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (9, 23, 1, 14, 6)]
    engine = InferenceEngine.create(models[name], SchedulerConfig(num_kv_pages=30, kv_block_size=4, max_batch_requests=3,
                                                                  max_prefill_tokens=5, cuda_graphs=graphs),
                                    dtype="float32")
    results = engine.generate_batch(prompts, GenerationConfig(max_new_tokens=20, ignore_eos=True))
    pcfg, w = KP.read_model(models[name], F64)
    for p, r in zip(prompts, results):
        assert r.finish_reason == "length"
        assert r.output_ids == KP.greedy(pcfg, w, p, 20)
    st = engine.cache_stats()
    assert st["live_requests"] == 0 and st["free_pages"] == st["pages_per_group"]


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_trace_program_on_a_kevatar_folder(models, tmp_path, dtype):
    cfg, _ = KT.CONFIGS["B"]
    requests = make_requests(cfg, [70, 9, 33, 50, 21], seed=6)
    steps = traces.mixed(requests, seed=1)
    need = traces.max_live_tokens(steps, round_to=64)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", models["B"], "--dtype", dtype,
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
    judge(got, expected_logits(models["B"], requests), dtype)


def test_command_line_programs_take_the_design(tmp_path, capsys):
    """From a bare config.json with weights drawn on the device: the bench program, continuous batching, and the
    consistency program, which returns 0 only if every float32 logit is the same bit pattern however the work is cut."""
    from zedinfer_b200.cli import batch_bench, bench, consistency
    path = tmp_path / "config.json"
    path.write_text(json.dumps(KT.KV_A))
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
