"""Helpers for tests that run one part of a layer alone on the device: a step's context on a cache manager, a schedule of
portions fed through mixers, random tensors bound to a part."""
import torch

DEV = "cuda:0"


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


def feed(mixers, views, cache, dtype, xs, schedule, table_width=64):
    """Run ``mixers`` (each on its own view of ``views``) over the requests ``xs = {id: [T, hidden]}`` cut as ``schedule =
    [[(id, tokens), ...], ...]`` says (a step may hold portions of several requests; ``"end:<id>"`` closes one); returns one
    ``{id: [T, hidden]}`` per mixer."""
    done = {rid: 0 for rid in xs}
    outs = [{rid: [] for rid in xs} for _ in mixers]
    for step in schedule:
        portions = [p for p in step if not isinstance(p, str)]
        if portions:
            ctx, entries, rcs = step_context(cache, dtype, portions, table_width)
            x = torch.cat([xs[rid][done[rid]:done[rid] + n] for rid, n in portions]).to(DEV)
            ys = [m.forward(x, ctx, v, owns_cache=True).cpu() for m, v in zip(mixers, views)]
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
    return [{rid: torch.cat(v) for rid, v in out.items() if v} for out in outs]


def bind_random(part, dtype, seed, scale=0.3, overrides=None):
    """Random tensors for a part (its own names), bound on the device; returns them as float64 on the host."""
    g = torch.Generator().manual_seed(seed)
    t = {k: (torch.randn(v.shape, generator=g) * scale).to(dtype) for k, v in part.tensor_specs().items()}
    for k, v in (overrides or {}).items():
        t[k] = v.to(dtype)
    part.bind({k: v.to(DEV) for k, v in t.items()})
    return {k: v.double() for k, v in t.items()}
