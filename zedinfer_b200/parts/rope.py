"""Rotary position encodings: rotate-half over the whole head (``rope``), and a span of the head in either pairing
(``rope_span``).

``rope``:

``inv_freq[k] = 1 / theta^(2k / head_dim)`` in float32, ``angle = float(position) * inv_freq[k]``,
``y[k] = a*cos - b*sin``, ``y[k + half] = b*cos + a*sin`` with ``a = x[k]``, ``b = x[k + half]``
(src/backend/ops/rope/cpu/rope_cpu.cpp:32-52 and :60-65).  Values are not rotated.  The kernel
that rotates also appends k and v to the cache pages of each token's request.
"""
from __future__ import annotations

import math
from typing import Mapping, Optional

import torch

from .. import ops
from ..cache.manager import CallCacheView
from .base import PositionEncoding, StepContext, register_position


@register_position("rope")
class RotaryPosition(PositionEncoding):
    capture_safe = True

    def __init__(self, head_dim: int, theta: float):
        if head_dim <= 0 or head_dim % 2:
            raise ValueError(f"rope: head_dim={head_dim} must be positive and even")
        if not theta > 0.0:
            raise ValueError(f"rope: theta={theta} must be positive")
        self.head_dim, self.theta = int(head_dim), float(theta)
        self._inv_freq: Optional[torch.Tensor] = None

    def inverse_frequencies(self) -> torch.Tensor:
        """float32 table on the CPU: 1 / powf(theta, float(2k) / float(head_dim))."""
        expo = torch.arange(0, self.head_dim, 2, dtype=torch.float32) / torch.tensor(float(self.head_dim),
                                                                                     dtype=torch.float32)
        return 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float32), expo)

    def _table(self, device: torch.device) -> torch.Tensor:
        if self._inv_freq is None or self._inv_freq.device != device:
            self._inv_freq = self.inverse_frequencies().to(device)
        return self._inv_freq

    def _angles_key(self) -> tuple:
        """What else the step's shared table of angles depends on, for rules derived from this one."""
        return ()

    def rotate_append(self, qkv: torch.Tensor, q_out: torch.Tensor, cache: CallCacheView, ctx: StepContext,
                      n_heads: int, n_kv_heads: int, head_dim: int, write_kv: bool) -> None:
        if head_dim != self.head_dim:
            raise ValueError(f"rope was built for head_dim={self.head_dim}, the mixer has {head_dim}")
        # few tokens (a decode step beyond what the product's epilogue takes): the step's angles, made once
        cs = self._step_angles(ctx, qkv.device) if qkv.shape[0] <= ops.ROPE_TABLE_MAX_TOKENS else None
        ops.rope_append(qkv, q_out, cache.tensor, ctx.tables[cache.group], ctx.tok_seg, ctx.positions,
                        self._table(qkv.device), n_heads, n_kv_heads, head_dim, cache.page_size, cache.page_stride,
                        cache.kv_stride, write_kv=write_kv, cs=cs)

    def _step_angles(self, ctx: StepContext, device: torch.device) -> torch.Tensor:
        """cos | sin of every token's angles, float32 ``[tokens, head_dim]``: made by the first layer of a step that
        asks, shared by every layer with the same theta and head size."""
        key = ("rope_cs", self.theta, self.head_dim) + self._angles_key()
        cs = ctx.step_cache.get(key)
        if cs is None:
            cs = torch.empty((ctx.positions.numel(), self.head_dim), dtype=torch.float32, device=device)
            ops.rope_table(ctx.positions, self._table(device), cs)
            ctx.step_cache[key] = cs
        return cs

    def project_rotate_append(self, x: torch.Tensor, w_qkv: torch.Tensor, b_qkv: Optional[torch.Tensor],
                              q_out: torch.Tensor, cache: CallCacheView, ctx: StepContext, n_heads: int,
                              n_kv_heads: int, head_dim: int, write_kv: bool) -> bool:
        """Steps of at most 16 tokens in bfloat16 (decode): rotation and append run in the epilogue of the q/k/v
        product.  The step's cosines and sines are made once and shared by every layer with the same theta and
        head size."""
        if not (write_kv and head_dim == self.head_dim
                and ops.can_fuse_rope_product(x, w_qkv, b_qkv, cache.tensor)):
            return False
        cs = self._step_angles(ctx, x.device)
        ops.gemm_smallm_rope(x, w_qkv, b_qkv, cs, q_out, cache.tensor, ctx.tables[cache.group], ctx.tok_seg,
                             ctx.positions, n_heads, n_kv_heads, head_dim, cache.page_size, cache.page_stride,
                             cache.kv_stride)
        return True


@register_position("rope_span")
class SpanRotaryPosition(PositionEncoding):
    """Only entries ``offset .. offset + dims`` of a head turn, the rest pass unchanged.  Pair i of the span is (entry i,
    entry i + dims / 2) (``interleaved=False``, the rotate-half pairing) or (entry 2i, entry 2i + 1) (``interleaved=True``);
    ``(lo, hi) -> (lo cos a - hi sin a, hi cos a + lo sin a)`` with ``a = float(position) * inv_freq[i]``, ``inv_freq[i] =
    1 / theta^(2i / dims)`` in float32.  The kernel that turns also appends the keys and the values to the cache; with
    ``value_from_key`` the values are the keys as they were before the turn (the product then has no value columns)."""
    capture_safe = True
    takes_value_from_key = True

    def __init__(self, head_dim: int, dims: int, theta: float, interleaved: bool = False, offset: int = 0,
                 scaling: Optional[Mapping[str, float]] = None, unit_rms_eps: Optional[float] = None):
        """``scaling`` (``factor``, ``original``, ``fast``, ``slow``): the frequencies are stretched for contexts longer than
        ``original`` positions, pair by pair (see :meth:`inverse_frequencies`), and cosines and sines are multiplied by
        ``0.1 ln(factor) + 1``.  ``unit_rms_eps``: after the turn every query and key head is divided by its root mean square
        ``sqrt(mean(x^2) + unit_rms_eps)``.  Either option, a cache whose rows are wider than a head or a value size of its
        own takes the kernel ``ops.rotary_norm`` (span at the start of the head); ``dims`` may then be 0 (nothing turns)."""
        plain = scaling is None and unit_rms_eps is None
        if head_dim <= 0 or dims < 0 or (dims == 0 and plain) or dims % 2 or offset < 0 or offset + dims > head_dim:
            raise ValueError(f"rope_span: a span of {dims} entries from {offset} must be even and fit a head of {head_dim}")
        if not theta > 0.0:
            raise ValueError(f"rope_span: theta={theta} must be positive")
        if not plain and offset:
            raise ValueError("rope_span: stretched frequencies and unit heads need the span at the start of the head")
        if unit_rms_eps is not None and not unit_rms_eps > 0.0:
            raise ValueError(f"rope_span: unit_rms_eps={unit_rms_eps} must be positive")
        self.head_dim, self.dims, self.theta = int(head_dim), int(dims), float(theta)
        self.interleaved, self.offset = bool(interleaved), int(offset)
        self.unit_rms_eps = float(unit_rms_eps) if unit_rms_eps is not None else None
        self.scaling = None
        self.magnitude = 1.0
        if scaling is not None:
            missing = [k for k in ("factor", "original", "fast", "slow") if k not in scaling]
            if missing:
                raise ValueError(f"rope_span: scaling lacks {missing}")
            self.scaling = {k: float(scaling[k]) for k in ("factor", "original", "fast", "slow")}
            if not (self.scaling["factor"] > 0.0 and self.scaling["original"] > 0.0 and self.scaling["fast"] > 0.0
                    and self.scaling["slow"] > 0.0 and self.theta != 1.0):
                raise ValueError(f"rope_span: scaling={dict(scaling)} must be positive throughout (and theta differ from 1)")
            self.magnitude = 0.1 * math.log(self.scaling["factor"]) + 1.0
        self._inv_freq: Optional[torch.Tensor] = None

    def inverse_frequencies(self) -> torch.Tensor:
        """float32 table on the CPU: ``f_i = theta^(-2i / dims)``.  With ``scaling``: let ``D(n) = dims ln(original / (2 pi
        n)) / (2 ln theta)`` be the pair that makes n full turns over ``original`` positions, ``lo = max(floor(D(fast)), 0)``,
        ``hi = min(ceil(D(slow)), dims - 1)`` and ``m_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)``; the table holds ``f_i
        / factor * m_i + f_i (1 - m_i)``: pairs below ``lo`` keep their frequency, pairs above ``hi`` turn ``factor`` times
        slower.  Formed in float64 and rounded once."""
        i = torch.arange(0, self.dims // 2, dtype=torch.float64)
        f = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / max(self.dims, 1))
        if self.scaling is not None:
            sc = self.scaling

            def pair_of(turns: float) -> float:
                return self.dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

            lo = max(math.floor(pair_of(sc["fast"])), 0)
            hi = min(math.ceil(pair_of(sc["slow"])), self.dims - 1)
            ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            f = f / sc["factor"] * ramp + f * (1.0 - ramp)
        return f.to(torch.float32)

    def table(self, device: torch.device) -> torch.Tensor:
        if self._inv_freq is None or self._inv_freq.device != device:
            self._inv_freq = self.inverse_frequencies().to(device)
        return self._inv_freq

    def rotate_append(self, qkv: torch.Tensor, q_out: torch.Tensor, cache: CallCacheView, ctx: StepContext,
                      n_heads: int, n_kv_heads: int, head_dim: int, write_kv: bool, value_from_key: bool = False,
                      v_dim: Optional[int] = None, row_dim: Optional[int] = None,
                      q_head_scale: Optional[torch.Tensor] = None) -> None:
        """``v_dim``: the value heads' size where it differs from ``head_dim``; ``row_dim``: the width of the cache's rows
        and of the heads of ``q_out`` where that is more than a head (the rest is written as zero); ``q_head_scale``
        (float32, one per query head): a factor on every query head as it is written."""
        if head_dim != self.head_dim:
            raise ValueError(f"rope_span was built for head_dim={self.head_dim}, the mixer has {head_dim}")
        v_dim = head_dim if v_dim is None else v_dim
        row_dim = head_dim if row_dim is None else row_dim
        if (self.scaling is not None or self.unit_rms_eps is not None or v_dim != head_dim or row_dim != head_dim or not self.dims
                or q_head_scale is not None):
            if value_from_key:
                raise ValueError("rope_span: unturned keys as values go with the plain span only")
            ops.rotary_norm(qkv, q_out, ctx.positions, self.table(qkv.device) if self.dims else None, self.magnitude, n_heads,
                            n_kv_heads, head_dim, v_dim, row_dim, self.dims, self.interleaved, self.unit_rms_eps,
                            cache=cache if write_kv else None, tables=ctx.tables[cache.group] if write_kv else None,
                            tok_seg=ctx.tok_seg if write_kv else None, q_head_scale=q_head_scale)
            return
        if not write_kv:
            ops.rotary(qkv, q_out, ctx.positions, self.table(qkv.device), n_heads, 0, head_dim, self.offset, self.dims,
                       self.interleaved)
            return
        ops.rotary(qkv, q_out, ctx.positions, self.table(qkv.device), n_heads, n_kv_heads, head_dim, self.offset, self.dims,
                   self.interleaved, cache=cache, tables=ctx.tables[cache.group], tok_seg=ctx.tok_seg,
                   v_mode=2 if value_from_key else 1)

    def rotate_queries(self, q: torch.Tensor, ctx: StepContext, n_heads: int) -> None:
        """In place, queries alone: ``q [tokens, n_heads * head_dim]`` (rows may be strided)."""
        ops.rotary(q, q, ctx.positions, self.table(q.device), n_heads, 0, self.head_dim, self.offset, self.dims, self.interleaved)


@register_position("rope_span_as_whole")
class SpanAsWholeRotaryPosition(RotaryPosition):
    """A rotate-half rotation of the first ``dims`` entries of a head, run by the kernels that turn whole heads.

    Those kernels pair entry k with k + head_dim / 2.  With the head's entries reordered as ``[first half of the span |
    first half of the rest | second half of the span | second half of the rest]`` (:meth:`head_order`; the mixer reorders
    the rows of its query and key weights and the columns of its output weight once, when it binds them) every pair of
    the span is such a pair, and the pairs of the rest get the frequency 0: angle 0, cosine 1, sine 0, and ``a * 1 - b * 0``
    is a.  Scores do not change under one reordering of queries and keys.  So the fused decode product (rotation and cache
    append in its epilogue) and the vectorised rotation of prompts serve a partly turned head as they are."""

    def __init__(self, head_dim: int, dims: int, theta: float):
        super().__init__(head_dim, theta)
        if dims <= 0 or dims % 2 or dims > head_dim:
            raise ValueError(f"rope_span_as_whole: a span of {dims} entries must be even and fit a head of {head_dim}")
        self.dims = int(dims)

    def inverse_frequencies(self) -> torch.Tensor:
        """float32: 1 / powf(theta, float(2i) / float(dims)) for the span's pairs, 0 for the others."""
        expo = torch.arange(0, self.dims, 2, dtype=torch.float32) / torch.tensor(float(self.dims), dtype=torch.float32)
        out = torch.zeros(self.head_dim // 2, dtype=torch.float32)
        out[:self.dims // 2] = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float32), expo)
        return out

    def _angles_key(self) -> tuple:
        return ("span", self.dims)

    def head_order(self) -> torch.Tensor:
        """``order[new] = old``: where each entry of a reordered head comes from."""
        d, r = self.head_dim, self.dims
        rest = (d - r) // 2
        return torch.tensor(list(range(0, r // 2)) + list(range(r, r + rest)) + list(range(r // 2, r)) + list(range(r + rest, d)),
                            dtype=torch.long)
