"""Mixers that carry a matrix state per head from token to token instead of cached keys and values.

``channel_delta`` (a gated delta rule with a decay per key entry).  With ``H`` heads, ``G`` query/key heads of ``dim``
entries (head a reads query/key head ``a // (H / G)``) and values of ``vdim`` entries:

    q, k, v = silu(conv(Wq h)), silu(conv(Wk h)), silu(conv(Wv h))    a short causal convolution per channel, no bias
    q <- q / sqrt(|q|^2 + 1e-6) / sqrt(dim),   k <- k / sqrt(|k|^2 + 1e-6)                       per head
    beta = sigmoid(Wb h);    g = exp(-exp(A_log_a) softplus(Wa2 Wa1 h + dt_bias))                 [H, dim]
    per head:   S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q            (S is dim x vdim, float32)
    out = Wo (unit_rms_per_head(o) * w_norm * sigmoid(Wg2 Wg1 h))                                w_norm [vdim], shared by heads

``gated_delta`` is the same rule with one decay per head, ``g = exp(-exp(A_log_a) softplus(Wa h + dt_bias_a))``, the decay's and
the gate's inputs projected in one step each, and a SiLU gate: ``out = Wo (unit_rms_per_head(o) * w_norm * silu(Wg h))``.

``forget_gate`` (one gate per key entry fades the state, and its complement stands where the other rules have a key):

    q = silu(Wq h);   v = Wv h;   f = l + (1 - l) sigmoid(Wf h + bf)          l [H, dim] a lower bound, f per head and key entry
    per head:   S <- diag(f) S + (1 - f) v^T;   o = S^T q
    out = Wo (unit_rms_per_head(o) * w_norm)                                   w_norm [vdim], shared by heads

``lightning`` (a constant decay per head):

    q, k, v = silu(Wq h), silu(Wk h), silu(Wv h);    per head   S <- decay_a S + k v^T;   o = S^T q
    out = Wo (unit_rms(concat(o)) * w_norm * sigmoid(Wg h))                                       w_norm [H * vdim]

What a request carries from step to step is one slot of fixed-size float32 state: S of every head laid out ``[H, vdim,
dim]`` and, for ``channel_delta``, the convolution's last ``taps - 1`` inputs behind it.  A step runs the tokens it brings
from that state and leaves the state behind its last token, so a prompt may be cut anywhere and a decoded token is a portion
of one.  Unit vectors, sigmoid, softplus, decays, the state and every sum of the recurrence are float32 whatever the step's
type; the projections, the convolution and the activations on them have the step's type.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Sequence

import torch

from .. import ops
from ..cache.manager import CallCacheView, StateNeed
from ..weights.loader import TensorSpec
from .base import Mixer, StepContext, register_mixer
from .ssm import step_segment_bounds

UNIT_EPS = 1e-6                  # inside the root of channel_delta's unit vectors


def _stack_padded(tensors: Sequence[torch.Tensor], multiple: int = 8):
    """Concatenate weight matrices along their rows, each padded with zero rows to a multiple of ``multiple``, so that
    every part of the product's output starts on a 16-byte boundary.  Returns the stacked weight and the parts' offsets."""
    dtype = torch.float32 if any(t.dtype == torch.float32 for t in tensors) else tensors[0].dtype
    rows, offsets, at = [], [], 0
    for t in tensors:
        offsets.append(at)
        pad = -t.shape[0] % multiple
        rows.append(t.to(dtype))
        if pad:
            rows.append(t.new_zeros((pad, t.shape[1]), dtype=dtype))
        at += t.shape[0] + pad
    return torch.cat(rows, dim=0).contiguous(), offsets


def _walk_workspace(rule: str, ctx: StepContext, n: int, heads: int, dim: int, vdim: int) -> Optional[torch.Tensor]:
    """The float32 workspace in which a step that brings portions of prompts makes its tokens ready before the walk; a step
    of single tokens needs none (its walk makes them ready itself, in one launch)."""
    if ctx.decode_only or n <= ctx.n_segments:
        return None
    return ctx.empty(ops.linear_state_work_floats(rule, n, heads, dim, vdim), dtype=torch.float32)


def _state_and_slots(cache: CallCacheView, ctx: StepContext, owns_cache: bool, what: str) -> torch.Tensor:
    if cache.kind != "state" or not owns_cache:
        raise RuntimeError(f"{what} needs a state slot of its own")
    if ctx.slots is None:
        raise RuntimeError(f"{what} needs the step's state slots")
    return cache.tensor


@register_mixer("channel_delta")
class ChannelDeltaMixer(Mixer):
    capture_safe = True

    def __init__(self, hidden_size: int, heads: int, kv_heads: int, dim: int, vdim: int, conv: int, decay_rank: Optional[int],
                 gate_rank: Optional[int], eps: float, names: Optional[Mapping[str, str]] = None, decay_per: str = "entry",
                 gate_act: str = "sigmoid"):
        """``decay_rank`` / ``gate_rank`` None: the decay's / the gate's input is one projection of the layer's input (tensors
        ``a`` / ``g``) instead of two through a low rank (``a1``, ``a2`` / ``g1``, ``g2``).  ``decay_per``: ``"entry"``, a decay per
        head and key entry, or ``"head"``, one per head (``dt_bias`` then has one entry per head).  ``gate_act``: ``"sigmoid"``
        or ``"silu"``."""
        if min(hidden_size, heads, kv_heads, dim, vdim, conv, decay_rank or 1, gate_rank or 1) <= 0:
            raise ValueError("channel_delta: every size must be positive")
        if decay_per not in ("entry", "head") or gate_act not in ("sigmoid", "silu"):
            raise ValueError(f"channel_delta: decay_per={decay_per!r} is not 'entry' or 'head', or gate_act={gate_act!r} not 'sigmoid' or 'silu'")
        if heads % kv_heads:
            raise ValueError(f"channel_delta: {heads} heads cannot share {kv_heads} query/key heads")
        if dim > 256:
            raise ValueError(f"channel_delta: dim={dim} is not supported; the recurrence kernel takes at most 256")
        self.hidden_size, self.heads, self.kv_heads, self.dim, self.vdim = int(hidden_size), int(heads), int(kv_heads), int(dim), int(vdim)
        self.taps, self.eps = int(conv), float(eps)
        self.decay_rank = int(decay_rank) if decay_rank is not None else None
        self.gate_rank = int(gate_rank) if gate_rank is not None else None
        self.decay_per, self.gate_act = decay_per, gate_act
        self.decay_width = self.heads * (self.dim if decay_per == "entry" else 1)       # decays per token
        self.qk_width, self.inner = self.kv_heads * self.dim, self.heads * self.vdim
        self.channels = 2 * self.qk_width + self.inner                          # what the convolution sees: q | k | v
        self.state_elems = self.heads * self.vdim * self.dim
        self.names = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "b": "b",
                      "a_log": "A_log", "norm": "norm", "a1": "a1", "a2": "a2", "dt_bias": "dt_bias", "g1": "g1", "g2": "g2",
                      "a": "a", "g": "g", "o": "o"}
        self.names.update(names or {})
        self.w_in = self.w_conv = self.w_a2 = self.w_g2 = self.dt_bias = self.a_log = self.g = self.w_o = None
        self._offsets: List[int] = []

    def cache_need(self):
        # the recurrent state [heads, vdim, dim], then the convolution's ring [taps - 1, channels]
        return StateNeed((self.state_elems + (self.taps - 1) * self.channels,), torch.float32)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        nm, h = self.names, self.hidden_size
        conv = ("normal", 0.3)
        specs = {nm["q"]: TensorSpec((self.qk_width, h)), nm["k"]: TensorSpec((self.qk_width, h)), nm["v"]: TensorSpec((self.inner, h)),
                 nm["q_conv"]: TensorSpec((self.qk_width, self.taps), init=conv), nm["k_conv"]: TensorSpec((self.qk_width, self.taps), init=conv),
                 nm["v_conv"]: TensorSpec((self.inner, self.taps), init=conv), nm["b"]: TensorSpec((self.heads, h)),
                 nm["a_log"]: TensorSpec((self.heads,)), nm["norm"]: TensorSpec((self.vdim,), init=("one_plus_normal", 0.01)),
                 nm["dt_bias"]: TensorSpec((self.decay_width,)), nm["o"]: TensorSpec((h, self.inner))}
        if self.decay_rank is None:
            specs[nm["a"]] = TensorSpec((self.decay_width, h))
        else:
            specs.update({nm["a1"]: TensorSpec((self.decay_rank, h)), nm["a2"]: TensorSpec((self.decay_width, self.decay_rank))})
        if self.gate_rank is None:
            specs[nm["g"]] = TensorSpec((self.inner, h))
        else:
            specs.update({nm["g1"]: TensorSpec((self.gate_rank, h)), nm["g2"]: TensorSpec((self.inner, self.gate_rank))})
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        nm = self.names
        # one product makes q | k | v | b | the decay's input (or its low rank) | the gate's input (or its low rank)
        self.w_in, self._offsets = _stack_padded([tensors[nm[r]] for r in ("q", "k", "v", "b", "a1" if self.decay_rank else "a",
                                                                            "g1" if self.gate_rank else "g")])
        self.w_conv = torch.cat([tensors[nm[r]] for r in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        self.w_a2 = tensors[nm["a2"]].contiguous() if self.decay_rank else None
        self.w_g2 = tensors[nm["g2"]].contiguous() if self.gate_rank else None
        # what enters the recurrence is float32
        self.dt_bias, self.a_log = tensors[nm["dt_bias"]].float().contiguous(), tensors[nm["a_log"]].float().contiguous()
        self.g, self.w_o = tensors[nm["norm"]].contiguous(), tensors[nm["o"]].contiguous()

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CallCacheView, owns_cache: bool) -> torch.Tensor:
        state = _state_and_slots(cache, ctx, owns_cache, "a delta-rule mixer")
        n = x.shape[0]
        proj = ctx.empty(n, self.w_in.shape[0])
        ops.linear(x, self.w_in, None, proj)
        o_q, o_k, o_v, o_b, o_a, o_g = self._offsets
        if o_k != self.qk_width or o_v != 2 * self.qk_width:
            # q, k and v must lie side by side for the convolution: sizes that are no multiples of 8 are laid out again
            raw = torch.cat([proj[:, o_q:o_q + self.qk_width], proj[:, o_k:o_k + self.qk_width], proj[:, o_v:o_v + self.inner]], dim=1)
        else:
            raw = proj[:, :self.channels]
        bounds = step_segment_bounds(ctx)
        single = ctx.decode_only
        tok_seg = None if single else ctx.tok_seg
        qkv = ctx.empty(n, self.channels)
        ops.causal_conv_silu(raw, self.w_conv, None, state, self.state_elems, ctx.slots, tok_seg, ctx.positions, qkv, update_state=single)
        if not single:
            ops.conv_state_update(raw, self.taps, state, self.state_elems, ctx.slots, bounds, ctx.positions, ctx.n_segments)
        if self.decay_rank is None:
            a = proj[:, o_a:o_a + self.decay_width]
        else:
            a = ctx.empty(n, self.decay_width)
            ops.linear(proj[:, o_a:o_a + self.decay_rank], self.w_a2, None, a)
        if self.gate_rank is None:
            gate = proj[:, o_g:o_g + self.inner]
        else:
            gate = ctx.empty(n, self.inner)
            ops.linear(proj[:, o_g:o_g + self.gate_rank], self.w_g2, None, gate)
        y = ctx.empty(n, self.inner, dtype=torch.float32)
        ops.linear_state("delta", qkv[:, :self.qk_width], qkv[:, self.qk_width:2 * self.qk_width], qkv[:, 2 * self.qk_width:], state,
                         ctx.slots, bounds, y, ctx.n_segments, self.heads, self.kv_heads, self.dim, self.vdim, a=a,
                         b=proj[:, o_b:o_b + self.heads], dt_bias=self.dt_bias, a_log=self.a_log, q_scale=self.dim ** -0.5,
                         unit_eps=UNIT_EPS, work=_walk_workspace("delta", ctx, n, self.heads, self.dim, self.vdim),
                         decay_per_head=self.decay_per == "head")
        normed = ctx.empty(n, self.inner)
        ops.group_rmsnorm_gate(y, gate, self.g, self.heads, self.eps, normed, gate=self.gate_act)
        out = ctx.empty(n, self.hidden_size)
        ops.linear(normed, self.w_o, None, out)
        return out


@register_mixer("gated_delta")
class GatedDeltaMixer(ChannelDeltaMixer):
    """The delta rule with one decay per head, the decay's and the gate's inputs as plain projections (``a`` ``[heads,
    hidden]``, ``g`` ``[heads * vdim, hidden]``) and a SiLU gate on the normed read-out."""

    def __init__(self, hidden_size: int, heads: int, kv_heads: int, dim: int, vdim: int, conv: int, eps: float,
                 names: Optional[Mapping[str, str]] = None):
        super().__init__(hidden_size, heads, kv_heads, dim, vdim, conv, None, None, eps, names=names, decay_per="head", gate_act="silu")


@register_mixer("forget_gate")
class ForgetGateMixer(Mixer):
    capture_safe = True

    def __init__(self, hidden_size: int, heads: int, dim: int, vdim: int, eps: float, names: Optional[Mapping[str, str]] = None):
        if min(hidden_size, heads, dim, vdim) <= 0:
            raise ValueError("forget_gate: every size must be positive")
        if dim > 256:
            raise ValueError(f"forget_gate: dim={dim} is not supported; the recurrence kernel takes at most 256")
        self.hidden_size, self.heads, self.dim, self.vdim, self.eps = int(hidden_size), int(heads), int(dim), int(vdim), float(eps)
        self.qk_width, self.inner = self.heads * self.dim, self.heads * self.vdim
        self.state_elems = self.heads * self.vdim * self.dim
        self.names = {"q": "q", "f": "f", "f_bias": "f.b", "lower": "lower", "v": "v", "norm": "norm", "o": "o"}
        self.names.update(names or {})
        self.w_in = self.b_in = self.lower = self.g = self.w_o = None
        self._offsets: List[int] = []

    def cache_need(self):
        return StateNeed((self.state_elems,), torch.float32)           # S of every head, [heads, vdim, dim]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        nm, h = self.names, self.hidden_size
        return {nm["q"]: TensorSpec((self.qk_width, h)), nm["f"]: TensorSpec((self.qk_width, h)), nm["f_bias"]: TensorSpec((self.qk_width,)),
                nm["lower"]: TensorSpec((self.qk_width,)), nm["v"]: TensorSpec((self.inner, h)),
                nm["norm"]: TensorSpec((self.vdim,), init=("one_plus_normal", 0.01)), nm["o"]: TensorSpec((h, self.inner))}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        nm = self.names
        # one product makes q | the gate's input | v; of the three only the gate's input has a bias
        self.w_in, self._offsets = _stack_padded([tensors[nm[r]] for r in ("q", "f", "v")])
        self.b_in = torch.zeros(self.w_in.shape[0], dtype=self.w_in.dtype, device=self.w_in.device)
        self.b_in[self._offsets[1]:self._offsets[1] + self.qk_width] = tensors[nm["f_bias"]].to(self.w_in.dtype)
        self.lower = tensors[nm["lower"]].float().contiguous()            # what enters the recurrence is float32
        self.g, self.w_o = tensors[nm["norm"]].contiguous(), tensors[nm["o"]].contiguous()

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CallCacheView, owns_cache: bool) -> torch.Tensor:
        state = _state_and_slots(cache, ctx, owns_cache, "a forget-gate mixer")
        n = x.shape[0]
        proj = ctx.empty(n, self.w_in.shape[0])
        ops.linear(x, self.w_in, self.b_in, proj)
        o_q, o_f, o_v = self._offsets
        y = ctx.empty(n, self.inner, dtype=torch.float32)
        ops.linear_state("forget", proj[:, o_q:o_q + self.qk_width], None, proj[:, o_v:o_v + self.inner], state, ctx.slots,
                         step_segment_bounds(ctx), y, ctx.n_segments, self.heads, self.heads, self.dim, self.vdim,
                         a=proj[:, o_f:o_f + self.qk_width], dt_bias=self.lower, act_silu="q",
                         work=_walk_workspace("forget", ctx, n, self.heads, self.dim, self.vdim))
        normed = ctx.empty(n, self.inner)
        ops.group_rmsnorm_gate(y, None, self.g, self.heads, self.eps, normed, gate=None)
        out = ctx.empty(n, self.hidden_size)
        ops.linear(normed, self.w_o, None, out)
        return out


@register_mixer("lightning")
class LightningMixer(Mixer):
    capture_safe = True

    def __init__(self, hidden_size: int, heads: int, dim: int, vdim: int, decay: Sequence[float], eps: float,
                 names: Optional[Mapping[str, str]] = None):
        if min(hidden_size, heads, dim, vdim) <= 0:
            raise ValueError("lightning: every size must be positive")
        if len(decay) != heads:
            raise ValueError(f"lightning: {len(decay)} decays for {heads} heads")
        if dim > 256:
            raise ValueError(f"lightning: dim={dim} is not supported; the recurrence kernel takes at most 256")
        self.hidden_size, self.heads, self.dim, self.vdim, self.eps = int(hidden_size), int(heads), int(dim), int(vdim), float(eps)
        self.decay_values = [float(d) for d in decay]
        self.qk_width, self.inner = self.heads * self.dim, self.heads * self.vdim
        self.state_elems = self.heads * self.vdim * self.dim
        self.names = {"q": "q", "k": "k", "v": "v", "g": "g", "norm": "norm", "o": "o"}
        self.names.update(names or {})
        self.w_in = self.g = self.w_o = self.decay = None
        self._offsets: List[int] = []

    def cache_need(self):
        return StateNeed((self.state_elems,), torch.float32)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        nm, h = self.names, self.hidden_size
        return {nm["q"]: TensorSpec((self.qk_width, h)), nm["k"]: TensorSpec((self.qk_width, h)), nm["v"]: TensorSpec((self.inner, h)),
                nm["g"]: TensorSpec((self.inner, h)), nm["norm"]: TensorSpec((self.inner,), init=("one_plus_normal", 0.01)),
                nm["o"]: TensorSpec((h, self.inner))}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        nm = self.names
        self.w_in, self._offsets = _stack_padded([tensors[nm[r]] for r in ("q", "k", "v", "g")])
        self.g, self.w_o = tensors[nm["norm"]].contiguous(), tensors[nm["o"]].contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.w_o.device)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CallCacheView, owns_cache: bool) -> torch.Tensor:
        state = _state_and_slots(cache, ctx, owns_cache, "a lightning mixer")
        n = x.shape[0]
        proj = ctx.empty(n, self.w_in.shape[0])
        ops.linear(x, self.w_in, None, proj)
        o_q, o_k, o_v, o_g = self._offsets
        y = ctx.empty(n, self.inner, dtype=torch.float32)
        ops.linear_state("decay", proj[:, o_q:o_q + self.qk_width], proj[:, o_k:o_k + self.qk_width], proj[:, o_v:o_v + self.inner],
                         state, ctx.slots, step_segment_bounds(ctx), y, ctx.n_segments, self.heads, self.heads, self.dim, self.vdim,
                         decay=self.decay, act_silu=True, work=_walk_workspace("decay", ctx, n, self.heads, self.dim, self.vdim))
        normed = ctx.empty(n, self.inner)
        ops.group_rmsnorm_gate(y, proj[:, o_g:o_g + self.inner], self.g, 1, self.eps, normed)
        out = ctx.empty(n, self.hidden_size)
        ops.linear(normed, self.w_o, None, out)
        return out
