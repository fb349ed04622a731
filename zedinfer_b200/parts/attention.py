"""Causal self-attention with grouped key/value heads over the paged cache.

Per token (src/frontend/models/transformer_forward.cpp:71-112, and
src/backend/ops/self_attention/cpu/paged_attention_cpu.cpp:113-159 for the scores):

    q, k, v = x Wq^T + bq, x Wk^T + bk, x Wv^T + bv       (one stacked product)
    q, k rotated by position; k, v appended to the request's cache pages
    s_j = (q . k_j) * scale for the keys j the query may see; softmax in float32; out = sum p_j v_j
    y = out Wo^T (+ bo)

A query at position P sees keys ``max(0, P - window + 1) .. P`` (all keys from 0 without a
window).  Query head ``h`` reads key/value head ``h // (num_heads // num_kv_heads)``.

Options beside the reference's form: ``value_from_key`` (there is no value projection: a token's value is its key as
projected, before the position rule turns it; the cache still has two planes, turned keys and plain ones),
``unit_sink`` (the softmax's denominator holds one more term, ``exp(0)``, that has no key and no value: ``p_j = exp(s_j) /
(1 + sum_j' exp(s_j'))``), ``names`` (the local tensor names by role), ``softcap`` c (a scaled score s becomes ``c tanh(s /
c)`` before the softmax), ``v_head_dim`` (value heads of another size than the query/key heads: the cache's rows and the
heads of the query are then ``row_dim`` wide, the larger of the two sizes rounded up to a multiple of 8, and what lies past
a head's own entries is zero, which changes no score and no output), ``shared_kv`` (the layer has no key and value
projections: it reads the cache that another layer's call wrote, with its own queries, window and everything else) and
``cache_window`` (the window the cache keeps pages for, where layers that read this layer's cache look further back than
the layer itself; ``"own"``: the layer's window, None: all keys) and ``head_scale`` (the local name of a tensor with one
number per query head that multiplies that head's scores, ``s = q . k * scale * t_h``; the query head is multiplied by it, in
float32, as the position rule's kernel writes it, so it goes with ``v_head_dim`` given).
"""
from __future__ import annotations

import math
from typing import Dict, Mapping, Optional

import torch

from .. import ops
from ..cache.manager import CallCacheView, PagedKVNeed
from ..config.spec import PartSpec
from ..weights.loader import TensorSpec
from .base import Mixer, StepContext, build_part, register_mixer
from .mlp import _stack


@register_mixer("attention")
class AttentionMixer(Mixer):
    @property
    def capture_safe(self) -> bool:        # as safe as the position rule it was built with
        return bool(getattr(self.position, "capture_safe", False))

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PartSpec, qkv_bias: bool = True, out_bias: bool = False,
                 scale: Optional[float] = None, window: Optional[int] = None, value_from_key: bool = False,
                 unit_sink: bool = False, names: Optional[Mapping[str, str]] = None, softcap: Optional[float] = None,
                 v_head_dim: Optional[int] = None, shared_kv: bool = False, cache_window="own", head_scale: Optional[str] = None):
        if num_heads <= 0 or num_kv_heads <= 0 or num_heads % num_kv_heads:
            raise ValueError(f"attention: {num_heads} query heads cannot share {num_kv_heads} key/value heads")
        if softcap is not None and not softcap > 0.0:
            raise ValueError(f"attention: softcap={softcap} must be positive (or None for no cap)")
        if v_head_dim is not None and (v_head_dim <= 0 or position.kind != "rope_span" or value_from_key):
            raise ValueError("attention: value heads of a size of their own need a positive size, the position rule 'rope_span' "
                             "and a value projection")
        if head_scale is not None and v_head_dim is None:
            raise ValueError("attention: a factor per query head goes with v_head_dim given (the size of the value heads)")
        self.head_scale_name = head_scale
        self.head_scale: Optional[torch.Tensor] = None
        if shared_kv and (value_from_key or qkv_bias):
            raise ValueError("attention: a layer without key and value projections has neither their biases nor keys as values")
        # a rule that turns a span of the head (its own kernel) takes steps of 8; the rotate-half kernels steps of 16
        step = 8 if position.kind == "rope_span" else 16
        self.v_head_dim = int(v_head_dim) if v_head_dim is not None else int(head_dim)
        # rows of the cache and heads of the query: a head's own size, or wide enough for keys and values alike
        self.row_dim = int(head_dim) if v_head_dim is None else (max(int(head_dim), int(v_head_dim)) + 7) // 8 * 8
        if v_head_dim is not None:
            if head_dim <= 0 or self.row_dim > 1024:
                raise ValueError(f"attention: head sizes {head_dim} and {v_head_dim} are not supported; rows of at most 1024 entries")
        elif head_dim <= 0 or head_dim % step:
            raise ValueError(f"attention: head_dim={head_dim} is not supported; the kernels take head sizes "
                             f"in steps of {step} ({step}, {2 * step}, ..., 256)")
        elif head_dim > 256:
            raise ValueError(f"attention: head_dim={head_dim} is not supported; the kernels take at most 256")
        if window is not None and window <= 0:
            raise ValueError(f"attention: window={window} must be positive (or None for all keys)")
        if cache_window != "own" and cache_window is not None and (window is None or int(cache_window) < window):
            raise ValueError(f"attention: cache_window={cache_window} must be at least the layer's own window {window} "
                             "(None: all keys)")
        self.softcap = float(softcap) if softcap is not None else None
        self.shared_kv = bool(shared_kv)
        # what the cache keeps: the layer's own window, or more where its readers look further back (all keys: None)
        self.cache_window = window if cache_window == "own" else cache_window
        self.cache_window = int(self.cache_window) if self.cache_window is not None else None
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim, self.window = int(head_dim), (int(window) if window is not None else None)
        self.qkv_bias, self.out_bias = bool(qkv_bias), bool(out_bias)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(float(head_dim))
        self.position = build_part("position", position)
        self.value_from_key, self.unit_sink = bool(value_from_key), bool(unit_sink)
        # A rotate-half span at the start of a head of a multiple of 16 entries runs on the kernels that turn whole heads,
        # with the head's entries reordered at bind (SpanAsWholeRotaryPosition); keys that are also values then come out
        # of the product twice (the key rows stand in the stacked weight a second time, as the value rows), so that the
        # fused decode product and the vectorised rotation append them as they append any values.
        if position.kind == "rope_span" and v_head_dim is None and (self.position.scaling is not None
                                                                   or self.position.unit_rms_eps is not None):
            raise ValueError("attention: stretched frequencies and unit heads go with v_head_dim given (the size of the value heads)")
        self._reordered = (position.kind == "rope_span" and not self.position.interleaved and self.position.offset == 0
                           and head_dim % 16 == 0 and v_head_dim is None)
        if self._reordered:
            self.position = build_part("position", PartSpec("rope_span_as_whole", {
                "head_dim": head_dim, "dims": self.position.dims, "theta": self.position.theta}))
        elif self.value_from_key and not getattr(self.position, "takes_value_from_key", False):
            raise ValueError(f"attention: the position rule {position.kind!r} cannot append unturned keys as values")
        self.names = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
                      "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias", "o_bias": "o_proj.bias"}
        self.names.update(names or {})
        self.q_dim, self.kv_dim = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        self.v_dim = self.num_kv_heads * self.v_head_dim
        self._wide = v_head_dim is not None
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = self.sinks = None

    def cache_need(self):
        return PagedKVNeed(self.num_kv_heads, self.row_dim, self.cache_window)

    def _roles(self):
        return ("q",) if self.shared_kv else (("q", "k") if self.value_from_key else ("q", "k", "v"))

    def _width(self, role: str) -> int:
        return {"q": self.q_dim, "k": self.kv_dim, "v": self.v_dim}[role]

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        h, nm = self.hidden_size, self.names
        roles = self._roles()
        specs = {nm[r]: TensorSpec((self._width(r), h)) for r in roles}
        specs[nm["o"]] = TensorSpec((h, self.num_heads * self.v_head_dim))
        if self.qkv_bias:
            specs.update({nm[r + "_bias"]: TensorSpec((self._width(r),)) for r in roles})
        if self.out_bias:
            specs[nm["o_bias"]] = TensorSpec((h,))
        if self.head_scale_name is not None:
            specs[self.head_scale_name] = TensorSpec((self.num_heads,), init=("one_plus_normal", 0.05))
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        nm = self.names
        roles = self._roles()
        if self._reordered:
            order = self.position.head_order().to(tensors[nm["q"]].device)

            def rows(t: torch.Tensor, heads: int) -> torch.Tensor:          # a projection's rows (or a bias), head by head
                return t.view(heads, self.head_dim, *t.shape[1:])[:, order].reshape(t.shape)

            tensors = dict(tensors)
            for r in roles:
                heads = self.num_heads if r == "q" else self.num_kv_heads
                if r != "v":                                              # values keep their order only if they are no keys
                    tensors[nm[r]] = rows(tensors[nm[r]], heads)
                    if self.qkv_bias:
                        tensors[nm[r + "_bias"]] = rows(tensors[nm[r + "_bias"]], heads)
            if self.value_from_key:
                # the output product reads the heads in the keys' new order
                w_o = tensors[nm["o"]]
                tensors[nm["o"]] = w_o.view(w_o.shape[0], self.num_heads, self.head_dim)[:, :, order].reshape(w_o.shape)
                roles = ("q", "k", "k")
        self.w_qkv = _stack([tensors[nm[r]] for r in roles])
        if self.qkv_bias:
            self.b_qkv = _stack([tensors[nm[r + "_bias"]] for r in roles])
            if self.b_qkv.dtype != self.w_qkv.dtype:
                # one product, one operand type: float32 wins
                self.w_qkv, self.b_qkv = self.w_qkv.float(), self.b_qkv.float()
        self.w_o = tensors[nm["o"]].contiguous()
        if self.row_dim != self.v_head_dim:
            # the attention's output has row_dim entries per head, zero past the value's own: the weight gets zero columns there
            w_o = self.w_o.new_zeros((self.hidden_size, self.num_heads, self.row_dim))
            w_o[:, :, :self.v_head_dim] = self.w_o.view(self.hidden_size, self.num_heads, self.v_head_dim)
            self.w_o = w_o.view(self.hidden_size, self.num_heads * self.row_dim)
        if self.out_bias:
            self.b_o = tensors[nm["o_bias"]].contiguous()
        if self.unit_sink:
            self.sinks = torch.zeros(self.num_heads, dtype=torch.float32, device=self.w_o.device)
        if self.head_scale_name is not None:
            self.head_scale = tensors[self.head_scale_name].float().contiguous()       # scores are float32

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CallCacheView, owns_cache: bool) -> torch.Tensor:
        out = ctx.empty(x.shape[0], self.hidden_size)
        ops.linear(self._attend(x, ctx, cache, owns_cache), self.w_o, self.b_o, out)
        return out

    def forward_for_residual(self, x: torch.Tensor, ctx: StepContext, cache: CallCacheView,
                             owns_cache: bool) -> torch.Tensor:
        return ops.linear_for_residual(self._attend(x, ctx, cache, owns_cache), self.w_o, self.b_o)

    def _attend(self, x: torch.Tensor, ctx: StepContext, cache: CallCacheView, owns_cache: bool) -> torch.Tensor:
        """Everything up to the output projection: ``[tokens, heads * head_dim]``."""
        if cache.kind != "paged":
            raise RuntimeError("attention needs a paged key/value cache")
        n = x.shape[0]
        if self.shared_kv == owns_cache:
            raise RuntimeError("attention: a layer with key and value projections writes a cache of its own, and only a "
                               "layer without them reads another's")
        if self._wide or self.shared_kv:
            # one product for whatever projections the layer has; the position rule's kernel turns, norms, pads and appends
            proj = ctx.empty(n, self.w_qkv.shape[0])
            ops.linear(x, self.w_qkv, self.b_qkv, proj)
            q = ctx.empty(n, self.num_heads, self.row_dim)
            if self._wide:
                self.position.rotate_append(proj, q, cache, ctx, self.num_heads, self.num_kv_heads, self.head_dim,
                                            write_kv=owns_cache, v_dim=self.v_head_dim, row_dim=self.row_dim,
                                            q_head_scale=self.head_scale)
            else:
                self.position.rotate_append(proj, q, cache, ctx, self.num_heads, self.num_kv_heads, self.head_dim, write_kv=False)
            attn = ctx.empty(n, self.num_heads * self.row_dim)
            ops.attention(q, cache, attn, ctx, self.num_heads, self.num_kv_heads, self.row_dim, self.window, self.scale,
                          sinks=self.sinks, softcap=self.softcap)
            return attn
        q = ctx.empty(n, self.num_heads, self.head_dim)
        if self.value_from_key and not self._reordered:
            qk = ctx.empty(n, self.q_dim + self.kv_dim)
            ops.linear(x, self.w_qkv, self.b_qkv, qk)
            self.position.rotate_append(qk, q, cache, ctx, self.num_heads, self.num_kv_heads, self.head_dim,
                                        write_kv=owns_cache, value_from_key=True)
        elif not self.position.project_rotate_append(x, self.w_qkv, self.b_qkv, q, cache, ctx, self.num_heads,
                                                     self.num_kv_heads, self.head_dim, write_kv=owns_cache):
            qkv = ctx.empty(n, self.q_dim + 2 * self.kv_dim)
            ops.linear(x, self.w_qkv, self.b_qkv, qkv)
            self.position.rotate_append(qkv, q, cache, ctx, self.num_heads, self.num_kv_heads, self.head_dim,
                                        write_kv=owns_cache)
        attn = ctx.empty(n, self.q_dim)
        ops.attention(q, cache, attn, ctx, self.num_heads, self.num_kv_heads, self.head_dim, self.window, self.scale,
                      sinks=self.sinks, softcap=self.softcap)
        return attn
