"""Routed feed-forward: every token runs ``top`` of ``experts`` small gated feed-forwards, weighted, plus an optional
shared one that every token runs.

    z = Wr x + b                     router logits, float32
    S = the ``top`` largest z        (lowest index wins a tie)
    y = sum_{e in S} softmax_S(z)_e * expert_e(x)   (+ shared(x))

Each expert has the form of :class:`~zedinfer_b200.parts.mlp.ClampedGatedMLP` (``activation="clamped_gate"``), or, with
``activation="relu2"``, of :class:`~zedinfer_b200.parts.mlp.SquaredReluMLP`: ``down(max(up x, 0)^2)``, no gate matrix.
``score="sigmoid"``: a chosen expert's weight is its own ``sigmoid(z_e)``, not renormalised (the choice is still by the
largest z, which is the largest score).  ``weight_on="input"``: the weight multiplies the expert's input instead of its
output, ``y = sum_e expert_e(w_e x)``, the scaled row rounded to the step's type before the first product.
``score="softmax_all"``: an expert's score is its share of the softmax over all experts; the choice goes by ``score +
choice_bias`` (a tensor of one number per expert, ``choice_bias_name``) and the weights are the chosen experts' scores
themselves, not renormalised.  ``identity`` n: the router has ``experts + n`` outputs, and the last n of them are experts
without tensors that return their input, ``y += s_e x``.  ``shared_gate_name``: the shared expert's output is multiplied by
``sigmoid(w_sg . x)``, one number per token (float32), ``w_sg`` a tensor ``[1, hidden]`` under the shared expert's prefix.

Nothing goes to the host: the step's
(token, choice) pairs are grouped by expert on the device, the two products run as grouped products over the sorted
rows (``csrc/moe.cu``, or the tcgen05 grouped product from a few hundred rows; the activation in the first one's epilogue), and one kernel adds a token's rows with its router
weights and the shared expert's output in float32.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from ..config.spec import PartSpec
from ..weights.loader import TensorSpec
from .base import FeedForward, StepContext, build_part, register_feed_forward


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, experts: int, top: int, limit: Optional[float] = None,
                 slope: float = 1.0, up_offset: float = 0.0, router_bias: bool = True, shared: Optional[PartSpec] = None,
                 expert_prefix: str = "e{e}.", router_name: str = "router", router_bias_name: str = "router.b",
                 shared_prefix: str = "shared.", gate_name: str = "gate", up_name: str = "up", down_name: str = "down",
                 activation: str = "clamped_gate", score: str = "softmax_chosen", weight_on: str = "output",
                 choice_bias_name: Optional[str] = None, identity: int = 0, shared_gate_name: Optional[str] = None):
        """``shared``: the spec of a feed-forward that every token runs as well (its tensors under ``shared_prefix``)."""
        if activation not in ("clamped_gate", "relu2"):
            raise ValueError(f"routed_experts: activation={activation!r} is not 'clamped_gate' or 'relu2'")
        if score not in ops.ROUTER_SCORES:
            raise ValueError(f"routed_experts: score={score!r} is not one of {sorted(ops.ROUTER_SCORES)}")
        if weight_on not in ("output", "input"):
            raise ValueError(f"routed_experts: weight_on={weight_on!r} is not 'output' or 'input'")
        if choice_bias_name is not None and score != "softmax_all":
            raise ValueError("routed_experts: a bias on the choice goes with score='softmax_all'")
        if identity < 0 or (identity and weight_on != "output"):
            raise ValueError("routed_experts: experts that return their input are counted from 0 and weigh their output")
        if shared_gate_name is not None and shared is None:
            raise ValueError("routed_experts: a gate on the shared expert needs a shared expert")
        self.choice_bias_name, self.identity, self.shared_gate_name = choice_bias_name, int(identity), shared_gate_name
        self.activation, self.score, self.weight_on = activation, score, weight_on
        self.gated = activation == "clamped_gate"
        if hidden_size <= 0 or intermediate_size <= 0:
            raise ValueError("routed_experts: sizes must be positive")
        if experts <= 0 or experts + identity > 1024 or not 0 < top <= experts + identity:
            raise ValueError(f"routed_experts: top={top} of {experts} + {identity} experts is not supported (1 <= top <= experts <= 1024)")
        if limit is not None and not limit > 0.0:
            raise ValueError(f"routed_experts: limit={limit} must be positive (or None)")
        self.hidden_size, self.intermediate_size, self.experts, self.top = int(hidden_size), int(intermediate_size), int(experts), int(top)
        self.limit, self.slope, self.up_offset = (float(limit) if limit is not None else 0.0), float(slope), float(up_offset)
        self.router_bias = bool(router_bias)
        self.expert_prefix, self.router_name, self.router_bias_name, self.shared_prefix = expert_prefix, router_name, router_bias_name, shared_prefix
        self.gate_name, self.up_name, self.down_name = gate_name, up_name, down_name
        self.shared = build_part("ffn", shared) if shared is not None else None
        self.w_router = self.b_router = self.w_gate_up = self.w_down = self.choice_bias = self.w_shared_gate = None
        self.outputs = self.experts + self.identity          # what the router chooses among

    @property
    def capture_safe(self) -> bool:
        return self.shared is None or bool(getattr(self.shared, "capture_safe", False))

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        h, i = self.hidden_size, self.intermediate_size
        specs = {self.router_name: TensorSpec((self.outputs, h))}
        if self.router_bias:
            specs[self.router_bias_name] = TensorSpec((self.outputs,))
        if self.choice_bias_name is not None:
            specs[self.choice_bias_name] = TensorSpec((self.outputs,), init=("normal", 0.01))
        if self.shared_gate_name is not None:
            specs[self.shared_prefix + self.shared_gate_name] = TensorSpec((1, h))
        for e in range(self.experts):
            p = self.expert_prefix.format(e=e)
            if self.gated:
                specs[p + self.gate_name] = TensorSpec((i, h))
            specs[p + self.up_name] = TensorSpec((i, h))
            specs[p + self.down_name] = TensorSpec((h, i))
        if self.shared is not None:
            for name, ts in self.shared.tensor_specs().items():
                specs[self.shared_prefix + name] = ts
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_router = tensors[self.router_name].contiguous()
        self.b_router = tensors[self.router_bias_name].float().contiguous() if self.router_bias else None
        self.choice_bias = tensors[self.choice_bias_name].float().contiguous() if self.choice_bias_name is not None else None
        if self.shared_gate_name is not None:
            self.w_shared_gate = tensors[self.shared_prefix + self.shared_gate_name].reshape(-1).contiguous()
        names = [self.expert_prefix.format(e=e) for e in range(self.experts)]
        first = (self.gate_name, self.up_name) if self.gated else (self.up_name,)
        dtype = torch.float32 if any(tensors[p + n].dtype == torch.float32 for p in names
                                     for n in first + (self.down_name,)) else tensors[names[0] + self.up_name].dtype
        # [experts, 2 * inner, hidden]: an expert's gate rows, then its up rows (without a gate: [experts, inner, hidden],
        # the up rows alone); [experts, hidden, inner]
        self.w_gate_up = torch.stack([torch.cat([tensors[p + n].to(dtype) for n in first], dim=0) for p in names]).contiguous()
        self.w_down = torch.stack([tensors[p + self.down_name].to(dtype) for p in names]).contiguous()
        if self.shared is not None:
            n = len(self.shared_prefix)
            self.shared.bind({k[n:]: v for k, v in tensors.items()
                              if k.startswith(self.shared_prefix) and k[n:] != self.shared_gate_name})

    def route(self, x: torch.Tensor):
        """(``idx`` int32 ``[tokens, top]``, ``wts`` float32 ``[tokens, top]``) of the step's tokens."""
        n = x.shape[0]
        idx = torch.empty((n, self.top), dtype=torch.int32, device=x.device)
        wts = torch.empty((n, self.top), dtype=torch.float32, device=x.device)
        ops.route(x, self.w_router, self.b_router, self.top, idx, wts, score=self.score,     # float32 logits whatever the operands' type
                  choice_bias=self.choice_bias)
        return idx, wts

    def _shared(self, x: torch.Tensor, ctx: StepContext):
        """(the shared expert's output, its gate per token), either of them None where the layer has none."""
        if self.shared is None:
            return None, None
        gate = None
        if self.w_shared_gate is not None:
            gate = torch.empty(x.shape[0], dtype=torch.float32, device=x.device)
            ops.row_gate(x, self.w_shared_gate, gate)
        return self.shared.forward(x, ctx), gate

    def _first_product(self) -> dict:
        """The activation of the experts' first product, as the grouped products' keywords."""
        return {"gated": (self.limit, self.slope, self.up_offset)} if self.gated else {"relu2": True}

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        n, pairs = x.shape[0], x.shape[0] * self.top
        idx, wts = self.route(x)
        if self._tcgen05_ok(x, pairs):
            return self._forward_tcgen05(x, ctx, idx, wts)
        offsets = torch.empty(self.experts + 1, dtype=torch.int32, device=x.device)
        row_pair = torch.empty(pairs, dtype=torch.int32, device=x.device)
        pair_row = torch.empty(pairs, dtype=torch.int32, device=x.device)
        ops.moe_group(idx, self.experts, offsets, row_pair, pair_row)
        act = ctx.empty(pairs, self.intermediate_size)
        on_input = self.weight_on == "input"
        ops.moe_gemm(x, row_pair, self.top, self.w_gate_up, offsets, act, a_scale=wts if on_input else None, **self._first_product())
        y = ctx.empty(pairs, self.hidden_size)
        ops.moe_gemm(act, None, 1, self.w_down, offsets, y)
        shared, gate = self._shared(x, ctx)
        out = ctx.empty(n, self.hidden_size)
        ops.moe_combine(y, pair_row.view(n, self.top), None if on_input else wts, shared, out, x=x if self.identity else None,
                        shared_gate=gate)
        return out

    def _tcgen05_ok(self, x: torch.Tensor, pairs: int) -> bool:
        return (ops.MOE_TENSOR_CORES and pairs >= ops.MOE_TCGEN05_MIN_PAIRS and x.dtype == torch.bfloat16
                and self.w_gate_up.dtype == torch.bfloat16 and self.hidden_size % 8 == 0 and self.intermediate_size % 8 == 0
                and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0)

    def _forward_tcgen05(self, x: torch.Tensor, ctx: StepContext, idx: torch.Tensor, wts: torch.Tensor) -> torch.Tensor:
        """Many rows: the step's rows are copied into sorted order, every expert's share padded to whole 128-row
        tiles, and both products run on the tcgen05 grouped kernel (the activation in the first one's epilogue)."""
        n, pairs, pad = x.shape[0], x.shape[0] * self.top, ops.GROUPED_TILE_ROWS
        tiles = (pairs + self.experts * (pad - 1) + pad - 1) // pad
        dev = x.device
        starts = torch.empty(self.experts + 1, dtype=torch.int32, device=dev)
        row_pair = torch.empty(tiles * pad, dtype=torch.int32, device=dev)
        pair_row = torch.empty(pairs, dtype=torch.int32, device=dev)
        tile_expert = torch.empty(tiles, dtype=torch.int32, device=dev)
        ops.moe_group_padded(idx, self.experts, pad, starts, row_pair, pair_row, tile_expert)
        xs = ctx.empty(tiles * pad, self.hidden_size)
        on_input = self.weight_on == "input"
        ops.moe_gather_rows(x, row_pair, self.top, xs, scale=wts if on_input else None)
        act = ctx.empty(tiles * pad, self.intermediate_size)
        ops.gemm_tcgen05_grouped(xs, self.w_gate_up, tile_expert, act, **self._first_product())
        y = ctx.empty(tiles * pad, self.hidden_size)
        ops.gemm_tcgen05_grouped(act, self.w_down, tile_expert, y)
        shared, gate = self._shared(x, ctx)
        out = ctx.empty(n, self.hidden_size)
        ops.moe_combine(y, pair_row.view(n, self.top), None if on_input else wts, shared, out, x=x if self.identity else None,
                        shared_gate=gate)
        return out
