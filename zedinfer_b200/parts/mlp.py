"""Gated feed-forward: ``down(up(x) * act(gate(x)))`` with SiLU, no biases unless asked
(src/frontend/models/transformer_forward.cpp:128-137, src/backend/ops/swiglu/cpu/swiglu_cpu.cpp:13-20).
Gate and up weights are stacked at load so one product makes both."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import FeedForward, StepContext, register_feed_forward


def _stack(tensors):
    """Concatenate along dim 0; if storage dtypes differ, float32 wins."""
    dtype = torch.float32 if any(t.dtype == torch.float32 for t in tensors) else tensors[0].dtype
    return torch.cat([t.to(dtype) for t in tensors], dim=0).contiguous()


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    capture_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu", bias: bool = False,
                 names: Optional[Mapping[str, str]] = None):
        """``names``: the local tensor names of the three weights by role (``gate``, ``up``, ``down``); a bias is the
        weight's name with ``.weight`` replaced by ``.bias``."""
        if activation != "silu":
            raise ValueError(f"gated_mlp: activation {activation!r} is not supported (only 'silu')")
        if hidden_size <= 0 or intermediate_size <= 0:
            raise ValueError("gated_mlp: sizes must be positive")
        self.hidden_size, self.intermediate_size, self.bias = int(hidden_size), int(intermediate_size), bool(bias)
        self.names = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}
        self.names.update(names or {})
        if self.bias and not all(n.endswith(".weight") for n in self.names.values()):
            raise ValueError("gated_mlp: biases are named after weights that end in '.weight'")
        self.w_gate_up: Optional[torch.Tensor] = None
        self.b_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None
        self.b_down: Optional[torch.Tensor] = None

    def _bias_name(self, role: str) -> str:
        return self.names[role][:-len("weight")] + "bias"

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        h, i, nm = self.hidden_size, self.intermediate_size, self.names
        specs = {nm["gate"]: TensorSpec((i, h)), nm["up"]: TensorSpec((i, h)), nm["down"]: TensorSpec((h, i))}
        if self.bias:
            specs.update({self._bias_name("gate"): TensorSpec((i,)), self._bias_name("up"): TensorSpec((i,)),
                          self._bias_name("down"): TensorSpec((h,))})
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        nm = self.names
        self.w_gate_up = _stack([tensors[nm["gate"]], tensors[nm["up"]]])
        self.w_down = tensors[nm["down"]].contiguous()
        if self.bias:
            self.b_gate_up = _stack([tensors[self._bias_name("gate")], tensors[self._bias_name("up")]])
            self.b_down = tensors[self._bias_name("down")].contiguous()

    def _activation(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        act = ctx.empty(x.shape[0], self.intermediate_size)
        ops.linear_silu_mul(x, self.w_gate_up, self.b_gate_up, act)     # activation in the product's epilogue where it can be
        return act

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        out = ctx.empty(x.shape[0], self.hidden_size)
        ops.linear(self._activation(x, ctx), self.w_down, self.b_down, out)
        return out

    def forward_for_residual(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return ops.linear_for_residual(self._activation(x, ctx), self.w_down, self.b_down)   # the product, or partial sums over K


@register_feed_forward("squared_relu_mlp")
class SquaredReluMLP(FeedForward):
    """``down(relu(up(x))^2)``, no gate, no biases."""
    capture_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, up_name: str = "up", down_name: str = "down"):
        if hidden_size <= 0 or intermediate_size <= 0:
            raise ValueError("squared_relu_mlp: sizes must be positive")
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.up_name, self.down_name = up_name, down_name
        self.w_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.up_name: TensorSpec((self.intermediate_size, self.hidden_size)),
                self.down_name: TensorSpec((self.hidden_size, self.intermediate_size))}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_up = tensors[self.up_name].contiguous()
        self.w_down = tensors[self.down_name].contiguous()

    def _activation(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        act = ctx.empty(x.shape[0], self.intermediate_size)
        ops.linear_relu2(x, self.w_up, act)               # the activation in the product's epilogue where it can be
        return act

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        out = ctx.empty(x.shape[0], self.hidden_size)
        ops.linear(self._activation(x, ctx), self.w_down, None, out)
        return out

    def forward_for_residual(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return ops.linear_for_residual(self._activation(x, ctx), self.w_down, None)


@register_feed_forward("poly_norm_mlp")
class PolyNormMLP(FeedForward):
    """``down(P(up(x)))`` with ``P(z) = c1 U(z) + c2 U(z^2) + c3 U(z^3) + c0``: powers entry by entry, each divided by its own
    root mean square over the row, ``U(v) = v / sqrt(mean(v^2) + eps)`` (float32).  The four numbers come from one tensor
    ``[c1, c2, c3, c0]``; no gate, no biases."""
    capture_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, eps: float, up_name: str = "up", down_name: str = "down",
                 coeff_name: str = "act"):
        if hidden_size <= 0 or intermediate_size <= 0:
            raise ValueError("poly_norm_mlp: sizes must be positive")
        if not eps > 0.0:
            raise ValueError(f"poly_norm_mlp: eps={eps} must be positive")
        self.hidden_size, self.intermediate_size, self.eps = int(hidden_size), int(intermediate_size), float(eps)
        self.up_name, self.down_name, self.coeff_name = up_name, down_name, coeff_name
        self.w_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None
        self.coeffs = (1.0, 0.0, 0.0, 0.0)

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.up_name: TensorSpec((self.intermediate_size, self.hidden_size)),
                self.down_name: TensorSpec((self.hidden_size, self.intermediate_size)),
                self.coeff_name: TensorSpec((4,), init=("normal", 0.5))}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_up = tensors[self.up_name].contiguous()
        self.w_down = tensors[self.down_name].contiguous()
        self.coeffs = tuple(float(c) for c in tensors[self.coeff_name].float().cpu().tolist())     # read once, at load

    def _activation(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        z = ctx.empty(x.shape[0], self.intermediate_size)
        ops.linear(x, self.w_up, None, z)
        act = ctx.empty(x.shape[0], self.intermediate_size)
        ops.poly_norm(z, self.coeffs, self.eps, act)
        return act

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        out = ctx.empty(x.shape[0], self.hidden_size)
        ops.linear(self._activation(x, ctx), self.w_down, None, out)
        return out


@register_feed_forward("clamped_gated_mlp")
class ClampedGatedMLP(FeedForward):
    """``down(g * sigmoid(slope * g) * (u + up_offset))`` with ``g = min(gate(x), limit)``, ``u = clamp(up(x), -limit,
    limit)``; no biases.  ``limit=None``: no clamping."""
    capture_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, limit: Optional[float], slope: float = 1.0,
                 up_offset: float = 0.0, gate_name: str = "gate", up_name: str = "up", down_name: str = "down"):
        if hidden_size <= 0 or intermediate_size <= 0:
            raise ValueError("clamped_gated_mlp: sizes must be positive")
        if limit is not None and not limit > 0.0:
            raise ValueError(f"clamped_gated_mlp: limit={limit} must be positive (or None)")
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.limit, self.slope, self.up_offset = (float(limit) if limit is not None else 0.0), float(slope), float(up_offset)
        self.gate_name, self.up_name, self.down_name = gate_name, up_name, down_name
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        h, i = self.hidden_size, self.intermediate_size
        return {self.gate_name: TensorSpec((i, h)), self.up_name: TensorSpec((i, h)), self.down_name: TensorSpec((h, i))}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_gate_up = _stack([tensors[self.gate_name], tensors[self.up_name]])
        self.w_down = tensors[self.down_name].contiguous()

    def _activation(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        act = ctx.empty(x.shape[0], self.intermediate_size)
        ops.linear_gated_clamp_mul(x, self.w_gate_up, act, self.limit, self.slope, self.up_offset)
        return act

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        out = ctx.empty(x.shape[0], self.hidden_size)
        ops.linear(self._activation(x, ctx), self.w_down, None, out)
        return out

    def forward_for_residual(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return ops.linear_for_residual(self._activation(x, ctx), self.w_down, None)


@register_feed_forward("token_gated_table")
class TokenGatedTable(FeedForward):
    """A token's own table entry, gated by the stream: ``proj(gelu_tanh(gate(x)) * table[token, col0 : col0 + dim])``, no
    biases.  The table has a row per token of the vocabulary and is the embedding's to load (``scaled_token_embedding``'s
    ``token_tables``); this part finds it under ``ctx.step_cache[("token_table", table)]`` and reads ``dim`` columns from
    ``col0`` on (a layer's share of a table that all layers divide among themselves)."""
    capture_safe = True

    def __init__(self, hidden_size: int, dim: int, table: str, col0: int = 0, gate_name: str = "gate", proj_name: str = "proj"):
        if hidden_size <= 0 or dim <= 0 or col0 < 0:
            raise ValueError("token_gated_table: sizes must be positive")
        self.hidden_size, self.dim, self.table, self.col0 = int(hidden_size), int(dim), str(table), int(col0)
        self.gate_name, self.proj_name = gate_name, proj_name
        self.w_gate: Optional[torch.Tensor] = None
        self.w_proj: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.gate_name: TensorSpec((self.dim, self.hidden_size)), self.proj_name: TensorSpec((self.hidden_size, self.dim))}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w_gate = tensors[self.gate_name].contiguous()
        self.w_proj = tensors[self.proj_name].contiguous()

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        table = ctx.step_cache.get(("token_table", self.table))
        if table is None:
            raise RuntimeError(f"token_gated_table: the model's embedding has left no table {self.table!r} for this step")
        n = x.shape[0]
        t = ctx.empty(n, self.dim)
        ops.linear(x, self.w_gate, None, t)
        g = ctx.empty(n, self.dim)
        ops.gelu_mul_rows(t, table, self.col0, ctx.token_ids, g)
        out = ctx.empty(n, self.hidden_size)
        ops.linear(g, self.w_proj, None, out)
        return out
