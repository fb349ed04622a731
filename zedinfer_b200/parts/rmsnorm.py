"""RMSNorm: ``y = (w * x) * rstd``, ``rstd = 1 / sqrt(mean(x^2) + eps)``, in float32
(src/backend/ops/rms_norm/cpu/rms_norm_cpu.cpp:24-28).  No ``+1`` on the weight, unless the model stores its norm
weights around zero (``unit_offset``): the factor is then ``1 + w``, formed once in float32 when the weight is bound."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Norm, ResidualStream, StepContext, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    capture_safe = True

    def __init__(self, size: int, eps: float, name: str = "weight", unit_offset: bool = False, float32_weight: bool = False):
        """``name``: the tensor's local name; ``unit_offset``: the stored weight is the factor's distance from one;
        ``float32_weight``: the weight is widened to float32 when it is bound (for kernels that take it so)."""
        if size <= 0:
            raise ValueError(f"rmsnorm: size={size} must be positive")
        if not eps > 0.0:
            raise ValueError(f"rmsnorm: eps={eps} must be positive")
        self.size, self.eps, self.name, self.unit_offset = int(size), float(eps), str(name), bool(unit_offset)
        self.float32_weight = bool(float32_weight)
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.size,), init=("normal", 0.01) if self.unit_offset else ("one_plus_normal", 0.01))}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        w = tensors[self.name]
        # 1 + w does not fit bfloat16 without losing w's low bits: the factor is kept in float32 (the kernels take it so)
        self.weight = (w.float() + 1.0).contiguous() if self.unit_offset else (w.float() if self.float32_weight else w).contiguous()

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> None:
        ops.rmsnorm(x, self.weight, self.eps, out)

    def forward_residual(self, stream: ResidualStream, out: torch.Tensor,
                         row_idx: Optional[torch.Tensor] = None) -> None:
        if stream.delta is not None and (stream.delta_norm is not None or stream.delta_join is not None):
            raise RuntimeError("rmsnorm cannot fold a branch output that must pass a norm of its own first")
        ops.add_rmsnorm(stream.h, stream.delta, self.weight, self.eps, out, row_idx=row_idx,
                        write_residual=row_idx is None, delta_scale=stream.delta_scale)
        if row_idx is None:
            if stream.delta is not None:
                stream.rounded = None           # h has changed
            stream.delta = None

    def forward_branch(self, stream: ResidualStream, y: torch.Tensor, ctx: StepContext) -> None:
        """``h += y / sqrt(mean(y^2) + eps) * w`` (float32), and the rounded copy of the new ``h`` for the next sublayer."""
        rounded = None if ctx.dtype == torch.float32 else ctx.empty(*stream.h.shape)
        ops.norm_add(stream.h, y, self.weight, self.eps, rounded)
        stream.rounded = rounded
