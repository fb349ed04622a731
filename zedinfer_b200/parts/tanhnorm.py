"""The tanh norm: ``y = tanh(alpha * x) * w + b`` with a scalar ``alpha`` and vectors ``w`` and ``b``, entry by entry in
float32.  It computes no mean and no variance, so it needs no epsilon.

It serves arrangements that norm a sublayer's input and its output (``sandwich_norm``): the norm *after* a sublayer rides
with the sublayer's output in the stream (``ResidualStream.delta_norm``) until the next norm *before* a sublayer folds
both into the float32 residual, one kernel for ``h += N_after(y); out = N_before(h)``.  Where ``y`` is the output of two branches
that are joined by their unit rows (``ResidualStream.delta_join``), the same kernel joins them on the way."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Norm, ResidualStream, StepContext, register_norm


@register_norm("tanh_norm")
class TanhNorm(Norm):
    capture_safe = True

    def __init__(self, size: int, name: str = "weight", alpha_name: Optional[str] = None, bias_name: Optional[str] = None):
        """``name``: the weight's local name; the scalar and the bias are ``<name>.alpha`` and ``<name>.b`` unless named."""
        if size <= 0:
            raise ValueError(f"tanh_norm: size={size} must be positive")
        self.size, self.name = int(size), str(name)
        self.alpha_name = alpha_name or self.name + ".alpha"
        self.bias_name = bias_name or self.name + ".b"
        self.alpha: float = 1.0
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.size,), init=("one_plus_normal", 0.01)),
                self.bias_name: TensorSpec((self.size,), init=("normal", 0.01)),
                self.alpha_name: TensorSpec((), init=("one_plus_normal", 0.01))}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        # norms are float32: widening the stored values is exact
        self.weight = tensors[self.name].float().contiguous()
        self.bias = tensors[self.bias_name].float().contiguous()
        self.alpha = float(tensors[self.alpha_name].float().reshape(-1)[0].item())      # read once, when the model is loaded

    def params(self):
        return self.alpha, self.weight, self.bias

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> None:
        ops.tanh_norm(x, self.alpha, self.weight, self.bias, out)

    def forward_residual(self, stream: ResidualStream, out: torch.Tensor, row_idx: Optional[torch.Tensor] = None) -> None:
        """Fold the pending branch output, through the norm that follows it, into the float32 stream, and write this
        norm of the new stream to ``out``.  With ``row_idx`` only those rows are produced and the stream is left as it is."""
        post = None
        if stream.delta is not None:
            if stream.delta.dim() != 2 or not isinstance(stream.delta_norm, TanhNorm):
                raise RuntimeError("tanh_norm folds a branch output [tokens, hidden] that brings the tanh norm that follows it")
            post = stream.delta_norm.params()
        ops.tanh_norm_fold(stream.h, stream.delta, post, self.params(), out, row_idx=row_idx, write_h=row_idx is None,
                           join=stream.delta_join if stream.delta is not None else None)
        if row_idx is None:
            if stream.delta is not None:
                stream.rounded = None           # h has changed
            stream.delta, stream.delta_norm, stream.delta_join = None, None, None

    def forward_branch(self, stream: ResidualStream, y: torch.Tensor, ctx: StepContext) -> None:
        """``h += tanh(alpha y) * w + b`` (float32) at once, nothing left pending."""
        if stream.delta is not None:
            raise RuntimeError("a branch output is still pending: fold it into the stream first")
        ops.tanh_norm_fold(stream.h, y, self.params(), None, None)
        stream.rounded = None
