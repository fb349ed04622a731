"""Pre-norm residual arrangement (src/frontend/models/transformer_forward.cpp:63-149):

    h = h + mixer(norm1(h));  h = h + ffn(norm2(h))

The adds are fused into the norm that follows them: a branch output stays "pending" in the
stream until the next norm folds it into the float32 residual.

``residual_scale`` m (default 1): ``h = h + m * mixer(norm1(h)); h = h + m * ffn(norm2(h))``, the product and the
sum in float32.  A layer without a feed-forward (no ``ffn``, no ``norm2``) is its first half alone.

``branch_norm`` puts the norm on each branch's output; ``sandwich_norm`` has one before and one after every sublayer and
may run two mixers side by side on the same input."""
from __future__ import annotations

from typing import Mapping

from ..cache.manager import CallCacheView
from .base import Block, ResidualStream, StepContext, register_block


@register_block("pre_norm")
class PreNormBlock(Block):
    capture_safe = True

    def __init__(self, parts, residual_scale: float = 1.0):
        super().__init__(parts)
        need = ("mixer", "norm1") + (("ffn", "norm2") if ("ffn" in self.parts() or "norm2" in self.parts()) else ())
        missing = [role for role in need if role not in self.parts()]
        if missing:
            raise ValueError(f"the pre_norm arrangement needs the parts {missing} as well")
        self.residual_scale = float(residual_scale)

    def forward(self, stream: ResidualStream, ctx: StepContext, caches: Mapping[str, CallCacheView],
                owns_cache: bool) -> None:
        n, hidden = stream.h.shape
        normed = ctx.empty(n, hidden)
        self.norms["norm1"].forward_residual(stream, normed)
        stream.delta = self.mixer.forward_for_residual(normed, ctx, caches["mixer"], owns_cache)
        stream.delta_scale = self.residual_scale
        if self.ffn is None:
            return
        normed2 = ctx.empty(n, hidden)
        self.norms["norm2"].forward_residual(stream, normed2)
        stream.delta = self.ffn.forward_for_residual(normed2, ctx)


@register_block("branch_norm")
class BranchNormBlock(Block):
    """The norm sits on each branch's *output*, and the branches read the stream itself:

        h = h + norm1(mixer(h));  h = h + norm2(ffn(h));  h = h + norm_side(side(h))

    ``ffn`` with ``norm2`` and ``side`` with ``norm_side`` are optional.  ``side`` is a feed-forward part (it may read
    the step's token ids, e.g. a gate on a per-token table entry).  The sums are float32; in a bfloat16 step the kernel
    that adds a normed branch also leaves the rounded stream for the next branch to read."""
    capture_safe = True

    def __init__(self, parts):
        super().__init__(parts)
        have = self.parts()
        need = ["mixer", "norm1"]
        for branch, norm in (("ffn", "norm2"), ("side", "norm_side")):
            if branch in have or norm in have:
                need += [branch, norm]
        missing = [role for role in need if role not in have]
        if missing:
            raise ValueError(f"the branch_norm arrangement needs the parts {missing} as well")
        self.side = have.get("side")

    def forward(self, stream: ResidualStream, ctx: StepContext, caches: Mapping[str, CallCacheView],
                owns_cache: bool) -> None:
        y = self.mixer.forward(stream.as_input(ctx), ctx, caches["mixer"], owns_cache)
        self.norms["norm1"].forward_branch(stream, y, ctx)
        if self.ffn is not None:
            self.norms["norm2"].forward_branch(stream, self.ffn.forward(stream.as_input(ctx), ctx), ctx)
        if self.side is not None:
            self.norms["norm_side"].forward_branch(stream, self.side.forward(stream.as_input(ctx), ctx), ctx)


@register_block("sandwich_norm")
class SandwichNormBlock(Block):
    """A norm before and a norm after every sublayer:

        h = h + norm1b(mixer(norm1(h)));  h = h + norm2b(ffn(norm2(h)))

    ``ffn`` with ``norm2`` and ``norm2b`` is optional.  A branch's output stays pending in the stream together with the norm
    that follows it (``ResidualStream.delta_norm``) until the next norm before a sublayer (or the model's last norm) folds both
    into the float32 residual, so every sublayer costs one norm kernel (``ops.tanh_norm_fold``).

    With a second mixer (role ``mixer2``, a cache of its own) the two read the same normed input and their outputs are
    joined as ``(U(y1) * w1 + U(y2) * w2) / 2``, ``U`` the division by the root mean square over the row, the weights those
    of the norms ``mix_out`` and ``mix2_out`` (built with ``float32_weight``); the join rides in the same pending state
    (``ResidualStream.delta_join``) and happens inside the kernel that folds (``ops.rms_pair_mean`` is the join on its own)."""
    capture_safe = True

    def __init__(self, parts):
        super().__init__(parts)
        have = self.parts()
        need = ["mixer", "norm1", "norm1b"]
        if any(role in have for role in ("ffn", "norm2", "norm2b")):
            need += ["ffn", "norm2", "norm2b"]
        if any(role in have for role in ("mixer2", "mix_out", "mix2_out")):
            need += ["mixer2", "mix_out", "mix2_out"]
        missing = [role for role in need if role not in have]
        if missing:
            raise ValueError(f"the sandwich_norm arrangement needs the parts {missing} as well")
        self.mixer2 = have.get("mixer2")
        if self.mixer2 is not None and self.norms["mix_out"].eps != self.norms["mix2_out"].eps:
            raise ValueError("the sandwich_norm arrangement joins two mixers with one epsilon")

    def forward(self, stream: ResidualStream, ctx: StepContext, caches: Mapping[str, CallCacheView],
                owns_cache: bool) -> None:
        n, hidden = stream.h.shape
        normed = ctx.empty(n, hidden)
        self.norms["norm1"].forward_residual(stream, normed)
        y = self.mixer.forward(normed, ctx, caches["mixer"], owns_cache)
        stream.delta, stream.delta_norm, stream.delta_scale, stream.delta_join = y, self.norms["norm1b"], 1.0, None
        if self.mixer2 is not None:
            # the two outputs are joined by whoever folds them into the stream (one kernel for join, norm, add and next norm)
            y2 = self.mixer2.forward(normed, ctx, caches["mixer2"], owns_cache)
            stream.delta_join = (y2, self.norms["mix_out"].weight, self.norms["mix2_out"].weight, self.norms["mix_out"].eps)
        if self.ffn is None:
            return
        normed2 = ctx.empty(n, hidden)
        self.norms["norm2"].forward_residual(stream, normed2)
        stream.delta, stream.delta_norm, stream.delta_scale, stream.delta_join = self.ffn.forward(normed2, ctx), self.norms["norm2b"], 1.0, None
