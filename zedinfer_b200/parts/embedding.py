"""Token embedding and output head.

``hidden[n, :] = table[ids[n], :]`` (src/frontend/models/transformer_forward.cpp:58-59);
``logits = norm(hidden) @ head^T`` without bias (:152-156), computed only for the rows that
are asked for and returned in float32.  With tied embeddings the head is the embedding table
(src/frontend/models/base.cpp:411-416).

Two more forms, for models that have them: an embedding that adds a learned vector per absolute position
(``learned_position_embedding``: ``hidden[n] = table[ids[n]] + positions[pos[n]]``), and a cap on the logits
(``softcap`` c of the head: ``logits = c * tanh(logits / c)``, in float32)."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Embedding, Head, register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Embedding):
    capture_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, name: str = "embed_tokens.weight"):
        self.vocab_size, self.hidden_size, self.name = int(vocab_size), int(hidden_size), name
        self.table: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.vocab_size, self.hidden_size))}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = tensors[self.name].contiguous()

    def forward(self, ids: torch.Tensor, out: torch.Tensor) -> None:
        ops.embedding(self.table, ids, out)

    def tied_weight(self) -> Optional[torch.Tensor]:
        return self.table


@register_embedding("scaled_token_embedding")
class ScaledTokenEmbedding(TokenEmbedding):
    """``hidden[n] = table[ids[n]] * scale`` (the product in float32); a tied head reads the table itself, without the
    scale.  ``token_tables`` names further tables with a row per token of the vocabulary (``{key: (tensor name, width)}``)
    that parts of the layers read by the step's token ids: the embedding loads them and leaves each under
    ``ctx.step_cache[("token_table", key)]`` for the step."""
    capture_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, scale: float = 1.0, name: str = "embed_tokens.weight",
                 token_tables: Optional[Mapping[str, tuple]] = None):
        super().__init__(vocab_size, hidden_size, name)
        self.scale = float(scale)
        self.token_tables = {key: (str(tname), int(width)) for key, (tname, width) in (token_tables or {}).items()}
        for key, (tname, width) in self.token_tables.items():
            if width <= 0:
                raise ValueError(f"scaled_token_embedding: the table {key!r} needs a positive width, got {width}")
        self.tables: Dict[str, torch.Tensor] = {}

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        specs = super().tensor_specs()
        specs.update({tname: TensorSpec((self.vocab_size, width)) for tname, width in self.token_tables.values()})
        return specs

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        super().bind(tensors)
        self.tables = {key: tensors[tname].contiguous() for key, (tname, _) in self.token_tables.items()}

    def forward(self, ids: torch.Tensor, out: torch.Tensor) -> None:
        ops.embedding(self.table, ids, out, scale=self.scale)

    def forward_step(self, ctx, out: torch.Tensor) -> None:
        self.forward(ctx.token_ids, out)
        for key, table in self.tables.items():
            ctx.step_cache[("token_table", key)] = table


@register_embedding("learned_position_embedding")
class LearnedPositionEmbedding(Embedding):
    """Token table plus a table of learned absolute positions (not scaled), added in float32."""
    capture_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, max_positions: int, name: str = "embed_tokens.weight",
                 position_name: str = "embed_positions.weight"):
        if max_positions <= 0:
            raise ValueError(f"learned_position_embedding: max_positions={max_positions} must be positive")
        self.vocab_size, self.hidden_size, self.max_positions = int(vocab_size), int(hidden_size), int(max_positions)
        self.name, self.position_name = name, position_name
        self.table: Optional[torch.Tensor] = None
        self.positions: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.vocab_size, self.hidden_size)),
                self.position_name: TensorSpec((self.max_positions, self.hidden_size))}

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = tensors[self.name].contiguous()
        self.positions = tensors[self.position_name].to(self.table.dtype).contiguous()

    def forward(self, ids: torch.Tensor, out: torch.Tensor) -> None:
        raise RuntimeError("learned_position_embedding needs the step's positions: call forward_step")

    def forward_step(self, ctx, out: torch.Tensor) -> None:
        ops.embedding_positions(self.table, self.positions, ctx.token_ids, ctx.positions, out)

    def tied_weight(self) -> Optional[torch.Tensor]:
        return self.table


@register_head("output_head")
class OutputHead(Head):
    capture_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, tied: bool, name: str = "lm_head.weight",
                 softcap: Optional[float] = None):
        if softcap is not None and not softcap > 0.0:
            raise ValueError(f"output_head: softcap={softcap} must be positive (or None for no cap)")
        self.vocab_size, self.hidden_size, self.tied, self.name = int(vocab_size), int(hidden_size), bool(tied), name
        self.softcap = float(softcap) if softcap is not None else None
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {self.name: TensorSpec((self.vocab_size, self.hidden_size), optional=self.tied)}

    def bind(self, tensors: Mapping[str, torch.Tensor], embedding: Optional[torch.Tensor] = None) -> None:
        if self.name in tensors:
            self.weight = tensors[self.name].contiguous()
        elif self.tied and embedding is not None:
            self.weight = embedding
        else:
            raise KeyError(self.name)

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> None:
        ops.linear(x, self.weight, None, out)
        if self.softcap is not None:
            ops.softcap(out, self.softcap)
