"""Token embedding into the float32 residual stream, and the LM head that gives
float32 logits for the wanted rows only (slipstream/models/causal_lm.py:93,140;
tied weights: slipstream/models/loader.py:91-93)."""

from __future__ import annotations

import torch

from slipstream_b200 import ops

from .base import EMBEDDINGS, HEADS, Embedding, Head, Runtime, WeightSpec


@EMBEDDINGS.register("token_table")
class TokenEmbedding(Embedding):
    cuda_graph_safe = True

    def __init__(self, name: str, vocab_size: int, hidden_size: int, scale: float = 1.0, copies: int = 1,
                 tensor: str | None = None) -> None:
        """``scale``: a constant the table's rows are multiplied by (in float32).  ``copies``: how many residual
        streams the model keeps; above 1 the result is [N, copies, hidden], every stream starting as the same
        row.  ``tensor``: the checkpoint's name of the table (default ``<name>.weight``)."""
        self.name = name
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.scale = float(scale)
        self.copies = int(copies)
        self.tensor = tensor or f"{name}.weight"

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(self.tensor, (self.vocab_size, self.hidden_size))]

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        self.weight = weights[self.tensor]

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        return ops.embedding(token_ids, self.weight, scale=self.scale, copies=self.copies)


@HEADS.register("linear")
class LMHead(Head):
    cuda_graph_safe = True
    takes_pending_norm = True  # ``forward`` hands x to ``ops.linear`` as it is

    def __init__(self, name: str, vocab_size: int, hidden_size: int, tied_to: str | None,
                 tensor: str | None = None, softcap: float | None = None) -> None:
        """``softcap`` c: the logits leave as ``c * tanh(logits / c)``."""
        self.softcap = float(softcap) if softcap else None
        self.name = name
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.tied_to = tied_to
        self.tensor = tensor or f"{name}.weight"

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(self.tensor, (self.vocab_size, self.hidden_size), alias_of=self.tied_to)]

    def bind(self, weights: dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(weights, runtime)
        self.weight = weights[self.tensor]

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = ops.linear(x, self.weight, None, out_dtype=torch.float32)
        return ops.soft_cap(logits, self.softcap) if self.softcap else logits
