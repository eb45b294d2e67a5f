"""Token embedding (x = E[token, :], src/forward.cpp:496-503) and the output head
(logits = W_lm · h, no bias, src/forward.cpp:849-853).  A tied head reads the embedding's
tensor instead of a copy of it (the reference copies: src/gguf_loader.cpp:436-443)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from ..config.registry import register_part
from .base import Part, TensorSpec
from .linear import Linear


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, name: str, vocab_size: int, hidden_size: int, tensor: str = "weight", scale: float = 1.0):
        """`tensor`: the table's name below the part's prefix.  `scale` multiplies every row as it is read (float32)."""
        super().__init__(name, vocab_size=vocab_size, hidden_size=hidden_size, tensor=tensor, scale=scale)
        self.vocab, self.hidden, self.scale = int(vocab_size), int(hidden_size), float(scale)
        self.tensor = self.name + tensor

    def tensors(self):
        return [TensorSpec(self.tensor, (self.vocab, self.hidden), role="table")]

    def bind(self, get, runtime):
        super().bind(get, runtime)
        self.table = get(self.tensor).contiguous()

    def weight_bytes(self) -> int:
        return 0      # a step touches one row per token, not the table

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        x = self.runtime.empty(token_ids.numel(), self.hidden, dtype=torch.float32)
        kernels.embed(self.table, token_ids, x, self.scale)
        return x


@register_part("head", "linear_head")
class LinearHead(Part):
    graph_safe = True

    def __init__(self, name: str, vocab_size: int, hidden_size: int, tied_to: Optional[str] = None,
                 tensor: str = "weight", softcap: Optional[float] = None):
        """`tensor`: the matrix's name below the part's prefix.  `softcap` c: logits ← c·tanh(logits / c), in float32."""
        super().__init__(name, vocab_size=vocab_size, hidden_size=hidden_size, tied_to=tied_to, tensor=tensor, softcap=softcap)
        self.vocab, self.hidden, self.tied_to = int(vocab_size), int(hidden_size), tied_to
        self.tensor = self.name + tensor
        self.softcap = float(softcap) if softcap else None
        if self.softcap is not None and not self.softcap > 0:
            raise ValueError(f"head: the soft cap must be positive, got {softcap}")

    def tensors(self):
        if self.tied_to:
            return [TensorSpec(self.tied_to, (self.vocab, self.hidden), role="table", stored=False)]
        return [TensorSpec(self.tensor, (self.vocab, self.hidden))]

    def ignorable_tensors(self):
        return [self.tensor] if self.tied_to else []

    def bind(self, get, runtime):
        super().bind(get, runtime)
        self.proj = Linear(get(self.tied_to or self.tensor), runtime)

    def weight_bytes(self) -> int:
        return self.proj.nbytes()

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        logits = self.proj(h, torch.float32)
        if self.softcap is not None:
            kernels.softcap(logits, self.softcap)
        return logits
