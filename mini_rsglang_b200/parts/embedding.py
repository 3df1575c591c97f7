"""Token embedding and output head (reference: crates/kernels/src/ops.cu:15-18;
crates/models/src/qwen3.rs:232-236).  The head's logits are float32; a tied head reads the
embedding table."""
from __future__ import annotations

import torch

from .. import kernels
from ..errors import InvalidRequest
from ..weights.spec import WeightSpec
from .base import EMBEDDINGS, HEADS, Embedding, Head
from .linear import linear


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Embedding):
    def __init__(self, prefix: str, vocab: int, width: int, leaf: str = "weight", scale: float = 1.0):
        """`scale`: a constant that multiplies every embedding on its way into the float32 stream (the table is unchanged)."""
        super().__init__(prefix)
        self.vocab, self.width, self.leaf, self.scale = int(vocab), int(width), leaf, float(scale)
        self.table = None

    def weight_specs(self):
        return [WeightSpec(self.name(self.leaf), (self.vocab, self.width))]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.table = tensors[self.name(self.leaf)]

    def forward(self, ctx) -> torch.Tensor:
        stream = torch.empty((ctx.num_tokens, self.width), dtype=torch.float32, device=self.table.device)
        kernels.embed(self.table, ctx.token_ids, stream, self.scale)
        return stream


@HEADS.register("linear_head")
class OutputHead(Head):
    def __init__(self, prefix: str, vocab: int, width: int, tied_to: str | None = None, leaf: str = "weight", scale: float = 1.0,
                 softcap: float = 0.0):
        """`leaf`: the matrix's name below the part's root ("": the root itself); `scale`: a constant that multiplies the logits;
        `softcap` > 0: the scaled logits are then bent into (-softcap, softcap), cap * tanh(logit / cap)."""
        super().__init__(prefix)
        self.vocab, self.width, self.tied_to, self.leaf, self.scale = int(vocab), int(width), tied_to, leaf, float(scale)
        self.softcap = float(softcap)
        if self.softcap < 0:
            raise InvalidRequest("a soft cap on the logits cannot be negative")
        self.weight = None

    def weight_specs(self):
        return [] if self.tied_to else [WeightSpec(self.name(self.leaf), (self.vocab, self.width))]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.weight = tensors[self.tied_to if self.tied_to else self.name(self.leaf)]

    def forward(self, hidden) -> torch.Tensor:
        """`hidden`: the normalised rows, or a `Prenormed` that the product finishes."""
        logits = linear(hidden, self.weight, out_dtype=torch.float32)
        if self.softcap > 0.0:
            kernels.scale_softcap_(logits, self.scale, self.softcap)
        elif self.scale != 1.0:
            kernels.scale_(logits, self.scale)
        return logits
