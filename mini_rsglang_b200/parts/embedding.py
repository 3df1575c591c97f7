"""Token embedding and output head (reference: crates/kernels/src/ops.cu:15-18;
crates/models/src/qwen3.rs:232-236).  The head's logits are float32; a tied head reads the
embedding table."""
from __future__ import annotations

import torch

from .. import kernels
from ..errors import InvalidRequest
from ..weights.spec import WeightSpec
from .base import EMBEDDINGS, HEADS, Embedding, Head, StateNeed
from .linear import linear


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Embedding):
    def __init__(self, prefix: str, vocab: int, width: int, leaf: str = "weight", scale: float = 1.0, pairs: dict | None = None):
        """`scale`: a constant that multiplies every embedding on its way into the float32 stream (the table is unchanged).
        `pairs`: a second table, of token pairs, whose row is added (unscaled): {"table": its checkpoint name, "buckets",
        "mul_prev", "mul_cur"}; a token takes row (previous token * mul_prev + token * mul_cur) mod buckets, the first token
        of a sequence row number `buckets` (the table has buckets + 1 rows).  The last token that a request brought is then
        part of the request's state (one int32 in its state slot): the next portion's first token pairs with it."""
        super().__init__(prefix)
        self.vocab, self.width, self.leaf, self.scale = int(vocab), int(width), leaf, float(scale)
        self.pairs = dict(pairs) if pairs else None
        if self.pairs is not None:
            missing = [k for k in ("table", "buckets", "mul_prev", "mul_cur") if k not in self.pairs]
            if missing or int(self.pairs["buckets"]) <= 0:
                raise InvalidRequest(f"a table of token pairs needs its name, a positive number of buckets and two multipliers; missing {missing}")
        self.table = self.pair_table = None

    def weight_specs(self):
        specs = [WeightSpec(self.name(self.leaf), (self.vocab, self.width))]
        if self.pairs is not None:
            specs.append(WeightSpec(self.pairs["table"], (int(self.pairs["buckets"]) + 1, self.width)))
        return specs

    def state_need(self):
        return StateNeed((), torch.int32) if self.pairs is not None else None

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.table = tensors[self.name(self.leaf)]
        if self.pairs is not None:
            self.pair_table = tensors[self.pairs["table"]]

    def forward(self, ctx, state=None) -> torch.Tensor:
        """`state`: the requests' last tokens, int32 [slots] (an embedding with a table of pairs)."""
        stream = torch.empty((ctx.num_tokens, self.width), dtype=torch.float32, device=self.table.device)
        if self.pairs is None:
            kernels.embed(self.table, ctx.token_ids, stream, self.scale)
        else:
            if state is None:
                raise InvalidRequest("an embedding with a table of token pairs needs the requests' state")
            p = self.pairs
            kernels.embed_pairs(self.table, self.pair_table, ctx, state, stream, self.scale, int(p["buckets"]), int(p["mul_prev"]),
                                int(p["mul_cur"]), write_state=not ctx.rehearsal)
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
