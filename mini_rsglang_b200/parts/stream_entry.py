"""Parts that stand before a run of a layer and act on the whole residual stream.

"rejoin_embedding": x <- W [x ; x0], one product over the stream joined with the embedding's output (W [width, 2 width],
the stream's columns first).  It stands where a group of layers is entered again and again with the same weights: every
pass starts from the stream so far and is shown the embedding anew.  The operand is the float32 stream and embedding
rounded once to the engine's dtype; the result is the product's float32 sums and becomes the stream."""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.spec import WeightSpec
from .base import STREAM_ENTRIES, StreamEntry
from .linear import linear


@STREAM_ENTRIES.register("rejoin_embedding")
class RejoinEmbedding(StreamEntry):
    def __init__(self, prefix: str, width: int, leaf: str = "weight"):
        super().__init__(prefix)
        self.width, self.leaf = int(width), leaf
        self.weight = None

    def weight_specs(self):
        return [WeightSpec(self.name(self.leaf), (self.width, 2 * self.width))]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.weight = tensors[self.name(self.leaf)].contiguous()

    def forward(self, stream, origin, ctx):
        joined = torch.empty((stream.shape[0], 2 * self.width), dtype=self.runtime.dtype, device=stream.device)
        kernels.concat_rows(stream, origin, joined)
        return linear(joined, self.weight, out_dtype=torch.float32)
