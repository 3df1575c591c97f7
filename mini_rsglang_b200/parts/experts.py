"""Routed experts: every token is sent to `top` of a layer's small gated feed-forwards and gets the weighted sum of
their outputs (no biases anywhere).

  z = W_router h  (float32),  s = softmax(z) over all experts (or sigmoid(z), one by one)
  chosen = the `top` experts with the largest s + correction   (the correction steers the choice only)
  weight_e = s_e / (sum of the chosen s + 1e-20) * scale
  out = sum over the chosen of weight_e * expert_e(h),   expert_e(h) = W_down silu(W_gate h) * (W_up h)

Variations, all parameters: `normalize` False leaves the weights as the chosen scores (times scale); `form` "plain" makes
an expert W_down act(W_up h) without a gate, `activation` one of `kernels.ACTIVATIONS`; `weight_on` "input" multiplies what
a chosen expert reads by its weight instead of what it returns: out = sum over the chosen of expert_e(weight_e * h).

The last `identity` experts of the router have no tensors: their output is their input.  A shared expert (any
registered feed-forward) may run for every token beside them, behind one sigmoid gate a token.

The shapes of every launch are fixed by the number of tokens, so a step can be recorded: one kernel lists the
(token, choice) pairs expert by expert, every expert's run filled up to whole tiles, and the two products of the
gated unit run over those tiles, each with the weights of its tile's expert; a last kernel sums a token's
choices in their order.  Which pairs share a tile does not enter a row's result."""
from __future__ import annotations

import torch

from .. import kernels
from ..errors import InvalidRequest
from ..weights.spec import WeightSpec
from .base import FEED_FORWARDS, FeedForward, PartSpec, plain
from .linear import linear


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, prefix: str, width: int, experts: int, top: int, inner: int, identity: int = 0, scale: float = 1.0,
                 score: str = "softmax", correction: bool = False, shared: PartSpec | None = None, shared_gate: bool = False,
                 normalize: bool = True, form: str = "gated", activation: str = "silu", weight_on: str = "output",
                 float32_out: bool = False, names: dict | None = None):
        """`experts` with tensors, then `identity` without; `shared`: the feed-forward that every token passes as well
        (its root is the leaf "shared" below this part's), `shared_gate`: behind a sigmoid gate of one number a token.
        `names`: leaves below the part's root; "expert" is a pattern with `{}` for the expert's number."""
        super().__init__(prefix)
        self.width, self.experts, self.identity = int(width), int(experts), int(identity)
        self.top, self.inner, self.scale = int(top), int(inner), float(scale)
        if self.experts < 0 or self.identity < 0 or not 0 < self.top <= self.experts + self.identity:
            raise InvalidRequest(f"{prefix}: {top} choices among {experts} + {identity} experts")
        if self.experts and self.inner <= 0 or self.width <= 0:
            raise InvalidRequest(f"{prefix}: sizes must be positive")
        if score not in ("softmax", "sigmoid"):
            raise InvalidRequest(f"{prefix}: router scores {score!r} are not built; softmax or sigmoid")
        self.score, self.correction = score, bool(correction)
        self.normalize, self.form, self.activation, self.weight_on = bool(normalize), form, activation, weight_on
        self.float32_out = bool(float32_out)       # the summed outputs leave as float32 (a float32 norm or sum reads them)
        if form not in ("gated", "plain") or weight_on not in ("output", "input"):
            raise InvalidRequest(f"{prefix}: experts are 'gated' or 'plain', their weights on the 'output' or the 'input'")
        if form == "gated" and activation != "silu":
            raise InvalidRequest(f"{prefix}: gated experts with {activation!r} are not built; only silu")
        if form == "plain" and activation not in kernels.ACTIVATIONS:
            raise InvalidRequest(f"{prefix}: activation {activation!r} is not built; known: {sorted(kernels.ACTIVATIONS)}")
        if weight_on == "input" and (form != "plain" or self.identity):
            raise InvalidRequest(f"{prefix}: weights on the experts' input are built for plain experts without identity experts")
        self.leaf = {"router": "router.weight", "correction": "router.correction", "expert": "experts.{}", "gate": "gate_proj.weight",
                     "up": "up_proj.weight", "down": "down_proj.weight", "shared": "shared", "shared_gate": "shared_gate.weight"}
        self.leaf.update(names or {})
        self.shared = FEED_FORWARDS.build(shared, self.name(self.leaf["shared"])) if shared is not None else None
        self.shared_gate = bool(shared_gate) and self.shared is not None
        self.router = self.correction_values = self.gate_up = self.down = None
        self.block = 0

    @property
    def all_experts(self) -> int:
        return self.experts + self.identity

    def _expert(self, number: int, which: str) -> str:
        return self.name(f"{self.leaf['expert'].format(number)}.{self.leaf[which]}")

    def weight_specs(self):
        n = self.leaf
        specs = []
        for number in range(self.experts):
            if self.form == "gated":
                specs.append(WeightSpec(self._expert(number, "gate"), (self.inner, self.width)))
            specs += [WeightSpec(self._expert(number, "up"), (self.inner, self.width)),
                      WeightSpec(self._expert(number, "down"), (self.width, self.inner))]
        specs.append(WeightSpec(self.name(n["router"]), (self.all_experts, self.width)))
        if self.correction:
            specs.append(WeightSpec(self.name(n["correction"]), (self.all_experts,), "bias"))
        if self.shared is not None:
            specs += self.shared.weight_specs()
        if self.shared_gate:
            specs.append(WeightSpec(self.name(n["shared_gate"]), (1, self.width)))
        return specs

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        n = self.leaf
        # When serving in bfloat16 and the inner size allows it, blocks of 64 gate rows alternate with the 64 matching up
        # rows: a weight tile of the product for many rows then holds both factors of its outputs.
        self.block = kernels.MOE_TC_BLOCK if runtime.is_bf16 and self.experts and self.inner % kernels.MOE_TC_BLOCK == 0 else 0
        if self.experts and self.form == "plain":
            self.block = 0
            self.gate_up = torch.stack([tensors[self._expert(e, "up")] for e in range(self.experts)]).contiguous()      # [experts, inner, width]
        elif self.experts and self.block:
            b = self.block
            self.gate_up = torch.stack([torch.stack([tensors[self._expert(e, "gate")].view(-1, b, self.width),
                                                     tensors[self._expert(e, "up")].view(-1, b, self.width)], dim=1)
                                        .reshape(2 * self.inner, self.width) for e in range(self.experts)]).contiguous()
        elif self.experts:
            self.gate_up = torch.stack([torch.cat([tensors[self._expert(e, "gate")], tensors[self._expert(e, "up")]], dim=0)
                                        for e in range(self.experts)]).contiguous()                         # [experts, 2 inner, width]
        if self.experts:
            self.down = torch.stack([tensors[self._expert(e, "down")] for e in range(self.experts)]).contiguous()   # [experts, width, inner]
        rows = [tensors[self.name(n["router"])]]
        if self.shared_gate:
            rows.append(tensors[self.name(n["shared_gate"])])
        # the shared expert's gate is one more row of the router's product; rows of zeros fill it up to a multiple of 8, so
        # that the float32 logits' rows start on 32-byte boundaries (the library then takes its aligned kernels)
        count = sum(r.shape[0] for r in rows)
        if count % 8:
            rows.append(torch.zeros((8 - count % 8, self.width), dtype=rows[0].dtype, device=rows[0].device))
        self.router = torch.cat(rows, dim=0).contiguous()
        self.correction_values = tensors[self.name(n["correction"])] if self.correction else None
        if self.shared is not None:
            self.shared.bind(tensors, runtime)

    def forward(self, h, ctx):
        h = plain(h)
        tokens = h.shape[0]
        device, dtype = h.device, self.runtime.dtype
        logits = linear(h, self.router, out_dtype=torch.float32)
        chosen = torch.empty((tokens, self.top), dtype=torch.int32, device=device)
        weights = torch.empty((tokens, self.top), dtype=torch.float32, device=device)
        shared_gate = torch.empty((tokens,), dtype=torch.float32, device=device) if self.shared_gate else None
        kernels.moe_route(logits, self.correction_values, chosen, weights, shared_gate, self.all_experts, self.top, self.scale,
                          sigmoid_scores=self.score == "sigmoid", normalize=self.normalize)
        on_input = self.weight_on == "input"
        y = None
        if self.experts:
            y = torch.empty((tokens * self.top, self.width), dtype=dtype, device=device)
            if self.form == "plain":
                kernels.moe_plain_experts(h, chosen, weights if on_input else None, self.gate_up, self.down, y, self.experts, self.activation)
            else:
                kernels.moe_experts(h, chosen, self.gate_up, self.down, y, self.experts, block=self.block)
        shared_out = self.shared.forward(h, ctx) if self.shared is not None else None       # no gate: it counts fully
        out = torch.empty((tokens, self.width), dtype=torch.float32 if self.float32_out else dtype, device=device)
        kernels.moe_combine(y, h, shared_out, chosen, None if on_input else weights, shared_gate, out, self.experts)
        return out
