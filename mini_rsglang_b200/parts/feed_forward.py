"""Dense gated feed-forward: down(silu(gate(x)) * up(x)) (reference:
crates/models/src/qwen3.rs:239-262; ops.cu:91-94).  Gate and up are one projection over the
row-concatenated matrices."""
from __future__ import annotations

import torch

from .. import kernels
from ..errors import InvalidRequest
from ..weights.spec import WeightSpec
from .base import FEED_FORWARDS, FeedForward, Prenormed, observing, plain
from .linear import few_rows, linear


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    adds_to_stream = True
    takes_prenormed = True

    def __init__(self, prefix: str, width: int, inner: int, activation: str = "silu", names: dict | None = None):
        """`names`: leaves of the three tensors below the part's root, under "gate", "up" and "down"."""
        super().__init__(prefix)
        if activation != "silu":
            raise InvalidRequest(f"activation {activation!r} is not built; only silu")
        self.width, self.inner = int(width), int(inner)
        self.leaf = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}
        self.leaf.update(names or {})
        self.gate_up = self.down = None

    def weight_specs(self):
        return [WeightSpec(self.name(self.leaf["gate"]), (self.inner, self.width)),
                WeightSpec(self.name(self.leaf["up"]), (self.inner, self.width)),
                WeightSpec(self.name(self.leaf["down"]), (self.width, self.inner))]

    BLOCK = 64     # gate rows of a 128-row weight tile of the tensor-core product; the other 64 are the up rows

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        gate, up = tensors[self.name(self.leaf["gate"])], tensors[self.name(self.leaf["up"])]
        # When serving in bfloat16 and the width allows it, blocks of 64 gate rows alternate with the 64
        # matching up rows: a weight tile of the product for few rows then holds both halves of its outputs,
        # and the product applies silu(gate) * up before it stores.
        self.block = self.BLOCK if runtime.is_bf16 and self.inner % self.BLOCK == 0 else 0
        if self.block:
            b = self.block
            self.gate_up = torch.stack([gate.view(-1, b, self.width), up.view(-1, b, self.width)], dim=1) \
                .reshape(2 * self.inner, self.width).contiguous()
        else:
            self.gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.down = tensors[self.name(self.leaf["down"])].contiguous()

    def forward(self, h, ctx, into=None):
        act = torch.empty((h.shape[0], self.inner), dtype=self.runtime.dtype, device=self.down.device)
        if self.block and few_rows(h, self.gate_up) and not observing(ctx):
            if isinstance(h, Prenormed):
                kernels.gemm_tc(h.scaled, self.gate_up, act, gated=True, row_sums=h.row_sums)
            else:
                kernels.gemm_tc(h, self.gate_up, act, gated=True)
        else:
            h = plain(h)
            if self.block == 64 and not observing(ctx) and kernels.gemm_gated_rows_wins(h, self.gate_up):
                kernels.gemm_gated_rows(h, self.gate_up, act)      # many rows: the tcgen05 product with the activation in it
            else:
                kernels.silu_mul(linear(h, self.gate_up), act, self.block)
        if observing(ctx):
            ctx.observe(f"{ctx.label}-swiglu", act)
        return linear(act, self.down, into=into)


@FEED_FORWARDS.register("clamped_glu")
class ClampedGLU(FeedForward):
    """A gated feed-forward with clamped branches: g = min(gate(x), limit), u = clamp(up(x), -limit, limit),
    down(g * sigmoid(alpha * g) * (u + 1)).  Gate and up are one projection over the row-concatenated matrices;
    the result keeps the product's float32 sums (the norm that follows a branch reads them)."""

    def __init__(self, prefix: str, width: int, inner: int, limit: float, alpha: float = 1.702, names: dict | None = None):
        super().__init__(prefix)
        self.width, self.inner, self.limit, self.alpha = int(width), int(inner), float(limit), float(alpha)
        self.leaf = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}
        self.leaf.update(names or {})
        self.gate_up = self.down = None

    def weight_specs(self):
        n = self.leaf
        return [WeightSpec(self.name(n["gate"]), (self.inner, self.width)),
                WeightSpec(self.name(n["up"]), (self.inner, self.width)),
                WeightSpec(self.name(n["down"]), (self.width, self.inner))]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        n = self.leaf
        self.gate_up = torch.cat([tensors[self.name(n["gate"])], tensors[self.name(n["up"])]], dim=0).contiguous()
        self.down = tensors[self.name(n["down"])].contiguous()

    def forward(self, h, ctx):
        h = plain(h)
        act = torch.empty((h.shape[0], self.inner), dtype=self.runtime.dtype, device=self.down.device)
        kernels.glu_clamped(linear(h, self.gate_up), act, self.limit, self.alpha)
        return linear(act, self.down, out_dtype=torch.float32)


@FEED_FORWARDS.register("dense_mlp")
class DenseMLP(FeedForward):
    """A plain feed-forward without a gate: down(act(up(x))), act one of `kernels.ACTIVATIONS` ("gelu_erf": the exact
    gelu 0.5 z (1 + erf(z / sqrt 2)); "gelu_tanh"; "silu"), computed in float32.  The result keeps the down product's
    float32 sums (the residual sum that follows reads them)."""

    def __init__(self, prefix: str, width: int, inner: int, activation: str = "gelu_erf", names: dict | None = None,
                 float32_out: bool = True):
        """`float32_out` False: the result is rounded to the engine's dtype (a part that sums it with others of that dtype)."""
        super().__init__(prefix)
        if activation not in kernels.ACTIVATIONS:
            raise InvalidRequest(f"activation {activation!r} is not built; known: {sorted(kernels.ACTIVATIONS)}")
        self.width, self.inner, self.activation, self.float32_out = int(width), int(inner), activation, bool(float32_out)
        self.leaf = {"up": "up_proj.weight", "down": "down_proj.weight"}
        self.leaf.update(names or {})
        self.up = self.down = None

    def weight_specs(self):
        return [WeightSpec(self.name(self.leaf["up"]), (self.inner, self.width)),
                WeightSpec(self.name(self.leaf["down"]), (self.width, self.inner))]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.up = tensors[self.name(self.leaf["up"])].contiguous()
        self.down = tensors[self.name(self.leaf["down"])].contiguous()

    def forward(self, h, ctx):
        x = plain(h)
        if kernels.gemm_act_rows_wins(x, self.up, self.activation):      # many rows: the activation in the product's epilogue
            z = torch.empty((x.shape[0], self.inner), dtype=x.dtype, device=x.device)
            kernels.gemm_act_rows(x, self.up, z, self.activation)
        else:
            z = linear(x, self.up)
            kernels.activation(z, z, self.activation)
        return linear(z, self.down, out_dtype=torch.float32 if self.float32_out else None)


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(FeedForward):
    """A gated feed-forward down(act(gate(x)) * up(x)) with the activation a parameter (one of `kernels.ACTIVATIONS`; float32
    arithmetic) whose result keeps the down product's float32 sums (the norm or residual sum that follows reads them).  Gate
    and up are one projection; when serving in bfloat16 with an inner size of a multiple of 64, blocks of 64 gate rows
    alternate with the 64 matching up rows, so that from 2,048 rows on the tcgen05 product may apply the activation in its
    epilogue (silu and relu gates; where it was timed ahead of the library's product and the activation kernel)."""

    BLOCK = 64

    def __init__(self, prefix: str, width: int, inner: int, activation: str = "silu", names: dict | None = None):
        super().__init__(prefix)
        if activation not in kernels.ACTIVATIONS:
            raise InvalidRequest(f"activation {activation!r} is not built; known: {sorted(kernels.ACTIVATIONS)}")
        self.width, self.inner, self.activation = int(width), int(inner), activation
        self.leaf = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}
        self.leaf.update(names or {})
        self.gate_up = self.down = None
        self.block = 0

    def weight_specs(self):
        n = self.leaf
        return [WeightSpec(self.name(n["gate"]), (self.inner, self.width)),
                WeightSpec(self.name(n["up"]), (self.inner, self.width)),
                WeightSpec(self.name(n["down"]), (self.width, self.inner))]

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        n = self.leaf
        gate, up = tensors[self.name(n["gate"])], tensors[self.name(n["up"])]
        self.block = self.BLOCK if runtime.is_bf16 and self.inner % self.BLOCK == 0 else 0
        if self.block:
            b = self.block
            self.gate_up = torch.stack([gate.view(-1, b, self.width), up.view(-1, b, self.width)], dim=1) \
                .reshape(2 * self.inner, self.width).contiguous()
        else:
            self.gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.down = tensors[self.name(n["down"])].contiguous()

    def forward(self, h, ctx):
        h = plain(h)
        act = torch.empty((h.shape[0], self.inner), dtype=self.runtime.dtype, device=self.down.device)
        if self.block and self.activation in kernels.GATE_ACTIVATIONS and not observing(ctx) \
                and kernels.gemm_gated_rows_wins(h, self.gate_up, self.activation):
            kernels.gemm_gated_rows(h, self.gate_up, act, self.activation)
        else:
            kernels.gated_activation(linear(h, self.gate_up), act, self.activation, self.block)
        return linear(act, self.down, out_dtype=torch.float32)
