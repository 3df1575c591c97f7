"""Rotary position encoding: split-half pairing (j, j + d/2) with every dimension rotary
(reference: crates/kernels/src/ops.cu:79-90) unless a part of the head (`rotary_dim`) or pairs of neighbours
(`pairing="interleaved"`) are asked for.  The part owns the table of inverse
frequencies; angle = position * f_j, its cosine and sine and the rotation are float32.  The
cosines and sines of a step's tokens are computed once and shared by every layer that rotates
by the same frequencies (`rotations`); kernels that have the angles at hand compute them
themselves from the frequencies of `rotation()`."""
from __future__ import annotations

import math

import torch

from .. import kernels
from ..errors import InvalidRequest
from .base import POSITION_ENCODINGS, PositionEncoding, Rotation


@POSITION_ENCODINGS.register("rope")
class RotaryPosition(PositionEncoding):
    def __init__(self, prefix: str, head_dim: int, theta: float, rotary_dim: int | None = None, pairing: str = "split_half"):
        """`rotary_dim`: the first so many elements of a head turn (None: all), pair j by position * theta^(-2j / rotary_dim);
        `pairing`: "split_half" (j with j + rotary_dim / 2) or "interleaved" (2j with 2j + 1)."""
        super().__init__(prefix)
        self.head_dim, self.theta = int(head_dim), float(theta)
        self.rotary_dim = self.head_dim if rotary_dim is None else int(rotary_dim)
        self.pairing = pairing
        if pairing not in ("split_half", "interleaved") or self.rotary_dim % 2 or not 0 <= self.rotary_dim <= self.head_dim:
            raise InvalidRequest("rotary positions: an even number of a head's elements turn, in split halves or interleaved pairs")
        self.inv_freq: torch.Tensor | None = None
        self.shared_key = None

    @staticmethod
    def inverse_frequencies(head_dim: int, theta: float) -> torch.Tensor:
        """f_j = 1 / float32(theta^(2j/d)): the power in float64, narrowed, then the reciprocal
        in float32 (reference: crates/kernels/src/lib.rs:612-614)."""
        j = torch.arange(head_dim // 2, dtype=torch.float64)
        power = torch.pow(torch.tensor(theta, dtype=torch.float64), 2.0 * j / head_dim)
        return 1.0 / power.to(torch.float32)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        frequencies = self.inverse_frequencies(self.rotary_dim, self.theta)
        self.inv_freq = frequencies.to(runtime.device)
        self.shared_key = ("rotations", frequencies.numpy().tobytes())     # layers with the same frequencies share a step's table

    def rotation(self):
        return Rotation(self.inv_freq, self.rotary_dim, self.pairing, 1.0)

    def rotations(self, ctx):
        """[tokens, rotary_dim / 2, 2] float32 (cos, sin) for the step's positions; kept in `ctx.shared` for the
        step's other layers (the model empties it when a step begins)."""
        shared = getattr(ctx, "shared", None)
        if shared is not None and self.shared_key in shared:
            return shared[self.shared_key]
        table = kernels.rotation_table(ctx.positions, self.inv_freq)
        if shared is not None:
            shared[self.shared_key] = table
        return table


@POSITION_ENCODINGS.register("yarn_rope")
class YarnRotaryPosition(PositionEncoding):
    """Rotary positions on the first `rotary_dim` elements of a head (element i with i + rotary_dim / 2), with
    frequencies stretched for contexts beyond the length the model was trained at: with d(t) = rotary_dim *
    ln(original / (2 pi t)) / (2 ln theta), the pair that makes t turns over the original length, lo =
    max(floor(d(fast)), 0), hi = min(ceil(d(slow)), rotary_dim - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
    pair i turns by f_i / factor * ramp_i + f_i * (1 - ramp_i), f_i = theta^(-2i / rotary_dim); cosines and sines are
    multiplied by `magnitude_slope` * ln(factor) + 1.  A factor of 1 (or none) leaves plain rotary positions.  The table
    is made on the host in float64 and held in float32; the angles are float32."""

    def __init__(self, prefix: str, rotary_dim: int, theta: float, factor: float = 1.0, original: float = 0.0, fast: float = 32.0,
                 slow: float = 1.0, magnitude_slope: float = 0.1):
        super().__init__(prefix)
        self.rotary_dim, self.theta = int(rotary_dim), float(theta)
        self.factor, self.original, self.fast, self.slow = float(factor), float(original), float(fast), float(slow)
        self.magnitude_slope = float(magnitude_slope)
        if self.rotary_dim % 2 or self.rotary_dim < 0 or self.theta <= 1.0:
            raise InvalidRequest("rotary positions need an even number of elements and a base above 1")
        self.scaled = self.factor != 1.0
        if self.scaled and (self.factor <= 0.0 or self.original <= 0.0 or self.fast <= 0.0 or self.slow <= 0.0):
            raise InvalidRequest("stretched rotary positions need a positive factor, original length and turn counts")
        self.inv_freq: torch.Tensor | None = None

    def frequencies(self) -> torch.Tensor:
        dims, half = self.rotary_dim, self.rotary_dim // 2
        plain = [self.theta ** (-2.0 * i / dims) for i in range(half)]
        if not self.scaled:
            return torch.tensor(plain, dtype=torch.float64)

        def pair_of(turns: float) -> float:
            return dims * math.log(self.original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

        lo = max(math.floor(pair_of(self.fast)), 0)
        hi = min(math.ceil(pair_of(self.slow)), dims - 1)
        out = []
        for i, f in enumerate(plain):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(f / self.factor * ramp + f * (1.0 - ramp))
        return torch.tensor(out, dtype=torch.float64)

    @property
    def magnitude(self) -> float:
        return self.magnitude_slope * math.log(self.factor) + 1.0 if self.scaled else 1.0

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        self.inv_freq = self.frequencies().to(torch.float32).to(runtime.device)

    def rotation(self):
        return Rotation(self.inv_freq, self.rotary_dim, "split_half", self.magnitude)


@POSITION_ENCODINGS.register("none")
class NoPosition(PositionEncoding):
    def __init__(self, prefix: str = ""):
        super().__init__(prefix)

    def rotation(self):
        return None

    def rotations(self, ctx):
        return None
