"""The gated delta rule: a recurrent mixer whose state is a matrix a head, S [d, e], that forgets by a scalar a token and
then corrects what it holds under the token's key towards the token's value.

With h the mixer's input, H heads of e value elements and G groups of d query/key elements (head j reads group
j // (H / G)):

  q = W_q h, k = W_k h  [G, d];  v = W_v h  [H, e];  each channel of q, k, v passes a short causal convolution over time
  (taps weights a channel, the last one the current token's, zeros before the sequence's start) and silu;
  q and k become unit vectors per group, x / sqrt(sum x^2 + unit_eps), q also times d^(-1/2);
  beta = sigmoid(W_b h), g = exp(-exp(A_log) * softplus(W_a h + dt_bias))          one each a head
  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q                      per head, in this order
  out = W_o (o / rms(o) * w_norm * silu(W_g h))                                     rms over a head's e elements

A request's state (the convolution's last taps - 1 inputs, then S of every head) lives in its state slot as one float32
vector; it counts as zero where a sequence starts at position 0.  One projection gives q | k | v | b | a | gate as float32
sums; convolution, unit norms, step sizes, decays, the recurrence and the head norm are float32.  Every size and constant
is a parameter."""
from __future__ import annotations

import torch

from .. import kernels
from ..errors import InvalidRequest
from ..weights.spec import WeightSpec
from .base import MIXERS, Mixer, StateNeed
from .linear import linear


@MIXERS.register("gated_delta_rule")
class GatedDeltaRule(Mixer):
    replayable = True      # the step's facts are read from device tensors only

    def __init__(self, prefix: str, width: int, heads: int, groups: int, head_dim: int, value_dim: int, conv: int, eps: float,
                 unit_eps: float = 1e-6, names: dict | None = None):
        """`groups`: query/key heads; `conv`: taps of the convolution; `eps`: of the head norm; `unit_eps`: inside the root
        of the unit norms.  `names`: leaves of the tensors below the part's root."""
        super().__init__(prefix)
        self.width, self.heads, self.groups, self.d, self.e = int(width), int(heads), int(groups), int(head_dim), int(value_dim)
        self.taps, self.eps, self.unit_eps = int(conv), float(eps), float(unit_eps)
        if min(self.width, self.heads, self.groups, self.d, self.e) <= 0 or self.heads % self.groups:
            raise InvalidRequest(f"{prefix}: sizes must be positive and heads a multiple of the query/key heads")
        if not 1 <= self.taps <= 16 or self.d > 512:
            raise InvalidRequest(f"{prefix}: convolutions of 1 to 16 taps and query/key heads of up to 512 elements are built")
        self.channels = 2 * self.groups * self.d + self.heads * self.e           # q | k | v
        self.leaf = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "q_conv": "q_conv.weight",
                     "k_conv": "k_conv.weight", "v_conv": "v_conv.weight", "b": "b_proj.weight", "a": "a_proj.weight",
                     "a_log": "A_log", "dt_bias": "dt_bias", "norm": "norm.weight", "gate": "g_proj.weight", "o": "o_proj.weight"}
        self.leaf.update(names or {})
        self.conv_floats = (self.taps - 1) * self.channels
        self.fused = self.w_o = None

    def weight_specs(self):
        n, qk, inner = self.leaf, self.groups * self.d, self.heads * self.e
        return [WeightSpec(self.name(n["q"]), (qk, self.width)), WeightSpec(self.name(n["q_conv"]), (qk, self.taps), "bias"),
                WeightSpec(self.name(n["k"]), (qk, self.width)), WeightSpec(self.name(n["k_conv"]), (qk, self.taps), "bias"),
                WeightSpec(self.name(n["v"]), (inner, self.width)), WeightSpec(self.name(n["v_conv"]), (inner, self.taps), "bias"),
                WeightSpec(self.name(n["b"]), (self.heads, self.width)), WeightSpec(self.name(n["a_log"]), (self.heads,), "bias"),
                WeightSpec(self.name(n["norm"]), (self.e,), "vector"), WeightSpec(self.name(n["a"]), (self.heads, self.width)),
                WeightSpec(self.name(n["dt_bias"]), (self.heads,), "bias"), WeightSpec(self.name(n["gate"]), (inner, self.width)),
                WeightSpec(self.name(n["o"]), (self.width, inner))]

    def state_need(self):
        return StateNeed((self.conv_floats + self.heads * self.d * self.e,), torch.float32)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        n = self.leaf
        self.fused = torch.cat([tensors[self.name(n[key])] for key in ("q", "k", "v", "b", "a", "gate")], dim=0).contiguous()
        self.w_o = tensors[self.name(n["o"])].contiguous()
        self.conv_w = torch.cat([tensors[self.name(n[key])].float() for key in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        self.a_log = tensors[self.name(n["a_log"])].float().contiguous()
        self.dt_bias = tensors[self.name(n["dt_bias"])].float().contiguous()
        self.norm_w = tensors[self.name(n["norm"])].float().contiguous()

    def forward(self, h, ctx, cache, write_cache=True):
        tokens = h.shape[0]
        device = self.w_o.device
        H, G, d, e, C = self.heads, self.groups, self.d, self.e, self.channels
        proj = linear(h, self.fused, out_dtype=torch.float32)            # q | k | v | b | a | gate
        slots = cache.state.shape[0]
        conv_state = cache.state[:, :self.conv_floats].view(slots, self.taps - 1, C)
        s_state = cache.state[:, self.conv_floats:].view(slots, H, d, e)
        qkv = torch.empty((tokens, C), dtype=torch.float32, device=device)
        kernels.causal_conv_silu(proj, 0, self.conv_w, None, conv_state, ctx.positions, ctx.seq_of_token, ctx.q_start,
                                 ctx.state_slots, qkv, update_state=write_cache)
        coef = torch.empty((tokens, 2 * H), dtype=torch.float32, device=device)
        kernels.delta_prepare(qkv, proj, C, C + H, self.a_log, self.dt_bias, coef, G, d, H, e, self.unit_eps, d ** -0.5)
        o = torch.zeros((tokens, H * e), dtype=torch.float32, device=device)
        kernels.delta_scan(qkv, coef, s_state, ctx.positions, ctx.q_start, ctx.state_slots, o, H, G, d, e, write_state=write_cache)
        normed = torch.empty((tokens, H * e), dtype=self.runtime.dtype, device=device)
        kernels.head_norm_gate(o, proj[:, C + 2 * H:], self.norm_w, self.eps, normed, H)
        return linear(normed, self.w_o, out_dtype=torch.float32)
