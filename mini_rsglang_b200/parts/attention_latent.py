"""Latent attention: keys and values of all heads are made from one small latent a token, and the cache keeps
that latent instead of them.

With h the mixer's input, H heads, per head d unrotated and r rotated query/key elements and e value elements,
and a latent of R elements:

  q = W_q h                         per head [d unrotated | r rotated]
  (c', k_r) = W_dkv h               c = c' / rms(c') * w_c  [R];  k_r [r], rotated, one for all heads
  k_head = W_uk[head] c  [d],  v_head = W_uv[head] c  [e]
  score(i, j) = (q_plain_i . k_head_j + q_rot_i . k_r_j) * scale,  softmax over the keys in sight (all earlier
  ones, or a sliding window), out_head = sum_j p_j v_head_j, times sigmoid(W_g h)_head where the layer gates,
  then W_o over the concatenated heads.

The cache holds one row a token, [c | k_r] (`KVNeed.values = False`: no value pages), and the attention runs in the
latent space, where every head reads the same rows: since q_plain . (W_uk c) = (W_uk^T q_plain) . c and
sum_j p_j W_uv c_j = W_uv sum_j p_j c_j, a head's query becomes [W_uk^T q_plain | q_rot] of R + r elements, its
"values" are the rows' first R elements, and W_uv is applied once to the result.  A layer may read the cache of
another layer that keeps one (`shares_cache`): it has no W_dkv, and uses that layer's rows with its own W_uk and
W_uv, queries, window and gate.

The queries may pass a latent of their own (`query_latent_dim`): c_q = W_dq h / rms(W_dq h) * w_q, q = W_uq c_q; such a layer
rotates nothing here.  The gate is one sigmoid a (token, head), or (`output_gate="elements"`) one a (token, head, value
element), W_g then having heads * e rows.

One projection gives q | c', k_r | gates (or c_q' | c' | gates) as float32 sums; one kernel norms the latent, rotates, gates and writes the
cache row; a batched product carries the queries into the latent space; one kernel attends; a batched product and the
output projection bring the heads back.  Every size and constant is a parameter."""
from __future__ import annotations

import torch

from .. import kernels
from ..errors import InvalidRequest
from ..weights.spec import WeightSpec
from .attention import attention_tile_lists, choose_splits, plan_attention_tiles
from .base import MIXERS, POSITION_ENCODINGS, KVNeed, Mixer, PartSpec, StepFacts
from .linear import linear


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    replayable = True      # everything that changes from step to step is read from device tensors

    def __init__(self, prefix: str, width: int, num_heads: int, head_dim: int, rotary_head_dim: int, value_dim: int,
                 latent_dim: int, scale: float, eps: float, position: PartSpec | None = None, window: int = 0,
                 cache_window: int | None = None, shares_cache: bool = False, output_gate: bool | str = False,
                 query_latent_dim: int = 0, float32_out: bool = False,
                 names: dict | None = None):
        """`position`: the encoding of the rotated part (None: nothing turns).  `window` 0: every earlier key is seen.
        `cache_window`: the window that the cache is kept for, where other layers read this layer's cache with wider
        windows (0: every key).  `shares_cache`: this layer reads another layer's cache and has no down-projection.
        `output_gate`: False, True or "heads" (one gate a head), or "elements" (one a value element of every head).
        `query_latent_dim` > 0: the queries are made from a normed latent of that size.
        `float32_out`: the output projection hands on its float32 sums (for a residual sum that reads them).
        `names`: leaves of the tensors below the part's root."""
        super().__init__(prefix)
        self.width, self.heads, self.d, self.r = int(width), int(num_heads), int(head_dim), int(rotary_head_dim)
        self.e, self.latent = int(value_dim), int(latent_dim)
        if min(self.width, self.heads, self.d, self.e, self.latent) <= 0 or self.r < 0:
            raise InvalidRequest(f"{prefix}: sizes of a latent attention must be positive")
        if self.latent + self.r > 1152 or self.latent > 1024:
            raise InvalidRequest(f"{prefix}: a latent of more than 1,024, or cache rows of more than 1,152 elements, are not built")
        self.scale, self.eps, self.window = float(scale), float(eps), int(window)
        self.cache_window = self.window if cache_window is None else int(cache_window)
        if self.window < 0 or (self.cache_window and (not self.window or self.cache_window < self.window)):
            raise InvalidRequest(f"{prefix}: the cache must keep at least the keys that the layer's window sees")
        if output_gate not in (False, True, "heads", "elements"):
            raise InvalidRequest(f"{prefix}: output_gate must be False, True, \"heads\" or \"elements\"")
        self.shares_cache, self.output_gate = bool(shares_cache), bool(output_gate)
        self.gate_elements = output_gate == "elements"
        self.float32_out = bool(float32_out)
        self.query_latent = int(query_latent_dim)
        if self.query_latent < 0 or (self.query_latent and (self.r or self.shares_cache or position is not None)):
            raise InvalidRequest(f"{prefix}: queries from a latent together with a rotated part or a borrowed cache are not built")
        if self.gate_elements and not self.query_latent:
            raise InvalidRequest(f"{prefix}: a gate a value element is built for layers whose queries pass a latent")
        self.position = POSITION_ENCODINGS.build(position, prefix) if position is not None else None
        self.leaf = {"q": "q_proj.weight", "down": "kv_down_proj.weight", "latent_norm": "kv_norm.weight", "up_k": "k_up_proj.weight",
                     "up_v": "v_up_proj.weight", "gate": "gate_proj.weight", "o": "o_proj.weight", "q_down": "q_down_proj.weight",
                     "q_norm": "q_norm.weight", "q_up": "q_up_proj.weight"}
        self.leaf.update(names or {})
        self.fused = self.latent_weight = self.up_k = self.up_v = self.o = self.q_up = self.q_latent_weight = None
        self.rotation = None
        self._plan_arguments = None

    @property
    def row(self) -> int:
        """Elements of a cache row, and of a query row in the latent space."""
        return self.latent + self.r

    def weight_specs(self):
        n = self.leaf
        if self.query_latent:
            specs = [WeightSpec(self.name(n["q_down"]), (self.query_latent, self.width)),
                     WeightSpec(self.name(n["q_norm"]), (self.query_latent,), "vector"),
                     WeightSpec(self.name(n["q_up"]), (self.heads * self.d, self.query_latent))]
        else:
            specs = [WeightSpec(self.name(n["q"]), (self.heads * (self.d + self.r), self.width))]
        if not self.shares_cache:
            specs += [WeightSpec(self.name(n["down"]), (self.row, self.width)),
                      WeightSpec(self.name(n["latent_norm"]), (self.latent,), "vector")]
        specs += [WeightSpec(self.name(n["up_k"]), (self.heads * self.d, self.latent)),
                  WeightSpec(self.name(n["up_v"]), (self.heads * self.e, self.latent))]
        if self.output_gate:
            specs.append(WeightSpec(self.name(n["gate"]), (self.heads * self.e if self.gate_elements else self.heads, self.width)))
        specs.append(WeightSpec(self.name(n["o"]), (self.width, self.heads * self.e)))
        return specs

    def cache_need(self):
        kind = "window" if self.cache_window else "full"
        return KVNeed(1, self.row, kind, self.cache_window, values=False)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        n = self.leaf
        rows = [tensors[self.name(n["q_down" if self.query_latent else "q"])]]
        if self.query_latent:
            self.q_latent_weight = tensors[self.name(n["q_norm"])]
            self.q_up = tensors[self.name(n["q_up"])].contiguous()
        if not self.shares_cache:
            rows.append(tensors[self.name(n["down"])])
            self.latent_weight = tensors[self.name(n["latent_norm"])]
        if self.output_gate:
            rows.append(tensors[self.name(n["gate"])])
        self.fused = torch.cat(rows, dim=0).contiguous()
        self.up_k = tensors[self.name(n["up_k"])].contiguous().view(self.heads, self.d, self.latent)
        self.up_v = tensors[self.name(n["up_v"])].contiguous().view(self.heads, self.e, self.latent).transpose(1, 2)
        self.o = tensors[self.name(n["o"])].contiguous()
        if self.position is not None:
            self.position.bind(tensors, runtime)
            self.rotation = self.position.rotation()
        if self.rotation is not None:
            if self.rotation.pairing != "split_half" or self.rotation.rotary_dim > self.r or self.rotation.rotary_dim % 2:
                raise InvalidRequest(f"{self.prefix}: the kernel turns an even number of the rotated part's first elements, "
                                     "element i with i + half of them")

    def forward(self, h, ctx, cache, write_cache=True):
        tokens = h.shape[0]
        device, dtype = self.o.device, self.runtime.dtype
        H, R, row = self.heads, self.latent, self.row
        proj = linear(h, self.fused, out_dtype=torch.float32)
        q_rows = torch.empty((tokens, H, row), dtype=dtype, device=device)
        keeps = write_cache and not self.shares_cache
        if self.query_latent:
            # c_q' | c' | gates: both latents normed by one kernel, the second into the cache; then the queries' up-projection
            q_latent = torch.empty((tokens, self.query_latent), dtype=dtype, device=device)
            kernels.latent_norms(proj, self.q_latent_weight, self.latent_weight, self.eps, ctx.slots[cache.group] if keeps else None,
                                 q_latent, cache.k if keeps else None)
            q_plain = linear(q_latent, self.q_up).view(tokens, H, self.d).transpose(0, 1)
            gate = None
        else:
            q_plain = torch.empty((H, tokens, self.d), dtype=dtype, device=device)
            gate = torch.empty((tokens, H), dtype=torch.float32, device=device) if self.output_gate else None
            rotation = self.rotation
            kernels.latent_prepare(proj, self.latent_weight, self.eps, rotation.inv_freq if rotation else None,
                                   rotation.magnitude if rotation else 1.0, ctx.positions, ctx.slots[cache.group] if keeps else None,
                                   q_plain, q_rows, cache.k if keeps else None, gate, H, self.d, self.r, R,
                                   rotation.rotary_dim if rotation else 0, not self.shares_cache)
        # the queries in the latent space: q_rows[:, head, :R] = q_plain[head] . W_uk[head]
        torch.bmm(q_plain, self.up_k, out=q_rows[:, :, :R].transpose(0, 1))
        q_rows = q_rows.view(tokens, H * row)
        mixed = torch.empty((tokens, H * R), dtype=dtype, device=device)
        table = ctx.block_tables[cache.group]
        arguments = self._tile_plan()
        if not arguments:
            # the 32-bit path and sizes that the tensor-core kernel does not take: one warp a (token, head)
            kernels.attention_biased_simt(q_rows, cache.k, None, ctx.positions, ctx.seq_of_token, table, mixed, H, 1, row, R,
                                          self.scale, window=self.window, gate=gate)
        else:
            narrow, wide, longest, _ = plan_attention_tiles(ctx, *arguments)
            few = kernels.MMA_ROWS_NARROW
            if ctx.decode_tiles is not None and narrow is None and H > few and H % few == 0:
                # single tokens of more heads than a tile of few rows holds: all heads read the same cache rows, so any
                # `few` of them are as good a group as all; a token becomes H / few rows of that many heads at its position,
                # each a narrow tile whose keys CTAs share (a wide tile would walk a request's keys alone)
                m = H // few
                tiles, positions = self._rows_of_few_heads(ctx, m)
                reach = min(longest, self.window) if self.window else longest
                splits = min(choose_splits(tiles.shape[0], 1, reach, arguments[5]), 16)
                kernels.attention_biased_mma(q_rows.view(tokens * m, few * row), cache.k, None, positions, table, tiles,
                                             mixed.view(tokens * m, few * R), few, 1, row, R, self.scale, window=self.window,
                                             gate=gate.view(tokens * m, few) if gate is not None else None, narrow=True, splits=splits)
                wide = None
            for tiles, is_narrow in ((narrow, True), (wide, False)):
                if tiles is not None:
                    splits = 1
                    if is_narrow:          # few rows: the keys in sight are shared among CTAs
                        reach = min(longest, self.window) if self.window else longest
                        splits = min(choose_splits(tiles.shape[0], 1, reach, arguments[5]), 16)
                    kernels.attention_biased_mma(q_rows, cache.k, None, ctx.positions, table, tiles, mixed, H, 1, row, R, self.scale,
                                                 window=self.window, gate=gate, narrow=is_narrow, splits=splits)
        # back to the heads' values: out[:, head] = mixed[:, head] . W_uv[head]^T
        out = torch.empty((tokens, H, self.e), dtype=dtype, device=device)
        torch.bmm(mixed.view(tokens, H, R).transpose(0, 1), self.up_v, out=out.transpose(0, 1))
        out = out.view(tokens, H * self.e)
        if self.query_latent and self.output_gate:
            gates = proj[:, self.query_latent + R:]
            if not self.gate_elements:             # one gate a head: spread over the head's value elements
                gates = gates.repeat_interleave(self.e, dim=1)
            kernels.sigmoid_gate_mul(out, gates)
        return linear(out, self.o, out_dtype=torch.float32 if self.float32_out else None)

    @staticmethod
    def _rows_of_few_heads(ctx, m: int):
        """A step of single tokens with every token as `m` rows: the step's tile list with tile (s, t, n, 0) as m tiles
        (s, t * m + j, n, 0), and every token's position m times.  Made on the device from the step's own arrays (a recorded
        step makes them anew: what its trial run made stays outside the recording); kept in the context for the other
        layers of the same pass."""
        made = ctx.__dict__.setdefault("_rows_of_few_heads", {})
        key = (m, ctx.rehearsal)
        if key not in made:
            base = ctx.decode_tiles
            tiles = base.repeat(1, m).view(-1, 4)
            tiles[:, 1] = tiles[:, 1] * m + torch.arange(m, dtype=torch.int32, device=base.device).repeat(base.shape[0])
            made[key] = (tiles, ctx.positions.view(-1, 1).expand(-1, m).contiguous().view(-1))
        return made[key]

    def _tile_plan(self) -> tuple:
        """What the tile planner is asked for this attention ((): no tiles, the CUDA-core kernel takes every row).  All
        heads read the same rows: they are one group."""
        if self._plan_arguments is None:
            if self.runtime.dtype is torch.bfloat16 and \
                    kernels.attention_biased_mma_supported(self.row, self.latent, self.heads, self.runtime.page_size, values_in_keys=True):
                self._plan_arguments = (self.heads, kernels.MMA_ROWS_WIDE, 1, self.window, 128, kernels.sm_count(self.o.device))
            else:
                self._plan_arguments = ()
        return self._plan_arguments

    def step_signature(self, facts: StepFacts):
        """The lengths of a step's two tile lists (None: no list is planned)."""
        arguments = self._tile_plan()
        return attention_tile_lists(facts, *arguments).signature() if arguments else None
