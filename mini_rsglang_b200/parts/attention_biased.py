"""Grouped-query attention with what some designs put around its scores and values:

  * biases on the q, k and v projections;
  * key heads of `head_dim` and value heads of `value_dim` elements;
  * a soft cap on the scaled scores, cap * tanh(score / cap), and after it a learned bias by the distance
    i - j, taken from a small table through buckets: one row a distance below half the table, then rows spaced
    evenly in the logarithm of the distance up to `bias_far`, the last row for everything beyond;
  * a sliding window that also keeps the first `keep_first` positions in sight (at their true distances); or sight in
    chunks: position i sees j <= i only where floor(i / chunk) = floor(j / chunk), chunks counted from position 0;
  * an RMS norm over every query and key head (one weight of the head's size for all query heads, one for all key heads,
    or no weight);
  * a rotation of query and key heads by their positions (any registered position encoding: all or part of a head, split
    halves or interleaved pairs), with the head norm before or after it;
  * values that are the key heads as projected (before norm and rotation): no value projection;
  * a softmax with a sink: one more term in the denominator that has no key and no value, exp(0) or exp of a learned
    number a head (not scaled);
  * values blended with those of the first layer that blends, (1 - m) v + m v_first per token; the blended values
    are what the cache holds;
  * an output gate from the same input as the projections: one sigmoid a (token, head), or one a (token, value element).

One projection gives q | k | v | gate (float32 sums), one kernel adds the biases, blends, gates and writes the
pages, one kernel attends.  Every constant is a parameter; none of the extras is tied to another."""
from __future__ import annotations

import math

import torch

from .. import kernels
from ..errors import InvalidRequest
from ..weights.spec import WeightSpec
from .attention import (attention_tile_lists, choose_splits, fast_kernels_take, paged_attention, plan_attention_tiles,
                        tile_plan_arguments)
from .base import MIXERS, POSITION_ENCODINGS, KVNeed, Mixer, PartSpec, StepFacts
from .linear import linear


def distance_buckets(rows: int, far: float) -> list[int]:
    """Row of a bias table of `rows` rows for the distances 0, 1, ..., up to the first distance that takes the
    last row (every larger one takes it too): n < rows // 2 -> n; else rows // 2 + floor(ln(n / half) /
    ln(far / half) * (rows - half)), at most rows - 1.  Computed in float64 on the host."""
    half = rows // 2
    out = []
    n = 0
    while True:
        if n < half:
            b = n
        else:
            b = min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))
        out.append(b)
        if b >= rows - 1 and n >= half:
            return out
        n += 1
        if n > 1 << 22:
            raise InvalidRequest("distance buckets: the last row is never reached")


@MIXERS.register("biased_window_attention")
class BiasedWindowAttention(Mixer):
    replayable = True      # everything that changes from step to step is read from device tensors

    def __init__(self, prefix: str, width: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int | None = None,
                 scale: float | None = None, softcap: float = 0.0, window: int = 0, keep_first: int = 0,
                 bias_rows: int = 0, bias_far: float = 0.0, sink: bool = False, projection_bias: bool = False,
                 value_mix: str | None = None, value_mix_source: bool = False, output_gate: bool = False,
                 chunk: int = 0, sink_logits: bool = False, head_norm_eps: float | None = None,
                 position: PartSpec | None = None, head_norm_place: str = "before_rotation", head_norm_weights: bool = True,
                 values_from_keys: bool = False, names: dict | None = None):
        """`position`: a position encoding that rotates query and key heads (None: none); `head_norm_place`: the head norm
        stands "before_rotation" or "after_rotation"; `head_norm_weights` False: it has no weights.  `values_from_keys`: no
        value projection, a value head is its key head as projected (`value_dim` = `head_dim`).  `output_gate`: True or
        "heads": one gate a (token, head); "elements": one a value element of every head.
        `chunk` > 0 (no window then): sight within the query's chunk of positions.  `sink_logits`: the sink's logit is a
        learned number a query head.  `head_norm_eps`: query and key heads pass an RMS norm with this epsilon (None: no norm).
        `value_mix`: a key under which the layers that blend values find the first one's values within a step
        (None: no blending); `value_mix_source`: this layer is that first one (its own mixing weight is unused).
        `names`: leaves of the tensors below the part's root."""
        super().__init__(prefix)
        if num_heads % num_kv_heads:
            raise InvalidRequest("query heads must be a multiple of key/value heads")
        self.width, self.nq, self.nkv, self.d = int(width), int(num_heads), int(num_kv_heads), int(head_dim)
        self.e = int(value_dim) if value_dim else self.d
        if not 0 < self.d <= 256 or not 0 < self.e <= 256:
            raise InvalidRequest("head sizes must lie between 1 and 256")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.d)
        self.softcap, self.window, self.keep_first = float(softcap), int(window), int(keep_first)
        self.bias_rows, self.bias_far, self.sink = int(bias_rows), float(bias_far), bool(sink)
        self.chunk, self.sink_logits = int(chunk), bool(sink_logits)
        self.head_norm_eps = None if head_norm_eps is None else float(head_norm_eps)
        self.sink = self.sink or self.sink_logits
        if self.window < 0 or self.keep_first < 0 or self.softcap < 0 or self.chunk < 0:
            raise InvalidRequest("window, chunk, kept first positions and soft cap cannot be negative")
        if self.chunk and (self.window or self.keep_first):
            raise InvalidRequest("sight in chunks together with a window or kept first positions is not built")
        if self.head_norm_eps is not None and value_mix:
            raise InvalidRequest("head norms together with blended values are not built")
        # bias_rows -1: as many rows as the checkpoint's table has
        if self.bias_rows > 0:
            self._check_bias_table(self.bias_rows)
        self.projection_bias = bool(projection_bias)
        self.output_gate = "heads" if output_gate is True else (output_gate or None)
        if self.output_gate not in (None, "heads", "elements"):
            raise InvalidRequest(f"{prefix}: an output gate is one a head ('heads') or one a value element ('elements')")
        self.position = POSITION_ENCODINGS.build(position, prefix) if position is not None else None
        self.head_norm_place, self.head_norm_weights = head_norm_place, bool(head_norm_weights)
        self.values_from_keys = bool(values_from_keys)
        if head_norm_place not in ("before_rotation", "after_rotation"):
            raise InvalidRequest(f"{prefix}: a head norm stands before_rotation or after_rotation")
        if self.values_from_keys and self.e != self.d:
            raise InvalidRequest(f"{prefix}: values taken from the keys have the keys' size")
        # what only the kernel with rotations does, and what only the one with biases and blending does
        self.rotary_store = (self.position is not None or self.values_from_keys or not self.head_norm_weights
                             or head_norm_place == "after_rotation" or self.output_gate == "elements")
        if self.rotary_store and (projection_bias or value_mix or self.output_gate == "heads"):
            raise InvalidRequest(f"{prefix}: rotation, values from keys, weightless or late head norms and gates a value element "
                                 "are not built together with projection biases, blended values or gates a head")
        if self.rotary_store and self.d > kernels.ROTARY_MAX_HEAD:
            raise InvalidRequest(f"{prefix}: rotated heads have at most {kernels.ROTARY_MAX_HEAD} elements")
        self.value_mix, self.value_mix_source = value_mix, bool(value_mix_source)
        self.leaf = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
                     "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias", "bias_table": "distance_bias",
                     "mix": "value_mix", "gate": "gate_proj.weight", "q_norm": "q_norm.weight", "k_norm": "k_norm.weight",
                     "sink": "sinks"}
        self.leaf.update(names or {})
        self.fused = self.o = self.bias = self.distance_bias = self.q_norm = self.k_norm = self.sinks = None
        self.mix = 0.0
        self._plan_arguments = None

    def _check_bias_table(self, rows: int) -> None:
        if rows < 2 or self.bias_far <= rows // 2:
            raise InvalidRequest("a distance bias needs at least two rows and a far distance beyond half the table")

    def weight_specs(self):
        n = self.leaf
        specs = [WeightSpec(self.name(n["q"]), (self.nq * self.d, self.width)),
                 WeightSpec(self.name(n["k"]), (self.nkv * self.d, self.width))]
        if not self.values_from_keys:
            specs.append(WeightSpec(self.name(n["v"]), (self.nkv * self.e, self.width)))
        specs.append(WeightSpec(self.name(n["o"]), (self.width, self.nq * self.e)))
        if self.projection_bias:
            specs += [WeightSpec(self.name(n["q_bias"]), (self.nq * self.d,), "bias"),
                      WeightSpec(self.name(n["k_bias"]), (self.nkv * self.d,), "bias"),
                      WeightSpec(self.name(n["v_bias"]), (self.nkv * self.e,), "bias")]
        if self.bias_rows:
            specs.append(WeightSpec(self.name(n["bias_table"]), (self.bias_rows, self.nq), "bias"))
        if self.value_mix:
            specs.append(WeightSpec(self.name(n["mix"]), (), "bias"))
        if self.output_gate:
            specs.append(WeightSpec(self.name(n["gate"]), (self.nq * (self.e if self.output_gate == "elements" else 1), self.width)))
        if self.head_norm_eps is not None and self.head_norm_weights:
            specs += [WeightSpec(self.name(n["q_norm"]), (self.d,), "vector"), WeightSpec(self.name(n["k_norm"]), (self.d,), "vector")]
        if self.sink_logits:
            specs.append(WeightSpec(self.name(n["sink"]), (self.nq,), "bias"))
        return specs

    def cache_need(self):
        # a window gives passed pages back; the pages of kept first positions stay with the request; a chunk never
        # reaches further back than its own length, so its cache is a window of that many keys
        if self.chunk:
            return KVNeed(self.nkv, self.d, "window", self.chunk, value_dim=self.e)
        if self.window:
            return KVNeed(self.nkv, self.d, "window", self.window, value_dim=self.e, keep_first=self.keep_first)
        return KVNeed(self.nkv, self.d, "full", 0, value_dim=self.e)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        n = self.leaf
        rows = [tensors[self.name(n[k])] for k in (("q", "k") if self.values_from_keys else ("q", "k", "v"))]
        if self.position is not None:
            self.position.bind(tensors, runtime)
        if self.output_gate:
            rows.append(tensors[self.name(n["gate"])])
        self.fused = torch.cat(rows, dim=0).contiguous()
        self.o = tensors[self.name(n["o"])].contiguous()
        if self.projection_bias:
            self.bias = torch.cat([tensors[self.name(n[k])].float() for k in ("q_bias", "k_bias", "v_bias")]).contiguous()
        if self.bias_rows:
            table = tensors[self.name(n["bias_table"])].float()
            self._check_bias_table(table.shape[0])
            rows_of = torch.tensor(distance_buckets(table.shape[0], self.bias_far), dtype=torch.long, device=table.device)
            self.distance_bias = table[rows_of].contiguous()         # [distances, heads]: the table, a row a distance
        if self.value_mix and not self.value_mix_source:
            self.mix = float(tensors[self.name(n["mix"])].float().item())
        if self.head_norm_eps is not None and self.head_norm_weights:
            self.q_norm = tensors[self.name(n["q_norm"])].float().contiguous()
            self.k_norm = tensors[self.name(n["k_norm"])].float().contiguous()
        if self.sink_logits:
            self.sinks = tensors[self.name(n["sink"])].float().contiguous()

    def forward(self, h, ctx, cache, write_cache=True):
        tokens = h.shape[0]
        device, dtype = self.o.device, self.runtime.dtype
        proj = linear(h, self.fused, out_dtype=torch.float32)
        q = torch.empty((tokens, self.nq * self.d), dtype=dtype, device=device)
        gate = torch.empty((tokens, self.nq), dtype=torch.float32, device=device) if self.output_gate == "heads" else None
        v_first, mode = None, 0
        if self.rotary_store:
            rotation = self.position.rotation() if self.position is not None else None
            if rotation is not None and rotation.rotary_dim == 0:
                rotation = None
            if rotation is not None and rotation.magnitude != 1.0:
                raise InvalidRequest(f"{self.prefix}: stretched cosines and sines are not built for this attention")
            kernels.qkv_rotary_store(proj, q, cache.k if write_cache else None, cache.v if write_cache else None,
                                     ctx.slots[cache.group] if write_cache else None, self.nq, self.nkv, self.d, self.e,
                                     rotations=self.position.rotations(ctx) if rotation is not None else None,
                                     rotary_dim=rotation.rotary_dim if rotation is not None else 0,
                                     pairing=rotation.pairing if rotation is not None else "split_half",
                                     norm_place=self.head_norm_place if self.head_norm_eps is not None else None,
                                     q_norm=self.q_norm, k_norm=self.k_norm, norm_eps=self.head_norm_eps or 0.0,
                                     values_from_keys=self.values_from_keys)
            return self._attend(q, proj, gate, ctx, cache)
        if self.value_mix:
            key = ("value_mix", self.value_mix)
            if self.value_mix_source:
                v_first = ctx.shared[key] = torch.empty((tokens, self.nkv * self.e), dtype=torch.float32, device=device)
                mode = 1
            else:
                if key not in ctx.shared:
                    raise InvalidRequest(f"{self.prefix}: no earlier layer of the step left values to blend with")
                v_first, mode = ctx.shared[key], 2
        kernels.qkv_bias_store(proj, self.bias, q, cache.k if write_cache else None, cache.v if write_cache else None,
                               ctx.slots[cache.group] if write_cache else None, self.nq, self.nkv, self.d, self.e,
                               v_first=v_first, mix_mode=mode, mix=self.mix, gate_out=gate, q_norm=self.q_norm, k_norm=self.k_norm,
                               norm_eps=self.head_norm_eps or 0.0)
        return self._attend(q, proj, gate, ctx, cache)

    def _attend(self, q, proj, gate, ctx, cache):
        """The attention over the pages and the output projection; `gate`: the heads' gates, if there are such."""
        tokens = q.shape[0]
        device, dtype = self.o.device, self.runtime.dtype
        out = torch.empty((tokens, self.nq * self.e), dtype=dtype, device=device)
        table = ctx.block_tables[cache.group]
        arguments = self._tile_plan()
        if self._plain_scores():
            # nothing but scale, cap and window around the scores: the kernels that are fed by bulk tensor copies take them
            paged_attention(q, cache, ctx, out, self.nq, self.nkv, self.d, self.window, scale=self.scale, cap=self.softcap)
        elif not arguments:
            # the 32-bit path and head sizes that the tensor-core kernel does not take: one warp a (token, head)
            kernels.attention_biased_simt(q, cache.k, cache.v, ctx.positions, ctx.seq_of_token, table, out, self.nq, self.nkv,
                                          self.d, self.e, self.scale, self.softcap, self.window, self.keep_first,
                                          self.distance_bias, gate, self.sink, self.sinks, self.chunk)
        else:
            # decoded tokens and short portions in tiles of 16 rows whose warps share the keys, longer portions in tiles of 64
            narrow, wide, longest, _ = plan_attention_tiles(ctx, *arguments)
            for tiles, is_narrow in ((narrow, True), (wide, False)):
                if tiles is not None:
                    splits = 1
                    if is_narrow:          # few rows: the keys in sight (the window and the kept tokens at most) are shared among CTAs
                        reach = min(longest, self.window + self.keep_first) if self.window else (min(longest, self.chunk) if self.chunk else longest)
                        splits = min(choose_splits(tiles.shape[0], self.nkv, reach, arguments[5]), 16)
                    kernels.attention_biased_mma(q, cache.k, cache.v, ctx.positions, table, tiles, out, self.nq, self.nkv, self.d,
                                                 self.e, self.scale, self.softcap, self.window, self.keep_first, self.distance_bias,
                                                 gate, self.sink, narrow=is_narrow, splits=splits, sink_logits=self.sinks, chunk=self.chunk)
        if self.output_gate == "elements":         # the gates are the projection's last columns, still float32 sums
            kernels.sigmoid_gate_mul(out, proj[:, proj.shape[1] - self.nq * self.e:])
        return linear(out, self.o, out_dtype=torch.float32)

    def _plain_scores(self) -> bool:
        """Whether this attention, as it is served, is scale, cap, window and softmax and nothing else (no bias table, no
        sink, no kept first positions, no chunks, no gate a head, values of the keys' size), at sizes that the kernels fed by
        bulk tensor copies take."""
        return (self.runtime.dtype is torch.bfloat16 and self.e == self.d and not self.bias_rows and not self.sink
                and not self.keep_first and not self.chunk and self.output_gate != "heads"
                and fast_kernels_take(self.d, self.nq // self.nkv, self.runtime.page_size))

    def _tile_plan(self) -> tuple:
        """What the tile planner is asked for this attention ((): no tiles, the CUDA-core kernel takes every row)."""
        if self._plan_arguments is None:
            group = self.nq // self.nkv
            if self._plain_scores():
                self._plan_arguments = tile_plan_arguments(self.d, group, self.runtime.page_size, self.nkv, self.window, self.o.device)
            elif self.runtime.dtype is torch.bfloat16 and \
                    kernels.attention_biased_mma_supported(self.d, self.e, group, self.runtime.page_size):
                # the window enters the plan only as the reach of a tile's keys; kept first tokens add a block at most
                self._plan_arguments = (group, kernels.MMA_ROWS_WIDE, self.nkv, self.window or self.chunk, 128, kernels.sm_count(self.o.device))
            else:
                self._plan_arguments = ()
        return self._plan_arguments

    def step_signature(self, facts: StepFacts):
        """The lengths of a step's two tile lists (None: no list is planned)."""
        arguments = self._tile_plan()
        return attention_tile_lists(facts, *arguments).signature() if arguments else None
