"""Typed model configurations read from a checkpoint's config.json.

`ModelConfig` is what every architecture's configuration offers to the rest of the engine;
`Qwen3Config` holds the keys of Qwen3 dense under their config.json names and applies the
reference's checks (crates/models/src/config.rs:8-137).  No size stands in code: every
number the model uses comes from here."""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, fields
from typing import Any, ClassVar

from ..errors import InvalidRequest

INT32_MAX = 2**31 - 1


@dataclass
class ModelConfig:
    """Base of all typed configurations: the keys every architecture has."""

    model_type: str
    architectures: list[str]
    vocab_size: int
    max_position_embeddings: int
    eos_token_id: Any = None

    # the config.json values of `model_type` that this class reads
    MODEL_TYPES: ClassVar[tuple[str, ...]] = ()

    @classmethod
    def from_dict(cls, raw: dict) -> "ModelConfig":
        raise NotImplementedError

    def validate(self) -> None:
        raise NotImplementedError

    def to_dict(self) -> dict:
        """The configuration under its config.json key names."""
        return {f.name: getattr(self, f.name) for f in fields(self)}

    def save(self, folder: str) -> None:
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(self.to_dict(), f, indent=1)

    def eos_ids(self, folder: str | None = None) -> list[int]:
        """End-of-sequence ids: generation_config.json's `eos_token_id` when the folder has
        one, else config.json's; an int or a list (config.rs:155-184)."""
        value = self.eos_token_id
        if folder is not None:
            path = os.path.join(folder, "generation_config.json")
            if os.path.exists(path):
                with open(path) as f:
                    value = json.load(f).get("eos_token_id", value)
        values = value if isinstance(value, list) else [value]
        if not values:
            raise InvalidRequest("empty EOS token list")
        for v in values:
            if isinstance(v, bool) or not isinstance(v, int) or not 0 <= v < self.vocab_size:
                raise InvalidRequest("invalid eos_token_id")
        return list(values)


def _require(raw: dict, key: str, kind, what: str):
    if key not in raw or raw[key] is None:
        raise InvalidRequest(f"config.json: missing key `{key}` ({what})")
    value = raw[key]
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, int):
            raise InvalidRequest(f"config.json: `{key}` must be an integer, got {value!r}")
    elif kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise InvalidRequest(f"config.json: `{key}` must be a number, got {value!r}")
        value = float(value)
    elif kind is bool:
        if not isinstance(value, bool):
            raise InvalidRequest(f"config.json: `{key}` must be true or false, got {value!r}")
    elif kind is str:
        if not isinstance(value, str):
            raise InvalidRequest(f"config.json: `{key}` must be a string, got {value!r}")
    return value


@dataclass
class Qwen3Config(ModelConfig):
    """Qwen3 dense (`Qwen3ForCausalLM`).  Required and optional keys as in the reference's
    serde struct (config.rs:8-47); a file that spells `rope_theta` inside `rope_parameters`
    and `dtype` for `torch_dtype` is accepted too."""

    hidden_size: int = 0
    intermediate_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    rms_norm_eps: float = 0.0
    rope_theta: float = 0.0
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    rope_scaling: Any = None
    sliding_window: Any = None
    use_sliding_window: bool = False
    attention_bias: bool = False
    torch_dtype: Any = None
    num_experts: int = 0

    MODEL_TYPES: ClassVar[tuple[str, ...]] = ("qwen3",)
    MAX_HEAD_DIM: ClassVar[int] = 256   # the attention kernels' limit (config.rs:101 has the same)

    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen3Config":
        architectures = raw.get("architectures")
        if not isinstance(architectures, list) or not all(isinstance(a, str) for a in architectures):
            raise InvalidRequest("config.json: `architectures` must be a list of names")
        theta = raw.get("rope_theta")
        scaling = raw.get("rope_scaling")
        params = raw.get("rope_parameters")
        if isinstance(params, dict):
            if theta is None:
                theta = params.get("rope_theta")
            kind = params.get("rope_type", params.get("type", "default"))
            if kind not in (None, "default"):
                scaling = params
        if theta is None:
            raise InvalidRequest("config.json: missing key `rope_theta` (rotary base)")
        heads = _require(raw, "num_attention_heads", int, "query heads")
        hidden = _require(raw, "hidden_size", int, "model width")
        head_dim = raw.get("head_dim")
        if head_dim is None:
            if heads <= 0 or hidden % heads:
                raise InvalidRequest("config.json: no `head_dim` and hidden_size is no multiple of "
                                     "num_attention_heads")
            head_dim = hidden // heads
        cfg = cls(
            model_type=_require(raw, "model_type", str, "architecture family"),
            architectures=list(architectures),
            vocab_size=_require(raw, "vocab_size", int, "vocabulary"),
            max_position_embeddings=_require(raw, "max_position_embeddings", int, "longest context"),
            eos_token_id=raw.get("eos_token_id"),
            hidden_size=hidden,
            intermediate_size=_require(raw, "intermediate_size", int, "feed-forward width"),
            num_hidden_layers=_require(raw, "num_hidden_layers", int, "layers"),
            num_attention_heads=heads,
            num_key_value_heads=_require(raw, "num_key_value_heads", int, "key/value heads"),
            head_dim=head_dim,
            rms_norm_eps=_require(raw, "rms_norm_eps", float, "norm epsilon"),
            rope_theta=float(theta),
            tie_word_embeddings=_require(raw, "tie_word_embeddings", bool, "shared head"),
            hidden_act=_require(raw, "hidden_act", str, "activation"),
            rope_scaling=scaling,
            sliding_window=raw.get("sliding_window"),
            use_sliding_window=bool(raw.get("use_sliding_window", False)),
            attention_bias=bool(raw.get("attention_bias", False)),
            torch_dtype=raw.get("torch_dtype", raw.get("dtype")),
            num_experts=int(raw.get("num_experts", 0) or 0),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.model_type != "qwen3" or self.architectures != ["Qwen3ForCausalLM"] or self.num_experts:
            raise InvalidRequest("only Qwen3ForCausalLM (dense, model_type qwen3) is supported, got "
                                 f"model_type {self.model_type!r}, architectures {self.architectures!r}, "
                                 f"num_experts {self.num_experts}")
        if (self.rope_scaling is not None or self.use_sliding_window
                or self.sliding_window is not None or self.attention_bias or self.hidden_act != "silu"):
            raise InvalidRequest("RoPE scaling, sliding window, biased attention, or non-SiLU "
                                 "architecture unsupported")
        sizes = (self.hidden_size, self.intermediate_size, self.num_hidden_layers,
                 self.num_attention_heads, self.num_key_value_heads, self.vocab_size,
                 self.max_position_embeddings, self.head_dim)
        if any(isinstance(v, bool) or not isinstance(v, int) or v <= 0 for v in sizes):
            raise InvalidRequest("invalid Qwen3 dimensions: every size must be a positive integer")
        if self.head_dim > self.MAX_HEAD_DIM or self.head_dim % 2:
            raise InvalidRequest(f"invalid Qwen3 dimensions: head_dim {self.head_dim} must be even "
                                 f"and at most {self.MAX_HEAD_DIM}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise InvalidRequest("invalid Qwen3 dimensions or GQA ratio: num_attention_heads must be "
                                 "a multiple of num_key_value_heads")
        for v in (self.rms_norm_eps, self.rope_theta):
            if not math.isfinite(v) or v <= 0:
                raise InvalidRequest("invalid normalization or RoPE parameters")
        for a, b in ((self.num_attention_heads, self.head_dim), (self.num_key_value_heads, self.head_dim),
                     (self.vocab_size, self.hidden_size), (self.hidden_size, self.intermediate_size)):
            if a * b > INT32_MAX:
                raise InvalidRequest("model dimensions exceed backend limits")
        self.eos_ids()

    def to_dict(self) -> dict:
        out = super().to_dict()
        for key in ("rope_scaling", "sliding_window", "torch_dtype"):
            if out[key] is None:
                del out[key]
        if not out["num_experts"]:
            del out["num_experts"]
        return out


@dataclass
class NiduvikConfig(ModelConfig):
    """Niduvik: a decoder of layers that each hold one mixer, attention (no rotation; biased, soft-capped, windowed
    with kept first tokens, a sink in the softmax, blended values, an output gate) or a state-space recurrence, and
    optionally a clamped gated feed-forward, with an RMS norm before and after each branch.  config.json names the
    design under `architecture` and lists the layers with their sizes and constants; the keys are read as they
    stand there:

      vocab, width, norm.eps
      layers[i].type = "attention": mixer.{heads, kv_heads, dim, vdim, scale, softcap, bias_max, v_mix, mask.{size, keep_first}}
      layers[i].type = "mamba2":    mixer.{heads, vdim, state, groups, conv, norm_groups}
      layers[i].mlp = null | {kind: "dense", ff, limit}

    A checkpoint's distance-bias table states its own length; `mixer.bias_rows` gives it for a model that is drawn at
    random.  The design states no longest context and no end-of-sequence token; `max_position_embeddings` and `eos_token_id`
    are read if a file has them."""

    width: int = 0
    norm_eps: float = 0.0
    layers: list = None

    MODEL_TYPES: ClassVar[tuple[str, ...]] = ("niduvik",)
    NO_CONTEXT_LIMIT: ClassVar[int] = 1 << 22
    MIXER_KEYS: ClassVar[dict] = {
        "attention": {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "scale": float, "softcap": float,
                      "bias_max": float, "v_mix": bool},
        "mamba2": {"heads": int, "vdim": int, "state": int, "groups": int, "conv": int, "norm_groups": int},
    }

    @classmethod
    def from_dict(cls, raw: dict) -> "NiduvikConfig":
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise InvalidRequest("config.json: missing key `norm` (an object with `eps`)")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise InvalidRequest("config.json: `layers` must be a list of layers")
        read = []
        for i, layer in enumerate(layers):
            if not isinstance(layer, dict):
                raise InvalidRequest(f"config.json: layers[{i}] must be an object")
            kind = _require(layer, "type", str, f"mixer of layer {i}")
            if kind not in cls.MIXER_KEYS:
                raise InvalidRequest(f"config.json: layers[{i}].type {kind!r}; known: {sorted(cls.MIXER_KEYS)}")
            mixer = layer.get("mixer")
            if not isinstance(mixer, dict):
                raise InvalidRequest(f"config.json: layers[{i}].mixer must be an object")
            sizes = {key: _require(mixer, key, want, f"layers[{i}].mixer") for key, want in cls.MIXER_KEYS[kind].items()}
            if kind == "attention":
                mask = mixer.get("mask")
                if not isinstance(mask, dict):
                    raise InvalidRequest(f"config.json: layers[{i}].mixer.mask must be an object")
                if mixer.get("bias_rows") is not None:          # not a key of the design: the table's rows, for models without a checkpoint
                    sizes["bias_rows"] = _require(mixer, "bias_rows", int, "rows of the distance-bias table")
                sizes["mask"] = {"size": _require(mask, "size", int, "window"), "keep_first": _require(mask, "keep_first", int, "kept first tokens")}
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise InvalidRequest(f"config.json: layers[{i}].mlp must be null or an object")
                mlp = {"kind": _require(mlp, "kind", str, "feed-forward kind"), "ff": _require(mlp, "ff", int, "feed-forward width"),
                       "limit": _require(mlp, "limit", float, "clamp")}
            read.append({"type": kind, "mixer": sizes, "mlp": mlp})
        cfg = cls(model_type="niduvik", architectures=["Niduvik"], vocab_size=_require(raw, "vocab", int, "vocabulary"),
                  max_position_embeddings=int(raw.get("max_position_embeddings") or cls.NO_CONTEXT_LIMIT),
                  eos_token_id=raw.get("eos_token_id"), width=_require(raw, "width", int, "model width"),
                  norm_eps=_require(norm, "eps", float, "norm epsilon"), layers=read)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.width <= 0 or self.max_position_embeddings <= 0:
            raise InvalidRequest("invalid Niduvik dimensions: every size must be a positive integer")
        if not math.isfinite(self.norm_eps) or self.norm_eps <= 0:
            raise InvalidRequest("invalid normalization parameters")
        for i, layer in enumerate(self.layers):
            m = layer["mixer"]
            for key, want in self.MIXER_KEYS[layer["type"]].items():
                if want is int and m[key] <= 0:
                    raise InvalidRequest(f"layers[{i}].mixer.{key} must be positive")
            if layer["type"] == "attention":
                if m["heads"] % m["kv_heads"]:
                    raise InvalidRequest(f"layers[{i}]: heads must be a multiple of kv_heads")
                if m["mask"]["size"] <= 0 or m["mask"]["keep_first"] < 0 or m["softcap"] <= 0 or m["scale"] <= 0:
                    raise InvalidRequest(f"layers[{i}]: window, kept tokens, soft cap or scale out of range")
            else:
                if m["heads"] % m["groups"] or (m["heads"] * m["vdim"]) % m["norm_groups"]:
                    raise InvalidRequest(f"layers[{i}]: heads must be a multiple of groups, heads * vdim of norm_groups")
            mlp = layer["mlp"]
            if mlp is not None and (mlp["kind"] != "dense" or mlp["ff"] <= 0 or mlp["limit"] <= 0):
                raise InvalidRequest(f"layers[{i}].mlp: only kind `dense` with positive `ff` and `limit` is built")
        if self.eos_token_id is not None:
            self.eos_ids()

    def eos_ids(self, folder: str | None = None) -> list[int]:
        if self.eos_token_id is None and (folder is None or not os.path.exists(os.path.join(folder, "generation_config.json"))):
            return []                # the design names no end-of-sequence token: generation ends by length
        return super().eos_ids(folder)

    def to_dict(self) -> dict:
        out = {"architecture": "Niduvik", "vocab": self.vocab_size, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": self.layers}
        if self.max_position_embeddings != self.NO_CONTEXT_LIMIT:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_id is not None:
            out["eos_token_id"] = self.eos_token_id
        return out


@dataclass
class SatedraConfig(ModelConfig):
    """Satedra: a decoder of pre-norm layers (layer norms with bias) that each hold a latent attention (keys and values
    made from one small latent a token, which is what the cache keeps; part of every head rotated with stretched rotary
    positions; a sliding window; gated heads; a layer may read the cache of an earlier one) and, optionally, a
    feed-forward: a dense gated unit, or routed experts with identity experts, a corrected choice and a gated shared
    expert.  The logits are scaled by a constant.  config.json names the design under `architecture`; its keys are read
    as they stand there:

      vocab, width, norm.eps, logit_scale
      layers[i].type = "latent_attention"
      layers[i].mixer.{heads, dim, rot_dim, vdim, kv_rank, scale, mask.size, rot.{base, dims, scaling.{factor, original, fast, slow}}, kv_from}
      layers[i].mlp = null | {kind: "dense", ff} | {kind: "moe", expert.ff, router.{experts, identity, top, scale}, shared.ff}

    `mask` (no window: every earlier key), `rot.scaling` (plain rotary positions), `kv_from`, `router.identity` and `shared`
    may be left out.  The design states no longest context and no end-of-sequence token; `max_position_embeddings` and
    `eos_token_id` are read if a file has them."""

    width: int = 0
    norm_eps: float = 0.0
    logit_scale: float = 1.0
    layers: list = None

    MODEL_TYPES: ClassVar[tuple[str, ...]] = ("satedra",)
    NO_CONTEXT_LIMIT: ClassVar[int] = 1 << 22

    @classmethod
    def _mixer(cls, i: int, mixer: dict) -> dict:
        where = f"layers[{i}].mixer"
        out = {key: _require(mixer, key, int, where) for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank")}
        out["scale"] = _require(mixer, "scale", float, where)
        mask = mixer.get("mask")
        if mask is not None:
            if not isinstance(mask, dict):
                raise InvalidRequest(f"config.json: {where}.mask must be an object")
            out["mask"] = {"size": _require(mask, "size", int, "window")}
        rot = mixer.get("rot")
        if not isinstance(rot, dict):
            raise InvalidRequest(f"config.json: {where}.rot must be an object")
        out["rot"] = {"base": _require(rot, "base", float, "rotary base"), "dims": _require(rot, "dims", int, "rotated elements")}
        scaling = rot.get("scaling")
        if scaling is not None:
            if not isinstance(scaling, dict):
                raise InvalidRequest(f"config.json: {where}.rot.scaling must be an object")
            out["rot"]["scaling"] = {key: _require(scaling, key, float, f"{where}.rot.scaling") for key in ("factor", "original", "fast", "slow")}
        if mixer.get("kv_from") is not None:
            out["kv_from"] = _require(mixer, "kv_from", int, "the layer whose cache is read")
        return out

    @classmethod
    def _mlp(cls, i: int, mlp) -> dict | None:
        if mlp is None:
            return None
        where = f"layers[{i}].mlp"
        if not isinstance(mlp, dict):
            raise InvalidRequest(f"config.json: {where} must be null or an object")
        kind = _require(mlp, "kind", str, "feed-forward kind")
        if kind == "dense":
            return {"kind": kind, "ff": _require(mlp, "ff", int, "feed-forward width")}
        if kind != "moe":
            raise InvalidRequest(f"config.json: {where}.kind {kind!r}; known: dense, moe")
        expert, router = mlp.get("expert"), mlp.get("router")
        if not isinstance(expert, dict) or not isinstance(router, dict):
            raise InvalidRequest(f"config.json: {where} needs the objects `expert` and `router`")
        out = {"kind": kind, "expert": {"ff": _require(expert, "ff", int, "expert width")},
               "router": {"experts": _require(router, "experts", int, "experts"), "top": _require(router, "top", int, "choices"),
                          "scale": _require(router, "scale", float, "weight scale"),
                          "identity": _require(router, "identity", int, "identity experts") if router.get("identity") is not None else 0}}
        shared = mlp.get("shared")
        if shared is not None:
            if not isinstance(shared, dict):
                raise InvalidRequest(f"config.json: {where}.shared must be an object")
            out["shared"] = {"ff": _require(shared, "ff", int, "shared expert width")}
        return out

    @classmethod
    def from_dict(cls, raw: dict) -> "SatedraConfig":
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise InvalidRequest("config.json: missing key `norm` (an object with `eps`)")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise InvalidRequest("config.json: `layers` must be a list of layers")
        read = []
        for i, layer in enumerate(layers):
            if not isinstance(layer, dict):
                raise InvalidRequest(f"config.json: layers[{i}] must be an object")
            kind = _require(layer, "type", str, f"mixer of layer {i}")
            if kind != "latent_attention":
                raise InvalidRequest(f"config.json: layers[{i}].type {kind!r}; known: latent_attention")
            if not isinstance(layer.get("mixer"), dict):
                raise InvalidRequest(f"config.json: layers[{i}].mixer must be an object")
            read.append({"type": kind, "mixer": cls._mixer(i, layer["mixer"]), "mlp": cls._mlp(i, layer.get("mlp"))})
        cfg = cls(model_type="satedra", architectures=["Satedra"], vocab_size=_require(raw, "vocab", int, "vocabulary"),
                  max_position_embeddings=int(raw.get("max_position_embeddings") or cls.NO_CONTEXT_LIMIT),
                  eos_token_id=raw.get("eos_token_id"), width=_require(raw, "width", int, "model width"),
                  norm_eps=_require(norm, "eps", float, "norm epsilon"),
                  logit_scale=_require(raw, "logit_scale", float, "logit scale") if raw.get("logit_scale") is not None else 1.0,
                  layers=read)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.width <= 0 or self.max_position_embeddings <= 0:
            raise InvalidRequest("invalid Satedra dimensions: every size must be a positive integer")
        if not math.isfinite(self.norm_eps) or self.norm_eps <= 0 or not math.isfinite(self.logit_scale):
            raise InvalidRequest("invalid normalization parameters or logit scale")
        for i, layer in enumerate(self.layers):
            m = layer["mixer"]
            if min(m["heads"], m["dim"], m["vdim"], m["kv_rank"]) <= 0 or m["rot_dim"] < 0 or m["scale"] <= 0:
                raise InvalidRequest(f"layers[{i}].mixer: sizes and scale must be positive")
            if "mask" in m and m["mask"]["size"] <= 0:
                raise InvalidRequest(f"layers[{i}].mixer.mask.size must be positive")
            rot = m["rot"]
            if rot["dims"] < 0 or rot["dims"] % 2 or rot["dims"] > m["rot_dim"] or rot["base"] <= 1:
                raise InvalidRequest(f"layers[{i}].mixer.rot: an even number of elements, at most rot_dim, and a base above 1")
            if "scaling" in rot and min(rot["scaling"].values()) <= 0:
                raise InvalidRequest(f"layers[{i}].mixer.rot.scaling: every number must be positive")
            if "kv_from" in m:
                j = m["kv_from"]
                if not 0 <= j < i or "kv_from" in self.layers[j]["mixer"]:
                    raise InvalidRequest(f"layers[{i}].mixer.kv_from must name an earlier layer that keeps a cache of its own")
                other = self.layers[j]["mixer"]
                if (other["kv_rank"], other["rot_dim"], other["rot"]) != (m["kv_rank"], m["rot_dim"], m["rot"]):
                    raise InvalidRequest(f"layers[{i}]: the layer whose cache is read must have the same latent, rotated part and rotation")
            mlp = layer["mlp"]
            if mlp is None:
                continue
            if mlp["kind"] == "dense":
                if mlp["ff"] <= 0:
                    raise InvalidRequest(f"layers[{i}].mlp.ff must be positive")
                continue
            r = mlp["router"]
            if r["experts"] < 0 or r["identity"] < 0 or not 0 < r["top"] <= r["experts"] + r["identity"] or mlp["expert"]["ff"] <= 0:
                raise InvalidRequest(f"layers[{i}].mlp: experts, identity experts and choices out of range")
            if "shared" in mlp and mlp["shared"]["ff"] <= 0:
                raise InvalidRequest(f"layers[{i}].mlp.shared.ff must be positive")
        if self.eos_token_id is not None:
            self.eos_ids()

    def eos_ids(self, folder: str | None = None) -> list[int]:
        if self.eos_token_id is None and (folder is None or not os.path.exists(os.path.join(folder, "generation_config.json"))):
            return []                # the design names no end-of-sequence token: generation ends by length
        return super().eos_ids(folder)

    def to_dict(self) -> dict:
        out = {"architecture": "Satedra", "vocab": self.vocab_size, "width": self.width, "norm": {"eps": self.norm_eps},
               "logit_scale": self.logit_scale, "layers": self.layers}
        if self.max_position_embeddings != self.NO_CONTEXT_LIMIT:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_id is not None:
            out["eos_token_id"] = self.eos_token_id
        return out


@dataclass
class NubipelConfig(ModelConfig):
    """Nubipel: a decoder of layers whose two branches, a mixer and a dense feed-forward, read one RMS norm's output side by
    side.  The mixer is an attention without rotation (query and key heads normed, sight in chunks of positions, a learned
    sink a head in the softmax), a latent attention without rotation (queries through a latent of their own, keys and values
    from one cached latent, every value element gated) or a gated delta rule (short convolutions, unit-length queries and
    keys, a matrix state a head).  Embeddings are scaled, the output head reads the embedding table, and the logits are
    scaled and bent by a tanh.  config.json names the design under `architecture`; its keys are read as they stand there:

      vocab, width, norm.eps, embedding.scale, logit_scale, logit_softcap
      layers[i].type = "attention":        mixer.{heads, kv_heads, dim, vdim, scale, mask.size}
      layers[i].type = "latent_attention": mixer.{heads, dim, vdim, kv_rank, q_rank, scale}
      layers[i].type = "delta":            mixer.{heads, kv_heads, dim, vdim, conv}
      layers[i].mlp = null | {kind: "dense", ff}

    `embedding.scale`, `logit_scale` (1), `logit_softcap` (none) and an attention's `mask` (every earlier key) may be left
    out.  The design states no longest context and no end-of-sequence token; `max_position_embeddings` and `eos_token_id`
    are read if a file has them."""

    width: int = 0
    norm_eps: float = 0.0
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    logit_softcap: float = 0.0
    layers: list = None

    MODEL_TYPES: ClassVar[tuple[str, ...]] = ("nubipel",)
    NO_CONTEXT_LIMIT: ClassVar[int] = 1 << 22
    MIXER_KEYS: ClassVar[dict] = {
        "attention": {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "scale": float},
        "latent_attention": {"heads": int, "dim": int, "vdim": int, "kv_rank": int, "q_rank": int, "scale": float},
        "delta": {"heads": int, "kv_heads": int, "dim": int, "vdim": int, "conv": int},
    }

    @classmethod
    def from_dict(cls, raw: dict) -> "NubipelConfig":
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise InvalidRequest("config.json: missing key `norm` (an object with `eps`)")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise InvalidRequest("config.json: `layers` must be a list of layers")
        read = []
        for i, layer in enumerate(layers):
            if not isinstance(layer, dict):
                raise InvalidRequest(f"config.json: layers[{i}] must be an object")
            kind = _require(layer, "type", str, f"mixer of layer {i}")
            if kind not in cls.MIXER_KEYS:
                raise InvalidRequest(f"config.json: layers[{i}].type {kind!r}; known: {sorted(cls.MIXER_KEYS)}")
            mixer = layer.get("mixer")
            if not isinstance(mixer, dict):
                raise InvalidRequest(f"config.json: layers[{i}].mixer must be an object")
            sizes = {key: _require(mixer, key, want, f"layers[{i}].mixer") for key, want in cls.MIXER_KEYS[kind].items()}
            if kind == "attention" and mixer.get("mask") is not None:
                if not isinstance(mixer["mask"], dict):
                    raise InvalidRequest(f"config.json: layers[{i}].mixer.mask must be an object")
                sizes["mask"] = {"size": _require(mixer["mask"], "size", int, "chunk of positions")}
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict):
                    raise InvalidRequest(f"config.json: layers[{i}].mlp must be null or an object")
                mlp = {"kind": _require(mlp, "kind", str, "feed-forward kind"), "ff": _require(mlp, "ff", int, "feed-forward width")}
            read.append({"type": kind, "mixer": sizes, "mlp": mlp})
        embedding = raw.get("embedding")
        if embedding is not None and not isinstance(embedding, dict):
            raise InvalidRequest("config.json: `embedding` must be an object")
        cfg = cls(model_type="nubipel", architectures=["Nubipel"], vocab_size=_require(raw, "vocab", int, "vocabulary"),
                  max_position_embeddings=int(raw.get("max_position_embeddings") or cls.NO_CONTEXT_LIMIT),
                  eos_token_id=raw.get("eos_token_id"), width=_require(raw, "width", int, "model width"),
                  norm_eps=_require(norm, "eps", float, "norm epsilon"),
                  embedding_scale=_require(embedding, "scale", float, "embedding scale") if embedding and embedding.get("scale") is not None else 1.0,
                  logit_scale=_require(raw, "logit_scale", float, "logit scale") if raw.get("logit_scale") is not None else 1.0,
                  logit_softcap=_require(raw, "logit_softcap", float, "logit cap") if raw.get("logit_softcap") is not None else 0.0,
                  layers=read)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.width <= 0 or self.max_position_embeddings <= 0:
            raise InvalidRequest("invalid Nubipel dimensions: every size must be a positive integer")
        if not math.isfinite(self.norm_eps) or self.norm_eps <= 0:
            raise InvalidRequest("invalid normalization parameters")
        if not all(math.isfinite(v) for v in (self.embedding_scale, self.logit_scale, self.logit_softcap)) or self.logit_softcap < 0:
            raise InvalidRequest("embedding scale, logit scale and logit cap must be finite, the cap not negative")
        for i, layer in enumerate(self.layers):
            m = layer["mixer"]
            for key, want in self.MIXER_KEYS[layer["type"]].items():
                if m[key] <= 0 or not math.isfinite(m[key]):
                    raise InvalidRequest(f"layers[{i}].mixer.{key} must be positive")
            if "kv_heads" in m and m["heads"] % m["kv_heads"]:
                raise InvalidRequest(f"layers[{i}]: heads must be a multiple of kv_heads")
            if "mask" in m and m["mask"]["size"] <= 0:
                raise InvalidRequest(f"layers[{i}].mixer.mask.size must be positive")
            mlp = layer["mlp"]
            if mlp is not None and (mlp["kind"] != "dense" or mlp["ff"] <= 0):
                raise InvalidRequest(f"layers[{i}].mlp: only kind `dense` with a positive `ff` is built")
        if self.eos_token_id is not None:
            self.eos_ids()

    def eos_ids(self, folder: str | None = None) -> list[int]:
        if self.eos_token_id is None and (folder is None or not os.path.exists(os.path.join(folder, "generation_config.json"))):
            return []                # the design names no end-of-sequence token: generation ends by length
        return super().eos_ids(folder)

    def to_dict(self) -> dict:
        out = {"architecture": "Nubipel", "vocab": self.vocab_size, "width": self.width, "norm": {"eps": self.norm_eps},
               "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale, "layers": self.layers}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        if self.max_position_embeddings != self.NO_CONTEXT_LIMIT:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_id is not None:
            out["eos_token_id"] = self.eos_token_id
        return out


@dataclass
class MigenexConfig(ModelConfig):
    """Migenex: a decoder of layers with an RMS norm before and after each branch, whose branches join the stream times a
    constant.  The mixer is an attention with normed and then rotated heads and capped scores ("attention") or one whose
    values are its keys as projected, with heads rotated in interleaved pairs and then divided by their root mean square, a
    sliding window and a gate a value element ("attention_2").  The feed-forward is a gated unit with a relu gate, or routed
    experts without a gate (the square of relu) whose sigmoid scores multiply what they read, beside a shared expert.  The
    embedding adds a row of a table of token pairs; a run of layers may be passed several times with the same weights, every
    pass opened by a product over the stream and the embedding.  config.json gives `vocab`, `width`, `norm.eps`,
    `residual_mult`, `embedding.{scale, bigram.{buckets, mul_prev, mul_cur}}`, `loop.{start, stop, times}` and, layer by
    layer, `layers[i].{type, mixer, mlp}`; what may be absent: the table of pairs, the loop, a layer's mask, cap and
    feed-forward, the shared expert."""

    width: int = 0
    norm_eps: float = 0.0
    residual_mult: float = 1.0
    embedding_scale: float = 1.0
    bigram: dict | None = None
    loop: dict | None = None
    layers: list = None

    MODEL_TYPES: ClassVar[tuple[str, ...]] = ("migenex",)
    NO_CONTEXT_LIMIT: ClassVar[int] = 1 << 22
    MIXERS: ClassVar[tuple[str, ...]] = ("attention", "attention_2")

    @classmethod
    def _mixer(cls, i: int, mixer: dict) -> dict:
        where = f"layers[{i}].mixer"
        out = {key: _require(mixer, key, int, where) for key in ("heads", "kv_heads", "dim", "vdim")}
        out["scale"] = _require(mixer, "scale", float, where)
        rot = mixer.get("rot")
        if not isinstance(rot, dict):
            raise InvalidRequest(f"config.json: {where}.rot must be an object")
        out["rot"] = {"base": _require(rot, "base", float, "rotary base"), "dims": _require(rot, "dims", int, "rotated elements")}
        mask = mixer.get("mask")
        if mask is not None:
            if not isinstance(mask, dict):
                raise InvalidRequest(f"config.json: {where}.mask must be an object")
            out["mask"] = {"size": _require(mask, "size", int, "window")}
        if mixer.get("softcap") is not None:
            out["softcap"] = _require(mixer, "softcap", float, "soft cap of the scores")
        return out

    @classmethod
    def _mlp(cls, i: int, mlp) -> dict | None:
        if mlp is None:
            return None
        where = f"layers[{i}].mlp"
        if not isinstance(mlp, dict):
            raise InvalidRequest(f"config.json: {where} must be null or an object")
        kind = _require(mlp, "kind", str, "feed-forward kind")
        if kind == "dense":
            return {"kind": kind, "ff": _require(mlp, "ff", int, "feed-forward width")}
        if kind != "moe":
            raise InvalidRequest(f"config.json: {where}.kind {kind!r}; known: dense, moe")
        expert, router = mlp.get("expert"), mlp.get("router")
        if not isinstance(expert, dict) or not isinstance(router, dict):
            raise InvalidRequest(f"config.json: {where} needs the objects `expert` and `router`")
        out = {"kind": kind, "expert": {"ff": _require(expert, "ff", int, "expert width")},
               "router": {"experts": _require(router, "experts", int, "experts"), "top": _require(router, "top", int, "choices")}}
        shared = mlp.get("shared")
        if shared is not None:
            if not isinstance(shared, dict):
                raise InvalidRequest(f"config.json: {where}.shared must be an object")
            out["shared"] = {"ff": _require(shared, "ff", int, "shared expert width")}
        return out

    @classmethod
    def from_dict(cls, raw: dict) -> "MigenexConfig":
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise InvalidRequest("config.json: missing key `norm` (an object with `eps`)")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise InvalidRequest("config.json: `layers` must be a list of layers")
        read = []
        for i, layer in enumerate(layers):
            if not isinstance(layer, dict):
                raise InvalidRequest(f"config.json: layers[{i}] must be an object")
            kind = _require(layer, "type", str, f"mixer of layer {i}")
            if kind not in cls.MIXERS:
                raise InvalidRequest(f"config.json: layers[{i}].type {kind!r}; known: {', '.join(cls.MIXERS)}")
            if not isinstance(layer.get("mixer"), dict):
                raise InvalidRequest(f"config.json: layers[{i}].mixer must be an object")
            read.append({"type": kind, "mixer": cls._mixer(i, layer["mixer"]), "mlp": cls._mlp(i, layer.get("mlp"))})
        embedding = raw.get("embedding") or {}
        if not isinstance(embedding, dict):
            raise InvalidRequest("config.json: `embedding` must be an object")
        bigram = embedding.get("bigram")
        if bigram is not None:
            if not isinstance(bigram, dict):
                raise InvalidRequest("config.json: `embedding.bigram` must be an object")
            bigram = {key: _require(bigram, key, int, "embedding.bigram") for key in ("buckets", "mul_prev", "mul_cur")}
        loop = raw.get("loop")
        if loop is not None:
            if not isinstance(loop, dict):
                raise InvalidRequest("config.json: `loop` must be an object")
            loop = {key: _require(loop, key, int, "loop") for key in ("start", "stop", "times")}
        cfg = cls(model_type="migenex", architectures=["Migenex"], vocab_size=_require(raw, "vocab", int, "vocabulary"),
                  max_position_embeddings=int(raw.get("max_position_embeddings") or cls.NO_CONTEXT_LIMIT),
                  eos_token_id=raw.get("eos_token_id"), width=_require(raw, "width", int, "model width"),
                  norm_eps=_require(norm, "eps", float, "norm epsilon"),
                  residual_mult=_require(raw, "residual_mult", float, "branch multiplier") if raw.get("residual_mult") is not None else 1.0,
                  embedding_scale=_require(embedding, "scale", float, "embedding scale") if embedding.get("scale") is not None else 1.0,
                  bigram=bigram, loop=loop, layers=read)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.width <= 0 or self.max_position_embeddings <= 0:
            raise InvalidRequest("invalid Migenex dimensions: every size must be a positive integer")
        if not math.isfinite(self.norm_eps) or self.norm_eps <= 0 or not math.isfinite(self.residual_mult) \
                or not math.isfinite(self.embedding_scale):
            raise InvalidRequest("invalid normalization parameters, branch multiplier or embedding scale")
        if self.bigram is not None and (self.bigram["buckets"] <= 0 or self.bigram["mul_prev"] < 0 or self.bigram["mul_cur"] < 0):
            raise InvalidRequest("embedding.bigram: a positive number of buckets and multipliers that are not negative")
        if self.loop is not None:
            lo, hi, times = self.loop["start"], self.loop["stop"], self.loop["times"]
            if not 0 <= lo < hi <= len(self.layers) or times < 1:
                raise InvalidRequest("loop: start < stop within the layers, and at least one pass")
        for i, layer in enumerate(self.layers):
            m = layer["mixer"]
            if min(m["heads"], m["kv_heads"], m["dim"], m["vdim"]) <= 0 or m["heads"] % m["kv_heads"] or not m["scale"] > 0:
                raise InvalidRequest(f"layers[{i}].mixer: sizes and scale must be positive, query heads a multiple of key/value heads")
            if m["dim"] > 256 or m["vdim"] > 256:
                raise InvalidRequest(f"layers[{i}].mixer: heads have at most 256 elements")
            if layer["type"] == "attention_2" and m["vdim"] != m["dim"]:
                raise InvalidRequest(f"layers[{i}].mixer: values that are the keys have the keys' size (vdim = dim)")
            if "mask" in m and m["mask"]["size"] <= 0:
                raise InvalidRequest(f"layers[{i}].mixer.mask.size must be positive")
            if "softcap" in m and not m["softcap"] > 0:
                raise InvalidRequest(f"layers[{i}].mixer.softcap must be positive")
            rot = m["rot"]
            if rot["dims"] < 0 or rot["dims"] % 2 or rot["dims"] > m["dim"] or not rot["base"] > 0:
                raise InvalidRequest(f"layers[{i}].mixer.rot: an even number of elements, at most dim, and a positive base")
            mlp = layer["mlp"]
            if mlp is None:
                continue
            if mlp["kind"] == "dense":
                if mlp["ff"] <= 0:
                    raise InvalidRequest(f"layers[{i}].mlp.ff must be positive")
                continue
            r = mlp["router"]
            if not 0 < r["top"] <= r["experts"] or mlp["expert"]["ff"] <= 0:
                raise InvalidRequest(f"layers[{i}].mlp: experts and choices out of range")
            if "shared" in mlp and mlp["shared"]["ff"] <= 0:
                raise InvalidRequest(f"layers[{i}].mlp.shared.ff must be positive")
        if self.eos_token_id is not None:
            self.eos_ids()

    def eos_ids(self, folder: str | None = None) -> list[int]:
        if self.eos_token_id is None and (folder is None or not os.path.exists(os.path.join(folder, "generation_config.json"))):
            return []                # the design names no end-of-sequence token: generation ends by length
        return super().eos_ids(folder)

    def to_dict(self) -> dict:
        embedding = {"scale": self.embedding_scale}
        if self.bigram is not None:
            embedding["bigram"] = self.bigram
        out = {"architecture": "Migenex", "vocab": self.vocab_size, "width": self.width, "norm": {"eps": self.norm_eps},
               "residual_mult": self.residual_mult, "embedding": embedding, "layers": self.layers}
        if self.loop is not None:
            out["loop"] = self.loop
        if self.max_position_embeddings != self.NO_CONTEXT_LIMIT:
            out["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_id is not None:
            out["eos_token_id"] = self.eos_token_id
        return out
