"""Nubipel as a composition of parts: every layer is a "parallel" block (one RMS norm whose output both branches read)
around one mixer, "biased_window_attention" (normed heads, sight in chunks, learned sinks), "latent_attention" (queries
through a latent, every value element gated) or "gated_delta_rule", and, where the layer has one, a "dense_mlp"
feed-forward; the embedding is scaled, the output head reads the embedding table, scales and caps its logits.  Sizes and
constants come from the configuration, layer by layer; the tensor names are the checkpoint's: `embed`, `final.norm`, and
below `l<i>.` the norm `norm1` (the tensor is the norm's root), `mix.*` and `mlp.*`.

What the design fixes: the exact (error function) gelu in the feed-forward, 1e-6 inside the root of the unit norms of the
delta rule's queries and keys, the scores of every attention without rotation and without a bias."""
from __future__ import annotations

from ..config.model_config import NubipelConfig
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec

FEED_FORWARD_ACTIVATION = "gelu_erf"
DELTA_UNIT_EPS = 1e-6

ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "sink": "sink"}
LATENT_NAMES = {"q_down": "dq", "q_norm": "dq.norm", "q_up": "uq", "down": "dkv", "latent_norm": "dkv.norm", "up_k": "uk",
                "up_v": "uv", "gate": "g", "o": "o"}
DELTA_NAMES = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "b": "b", "a": "a",
               "a_log": "A_log", "dt_bias": "dt_bias", "norm": "norm", "gate": "g", "o": "o"}
MLP_NAMES = {"up": "up", "down": "down"}


def nubipel_spec(config: NubipelConfig) -> ModelSpec:
    c = config
    norm = PartSpec("rmsnorm", {"width": c.width, "eps": c.norm_eps, "leaf": ""})
    layers = []
    for i, layer in enumerate(c.layers):
        m = layer["mixer"]
        if layer["type"] == "attention":
            mixer = PartSpec("biased_window_attention", {
                "width": c.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
                "scale": m["scale"], "chunk": (m.get("mask") or {}).get("size", 0), "sink_logits": True,
                "head_norm_eps": c.norm_eps, "names": ATTENTION_NAMES})
        elif layer["type"] == "latent_attention":
            mixer = PartSpec("latent_attention", {
                "width": c.width, "num_heads": m["heads"], "head_dim": m["dim"], "rotary_head_dim": 0, "value_dim": m["vdim"],
                "latent_dim": m["kv_rank"], "query_latent_dim": m["q_rank"], "scale": m["scale"], "eps": c.norm_eps,
                "output_gate": "elements", "float32_out": True, "names": LATENT_NAMES})
        else:
            mixer = PartSpec("gated_delta_rule", {
                "width": c.width, "heads": m["heads"], "groups": m["kv_heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
                "conv": m["conv"], "eps": c.norm_eps, "unit_eps": DELTA_UNIT_EPS, "names": DELTA_NAMES})
        parts = {"norm1": norm, "mixer": mixer}
        names = {"norm1": "norm1", "mixer": "mix"}
        if layer["mlp"] is not None:
            parts["feed_forward"] = PartSpec("dense_mlp", {"width": c.width, "inner": layer["mlp"]["ff"],
                                                           "activation": FEED_FORWARD_ACTIVATION, "names": MLP_NAMES})
            names["feed_forward"] = "mlp"
        layers.append(LayerSpec(f"l{i}", "parallel", parts, names))
    table = {"vocab": c.vocab_size, "width": c.width}
    return ModelSpec(vocab_size=c.vocab_size, width=c.width,
                     embedding=PartSpec("token_embedding", dict(table, leaf="", scale=c.embedding_scale)), embedding_prefix="embed",
                     layers=layers, final_norm=norm, final_norm_prefix="final.norm",
                     head=PartSpec("linear_head", dict(table, tied_to="embed", scale=c.logit_scale, softcap=c.logit_softcap)),
                     head_prefix="head")
