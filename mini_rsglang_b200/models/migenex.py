"""Migenex as a composition of parts: every layer is a "sandwich_norm" block (an RMS norm before and after each branch,
the branches joining the stream times the configuration's multiplier) around a "biased_window_attention" in one of two
dresses and, where the layer has one, a "gated_mlp" or "routed_experts" feed-forward; the embedding is scaled and adds a
row of a table of token pairs; the layers of the loop appear in the run order once a pass, every pass with caches of its
own and opened by the "rejoin_embedding" stream entry; the output head has a matrix of its own.  Sizes and constants come
from the configuration, layer by layer; the tensor names are the checkpoint's: `embed`, `bigram`, `loop.in`, `final.norm`,
`head`, and below `l<i>.` the norms `norm1`, `norm1b`, `norm2`, `norm2b` (the tensor is the norm's root), `mix.*`, `mlp.*`.

What the design fixes: "attention" norms its heads with weights before it rotates split halves, and sees every earlier
position unless the layer states a mask; "attention_2" has no value projection, rotates interleaved pairs, then divides
the heads by their root mean square without weights, and gates every value element; the dense feed-forward's gate is a
relu, an expert is the square of a relu between two matrices, the router's scores are sigmoids that are not normalised and
multiply what the chosen experts read."""
from __future__ import annotations

from ..config.model_config import MigenexConfig
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec, RunEntry

DENSE_GATE = "relu"
EXPERT_ACTIVATION = "relu2"

ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "gate": "g"}
MLP_NAMES = {"gate": "gate", "up": "up", "down": "down"}
EXPERT_NAMES = {"router": "router", "expert": "e{}", "up": "up", "down": "down", "shared": "shared"}


def migenex_run_order(config: MigenexConfig) -> list[RunEntry]:
    """Layers before the loop, then the loop's layers once a pass (each pass enters through stream entry 0), then the rest."""
    n, loop = len(config.layers), config.loop
    if loop is None:
        return [RunEntry(i) for i in range(n)]
    order = [RunEntry(i) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        order += [RunEntry(i, enter=0 if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return order + [RunEntry(i) for i in range(loop["stop"], n)]


def migenex_spec(config: MigenexConfig) -> ModelSpec:
    c = config
    norm = PartSpec("rmsnorm", {"width": c.width, "eps": c.norm_eps, "leaf": ""})
    layers = []
    for i, layer in enumerate(c.layers):
        m = layer["mixer"]
        common = {"width": c.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
                  "scale": m["scale"], "softcap": m.get("softcap", 0.0), "window": (m.get("mask") or {}).get("size", 0),
                  "head_norm_eps": c.norm_eps, "names": ATTENTION_NAMES}
        position = {"head_dim": m["dim"], "theta": m["rot"]["base"], "rotary_dim": m["rot"]["dims"]}
        if layer["type"] == "attention":
            mixer = PartSpec("biased_window_attention", dict(common, position=PartSpec("rope", dict(position, pairing="split_half")),
                                                             head_norm_place="before_rotation"))
        else:
            mixer = PartSpec("biased_window_attention", dict(common, position=PartSpec("rope", dict(position, pairing="interleaved")),
                                                             head_norm_place="after_rotation", head_norm_weights=False,
                                                             values_from_keys=True, output_gate="elements"))
        parts = {"norm1": norm, "mixer": mixer, "norm1b": norm}
        names = {"norm1": "norm1", "mixer": "mix", "norm1b": "norm1b"}
        mlp = layer["mlp"]
        if mlp is not None:
            if mlp["kind"] == "dense":
                feed_forward = PartSpec("gated_mlp", {"width": c.width, "inner": mlp["ff"], "activation": DENSE_GATE, "names": MLP_NAMES})
            else:
                shared = None
                if "shared" in mlp:
                    shared = PartSpec("dense_mlp", {"width": c.width, "inner": mlp["shared"]["ff"], "activation": EXPERT_ACTIVATION,
                                                    "names": MLP_NAMES, "float32_out": False})
                feed_forward = PartSpec("routed_experts", {
                    "width": c.width, "experts": mlp["router"]["experts"], "top": mlp["router"]["top"], "inner": mlp["expert"]["ff"],
                    "score": "sigmoid", "normalize": False, "form": "plain", "activation": EXPERT_ACTIVATION, "weight_on": "input",
                    "float32_out": True, "shared": shared, "names": EXPERT_NAMES})
            parts.update(norm2=norm, norm2b=norm, feed_forward=feed_forward)
            names.update(norm2="norm2", norm2b="norm2b", feed_forward="mlp")
        layers.append(LayerSpec(f"l{i}", "sandwich_norm", parts, names, {"branch_scale": c.residual_mult}))
    table = {"vocab": c.vocab_size, "width": c.width}
    pairs = dict(c.bigram, table="bigram") if c.bigram is not None else None
    return ModelSpec(vocab_size=c.vocab_size, width=c.width,
                     embedding=PartSpec("token_embedding", dict(table, leaf="", scale=c.embedding_scale, pairs=pairs)),
                     embedding_prefix="embed", layers=layers, final_norm=norm, final_norm_prefix="final.norm",
                     head=PartSpec("linear_head", dict(table, leaf="")), head_prefix="head", run_order=migenex_run_order(c),
                     stream_entries=[(PartSpec("rejoin_embedding", {"width": c.width, "leaf": ""}), "loop.in")] if c.loop is not None else [])
