"""Migenex's configuration, model spec and run order (no GPU): the keys of config.json as the design has them, what may be
absent, what is refused, the checkpoint's tensor names and shapes, the layers of the loop once a pass."""
import copy

import pytest

from mini_rsglang_b200.errors import InvalidRequest
from mini_rsglang_b200.models import config_from_dict
from mini_rsglang_b200.models.migenex import migenex_run_order, migenex_spec
from mini_rsglang_b200.models.spec import ModelSpec, RunEntry
from mini_rsglang_b200.parts.base import PartSpec

RAW = {"architecture": "Migenex", "vocab": 211, "width": 72, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
       "embedding": {"scale": 3.0, "bigram": {"buckets": 53, "mul_prev": 7, "mul_cur": 3}},
       "loop": {"start": 1, "stop": 3, "times": 3}, "layers": [
           {"type": "attention_2", "mixer": {"heads": 6, "kv_heads": 2, "dim": 24, "vdim": 24, "scale": 0.2, "mask": {"size": 19},
                                             "rot": {"base": 100.0, "dims": 12}}, "mlp": {"kind": "dense", "ff": 100}},
           {"type": "attention", "mixer": {"heads": 3, "kv_heads": 1, "dim": 12, "vdim": 28, "scale": 0.3, "softcap": 5.0,
                                           "rot": {"base": 10000.0, "dims": 12}},
            "mlp": {"kind": "moe", "expert": {"ff": 20}, "router": {"experts": 5, "top": 2}, "shared": {"ff": 36}}},
           {"type": "attention_2", "mixer": {"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 8, "scale": 0.3, "rot": {"base": 50.0, "dims": 8}},
            "mlp": None},
           {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 40, "vdim": 20, "scale": 0.1, "mask": {"size": 33},
                                           "rot": {"base": 500.0, "dims": 20}},
            "mlp": {"kind": "moe", "expert": {"ff": 12}, "router": {"experts": 3, "top": 3}}}]}


def test_reads_the_file_and_writes_it_back():
    c = config_from_dict(RAW)
    assert c.model_type == "migenex" and c.vocab_size == 211 and c.width == 72 and c.residual_mult == 0.5
    assert c.embedding_scale == 3.0 and c.bigram == {"buckets": 53, "mul_prev": 7, "mul_cur": 3}
    assert c.loop == {"start": 1, "stop": 3, "times": 3} and c.eos_ids() == []
    assert c.layers[1]["mixer"]["softcap"] == 5.0 and "mask" not in c.layers[1]["mixer"] and c.layers[2]["mlp"] is None
    again = config_from_dict(c.to_dict())
    assert again.to_dict() == c.to_dict()


def test_what_a_file_may_leave_out():
    raw = copy.deepcopy(RAW)
    del raw["loop"], raw["residual_mult"], raw["embedding"]["bigram"]
    c = config_from_dict(raw)
    assert c.loop is None and c.bigram is None and c.residual_mult == 1.0
    spec = migenex_spec(c)
    assert [(e.layer, e.enter) for e in spec.run_order] == [(0, None), (1, None), (2, None), (3, None)]
    names = {w.name for w in spec.weight_specs()}
    assert "bigram" not in names and "loop.in" not in names and spec.stream_entries == []
    assert spec.build_parts()[0].state_need() is None


def test_the_loop_in_the_run_order():
    c = config_from_dict(RAW)
    assert [(e.layer, e.enter) for e in migenex_run_order(c)] == \
        [(0, None), (1, 0), (2, None), (1, 0), (2, None), (1, 0), (2, None), (3, None)]
    raw = copy.deepcopy(RAW)
    raw["loop"] = {"start": 0, "stop": 4, "times": 1}
    assert [(e.layer, e.enter) for e in migenex_run_order(config_from_dict(raw))] == [(0, 0), (1, None), (2, None), (3, None)]


def test_tensor_names_and_shapes():
    spec = migenex_spec(config_from_dict(RAW))
    shapes = {w.name: w.shape for w in spec.weight_specs()}
    assert shapes["embed"] == (211, 72) and shapes["bigram"] == (54, 72) and shapes["loop.in"] == (72, 144)
    assert shapes["head"] == (211, 72) and shapes["final.norm"] == (72,)
    assert shapes["l0.mix.q"] == (144, 72) and shapes["l0.mix.k"] == (48, 72) and shapes["l0.mix.g"] == (144, 72)
    assert shapes["l0.mix.o"] == (72, 144) and "l0.mix.v" not in shapes and "l0.mix.q.norm" not in shapes
    assert shapes["l1.mix.v"] == (28, 72) and shapes["l1.mix.o"] == (72, 84) and shapes["l1.mix.q.norm"] == (12,)
    assert "l1.mix.g" not in shapes
    assert shapes["l0.mlp.gate"] == (100, 72) and shapes["l0.mlp.down"] == (72, 100)
    assert shapes["l1.mlp.router"] == (5, 72) and shapes["l1.mlp.e4.up"] == (20, 72) and shapes["l1.mlp.e0.down"] == (72, 20)
    assert shapes["l1.mlp.shared.up"] == (36, 72) and "l1.mlp.e0.gate" not in shapes and "l3.mlp.shared.up" not in shapes
    assert not any(name.startswith("l2.mlp") or name.startswith("l2.norm2") for name in shapes)
    assert {f"l{i}.{n}" for i in (0, 1, 3) for n in ("norm1", "norm1b", "norm2", "norm2b")} <= set(shapes)
    embedding = spec.build_parts()[0]
    assert embedding.state_need().shape == ()


@pytest.mark.parametrize("change,message", [
    (lambda r: r["layers"][0].__setitem__("type", "attention_3"), "known: attention, attention_2"),
    (lambda r: r["layers"][0]["mixer"].__setitem__("vdim", 12), "vdim = dim"),
    (lambda r: r["layers"][1]["mixer"]["rot"].__setitem__("dims", 13), "even number"),
    (lambda r: r["layers"][1]["mixer"]["rot"].__setitem__("dims", 14), "at most dim"),
    (lambda r: r["layers"][0]["mixer"].__setitem__("kv_heads", 4), "multiple of key/value heads"),
    (lambda r: r["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "mask.size"),
    (lambda r: r["layers"][1]["mlp"]["router"].__setitem__("top", 6), "choices out of range"),
    (lambda r: r["loop"].__setitem__("stop", 5), "loop"),
    (lambda r: r["loop"].__setitem__("times", 0), "loop"),
    (lambda r: r["embedding"]["bigram"].__setitem__("buckets", 0), "buckets"),
    (lambda r: r["embedding"]["bigram"].pop("mul_cur"), "mul_cur"),
    (lambda r: r.pop("norm"), "norm"),
    (lambda r: r["layers"][1]["mlp"].__setitem__("kind", "sparse"), "known: dense, moe"),
])
def test_refused(change, message):
    raw = copy.deepcopy(RAW)
    change(raw)
    with pytest.raises(InvalidRequest, match=message):
        config_from_dict(raw)


def test_a_run_may_name_only_a_stream_entry_that_the_model_has():
    spec = migenex_spec(config_from_dict(RAW))
    with pytest.raises(InvalidRequest, match="stream entry"):
        ModelSpec(vocab_size=spec.vocab_size, width=spec.width, embedding=spec.embedding, embedding_prefix="embed", layers=spec.layers,
                  final_norm=spec.final_norm, final_norm_prefix="final.norm", head=spec.head, head_prefix="head",
                  run_order=[RunEntry(0, enter=1)], stream_entries=[(PartSpec("rejoin_embedding", {"width": 72, "leaf": ""}), "loop.in")])


def test_parts_refuse_what_is_not_built():
    from mini_rsglang_b200.parts.attention_biased import BiasedWindowAttention
    from mini_rsglang_b200.parts.experts import RoutedExperts

    rope = PartSpec("rope", {"head_dim": 16, "theta": 100.0})
    with pytest.raises(InvalidRequest, match="not built together"):
        BiasedWindowAttention("m", 64, 4, 2, 16, position=rope, projection_bias=True)
    with pytest.raises(InvalidRequest, match="keys' size"):
        BiasedWindowAttention("m", 64, 4, 2, 16, value_dim=32, values_from_keys=True)
    with pytest.raises(InvalidRequest, match="plain experts"):
        RoutedExperts("f", 64, 4, 2, 16, weight_on="input")
    with pytest.raises(InvalidRequest, match="identity"):
        RoutedExperts("f", 64, 4, 2, 16, identity=1, form="plain", activation="relu2", weight_on="input")
    with pytest.raises(InvalidRequest, match="split halves or interleaved"):
        from mini_rsglang_b200.parts.position import RotaryPosition
        RotaryPosition("p", 16, 100.0, rotary_dim=6, pairing="pairs")
