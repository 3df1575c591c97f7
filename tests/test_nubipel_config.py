"""Nubipel without a GPU: the configuration reader and its checks, the model's spec (tensor names and shapes, which
layer keeps which kind of cache or state), and the plain implementation against independent restatements of its own
mechanisms (the delta rule as a sum over earlier tokens, the sink as one more key without a value, the chunks as
separate sequences, the convolution against the library's)."""
import copy
import json
import math

import pytest
import torch

import plain_nubipel as P
from mini_rsglang_b200.errors import InvalidRequest
from mini_rsglang_b200.models import config_from_dict, model_spec_for


def attention(heads=6, kv_heads=2, dim=24, vdim=20, scale=0.2, size=19):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size:
        mixer["mask"] = {"size": size}
    return {"type": "attention", "mixer": mixer}


def latent(heads=3, dim=12, vdim=20, kv_rank=40, q_rank=28, scale=0.3):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale}}


def delta(heads=4, kv_heads=2, dim=24, vdim=12, conv=3):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


RAW = {"architecture": "Nubipel", "vocab": 211, "width": 72, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0}, "logit_scale": 0.7,
       "logit_softcap": 9.0, "layers": [
           dict(latent(), mlp={"kind": "dense", "ff": 100}),
           dict(delta(), mlp=None),
           dict(attention(), mlp={"kind": "dense", "ff": 52}),
           dict(attention(size=0, heads=2, kv_heads=2), mlp=None)]}


def test_reads_every_key_and_writes_them_back():
    config = config_from_dict(copy.deepcopy(RAW))
    assert config.model_type == "nubipel" and config.vocab_size == 211 and config.width == 72
    assert config.embedding_scale == 3.0 and config.logit_scale == 0.7 and config.logit_softcap == 9.0 and config.norm_eps == 1e-5
    assert config.layers[1]["mlp"] is None and config.layers[2]["mixer"]["mask"]["size"] == 19 and "mask" not in config.layers[3]["mixer"]
    assert config.layers[0]["mixer"]["q_rank"] == 28 and config.layers[1]["mixer"]["conv"] == 3
    assert config.eos_ids() == []
    again = config_from_dict(json.loads(json.dumps(config.to_dict())))
    assert again.to_dict() == config.to_dict()


def test_constants_that_may_be_left_out():
    raw = copy.deepcopy(RAW)
    del raw["embedding"], raw["logit_scale"], raw["logit_softcap"]
    config = config_from_dict(raw)
    assert config.embedding_scale == 1.0 and config.logit_scale == 1.0 and config.logit_softcap == 0.0
    head = model_spec_for(config).head.params
    assert head["softcap"] == 0.0 and head["scale"] == 1.0


@pytest.mark.parametrize("path,value", [
    (("layers", 2, "mixer", "kv_heads"), 4), (("layers", 1, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "q_rank"), 0),
    (("layers", 0, "mlp", "kind"), "moe"), (("layers", 0, "type"), "recurrent"), (("layers", 2, "mixer", "mask", "size"), 0),
    (("norm", "eps"), 0.0), (("layers", 0, "mixer", "heads"), 0), (("layers", 0, "mlp", "ff"), 0), (("layers", 1, "mixer", "conv"), 0),
    (("logit_softcap",), -1.0), (("vocab",), 0), (("layers", 2, "mixer", "scale"), "big")])
def test_refuses_what_does_not_fit(path, value):
    raw = copy.deepcopy(RAW)
    at = raw
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(InvalidRequest):
        config_from_dict(raw)


@pytest.mark.parametrize("missing", [("norm",), ("layers",), ("width",), ("layers", 0, "mixer", "kv_rank"), ("layers", 1, "mixer", "conv"),
                                     ("layers", 2, "mixer", "scale"), ("layers", 2, "type")])
def test_names_the_key_that_is_missing(missing):
    raw = copy.deepcopy(RAW)
    at = raw
    for key in missing[:-1]:
        at = at[key]
    del at[missing[-1]]
    with pytest.raises(InvalidRequest, match=str(missing[-1])):
        config_from_dict(raw)


def test_spec_names_shapes_and_what_each_layer_keeps():
    spec = model_spec_for(config_from_dict(copy.deepcopy(RAW)))
    names = {s.name: tuple(s.shape) for s in spec.weight_specs()}
    assert names["embed"] == (211, 72) and names["final.norm"] == (72,) and "head" not in names and "head.weight" not in names
    assert names["l0.norm1"] == (72,) and "l0.norm2" not in names
    assert names["l0.mix.dq"] == (28, 72) and names["l0.mix.dq.norm"] == (28,) and names["l0.mix.uq"] == (36, 28)
    assert names["l0.mix.dkv"] == (40, 72) and names["l0.mix.dkv.norm"] == (40,) and names["l0.mix.uk"] == (36, 40)
    assert names["l0.mix.uv"] == (60, 40) and names["l0.mix.g"] == (60, 72) and names["l0.mix.o"] == (72, 60)
    assert names["l0.mlp.up"] == (100, 72) and names["l0.mlp.down"] == (72, 100) and "l1.mlp.up" not in names
    assert names["l1.mix.q"] == (48, 72) and names["l1.mix.k.conv"] == (48, 3) and names["l1.mix.v"] == (48, 72) and names["l1.mix.v.conv"] == (48, 3)
    assert names["l1.mix.b"] == (4, 72) and names["l1.mix.a"] == (4, 72) and names["l1.mix.A_log"] == (4,) and names["l1.mix.dt_bias"] == (4,)
    assert names["l1.mix.norm"] == (12,) and names["l1.mix.g"] == (48, 72) and names["l1.mix.o"] == (72, 48)
    assert names["l2.mix.q"] == (144, 72) and names["l2.mix.k"] == (48, 72) and names["l2.mix.v"] == (40, 72) and names["l2.mix.o"] == (72, 120)
    assert names["l2.mix.q.norm"] == (24,) and names["l2.mix.k.norm"] == (24,) and names["l2.mix.sink"] == (6,)
    assert len(names) == sum(1 for _ in spec.weight_specs())            # no name twice
    assert [layer.block for layer in spec.layers] == ["parallel"] * 4
    mixers = [layer.parts["mixer"] for layer in spec.layers]
    assert [m.kind for m in mixers] == ["latent_attention", "gated_delta_rule", "biased_window_attention", "biased_window_attention"]
    assert mixers[2].params["chunk"] == 19 and mixers[3].params["chunk"] == 0 and mixers[2].params["sink_logits"]
    assert mixers[1].params["unit_eps"] == 1e-6 and spec.layers[0].parts["feed_forward"].params["activation"] == "gelu_erf"
    assert "feed_forward" not in spec.layers[1].parts


def test_needs_of_cache_and_state():
    """The chunked attention keeps a window of one chunk, the one without a mask and the latent attention every key (the latter one
    row a token for all heads), the delta rule a float32 state of the convolutions' last inputs and a matrix a head."""
    from mini_rsglang_b200.parts.base import MIXERS

    spec = model_spec_for(config_from_dict(copy.deepcopy(RAW)))
    parts = [MIXERS.build(layer.parts["mixer"], f"l{i}.mix") for i, layer in enumerate(spec.layers)]
    need = parts[0].cache_need()
    assert (need.kind, need.kv_heads, need.head_dim, need.values) == ("full", 1, 40, False) and parts[0].state_need() is None
    state = parts[1].state_need()
    assert parts[1].cache_need() is None and state.dtype is torch.float32
    assert tuple(state.shape) == ((3 - 1) * (2 * 2 * 24 + 4 * 12) + 4 * 24 * 12,)
    need = parts[2].cache_need()
    assert (need.kind, need.window, need.kv_heads, need.head_dim, need.value_dim) == ("window", 19, 2, 24, 20)
    assert parts[3].cache_need().kind == "full"


# ----------------------------------------------------------------------------------------------------------------
# the plain implementation against restatements of its own mechanisms
# ----------------------------------------------------------------------------------------------------------------
def test_delta_recurrence_is_a_corrected_sum_over_earlier_tokens():
    """With the decay 1 and beta 1 and orthonormal keys the state holds every value under its key, and a query equal to
    key j reads value j; with a repeated key the later value replaces the earlier one; a decay g scales what older
    tokens wrote by the product of the decays since."""
    torch.manual_seed(1)
    d, e, T = 8, 5, 6
    keys = torch.linalg.qr(torch.randn(d, d).double())[0][:T]
    v = torch.randn(T, e).double()
    ones = torch.ones(T).double()
    o, S = P.delta_recurrence(keys, keys, v, ones, ones)
    assert (o - v).abs().max() < 1e-12                              # the read-out sees the token's own write
    assert (S.T @ keys[2] - v[2]).abs().max() < 1e-12
    keys2 = keys.clone()
    keys2[4] = keys[1]
    _, S = P.delta_recurrence(keys2, keys2, v, ones, ones)
    assert (S.T @ keys[1] - v[4]).abs().max() < 1e-12               # corrected towards the later value
    decay = torch.rand(T).double() * 0.5 + 0.4
    _, S = P.delta_recurrence(keys, keys, v, ones, decay)
    assert (S.T @ keys[1] - v[1] * decay[2:].prod()).abs().max() < 1e-12
    half = 0.5 * ones
    _, S = P.delta_recurrence(keys, keys, v, half, ones)
    assert (S.T @ keys[3] - 0.5 * v[3]).abs().max() < 1e-12
    # carried state: two halves give what the whole gives
    q = torch.randn(T, d).double()
    whole, S_whole = P.delta_recurrence(q, keys2, v, half, decay)
    first, S_mid = P.delta_recurrence(q[:3], keys2[:3], v[:3], half[:3], decay[:3])
    second, S_end = P.delta_recurrence(q[3:], keys2[3:], v[3:], half[3:], decay[3:], S_mid)
    assert (torch.cat([first, second]) - whole).abs().max() < 1e-12 and (S_end - S_whole).abs().max() < 1e-12


def test_sink_is_a_key_of_its_own_logit_without_a_value():
    torch.manual_seed(2)
    T = 9
    scores = torch.randn(T, T).double() * 2
    seen = P.chunk_mask(T, 4)
    sink = torch.tensor(0.8, dtype=torch.float64)
    got = P.softmax_with_sink(scores, seen, sink)
    wide = torch.cat([torch.where(seen, scores, torch.tensor(-math.inf, dtype=torch.float64)), sink.expand(T, 1)], dim=1)
    assert (got - torch.softmax(wide, dim=-1)[:, :T]).abs().max() < 1e-14
    assert (got.sum(dim=-1) < 1.0).all() and (got[~seen] == 0).all()
    assert (P.softmax_with_sink(scores, seen, None).sum(dim=-1) - 1.0).abs().max() < 1e-14
    far = P.softmax_with_sink(scores, seen, torch.tensor(40.0, dtype=torch.float64))       # a sink that outweighs every key
    assert far.max() < 1e-12


def test_chunks_are_sequences_of_their_own_for_the_attention():
    """Cutting the input at the chunk borders and attending within each piece gives the whole sequence's output."""
    torch.manual_seed(3)
    c = attention(heads=4, kv_heads=2, dim=6, vdim=5, size=7)["mixer"]
    W, T = 10, 23
    w = {"m.q": torch.randn(24, W).double(), "m.k": torch.randn(12, W).double(), "m.v": torch.randn(10, W).double(),
         "m.q.norm": torch.rand(6).double() + 0.5, "m.k.norm": torch.rand(6).double() + 0.5, "m.sink": torch.randn(4).double(),
         "m.o": torch.randn(W, 20).double()}
    h = torch.randn(T, W).double()
    whole = P.chunked_attention(h, w, "m.", c, 1e-5)
    no_mask = dict(c)
    del no_mask["mask"]
    pieces = torch.cat([P.chunked_attention(h[s:s + 7], w, "m.", no_mask, 1e-5) for s in range(0, T, 7)])
    assert (whole - pieces).abs().max() < 1e-12
    assert (P.chunked_attention(h, w, "m.", no_mask, 1e-5)[7:] - whole[7:]).abs().max() > 1e-3        # and the mask matters


def test_convolution_is_the_library_one_with_zeros_before_the_start():
    torch.manual_seed(4)
    T, channels, taps = 11, 6, 4
    x, weight = torch.randn(T, channels).double(), torch.randn(channels, taps).double()
    lib = torch.nn.functional.conv1d(x.T[None], weight[:, None, :], padding=taps - 1, groups=channels)[0, :, :T].T
    assert (P.causal_conv_silu(x, weight) - P.silu(lib)).abs().max() < 1e-13
    assert (P.causal_conv_silu(x, weight)[0] - P.silu(x[0] * weight[:, -1])).abs().max() < 1e-13       # the last tap is the current token's


def test_gelu_is_the_exact_one():
    z = torch.linspace(-6, 6, 101).double()
    assert (P.gelu_erf(z) - torch.nn.functional.gelu(z)).abs().max() < 1e-15
    assert (P.gelu_erf(z) - torch.nn.functional.gelu(z, approximate="tanh")).abs().max() > 1e-4
