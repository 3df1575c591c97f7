"""Migenex on the GPU against the plain implementation (`plain_migenex.py`): every mechanism's kernel alone, then whole
models of several small shapes through `bin/trace_run` in every cutting (whole, a decoded tail, portions down to two
tokens, requests mixed in a pool so small that pages and state slots are used again), in float32 and bfloat16, and greedy
generation through the engine's entry point and scheduler.  Where random weights would hide a fault (a far key, a window's
edge, a page border, the token before a portion), inputs are made so that it shows.

Routing in whole models: in float32 the router chooses freely (the engine's float32 scores and the plain implementation's
float64 ones order the experts alike unless two scores agree to six digits).  In bfloat16 a rounded input may turn a close
call, which is no fault, so the bfloat16 models choose all of their experts: every token's own scores still weight what
every expert reads; free routing in bfloat16 is covered kernel by kernel."""
import copy
import functools
import json
import os
import types

import pytest
import torch

import plain_migenex as P
import trace_tools as T

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

SHARPEN = 4.0          # the query heads' norm weights are scaled by this
PEAK = 1.5             # the spread of the scores that the models' scales are set for: attention becomes peaked


def full(heads, kv_heads, dim, vdim, dims, base=10000.0, cap=None, size=0, scale=None):
    """An "attention" layer's mixer: heads normed with weights (the queries' around SHARPEN), then rotated in split halves."""
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or PEAK / (SHARPEN * dim ** 0.5),
             "rot": {"base": base, "dims": dims}}
    if cap:
        mixer["softcap"] = cap
    if size:
        mixer["mask"] = {"size": size}
    return {"type": "attention", "mixer": mixer}


def keyed(heads, kv_heads, dim, dims, size, base=10000.0, cap=None, scale=None):
    """An "attention_2" layer's mixer: values are the keys, heads of unit root mean square after interleaved rotation."""
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale or PEAK / dim ** 0.5,
             "rot": {"base": base, "dims": dims}}
    if cap:
        mixer["softcap"] = cap
    if size:
        mixer["mask"] = {"size": size}
    return {"type": "attention_2", "mixer": mixer}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


# X: sizes that no tensor-core kernel takes (the CUDA-core kernels in both dtypes): every per-head size different, odd
# width and vocabulary, windows of 19 and 7 positions (no multiple of the page size 4), a part of the head rotated, an
# "attention" with a window and without a cap, an "attention_2" without a window and with a cap, layers without
# feed-forward, groups of 3, 2 and 1 query heads a key head, 2 of 5 and 3 of 3 experts, with and without a shared expert,
# three passes over three layers.
SHAPE_X = {"architecture": "Migenex", "vocab": 211, "width": 72, "norm": {"eps": 1e-5}, "residual_mult": 0.5,
           "embedding": {"scale": 3.0, "bigram": {"buckets": 53, "mul_prev": 7, "mul_cur": 3}},
           "loop": {"start": 1, "stop": 4, "times": 3}, "layers": [
               dict(keyed(6, 2, 24, 12, 19, base=100.0), mlp=dense(100)),
               dict(full(3, 1, 12, 28, 12, cap=5.0), mlp=moe(5, 2, 20, shared=36)),
               dict(keyed(2, 2, 8, 8, 7), mlp=None),
               dict(full(4, 2, 40, 20, 20, size=33, base=500.0), mlp=moe(3, 3, 12)),
               dict(keyed(3, 3, 20, 20, 0, cap=3.0), mlp=dense(44))]}
# Y: sizes of the tensor-core kernels (multiples of 16), values that a model may happen to make equal or 1: a window of one
# position (a token sees itself), a window longer than any request, a window of the page size 16, no rotation at all (zero
# elements turn), one expert, one pass of a loop that begins at the first layer, one bucket of token pairs, multipliers
# and constants of 1, one key head for 16 query heads, as many key heads as query heads.
SHAPE_Y = {"architecture": "Migenex", "vocab": 97, "width": 64, "norm": {"eps": 1e-6}, "residual_mult": 1.0,
           "embedding": {"scale": 1.0, "bigram": {"buckets": 1, "mul_prev": 1, "mul_cur": 1}},
           "loop": {"start": 0, "stop": 2, "times": 1}, "layers": [
               dict(keyed(4, 1, 16, 16, 1), mlp=dense(64)),
               dict(full(16, 1, 64, 64, 32, cap=2.0), mlp=moe(1, 1, 64, shared=64)),
               dict(keyed(2, 2, 32, 0, 1000), mlp=moe(8, 2, 16)),
               dict(full(2, 1, 128, 32, 128, size=16), mlp=None),
               dict(keyed(8, 8, 16, 16, 16), mlp=dense(128))]}
# Z: no loop, no table of token pairs, no multiplier (what a file may leave out); heads of 80 and 112 elements; the loop's
# layers at the model's end in W, which differs from Z by that alone.
SHAPE_Z = {"architecture": "Migenex", "vocab": 131, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.6}, "layers": [
    dict(full(4, 2, 80, 112, 80, cap=30.0), mlp=moe(4, 1, 32, shared=24)),
    dict(keyed(4, 2, 112, 56, 44), mlp=dense(160)),
    dict(keyed(2, 1, 80, 80, 5, base=50.0), mlp=moe(6, 2, 24))]}
SHAPE_W = dict(copy.deepcopy(SHAPE_Z), loop={"start": 1, "stop": 3, "times": 2}, residual_mult=0.75,
               embedding={"scale": 0.6, "bigram": {"buckets": 300, "mul_prev": 1000003, "mul_cur": 31}})
# V: heads of 64 and 128 whose attentions take the kernels fed by bulk tensor copies (in bfloat16): windows of 24 and 70
# positions whose passed pages go back to the pool while a request runs, a capped attention over everything, two passes
# over all three layers.
SHAPE_V = {"architecture": "Migenex", "vocab": 151, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 0.6,
           "embedding": {"scale": 1.5, "bigram": {"buckets": 77, "mul_prev": 13, "mul_cur": 5}},
           "loop": {"start": 0, "stop": 3, "times": 2}, "layers": [
               dict(keyed(4, 2, 64, 64, 24), mlp=dense(192)),
               dict(full(4, 1, 128, 128, 128, cap=5.0), mlp=moe(4, 2, 32, shared=64)),
               dict(keyed(2, 1, 128, 64, 70, base=300.0), mlp=None)]}
SHAPES = {"X": (SHAPE_X, 4), "Y": (SHAPE_Y, 16), "Z": (SHAPE_Z, 16), "W": (SHAPE_W, 8), "V": (SHAPE_V, 16)}
LENGTHS = {"X": [70, 45, 33, 100, 130, 64, 37, 90], "Y": [1, 7, 17, 40, 129, 65, 96, 50], "Z": [40, 75, 23, 58, 66, 31],
           "W": [50, 2, 81, 64, 33, 47], "V": [150, 40, 97, 200, 64, 130]}
MODES = ("whole", "decode_tail", "portions", "mixed")


def choosing_all(raw):
    """The same model with every routed layer choosing all its experts (for bfloat16: no close calls)."""
    out = copy.deepcopy(raw)
    for layer in out["layers"]:
        if layer["mlp"] is not None and layer["mlp"]["kind"] == "moe":
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return out


def write_model(folder, raw, seed):
    """A seeded random model: its attentions sharpened, its routers' scores spread, its table of token pairs as large as the
    embeddings (a wrong row shows)."""
    from mini_rsglang_b200.models import config_from_dict
    from mini_rsglang_b200.weights import write_random_model, write_safetensors
    from mini_rsglang_b200.weights.safetensors_io import SafetensorsFile

    write_random_model(folder, config_from_dict(raw), seed=seed, dtype=torch.bfloat16)
    path = os.path.join(folder, "model.safetensors")
    tensors = {k: t.read() for k, t in SafetensorsFile(path).tensors.items()}
    for name, t in tensors.items():
        if name.endswith(".mix.q.norm"):
            tensors[name] = (t.float() * SHARPEN).to(t.dtype)
        elif name.endswith(".mlp.router"):
            tensors[name] = (t.float() * 12.0).to(t.dtype)
        elif name == "bigram":
            tensors[name] = (t.float() * 2.0).to(t.dtype)
    write_safetensors(path, tensors)
    return folder


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for i, (name, (raw, _)) in enumerate(SHAPES.items()):
        out[(name, "float32")] = write_model(str(tmp_path_factory.mktemp(f"migenex_{name}")), raw, 71 + i)
        out[(name, "bfloat16")] = write_model(str(tmp_path_factory.mktemp(f"migenex_{name}_all")), choosing_all(raw), 71 + i)
    return out


def load_plain(folder):
    from mini_rsglang_b200.weights.safetensors_io import SafetensorsFile

    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    weights = {k: t.read() for k, t in SafetensorsFile(os.path.join(folder, "model.safetensors")).tensors.items()}
    return config, weights


@functools.lru_cache(maxsize=None)
def plain_logits(folder, name):
    config, weights = load_plain(folder)
    reqs = T.requests_for(config["vocab"], LENGTHS[name], seed=600 + ord(name))
    return reqs, {r: P.forward(tokens, weights, config) for r, tokens in reqs.items()}


_results = {}
# bfloat16 rows against the float64 plain implementation.  The models' attentions are sharpened, so a rounded score moves a
# weight by its own size; the experts square what they compute, which doubles its relative rounding; a layer that is passed
# several times adds its roundings as often; every pass begins with a product whose operand is the whole stream rounded to
# bfloat16; and the norm behind a branch brings a branch's output to unit size together with its rounding, however small
# the output was (a token whose few expert units are nearly all switched off).  With scores spread by 2 the error of a row's
# logits, relative to their root mean square, reached 0.023 in the models without a loop and 0.036 in the one that passes
# two layers twice; the models are set to 1.5, and a single row still reached 0.033.  So the gate is one of many rows, as
# the gates of whole models usually are: no row beyond one and a half times the limit, at most one row in fifty (or one)
# beyond it.  A key taken from a wrong place moves the sharpened attention's logits by far more.
BF16_NRMSE = 0.03


def check_rows(got, want, dtype, what, tally=None):
    """`tally`: a list that collects the rows' errors (the caller then weighs them together with `settle`)."""
    if dtype == "float32":
        return T.check_rows(got, want, dtype, what)
    assert got.shape == want.shape and torch.isfinite(got).all(), what
    own = tally if tally is not None else []
    for i in range(got.shape[0]):
        nrmse = ((got[i] - want[i]).pow(2).mean().sqrt() / want[i].pow(2).mean().sqrt()).item()
        cosine = torch.nn.functional.cosine_similarity(got[i], want[i], dim=0).item()
        assert nrmse <= 1.5 * BF16_NRMSE and cosine >= T.BF16_COSINE, f"{what} row {i}: NRMSE {nrmse:.4f}, cosine {cosine:.5f}"
        own.append((nrmse, f"{what} row {i}"))
    if tally is None:
        settle(own)


def settle(tally):
    over = [entry for entry in tally if entry[0] > BF16_NRMSE]
    assert len(over) <= max(1, len(tally) // 50), f"{len(over)} of {len(tally)} rows beyond {BF16_NRMSE}: {over[:5]}"


def replay(folders, name, dtype, tmp_path_factory):
    key = (name, dtype)
    if key in _results:
        return _results[key]
    folder = folders[key]
    reqs, want = plain_logits(folder, name)
    raw, page = SHAPES[name]
    mixed, peak = T.trace_mixed(reqs, seed=9)
    traces = {"whole": T.trace_whole(reqs), "decode_tail": T.trace_decode_tail(reqs, tail=40),
              "portions": T.trace_portions(reqs, seed=6), "mixed": mixed}
    max_tokens = max(peak, max(T.rounded(len(t)) for t in reqs.values()))
    assert sum(T.rounded(len(t)) for t in reqs.values()) > max_tokens, "the pool must force pages to be used again"
    run = T.TraceRun(folder, dtype, str(tmp_path_factory.mktemp(f"out_{name}_{dtype}")), max_tokens, extra=("--page-size", str(page)))
    out, first = {}, 0
    for mode in MODES:
        trace = T.renumber(traces[mode], first, f"{mode}-")
        first += len(trace.steps)
        rows = []
        for step, places in zip(trace.steps, trace.rows):
            got = run.step(step, raw["vocab"])
            if places:
                rows.append((step["step"], got, torch.stack([want[r][p] for r, p in places]), places))
        out[mode] = rows
    assert run.close() == 0
    _results[key] = out
    return out


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["X", "Y", "Z", "W", "V"])
def test_replay_matches_plain(folders, tmp_path_factory, name, dtype, mode):
    """Prefill against token-by-token decoding (the tail of 40 tokens lets the windows of 1, 5, 7, 16, 19 and 33 pass over
    decoded tokens), portions of every size (the token before a portion comes from the request's state), batches against
    each request alone, pages and state slots used again."""
    rows = replay(folders, name, dtype, tmp_path_factory)[mode]
    assert rows
    tally = []
    for step, got, want, _ in rows:
        check_rows(got, want, dtype, f"{name} {dtype} {mode} step {step}", tally)
    settle(tally)


@pytest.mark.parametrize("name", ["X", "Y"])
def test_float32_logits_do_not_depend_on_the_cutting(folders, tmp_path_factory, name):
    """The same position whole, decoded, in portions and mixed with other requests on pages and slots used again: within the
    rounding of float32 sums."""
    result = replay(folders, name, "float32", tmp_path_factory)
    whole = {place: row for _, got, _, places in result["whole"] for row, place in zip(got, places)}
    compared = 0
    for mode in MODES[1:]:
        for step, got, _, places in result[mode]:
            for row, place in zip(got, places):
                assert (row - whole[place]).abs().max() <= 2e-5 * max(1.0, whole[place].abs().max().item()), (mode, step, place)
                compared += 1
    assert compared > 50


def test_a_prompt_of_more_rows_than_a_recorded_step_holds(tmp_path_factory):
    """2,100 tokens in one step: the step is queued kernel by kernel, the gated unit's first product takes the tensor-core
    kernel for many rows with the relu gate in its epilogue and the shared expert's the one with the squared relu (the
    variable makes them the choice whatever the timing says), the experts' products the one for many rows, the windows pass
    over the prompt and the full attention reaches 2,099 tokens back."""
    raw = {"architecture": "Migenex", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 0.8,
           "embedding": {"scale": 2.0, "bigram": {"buckets": 40, "mul_prev": 5, "mul_cur": 9}}, "loop": {"start": 0, "stop": 2, "times": 2},
           "layers": [dict(keyed(2, 1, 16, 16, 700), mlp=dense(128)),
                      dict(full(2, 1, 16, 16, 16, cap=4.0), mlp=moe(2, 2, 64, shared=64))]}
    folder = write_model(str(tmp_path_factory.mktemp("migenex_long")), raw, 61)
    config, weights = load_plain(folder)
    reqs = T.requests_for(raw["vocab"], [2100], seed=12)
    want = P.forward(reqs["r0"], weights, config)
    trace = T.Trace()
    places = list(range(0, 2100, 37)) + [2099]
    trace.add([("r0", 0, reqs["r0"], places)], end=["r0"])
    run = T.TraceRun(folder, "bfloat16", str(tmp_path_factory.mktemp("out_long")), T.rounded(2100),
                     env=dict(os.environ, MRS_GEMM_GATED_ROWS_MIN="2048"), extra=("--page-size", "16"))
    got = run.step(trace.steps[0], raw["vocab"])
    assert run.close() == 0
    check_rows(got, torch.stack([want[p] for p in places]), "bfloat16", "a prompt of 2,100 tokens")


# ----------------------------------------------------------------------------------------------------------------
# each mechanism alone
# ----------------------------------------------------------------------------------------------------------------
def rotation_table(positions, dims, base):
    from mini_rsglang_b200 import kernels

    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float32, device=DEV)
    return kernels.rotation_table(positions, f)


@pytest.mark.parametrize("far", [False, True])
@pytest.mark.parametrize("place,weights", [("before_rotation", True), ("after_rotation", False), ("after_rotation", True), (None, False)])
@pytest.mark.parametrize("pairing", ["split_half", "interleaved"])
@pytest.mark.parametrize("H,G,d,e,dims,page,from_keys", [(6, 2, 24, 20, 12, 4, False), (2, 2, 8, 8, 8, 8, True), (16, 2, 64, 64, 32, 16, True),
                                                         (1, 1, 130, 16, 130, 4, False), (3, 1, 48, 48, 0, 16, True), (5, 5, 256, 256, 2, 16, False),
                                                         (2, 1, 16, 16, 6, 4, True), (4, 2, 128, 128, 128, 16, True), (2, 2, 128, 64, 64, 8, False)])
def test_rotated_and_normed_heads_on_the_way_into_the_cache(H, G, d, e, dims, page, from_keys, pairing, place, weights, far):
    """The kernel after the fused projection: rotation of all, a part or none of a head in either pairing, at positions up
    to thousands; the head norm before or after it, with or without weights; keys at scattered slots; values from columns
    of their own or the keys as projected; a token that keeps nothing (slot -1); columns behind (gates) left alone."""
    from mini_rsglang_b200 import kernels

    torch.manual_seed(H + d + dims)
    tokens, pool, extra = 11, 5, 7
    width = H * d + G * d + (0 if from_keys else G * e) + extra
    proj = torch.randn(tokens, width) * 2
    qw, kw = (torch.rand(d) + 0.5, torch.rand(d) + 0.5) if weights else (None, None)
    # float32 angles: position * frequency carries a relative rounding of 6e-8, so far positions get a tolerance of their own
    positions = torch.tensor([0, 1, 2, 3, 17, 18, 63, 64, 1000, 4095, 7001] if far else [0, 1, 2, 3, 17, 18, 31, 32, 33, 63, 64], dtype=torch.int32)
    slots = torch.randperm(pool * page)[:tokens].to(torch.int32)
    slots[4] = -1
    p64 = proj.double()
    layout = "half" if pairing == "split_half" else "interleaved"

    def shaped(x, heads, w):
        x = x.view(tokens, heads, d)
        out = []
        for t in range(tokens):             # one row at a time, at its own position
            row = x[t:t + 1]
            if place == "before_rotation":
                row = P.rms_norm(row, w.double() if w is not None else None, 1e-5)
            row = P.rotate(row, 777.0, dims, layout, start=int(positions[t]))
            if place == "after_rotation":
                row = P.rms_norm(row, w.double() if w is not None else None, 1e-5)
            out.append(row)
        return torch.cat(out)

    want_q = shaped(p64[:, :H * d], H, qw).reshape(tokens, H * d)
    want_k = shaped(p64[:, H * d:H * d + G * d], G, kw)
    want_v = p64[:, H * d:H * d + G * d].view(tokens, G, d) if from_keys else p64[:, H * d + G * d:H * d + G * d + G * e].view(tokens, G, e)
    table = rotation_table(positions.to(DEV), dims, 777.0) if dims else None
    for dtype, tol in ((torch.float32, 2e-3 if far and dims else 2e-5), (torch.bfloat16, 8e-3)):
        q = torch.empty(tokens, H * d, dtype=dtype, device=DEV)
        kc = torch.full((pool, G, page, d), 1024.0, dtype=dtype, device=DEV)
        vc = torch.full((pool, G, page, e), -2048.0, dtype=dtype, device=DEV)
        kernels.qkv_rotary_store(proj.to(DEV), q, kc, vc, slots.to(DEV), H, G, d, e, rotations=table, rotary_dim=dims, pairing=pairing,
                                 norm_place=place, q_norm=qw.to(DEV) if weights else None, k_norm=kw.to(DEV) if weights else None,
                                 norm_eps=1e-5, values_from_keys=from_keys)
        assert (q.double().cpu() - want_q).abs().max() < tol * want_q.abs().max()
        written = 0
        for t in range(tokens):
            if slots[t] < 0:
                continue
            pg, at = int(slots[t]) // page, int(slots[t]) % page
            assert (kc[pg, :, at].double().cpu() - want_k[t]).abs().max() < tol * want_k.abs().max(), t
            assert (vc[pg, :, at].double().cpu() - want_v[t]).abs().max() < tol * want_v.abs().max(), t
            written += 1
        assert (kc == 1024.0).sum() == (pool * page - written) * G * d and (vc == -2048.0).sum() == (pool * page - written) * G * e
        kernels.qkv_rotary_store(proj.to(DEV), q, None, None, None, H, G, d, e, rotations=table, rotary_dim=dims, pairing=pairing,
                                 norm_place=place, q_norm=qw.to(DEV) if weights else None, k_norm=kw.to(DEV) if weights else None,
                                 norm_eps=1e-5, values_from_keys=from_keys)                 # a run that keeps nothing
        assert (q.double().cpu() - want_q).abs().max() < tol * want_q.abs().max()


class StepFacts:
    """What `kernels.embed_pairs` reads of a step's context."""

    def __init__(self, ids, positions, seq_of_token, q_start, state_slots):
        as_int = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)      # noqa: E731
        self.token_ids, self.positions, self.seq_of_token = as_int(ids), as_int(positions), as_int(seq_of_token)
        self.q_start, self.state_slots = as_int(q_start), as_int(state_slots)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("buckets,mul_prev,mul_cur", [(53, 7, 3), (1, 1, 1), (499, 1000003, 65537), (17, 0, 5)])
def test_token_pair_embedding_across_portions_and_slots(dtype, buckets, mul_prev, mul_cur):
    """Two requests in portions of unequal sizes (down to one token) in one batch, a third that takes over a slot afterwards:
    every token pairs with the one before it, also across steps; a sequence's first token takes the last row; a run that
    keeps nothing leaves the state alone; padding rows (slot -1) touch nothing."""
    from mini_rsglang_b200 import kernels

    torch.manual_seed(buckets)
    vocab, width = 90, 40
    table = torch.randn(vocab, width).to(dtype)
    pairs = torch.randn(buckets + 1, width).to(dtype)
    config = {"embedding": {"scale": 1.5, "bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}}
    weights = {"embed": table.double(), "bigram": pairs.double()}
    a = [int(v) for v in torch.randint(0, vocab, (23,))]
    b = [int(v) for v in torch.randint(0, vocab, (9,))]
    c = [int(v) for v in torch.randint(0, vocab, (6,))]
    want = {n: P.embed(torch.tensor(t), weights, config) for n, t in (("a", a), ("b", b), ("c", c))}
    state = torch.full((4,), 77, dtype=torch.int32, device=DEV)            # slots that an earlier request left dirty
    slot = {"a": 2, "b": 0, "c": 2}
    fed = {"a": 0, "b": 0, "c": 0}
    tokens = {"a": a, "b": b, "c": c}
    schedule = [[("a", 5), ("b", 1)], [("b", 1), ("a", 1)], [("a", 2), ("b", 7)], [("a", 15)], [("c", 2)], [("c", 1)], [("c", 3)]]
    for step in schedule:
        ids, positions, seq, q_start, slots = [], [], [], [0], []
        for i, (name, count) in enumerate(step):
            ids += tokens[name][fed[name]:fed[name] + count]
            positions += list(range(fed[name], fed[name] + count))
            seq += [i] * count
            q_start.append(len(ids))
            slots.append(slot[name])
        real = len(ids)
        ids, positions, seq = ids + [0, 0], positions + [0, 0], seq + [len(step), len(step)]       # two padding rows of a sequence without a slot
        q_start.append(len(ids))
        slots.append(-1)
        facts = StepFacts(ids, positions, seq, q_start, slots)
        for write in (False, True):           # the trial run first: it must not move the state
            stream = torch.empty(len(ids), width, device=DEV)
            kernels.embed_pairs(table.to(DEV), pairs.to(DEV), facts, state, stream, 1.5, buckets, mul_prev, mul_cur, write_state=write)
            row = 0
            for name, count in step:
                ref = want[name][fed[name]:fed[name] + count]
                assert (stream[row:row + count].double().cpu() - ref).abs().max() < 1e-5, (step, name, write)
                row += count
            assert row == real
        for name, count in step:
            fed[name] += count
            assert int(state[slot[name]]) == tokens[name][fed[name] - 1]
    assert int(state[1]) == 77 and int(state[3]) == 77


@pytest.mark.parametrize("width", [72, 320, 1001, 4100])
@pytest.mark.parametrize("mult", [1.0, 0.7, 0.25])
def test_normed_branch_joins_the_stream_times_a_constant(width, mult):
    from mini_rsglang_b200 import kernels

    torch.manual_seed(width)
    stream = torch.randn(9, width, device=DEV) * 3
    branch = torch.randn(9, width, device=DEV) * 5
    post, following = torch.rand(width, device=DEV) + 0.5, torch.rand(width, device=DEV) + 0.5
    total = stream.double().cpu() + mult * P.rms_norm(branch.double().cpu(), post.double().cpu(), 1e-5)
    want = P.rms_norm(total, following.double().cpu(), 1e-6)
    for dtype, tol in ((torch.float32, 3e-6), (torch.bfloat16, 8e-3)):
        s, out = stream.clone(), torch.empty(9, width, dtype=dtype, device=DEV)
        kernels.postnorm_add_norm(s, branch, post, 1e-5, following, 1e-6, out, mult)
        assert (s.double().cpu() - total).abs().max() < 1e-6 * total.abs().max()
        assert (out.double().cpu() - want).abs().max() < tol * want.abs().max()
    s = stream.clone()
    kernels.postnorm_add_norm(s, branch, post, 1e-5, None, 0.0, None, mult)                 # the sum alone
    assert (s.double().cpu() - total).abs().max() < 1e-6 * total.abs().max()


def test_stream_joined_with_the_embedding_before_a_pass():
    """x <- W [x ; x0] through the part itself, in both dtypes."""
    from mini_rsglang_b200.parts.base import Runtime
    from mini_rsglang_b200.parts.stream_entry import RejoinEmbedding

    torch.manual_seed(8)
    for width, rows in ((72, 5), (64, 40), (200, 3)):
        w = (torch.randn(width, 2 * width) * 0.1).bfloat16()
        x, x0 = torch.randn(rows, width, device=DEV) * 3, torch.randn(rows, width, device=DEV)
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
            part = RejoinEmbedding("loop.in", width, leaf="")
            part.bind({"loop.in": w.to(DEV).to(dtype)}, Runtime(torch.device(DEV), dtype))
            kept = x.clone()
            got = part.forward(x, x0, None)
            want = torch.cat([x.double().cpu(), x0.double().cpu()], dim=-1) @ w.double().T
            assert got.dtype is torch.float32 and torch.equal(x, kept)
            assert (got.double().cpu() - want).abs().max() < tol * want.abs().max()


@pytest.mark.parametrize("kind", ["relu", "relu2", "silu"])
def test_gated_activations_and_the_relu_family(kind):
    from mini_rsglang_b200 import kernels

    torch.manual_seed(5)
    plain = {"relu": torch.relu, "relu2": lambda z: torch.relu(z) ** 2, "silu": lambda z: z * torch.sigmoid(z)}[kind]
    for tokens, inter, block in ((7, 50, 0), (3, 1001, 0), (16, 512, 64), (5, 192, 64), (2, 64, 64)):
        gate_up = torch.randn(tokens, 2 * inter, device=DEV) * 2
        g64 = gate_up.double().cpu()
        if block:
            cut = g64.view(tokens, inter // block, 2, block)
            gate, up = cut[:, :, 0].reshape(tokens, inter), cut[:, :, 1].reshape(tokens, inter)
        else:
            gate, up = g64[:, :inter], g64[:, inter:]
        want = plain(gate) * up
        out = torch.empty(tokens, inter, device=DEV)
        kernels.gated_activation(gate_up, out, kind, block)
        assert (out.double().cpu() - want).abs().max() < 3e-6 * max(1.0, want.abs().max().item())
        out16 = torch.empty(tokens, inter, dtype=torch.bfloat16, device=DEV)
        kernels.gated_activation(gate_up.bfloat16(), out16, kind, block)
        g16 = gate_up.bfloat16().double().cpu()
        if block:
            cut = g16.view(tokens, inter // block, 2, block)
            gate, up = cut[:, :, 0].reshape(tokens, inter), cut[:, :, 1].reshape(tokens, inter)
        else:
            gate, up = g16[:, :inter], g16[:, inter:]
        want = plain(gate) * up
        assert (out16.double().cpu() - want).abs().max() < 8e-3 * max(1.0, want.abs().max().item())
    z = torch.randn(6, 100, device=DEV) * 3
    out = torch.empty_like(z)
    kernels.activation(z, out, kind)
    assert (out.double().cpu() - plain(z.double().cpu())).abs().max() < 3e-6 * 10


@pytest.mark.parametrize("rows,n,k", [(300, 128, 72), (129, 640, 200), (2048, 512, 256), (1, 128, 64)])
def test_relu_gate_and_squared_relu_in_the_epilogue_of_the_product_for_many_rows(rows, n, k):
    """The tensor-core products whose epilogues apply relu(gate) * up (blocks of 64 gate and 64 up rows) and the square of
    relu to the float32 sums, against float64."""
    from mini_rsglang_b200 import kernels

    torch.manual_seed(19)
    x = torch.randn(rows, k, device=DEV).bfloat16()
    w = (torch.randn(n, k, device=DEV) * (2.0 / k ** 0.5)).bfloat16()
    sums = x.double().cpu() @ w.double().cpu().T
    out = torch.full((rows, n), 77.0, dtype=torch.bfloat16, device=DEV)
    kernels.gemm_act_rows(x, w, out, "relu2")
    kernels.check_device_errors()
    want = torch.relu(sums) ** 2
    assert (out.double().cpu() - want).abs().max() < 8e-3 * max(1.0, want.abs().max().item())
    cut = sums.view(rows, n // 128, 2, 64)
    want = torch.relu(cut[:, :, 0]).reshape(rows, n // 2) * cut[:, :, 1].reshape(rows, n // 2)
    out = torch.full((rows, n // 2), 77.0, dtype=torch.bfloat16, device=DEV)
    kernels.gemm_gated_rows(x, w, out, "relu")
    kernels.check_device_errors()
    assert (out.double().cpu() - want).abs().max() < 8e-3 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("experts,top", [(5, 2), (3, 3), (1, 1), (8, 1), (40, 6)])
def test_sigmoid_scores_that_are_not_normalised(experts, top):
    """The router's choice and weights: sigmoids of the logits, the `top` largest (the lower number wins a tie), the weights
    the scores themselves."""
    from mini_rsglang_b200 import kernels

    torch.manual_seed(experts)
    tokens = 50
    logits = torch.randn(tokens, experts + 3, device=DEV) * 2
    logits[7, :experts] = 0.25                                   # all scores equal: the first `top` experts
    chosen = torch.empty(tokens, top, dtype=torch.int32, device=DEV)
    weights = torch.empty(tokens, top, device=DEV)
    kernels.moe_route(logits, None, chosen, weights, None, experts, top, 1.0, sigmoid_scores=True, normalize=False)
    s = torch.sigmoid(logits[:, :experts].double().cpu())
    for t in range(tokens):
        order = sorted(range(experts), key=lambda e: (-float(s[t, e]), e))[:top]
        assert chosen[t].tolist() == order, t
        assert (weights[t].double().cpu() - s[t, order]).abs().max() < 1e-6


@pytest.mark.parametrize("kernel", ["simt", "rows", "mma", "tc"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,width,experts,top,inner", [(9, 72, 5, 2, 20), (70, 64, 8, 1, 64), (300, 128, 3, 3, 48), (33, 256, 16, 4, 8)])
def test_ungated_experts_that_read_weighted_tokens(kernel, dtype, tokens, width, experts, top, inner):
    """y[pair] = W_down relu(W_up (w h))^2 with every kernel that takes the sizes, free choices, experts that no token chose,
    runs filled up to whole tiles; and the sum over a token's choices with a shared expert added unweighted."""
    from mini_rsglang_b200 import kernels

    if kernel in ("mma", "tc") and dtype is torch.float32:
        pytest.skip("the tensor-core products are bfloat16")
    torch.manual_seed(tokens + width)
    h = torch.randn(tokens, width, device=DEV).to(dtype)
    up = (torch.randn(experts, inner, width, device=DEV) * (1.5 / width ** 0.5)).to(dtype)
    down = (torch.randn(experts, width, inner, device=DEV) / inner ** 0.5).to(dtype)
    if kernel == "rows" and not kernels.moe_rows_supported(h, inner) or kernel == "mma" and not kernels.moe_mma_supported(h, inner) \
            or kernel == "tc" and not kernels.moe_plain_tc_supported(h, up, down):
        pytest.skip("sizes that this kernel does not take")
    chosen = torch.stack([torch.randperm(experts)[:top] for _ in range(tokens)]).to(torch.int32).to(DEV)
    if experts > 2 and top == 1:
        chosen[chosen == 1] = 0                                              # expert 1 gets no row
    weights = torch.rand(tokens, top, device=DEV) * 0.9 + 0.05
    y = torch.zeros(tokens * top, width, dtype=dtype, device=DEV)
    kernels.moe_plain_experts(h, chosen, weights, up, down, y, experts, "relu2", kernel=kernel)
    kernels.check_device_errors()
    h64, up64, down64 = h.double().cpu(), up.double().cpu(), down.double().cpu()
    want = torch.zeros(tokens * top, width, dtype=torch.float64)
    for t in range(tokens):
        for c in range(top):
            e = int(chosen[t, c])
            x = h64[t] * float(weights[t, c])
            want[t * top + c] = down64[e] @ torch.relu(up64[e] @ x) ** 2
    tol = 2e-5 if dtype is torch.float32 else 2e-2
    assert (y.double().cpu() - want).abs().max() < tol * max(1.0, want.abs().max().item())
    shared = torch.randn(tokens, width, device=DEV).to(dtype)
    out = torch.empty(tokens, width, dtype=dtype, device=DEV)
    kernels.moe_combine(y, h, shared, chosen, None, None, out, experts)
    total = y.double().cpu().view(tokens, top, width).sum(1) + shared.double().cpu()
    assert (out.double().cpu() - total).abs().max() < (1e-5 if dtype is torch.float32 else 2e-2) * max(1.0, total.abs().max().item())
    sums = torch.empty(tokens, width, dtype=torch.float32, device=DEV)              # the sums as they are, whatever the parts' dtype
    kernels.moe_combine(y, h, shared, chosen, None, None, sums, experts)
    assert (sums.double().cpu() - total).abs().max() < 1e-5 * max(1.0, total.abs().max().item())


def attend_through_the_part(dtype, kind, H, G, d, window, page, tokens, portions, proj):
    """Runs a `biased_window_attention` in one of the design's two dresses over given projection rows (the part's fused
    matrix is the identity, its output matrix too), portion by portion through a cache of its own; returns the heads' outputs."""
    from mini_rsglang_b200 import kernels
    from mini_rsglang_b200.parts.attention_biased import BiasedWindowAttention
    from mini_rsglang_b200.parts.base import PartSpec, Runtime

    assert kind == "keyed"
    width_in = proj.shape[1]
    part = BiasedWindowAttention("m", width_in, H, G, d, d, scale=1.0, window=window, head_norm_eps=None,
                                 position=PartSpec("rope", {"head_dim": d, "theta": 10000.0, "rotary_dim": 0}), values_from_keys=True,
                                 names={"q": "q", "k": "k", "o": "o"})
    eye = torch.eye(width_in, device=DEV, dtype=dtype)
    part.bind({"m.q": eye[:H * d], "m.k": eye[H * d:], "m.o": torch.eye(H * d, device=DEV, dtype=dtype)}, Runtime(torch.device(DEV), dtype, page))
    pages = -(-tokens // page)
    order = torch.randperm(pages + 3)[:pages].to(torch.int32)           # the request's pages lie scattered in the pool

    class Cache:
        group = 0
        k = torch.zeros(pages + 3, G, page, d, dtype=dtype, device=DEV)
        v = torch.zeros(pages + 3, G, page, d, dtype=dtype, device=DEV)

    out, start = [], 0
    for count in portions:
        ctx = types.SimpleNamespace(shared={}, rehearsal=False, facts=None, plan_views=None, observe=None)
        ctx.num_tokens, ctx.num_sequences, ctx.real_sequences = count, 1, 1
        ctx.positions = torch.arange(start, start + count, dtype=torch.int32, device=DEV)
        ctx.seq_of_token = torch.zeros(count, dtype=torch.int32, device=DEV)
        ctx.q_start = torch.tensor([0, count], dtype=torch.int32, device=DEV)
        ctx.context_len = torch.tensor([start + count], dtype=torch.int32, device=DEV)
        ctx.block_tables = [order.view(1, -1).to(DEV)]
        at = torch.arange(start, start + count)
        ctx.slots = [(order[at // page].long() * page + at % page).to(torch.int32).to(DEV)]
        ctx.host_q_start, ctx.host_start_pos = [0, count], [start]
        ctx.max_query_len, ctx.max_context_len = count, start + count
        ctx.decode_tiles = torch.tensor([[0, 0, 1, 0]], dtype=torch.int32, device=DEV) if count == 1 else None
        out.append(part.forward(proj[start:start + count].to(DEV).to(dtype), ctx, Cache, True).double().cpu())
        start += count
        kernels.check_device_errors()
    return torch.cat(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,page,tokens", [(19, 4, 90), (16, 16, 70), (40, 16, 150), (1, 8, 20), (0, 16, 400)])
def test_a_window_sees_exactly_its_keys_whose_values_are_the_keys(dtype, window, page, tokens):
    """One key at a time is made to stand out for the last query (a score far above the others): just inside the window,
    just outside it, at page borders, the first token, a far token without a window; prompts in portions and decoded
    tokens.  The output is then that key itself, as projected, or (outside) shows nothing of it."""
    H, G, d = 4, 2, 16
    torch.manual_seed(window + tokens)
    last = tokens - 1
    first_seen = max(0, last - window + 1) if window else 0
    candidates = {first_seen, last, max(first_seen - 1, 0), (last // page) * page, max((last // page) * page - 1, 0), 0}
    for target in sorted(candidates):
        k = torch.randn(tokens, G, d) * 0.1
        marker = torch.zeros(d)
        marker[3] = 6.0
        k[target] += marker                                   # the key that stands out, in both key heads
        q = torch.randn(tokens, H, d) * 0.1
        q[last] = marker * 2.0                                # the last query asks for it: a score of 72 against about 0
        proj = torch.cat([q.view(tokens, -1), k.view(tokens, -1)], dim=1).bfloat16().float()
        for portions in ([tokens], [tokens - 3, 1, 1, 1], [5, 2, tokens - 7]):
            got = attend_through_the_part(dtype, "keyed", H, G, d, window, page, tokens, portions, proj)[last].view(H, d)
            seen = target >= first_seen
            value = proj[target, H * d:].view(G, d).double()
            for h in range(H):
                if seen:
                    assert (got[h] - value[h // 2]).abs().max() < 0.05, (target, portions, h)
                else:
                    assert got[h][3].abs() < 1.0, (target, portions, h)


@pytest.mark.parametrize("cap", [0.0, 2.0, 30.0])
@pytest.mark.parametrize("H,G,d,window,page", [(4, 2, 64, 0, 16), (16, 1, 64, 40, 16), (8, 2, 128, 0, 16), (2, 2, 128, 100, 8)])
def test_scale_and_cap_in_the_kernels_fed_by_bulk_copies(H, G, d, window, page, cap):
    """The attention of plain scores (scale, cap, window) through the kernel for few rows and the tcgen05 kernel for prompt
    portions, against the CUDA-core kernel on the same pages: a prompt of 300 tokens in one step, then a portion of 7 and
    single tokens; scores of a size that the small cap bends hard."""
    from mini_rsglang_b200 import kernels
    from mini_rsglang_b200.parts.attention import fast_kernels_take, paged_attention

    assert fast_kernels_take(d, H // G, page)
    torch.manual_seed(H + d + window)
    tokens, scale = 320, 2.5 / d ** 0.5
    pages = -(-tokens // page)
    order = torch.randperm(pages + 2)[:pages].to(torch.int32)
    k = torch.randn(pages + 2, G, page, d, device=DEV).bfloat16()
    v = torch.randn(pages + 2, G, page, d, device=DEV).bfloat16()
    q_all = (torch.randn(tokens, H * d, device=DEV) * 1.5).bfloat16()
    cache = types.SimpleNamespace(group=0, k=k, v=v)
    start = 0
    for count in (300, 7, 1, 1, 11):
        ctx = types.SimpleNamespace(shared={}, rehearsal=False, facts=None, plan_views=None, observe=None)
        ctx.num_tokens, ctx.num_sequences, ctx.real_sequences = count, 1, 1
        ctx.positions = torch.arange(start, start + count, dtype=torch.int32, device=DEV)
        ctx.seq_of_token = torch.zeros(count, dtype=torch.int32, device=DEV)
        ctx.block_tables = [order.view(1, -1).to(DEV)]
        ctx.host_q_start, ctx.host_start_pos = [0, count], [start]
        ctx.max_query_len, ctx.max_context_len = count, start + count
        ctx.decode_tiles = torch.tensor([[0, 0, 1, 0]], dtype=torch.int32, device=DEV) if count == 1 else None
        q = q_all[start:start + count].contiguous()
        got, want = torch.empty_like(q), torch.empty_like(q)
        paged_attention(q, cache, ctx, got, H, G, d, window, scale=scale, cap=cap)
        kernels.attention_biased_simt(q, k, v, ctx.positions, ctx.seq_of_token, ctx.block_tables[0], want, H, G, d, d, scale, cap, window)
        kernels.check_device_errors()
        assert (got.float() - want.float()).abs().max() < 0.03, (count, start)
        start += count


# ----------------------------------------------------------------------------------------------------------------
# the engine's own entry point and scheduler
# ----------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["X", "Y"])
def test_greedy_generation_through_the_engine(folders, name, dtype):
    """Prompts of unequal lengths, more requests than run at a time (state slots are used again), prompt portions under a small
    token budget beside decoded tokens, 40 generated tokens each (the windows pass over decoded tokens, every decoded token
    pairs with the one sampled before it): every token is the plain implementation's arg-max, or within rounding of it."""
    from mini_rsglang_b200 import RuntimeConfig, SamplingParams
    from mini_rsglang_b200.engine import EngineHandle

    folder = folders[(name, dtype)]
    config, weights = load_plain(folder)
    prompts = [T.requests_for(config["vocab"], [n], seed=700 + n)["r0"] for n in (3, 50, 1, 77, 20, 31)]
    engine = EngineHandle.load(folder, 0, config=RuntimeConfig(max_seq_len=160, prefill_budget=24, max_running=3, page_size=SHAPES[name][1]),
                               dtype=dtype, num_pages=120 if name == "X" else 40)
    results = engine.generate_many(prompts, SamplingParams(max_tokens=40, ignore_eos=True))
    engine.shutdown()
    for prompt, result in zip(prompts, results):
        assert len(result.token_ids) == 40
        tokens = list(prompt)
        for token in result.token_ids:
            logits = P.forward(tokens, weights, config)[-1]
            best = int(logits.argmax())
            gap = (logits[best] - logits[token]).item()
            limit = 2e-5 * max(1.0, logits.abs().max().item()) if dtype == "float32" else 0.02 * logits.abs().max().item()
            assert token == best or gap <= limit, f"{dtype}: engine chose {token}, plain {best}, gap {gap}"
            tokens.append(token)


def test_command_line_generates_the_plain_tokens(folders):
    """`bin/mini-rsglang generate` on a Migenex folder: the architecture is found by config.json, prefix sharing (on by
    default on the command line) is switched off with a note because the model keeps windows of keys and the last token of
    every request, and the tokens are the plain implementation's."""
    import subprocess
    import sys

    folder = folders[("X", "float32")]
    prompt = [3, 1, 4, 1, 5, 9, 2, 6]
    cmd = [sys.executable, os.path.join(T.ROOT, "bin", "mini-rsglang"), "--model", folder, "--dtype", "float32", "--page-size", "4",
           "--max-seq-len", "128", "--num-pages", "40", "generate", "--token-ids", ",".join(map(str, prompt)), "--max-tokens", "12",
           "--ignore-eos", "--json"]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    assert "prefix sharing is off" in proc.stderr
    events = [json.loads(line) for line in proc.stdout.splitlines() if line.startswith("{")]
    tokens = [e["Token"]["token_id"] for e in events if "Token" in e]
    done = events[-1]["Finished"]
    assert done["reason"] == "length" and done["prompt_tokens"] == len(prompt) and done["completion_tokens"] == 12
    config, weights = load_plain(folder)
    sequence = list(prompt)
    for token in tokens:
        logits = P.forward(sequence, weights, config)[-1]
        best = int(logits.argmax())
        assert token == best or (logits[best] - logits[token]).item() <= 2e-5 * max(1.0, logits.abs().max().item()), (token, best)
        sequence.append(token)
