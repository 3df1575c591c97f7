"""Nubipel on the GPU against the plain implementation (`plain_nubipel.py`): every mechanism's kernel alone, then
whole models of several small shapes through `bin/trace_run` in every cutting (whole, a decoded tail, portions
down to two tokens, requests mixed in a pool so small that pages and state slots are used again), in float32 and
bfloat16, and greedy generation through the engine's entry point and scheduler.  Where random weights would hide a
fault (a far key, a chunk's edge, a page border, a sink, an old token in a recurrent state), inputs are made so that
it shows."""
import functools
import json
import math
import os

import pytest
import torch

import plain_nubipel as P
import trace_tools as T

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


SHARPEN = 4.0          # the queries' head norm weights and the latent attention's query up-projection are scaled by this
PEAK = 2.0             # the spread of the scores that the models' scales are set for: attention becomes peaked, and bfloat16 still resolves it


def attention(heads, kv_heads, dim, vdim, size, scale=None):
    """`scale` None: such that the scores of normed heads (queries with weights around SHARPEN, keys around 1) spread by PEAK."""
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or PEAK / (SHARPEN * dim ** 0.5)}
    if size:
        mixer["mask"] = {"size": size}
    return {"type": "attention", "mixer": mixer}


def latent(heads, dim, vdim, kv_rank, q_rank, scale=None):
    """`scale` None: such that the scores spread by PEAK with up-projections drawn from N(0, 0.02) (the queries' times SHARPEN)
    on normed latents."""
    spread = (0.02 * SHARPEN * q_rank ** 0.5) * (0.02 * kv_rank ** 0.5) * dim ** 0.5
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                                                  "scale": scale or PEAK / spread}}


def delta(heads, kv_heads, dim, vdim, conv):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


# X: sizes that no tensor-core kernel takes (the CUDA-core kernels in both dtypes): every per-head size different, odd
# widths and vocabulary, chunks of 19 and 7 positions (no multiple of the page size 4) and an attention without chunks,
# layers without feed-forward, groups of 3 and of 1 query heads a key head, convolutions of 3 and 2 taps, a delta rule
# whose every head has its own query/key head.
SHAPE_X = {"architecture": "Nubipel", "vocab": 211, "width": 72, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
           "logit_scale": 0.7, "logit_softcap": 9.0, "layers": [
               dict(delta(4, 2, 24, 12, 3), mlp=dense(100)),
               dict(attention(6, 2, 24, 20, 19), mlp=None),
               dict(latent(3, 12, 20, 40, 28), mlp=dense(52)),
               dict(attention(2, 2, 8, 12, 7, scale=0.25), mlp=dense(36)),
               dict(delta(3, 3, 40, 10, 2), mlp=None),
               dict(latent(5, 8, 8, 18, 10), mlp=None),
               dict(attention(3, 1, 12, 28, 0), mlp=dense(44))]}
# Y: sizes of the tensor-core kernels (multiples of 16), values that a model may happen to make equal or 1: one head, a chunk
# of one position (a token sees itself and the sink), a chunk longer than any request, a chunk of the page size 16, a
# convolution of one tap (no inputs to keep), a vocabulary that is no multiple of 8, constants of 1, no cap on the logits,
# a group of 8 query heads a key head.
SHAPE_Y = {"architecture": "Nubipel", "vocab": 97, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
           "logit_scale": 1.0, "layers": [
               dict(attention(4, 1, 16, 32, 24), mlp=dense(64)),
               dict(latent(4, 16, 16, 64, 32), mlp=dense(32)),
               dict(delta(1, 1, 16, 16, 1), mlp=dense(48)),
               dict(attention(16, 2, 64, 64, 1), mlp=None),
               dict(attention(2, 2, 32, 16, 1000), mlp=dense(80)),
               dict(delta(4, 1, 64, 32, 4), mlp=None),
               dict(latent(1, 32, 48, 32, 16), mlp=dense(16)),
               dict(attention(2, 1, 128, 128, 16), mlp=None)]}
# Z: latent attentions of more heads than a tensor-core tile of few rows holds (32 and 48: decoded tokens go as two and three
# rows of 16 heads), and one of 24 heads (no multiple of 16: a wide tile a token).
SHAPE_Z = {"architecture": "Nubipel", "vocab": 131, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
           "logit_scale": 0.5, "logit_softcap": 12.0, "layers": [
               dict(latent(32, 16, 16, 32, 16), mlp=dense(48)),
               dict(latent(48, 16, 32, 48, 32), mlp=None),
               dict(latent(24, 32, 16, 64, 48), mlp=dense(32))]}
SHAPES = {"X": (SHAPE_X, 4), "Y": (SHAPE_Y, 16), "Z": (SHAPE_Z, 16)}
LENGTHS = {"X": [70, 45, 33, 100, 130, 64, 37, 90], "Y": [1, 7, 17, 40, 129, 65, 96, 50], "Z": [40, 75, 23, 58, 66, 31]}
MODES = ("whole", "decode_tail", "portions", "mixed")


def write_model(folder, raw, seed):
    """A seeded random model: its attentions sharpened, its recurrent heads slowed down (a state that remembers dozens of
    tokens shows a state that was lost or mixed up), its sinks of the size of the scores."""
    from mini_rsglang_b200.models import config_from_dict
    from mini_rsglang_b200.weights import write_random_model, write_safetensors
    from mini_rsglang_b200.weights.safetensors_io import SafetensorsFile

    write_random_model(folder, config_from_dict(raw), seed=seed, dtype=torch.bfloat16)
    path = os.path.join(folder, "model.safetensors")
    tensors = {k: t.read() for k, t in SafetensorsFile(path).tensors.items()}
    for name, t in tensors.items():
        if name.endswith(".mix.q.norm") or name.endswith(".mix.uq"):
            tensors[name] = (t.float() * SHARPEN).to(t.dtype)
        elif name.endswith(".mix.A_log"):
            tensors[name] = (t.float() - 3.0).to(t.dtype)
        elif name.endswith(".mix.sink"):
            tensors[name] = (t.float() * 3.0).to(t.dtype)
        elif name.endswith(".mix.b") or name.endswith(".mix.a"):
            tensors[name] = (t.float() * 8.0).to(t.dtype)          # step sizes and decays that differ from token to token
    write_safetensors(path, tensors)
    return folder


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: write_model(str(tmp_path_factory.mktemp(f"nubipel_{name}")), raw, 51 + i) for i, (name, (raw, _)) in enumerate(SHAPES.items())}


def load_plain(folder):
    from mini_rsglang_b200.weights.safetensors_io import SafetensorsFile

    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    weights = {k: t.read() for k, t in SafetensorsFile(os.path.join(folder, "model.safetensors")).tensors.items()}
    return config, weights


@functools.lru_cache(maxsize=None)
def plain_logits(folder, name):
    config, weights = load_plain(folder)
    reqs = T.requests_for(config["vocab"], LENGTHS[name], seed=400 + ord(name))
    return reqs, {r: P.forward(config, weights, tokens) for r, tokens in reqs.items()}


_results = {}


def replay(folders, name, dtype, tmp_path_factory):
    key = (name, dtype)
    if key in _results:
        return _results[key]
    folder = folders[name]
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
@pytest.mark.parametrize("name", ["X", "Y"])
def test_replay_matches_plain(folders, tmp_path_factory, name, dtype, mode):
    """Prefill against token-by-token decoding (the tail of 40 tokens lets the chunks of 1, 7, 16, 19 and 24 begin anew among
    decoded tokens), portions of every size, batches against each request alone, pages and state slots used again."""
    rows = replay(folders, name, dtype, tmp_path_factory)[mode]
    assert rows
    for step, got, want, _ in rows:
        T.check_rows(got, want, dtype, f"{name} {dtype} {mode} step {step}")


@pytest.mark.parametrize("mode", MODES)
def test_latent_attention_of_many_heads(folders, tmp_path_factory, mode):
    """Decoded tokens whose heads fill several tiles of few rows, alone and beside portions of other requests, against the
    plain implementation."""
    rows = replay(folders, "Z", "bfloat16", tmp_path_factory)[mode]
    assert rows
    for step, got, want, _ in rows:
        T.check_rows(got, want, "bfloat16", f"Z bfloat16 {mode} step {step}")


def test_a_prompt_of_more_rows_than_a_recorded_step_holds(tmp_path_factory):
    """2,100 tokens in one step: the step is queued kernel by kernel, the feed-forward's first product takes the kernel for
    many rows with the activation in its epilogue (the variable makes it the choice whatever the timing says), the
    chunked attention crosses its chunk's edge twice, the recurrence walks 2,100 tokens from an empty state."""
    raw = {"architecture": "Nubipel", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
           "logit_scale": 0.5, "logit_softcap": 12.0, "layers": [
               dict(latent(2, 16, 16, 32, 16), mlp=dense(64)),
               dict(attention(2, 1, 16, 16, 700), mlp=dense(96)),
               dict(delta(2, 1, 16, 16, 2), mlp=dense(32))]}
    folder = write_model(str(tmp_path_factory.mktemp("nubipel_long")), raw, 61)
    config, weights = load_plain(folder)
    reqs = T.requests_for(raw["vocab"], [2100], seed=12)
    want = P.forward(config, weights, reqs["r0"])
    trace = T.trace_whole(reqs)
    run = T.TraceRun(folder, "bfloat16", str(tmp_path_factory.mktemp("out_long")), T.rounded(2100),
                     env=dict(os.environ, MRS_GEMM_GATED_ROWS_MIN="2048"), extra=("--page-size", "16"))
    got = run.step(trace.steps[0], raw["vocab"])
    assert run.close() == 0
    T.check_rows(got, torch.stack([want[p] for _, p in trace.rows[0]]), "bfloat16", "a prompt of 2,100 tokens")


@pytest.mark.parametrize("name", ["X", "Y"])
def test_float32_logits_do_not_depend_on_the_cutting(folders, tmp_path_factory, name):
    """The same position whole, decoded, in portions and mixed with other requests on pages and slots used again: within the
    rounding of float32 sums (the batched library products may sum in another order for another number of rows)."""
    result = replay(folders, name, "float32", tmp_path_factory)
    whole = {place: row for _, got, _, places in result["whole"] for row, place in zip(got, places)}
    compared = 0
    for mode in MODES[1:]:
        for step, got, _, places in result[mode]:
            for row, place in zip(got, places):
                assert (row - whole[place]).abs().max() <= 2e-5 * max(1.0, whole[place].abs().max().item()), (mode, step, place)
                compared += 1
    assert compared > 50


# ----------------------------------------------------------------------------------------------------------------
# each mechanism alone
# ----------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("width", [72, 320, 1001, 4100, 8200])
def test_sum_of_both_branches_and_the_next_norm(width):
    from mini_rsglang_b200 import kernels

    torch.manual_seed(width)
    stream = torch.randn(9, width, device=DEV) * 3
    a, b = torch.randn(9, width, device=DEV) * 2, torch.randn(9, width, device=DEV) * 5
    weight = torch.rand(width, device=DEV) + 0.5
    for second in (b, None):
        total = stream.double().cpu() + a.double().cpu() + (second.double().cpu() if second is not None else 0.0)
        want = P.rms_norm(total, weight.double().cpu(), 1e-5)
        for dtype, tol in ((torch.float32, 3e-6), (torch.bfloat16, 8e-3)):
            s, out = stream.clone(), torch.empty(9, width, dtype=dtype, device=DEV)
            kernels.add_branches_norm(s, a, second, weight, 1e-5, out)
            assert (s.double().cpu() - total).abs().max() < 1e-6 * total.abs().max()
            assert (out.double().cpu() - want).abs().max() < tol * want.abs().max()
        s = stream.clone()
        kernels.add_branches_norm(s, a, second, None, 0.0, None)                 # the sum alone (the last layer's)
        assert (s.double().cpu() - total).abs().max() < 1e-6 * total.abs().max()


@pytest.mark.parametrize("kind", ["gelu_erf", "gelu_tanh", "silu"])
def test_activations(kind):
    from mini_rsglang_b200 import kernels

    torch.manual_seed(3)
    plain = {"gelu_erf": P.gelu_erf, "silu": P.silu,
             "gelu_tanh": lambda z: 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))}[kind]
    for shape in ((7, 50), (3, 1001), (16, 512)):
        z = torch.randn(*shape, device=DEV) * 3
        out = torch.empty_like(z)
        kernels.activation(z, out, kind)
        assert (out.double().cpu() - plain(z.double().cpu())).abs().max() < 2e-6
        z16 = z.bfloat16()
        kernels.activation(z16, z16, kind)                                     # in place
        want = plain(z.bfloat16().double().cpu())
        assert (z16.double().cpu() - want).abs().max() < 8e-3 * max(1.0, want.abs().max().item())
    far = torch.tensor([[-40.0, -9.0, 0.0, 9.0, 40.0, 1e4, -1e4]], device=DEV)
    out = torch.empty_like(far)
    kernels.activation(far, out, kind)
    assert torch.isfinite(out).all() and out[0, 2] == 0 and out[0, 5] == 1e4 and out[0, 6].abs() == 0


@pytest.mark.parametrize("kind", ["gelu_erf", "gelu_tanh", "silu"])
@pytest.mark.parametrize("rows,n,k", [(300, 96, 72), (129, 544, 200), (2048, 512, 256), (1, 32, 64)])
def test_activation_in_the_epilogue_of_the_product_for_many_rows(kind, rows, n, k):
    """act(x . w^T) from the tensor-core product whose epilogue applies the activation to the float32 sums, against float64:
    row and column counts that leave tiles partly empty, a K that is no multiple of the copies' 64 columns."""
    from mini_rsglang_b200 import kernels

    torch.manual_seed(17)
    plain = {"gelu_erf": P.gelu_erf, "silu": P.silu,
             "gelu_tanh": lambda z: 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))}[kind]
    x = torch.randn(rows, k, device=DEV).bfloat16()
    w = (torch.randn(n, k, device=DEV) * (2.0 / k ** 0.5)).bfloat16()
    assert kernels.gemm_act_rows_supported(x, w)
    out = torch.full((rows, n), 77.0, dtype=torch.bfloat16, device=DEV)
    kernels.gemm_act_rows(x, w, out, kind)
    kernels.check_device_errors()
    want = plain(x.double().cpu() @ w.double().cpu().T)
    assert (out.double().cpu() - want).abs().max() < 8e-3 * max(1.0, want.abs().max().item())


def test_scaled_embeddings_and_capped_logits():
    from mini_rsglang_b200 import kernels

    torch.manual_seed(4)
    for dtype in (torch.float32, torch.bfloat16):
        table = torch.randn(37, 72, device=DEV).to(dtype)
        ids = torch.tensor([36, 0, 5, 5, 17], dtype=torch.int32, device=DEV)
        stream = torch.empty(5, 72, device=DEV)
        kernels.embed(table, ids, stream, 3.5)
        assert (stream.double().cpu() - table.double().cpu()[ids.cpu().long()] * 3.5).abs().max() < 1e-6
    logits = torch.randn(6, 211, device=DEV) * 30
    want = 9.0 * torch.tanh(logits.double().cpu() * 0.7 / 9.0)
    kernels.scale_softcap_(logits, 0.7, 9.0)
    assert (logits.double().cpu() - want).abs().max() < 5e-6 and logits.abs().max() <= 9.0


@pytest.mark.parametrize("H,G,d,e,page", [(6, 2, 24, 20, 4), (2, 2, 8, 12, 8), (16, 2, 64, 64, 16), (1, 1, 130, 16, 4)])
def test_head_norms_on_the_way_into_the_cache(H, G, d, e, page):
    """The kernel after the fused projection: every query and key head over its root mean square times one weight for all
    query (key) heads, keys and values at scattered slots, a token that keeps nothing (slot -1)."""
    from mini_rsglang_b200 import kernels

    torch.manual_seed(H + d)
    tokens, pool = 11, 5
    proj = torch.randn(tokens, H * d + G * d + G * e) * 2
    qw, kw = torch.rand(d) + 0.5, torch.rand(d) + 0.5
    slots = torch.randperm(pool * page)[:tokens].to(torch.int32)
    slots[4] = -1
    p64 = proj.double()
    want_q = P.rms_norm(p64[:, :H * d].view(tokens, H, d), qw.double(), 1e-5).reshape(tokens, H * d)
    want_k = P.rms_norm(p64[:, H * d:H * d + G * d].view(tokens, G, d), kw.double(), 1e-5)
    want_v = p64[:, H * d + G * d:].view(tokens, G, e)
    for dtype, tol in ((torch.float32, 3e-6), (torch.bfloat16, 8e-3)):
        q = torch.empty(tokens, H * d, dtype=dtype, device=DEV)
        kc = torch.full((pool, G, page, d), 7.0, dtype=dtype, device=DEV)
        vc = torch.full((pool, G, page, e), -9.0, dtype=dtype, device=DEV)
        kernels.qkv_bias_store(proj.to(DEV), None, q, kc, vc, slots.to(DEV), H, G, d, e, q_norm=qw.to(DEV), k_norm=kw.to(DEV), norm_eps=1e-5)
        assert (q.double().cpu() - want_q).abs().max() < tol * want_q.abs().max()
        for t in range(tokens):
            if slots[t] < 0:
                continue
            pg, at = int(slots[t]) // page, int(slots[t]) % page
            assert (kc[pg, :, at].double().cpu() - want_k[t]).abs().max() < tol * want_k.abs().max(), t
            assert (vc[pg, :, at].double().cpu() - want_v[t]).abs().max() < tol * want_v.abs().max(), t
        used = {int(s) for s in slots if s >= 0}
        for s in set(range(pool * page)) - used:
            assert (kc[s // page, :, s % page] == 7.0).all() and (vc[s // page, :, s % page] == -9.0).all()


def plain_chunk_attention(q, k, v, sinks, scale, chunk):
    """q [T, H, d], k [T, G, d], v [T, G, e] as the cache holds them (normed already), sinks [H] or None."""
    T_, H, G = q.shape[0], q.shape[1], k.shape[1]
    seen = P.chunk_mask(T_, chunk)
    return torch.stack([P.softmax_with_sink(q[:, h] @ k[:, h // (H // G)].T * scale, seen, None if sinks is None else sinks[h])
                        @ v[:, h // (H // G)] for h in range(H)], dim=1)


def run_chunk_attention(dtype, q, k, v, sinks, scale, chunk, page, seed, kernel, give_back=0, rows_from=0):
    """The attention kernels on one sequence whose pages lie scattered in a larger pool.  `kernel`: "simt" (one warp a row),
    "rows", "keys" or "split" (the tensor-core kernel over tiles of 64 rows, of 16 rows, of 16 rows with three CTAs a tile).
    `give_back`: so many of the first pages are -1 in the table, as a cache that keeps one chunk's length leaves them;
    `rows_from`: only the rows from there on are computed (decoded tokens and portions late in a sequence)."""
    from mini_rsglang_b200 import kernels

    T_, H, d = q.shape
    G, e = k.shape[1], v.shape[2]
    gen = torch.Generator().manual_seed(seed)
    pages = -(-T_ // page)
    pool = pages + 5
    table = torch.randperm(pool, generator=gen)[:pages].to(torch.int32)
    kc = torch.full((pool, G, page, d), 7.0, dtype=dtype, device=DEV)         # other pages hold values that would show
    vc = torch.full((pool, G, page, e), -9.0, dtype=dtype, device=DEV)
    place = torch.arange(T_)
    page_of, at = table.long()[place // page].to(DEV), (place % page).to(DEV)
    kc[page_of, :, at] = k.to(dtype).to(DEV)
    vc[page_of, :, at] = v.to(dtype).to(DEV)
    table[:give_back] = -1
    n = T_ - rows_from
    qd = q[rows_from:].to(dtype).to(DEV).reshape(n, H * d).contiguous()
    sink_d = sinks.float().to(DEV).contiguous() if sinks is not None else None
    out = torch.empty(n, H * e, dtype=dtype, device=DEV)
    positions = torch.arange(rows_from, T_, dtype=torch.int32, device=DEV)
    if kernel == "simt":
        kernels.attention_biased_simt(qd, kc, vc, positions, torch.zeros(n, dtype=torch.int32, device=DEV), table.view(1, -1).to(DEV),
                                      out, H, G, d, e, scale, sink_logits=sink_d, chunk=chunk)
    else:
        per = (64 if kernel == "rows" else 16) // (H // G)
        tiles = torch.tensor([[0, first, min(per, n - first), 0] for first in range(0, n, per)] + [[0, 0, 0, 0]],
                             dtype=torch.int32, device=DEV)                  # and an entry without tokens, as padded lists have
        kernels.attention_biased_mma(qd, kc, vc, positions, table.view(1, -1).to(DEV), tiles, out, H, G, d, e, scale,
                                     narrow=kernel != "rows", splits=3 if kernel == "split" else 1, sink_logits=sink_d, chunk=chunk)
    return out.double().cpu().view(n, H, e)


@pytest.mark.parametrize("H,G,d,e,chunk,page", [(6, 2, 24, 20, 19, 4), (2, 2, 8, 12, 7, 16), (3, 1, 12, 28, 0, 8), (1, 1, 48, 72, 1, 4),
                                                (4, 1, 130, 16, 64, 16), (2, 2, 256, 256, 50, 16)])
def test_chunked_attention_kernel_random(H, G, d, e, chunk, page):
    T_ = 150
    torch.manual_seed(H * 100 + d)
    q, k, v = torch.randn(T_, H, d).double(), torch.randn(T_, G, d).double(), torch.randn(T_, G, e).double()
    sinks = torch.randn(H).double() * 2
    scale = 1.5 / d ** 0.5
    want = plain_chunk_attention(q, k, v, sinks, scale, chunk)
    got = run_chunk_attention(torch.float32, q, k, v, sinks, scale, chunk, page, 3, "simt")
    assert (got - want).abs().max() < 2e-5 * max(1.0, want.abs().max().item())
    no_sink = run_chunk_attention(torch.float32, q, k, v, None, scale, chunk, page, 3, "simt")
    assert (no_sink - plain_chunk_attention(q, k, v, None, scale, chunk)).abs().max() < 2e-5 * max(1.0, want.abs().max().item())
    q16, k16, v16 = (x.bfloat16().double() for x in (q, k, v))
    want16 = plain_chunk_attention(q16, k16, v16, sinks, scale, chunk)
    got16 = run_chunk_attention(torch.bfloat16, q, k, v, sinks, scale, chunk, page, 4, "simt")
    assert (got16 - want16).abs().max() < 0.02 * max(1.0, want16.abs().max().item())


@pytest.mark.parametrize("kernel", ["rows", "keys", "split"])
@pytest.mark.parametrize("H,G,d,e,chunk,page", [(4, 1, 16, 32, 24, 16), (16, 2, 64, 64, 1, 16), (2, 2, 32, 16, 1000, 8), (2, 1, 128, 128, 16, 16),
                                                (8, 8, 64, 48, 33, 4), (32, 2, 128, 64, 100, 16), (3, 3, 256, 256, 70, 16)])
def test_tensor_core_chunked_attention_kernel_random(kernel, H, G, d, e, chunk, page):
    if kernel != "rows" and H // G > 16:
        pytest.skip("tiles of 16 rows hold up to 16 query heads a key head")
    T_ = 200
    torch.manual_seed(H * 100 + d)
    q, k, v = torch.randn(T_, H, d), torch.randn(T_, G, d), torch.randn(T_, G, e)
    sinks = (torch.randn(H) * 2).double() if H != 2 else None
    scale = 1.5 / d ** 0.5
    want = plain_chunk_attention(q.bfloat16().double(), k.bfloat16().double(), v.bfloat16().double(), sinks, scale, chunk)
    got = run_chunk_attention(torch.bfloat16, q, k, v, sinks, scale, chunk, page, 4, kernel)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() < 0.02 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("kernel", ["simt", "rows", "keys", "split"])
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("chunk,page,T_", [(19, 4, 210), (64, 16, 210), (7, 8, 100), (120, 16, 300), (16, 16, 210), (0, 16, 700), (1, 16, 70)])
def test_chunked_attention_sees_exactly_its_chunk(kernel, decoded, chunk, page, T_):
    """One key stands out for the query (the others score far below): the first key of the query's chunk, the last of the
    chunk before, the query's own, the one before it, the sequence's very first, keys at page and key-block borders, and
    without chunks a key hundreds of tokens back.  The query is the last token, a token in the middle of its chunk, the first
    and the last of a chunk; it is part of a prompt's portion (`decoded` False: the rows from the chunk before on are one
    portion) or decoded alone.  Pages that lie wholly more than a chunk's length before the first row are given back.  With a wrong edge the
    output is another token's value row, or the sink's nothing."""
    H, G, d, e = 2, 1, 16, 16
    dtype, tol = (torch.float32, 1e-5) if kernel == "simt" else (torch.bfloat16, 0.03)
    size = chunk or T_
    queries = sorted({T_ - 1, (T_ - 1) // size * size, (T_ - 1) // size * size - 1, max((T_ - 1) // size * size - size // 2 - 1, 0)} & set(range(T_)))
    for i in queries:
        start = i // size * size
        targets = sorted({start, start - 1, i, i - 1, 0, 3, start // page * page, start // page * page - 1, (i // page) * page - 1,
                          (i // page) * page, i - 63, i - 64, i - 65, 127, 128} & set(range(i + 1)))
        first_row = i if decoded else max(start - size, 0)
        give_back = max(first_row - size + 1, 0) // page if chunk else 0          # what a cache that keeps `chunk` keys has let go
        for target in targets:
            torch.manual_seed(chunk * 1000 + target)
            q, k, v = 0.01 * torch.randn(i + 1, H, d).double(), 0.01 * torch.randn(i + 1, G, d).double(), torch.randn(i + 1, G, e).double()
            direction = torch.randn(d).double()
            direction /= direction.norm()
            q[i] = 30.0 * direction
            k[target, 0] = 30.0 * direction
            sinks = torch.tensor([2.0, -1.0]).double()
            if dtype is torch.bfloat16:
                q, k, v = q.bfloat16().double(), k.bfloat16().double(), v.bfloat16().double()
            want = plain_chunk_attention(q, k, v, sinks, 1.0, chunk)
            got = run_chunk_attention(dtype, q, k, v, sinks, 1.0, chunk, page, target, kernel, give_back, first_row)
            seen = start <= target <= i
            alone = (want[i, 0] - v[target, 0]).abs().max()
            assert (alone < 1e-2) == seen, f"query {i}, key {target}: the plain implementation itself does not single the key out"
            assert (got - want[first_row:]).abs().max() < tol, f"query {i}, key {target} (seen: {seen}) with chunks of {chunk}"


def test_a_heavy_sink_takes_the_weight_from_the_keys():
    """A sink far above every score leaves next to nothing of the values, one far below changes nothing, and each head has its own."""
    torch.manual_seed(8)
    T_, H, G, d, e = 40, 4, 2, 16, 16
    q, k, v = torch.randn(T_, H, d).double(), torch.randn(T_, G, d).double(), torch.randn(T_, G, e).double() + 3.0
    sinks = torch.tensor([25.0, -25.0, 0.0, 3.0]).double()
    for kernel, dtype in (("simt", torch.float32), ("rows", torch.bfloat16), ("keys", torch.bfloat16), ("split", torch.bfloat16)):
        got = run_chunk_attention(dtype, q, k, v, sinks, 0.25, 9, 4 if kernel == "simt" else 16, 1, kernel)
        qq, kk, vv = (q, k, v) if dtype is torch.float32 else (q.bfloat16().double(), k.bfloat16().double(), v.bfloat16().double())
        want = plain_chunk_attention(qq, kk, vv, sinks, 0.25, 9)
        without = plain_chunk_attention(qq, kk, vv, None, 0.25, 9)
        tol = 2e-5 if dtype is torch.float32 else 0.03
        assert (got - want).abs().max() < tol * max(1.0, want.abs().max().item())
        assert got[:, 0].abs().max() < 1e-6 and (got[:, 1] - without[:, 1]).abs().max() < tol * 5
        assert (got[:, 2] - without[:, 2]).abs().max() > 0.1


@pytest.mark.parametrize("q_rank,R,extra,page", [(28, 40, 60, 4), (10, 18, 0, 8), (32, 64, 64, 16), (130, 300, 7, 16)])
def test_both_latents_normed_and_the_gate_of_every_value_element(q_rank, R, extra, page):
    from mini_rsglang_b200 import kernels

    torch.manual_seed(q_rank)
    tokens, pool = 13, 6
    proj = torch.randn(tokens, q_rank + R + extra) * 3
    qw, cw = torch.rand(q_rank) + 0.5, torch.rand(R) + 0.5
    slots = torch.randperm(pool * page)[:tokens].to(torch.int32)
    slots[7] = -1
    want_q = P.rms_norm(proj[:, :q_rank].double(), qw.double(), 1e-5)
    want_c = P.rms_norm(proj[:, q_rank:q_rank + R].double(), cw.double(), 1e-5)
    for dtype, tol in ((torch.float32, 3e-6), (torch.bfloat16, 8e-3)):
        q_latent = torch.empty(tokens, q_rank, dtype=dtype, device=DEV)
        cache = torch.full((pool, 1, page, R), 7.0, dtype=dtype, device=DEV)
        kernels.latent_norms(proj.to(DEV), qw.to(DEV), cw.to(DEV), 1e-5, slots.to(DEV), q_latent, cache)
        assert (q_latent.double().cpu() - want_q).abs().max() < tol * want_q.abs().max()
        flat = cache.double().cpu().view(pool * page, R)
        for t in range(tokens):
            if slots[t] >= 0:
                assert (flat[slots[t]] - want_c[t]).abs().max() < tol * want_c.abs().max(), t
        untouched = sorted(set(range(pool * page)) - {int(s) for s in slots if s >= 0})
        assert (flat[untouched] == 7.0).all()
        kernels.latent_norms(proj.to(DEV), qw.to(DEV), cw.to(DEV), 1e-5, None, q_latent, None)           # a step that keeps nothing
        assert (q_latent.double().cpu() - want_q).abs().max() < tol * want_q.abs().max()
        if extra:
            x = torch.randn(tokens, extra, device=DEV).to(dtype)
            want = x.double().cpu() * torch.sigmoid(proj[:, q_rank + R:].double())
            kernels.sigmoid_gate_mul(x, proj.to(DEV)[:, q_rank + R:])
            assert (x.double().cpu() - want).abs().max() < tol * max(1.0, want.abs().max().item())


def delta_inputs(T_, H, G, d, e, taps, seed):
    gen = torch.Generator().manual_seed(seed)
    channels = 2 * G * d + H * e
    proj = torch.randn(T_, channels + 2 * H + H * e, generator=gen)
    proj[:, channels:channels + 2 * H] *= 3.0
    return proj, dict(conv=torch.randn(channels, taps, generator=gen) * 0.5, a_log=torch.randn(H, generator=gen) * 0.5 - 2.0,
                      dt_bias=torch.randn(H, generator=gen), norm=torch.rand(e, generator=gen) + 0.5)


def plain_delta(proj, w, H, G, d, e, eps):
    """The recurrent mixer between its two projections, from the float64 rows q | k | v | b | a | gate."""
    T_ = proj.shape[0]
    channels = 2 * G * d + H * e
    p = proj.double()
    qkv = P.causal_conv_silu(p[:, :channels], w["conv"].double())
    q = P.unit(qkv[:, :G * d].view(T_, G, d)) * d ** -0.5
    k = P.unit(qkv[:, G * d:2 * G * d].view(T_, G, d))
    v = qkv[:, 2 * G * d:].view(T_, H, e)
    beta = torch.sigmoid(p[:, channels:channels + H])
    decay = torch.exp(-torch.exp(w["a_log"].double()) * torch.nn.functional.softplus(p[:, channels + H:channels + 2 * H] + w["dt_bias"].double()))
    o = torch.stack([P.delta_recurrence(q[:, h // (H // G)], k[:, h // (H // G)], v[:, h], beta[:, h], decay[:, h])[0] for h in range(H)], dim=1)
    return P.rms_norm(o, w["norm"].double(), eps).reshape(T_, H * e) * P.silu(p[:, channels + 2 * H:])


def run_delta(rows, w, state, H, G, d, e, taps, positions, seq_of, q_start, slot_of, eps, dtype=torch.float32, write=True):
    from mini_rsglang_b200 import kernels

    channels = 2 * G * d + H * e
    slots = state.shape[0]
    conv_floats = (taps - 1) * channels
    conv_state = state[:, :conv_floats].view(slots, taps - 1, channels)
    s_state = state[:, conv_floats:].view(slots, H, d, e)
    qkv = torch.empty(rows.shape[0], channels, device=DEV)
    kernels.causal_conv_silu(rows, 0, w["conv"], None, conv_state, positions, seq_of, q_start, slot_of, qkv, update_state=write)
    coef = torch.empty(rows.shape[0], 2 * H, device=DEV)
    kernels.delta_prepare(qkv, rows, channels, channels + H, w["a_log"], w["dt_bias"], coef, G, d, H, e, 1e-6, d ** -0.5)
    o = torch.zeros(rows.shape[0], H * e, device=DEV)
    kernels.delta_scan(qkv, coef, s_state, positions, q_start, slot_of, o, H, G, d, e, write_state=write)
    out = torch.empty(rows.shape[0], H * e, dtype=dtype, device=DEV)
    kernels.head_norm_gate(o, rows[:, channels + 2 * H:], w["norm"], eps, out, H)
    return out


@pytest.mark.parametrize("H,G,d,e,taps", [(4, 2, 24, 12, 3), (3, 3, 40, 10, 2), (1, 1, 16, 16, 1), (4, 1, 64, 32, 4), (2, 1, 130, 70, 4),
                                          (8, 2, 128, 128, 4), (6, 3, 256, 64, 5), (2, 2, 8, 200, 2)])
def test_delta_rule_kernels_in_portions_with_slots_used_again(H, G, d, e, taps):
    """Convolution, unit norms, step sizes and decays, the recurrence and the gated head norm against the plain functions: two
    sequences side by side, cut into portions of 1 to 40 tokens (also shorter than the convolution), in state slots that
    held another sequence's state before; a padding sequence (slot -1) beside them; a step that must leave the state as it is."""
    lengths, cuts = [97, 61], [[40, 1, 2, 1, 1, 33, 19], [1, 1, 3, 56]]
    channels = 2 * G * d + H * e
    slots = 3
    state = torch.full((slots, (taps - 1) * channels + H * d * e), 11.0, device=DEV)        # stale contents
    data = [delta_inputs(n, H, G, d, e, taps, 70 + s) for s, n in enumerate(lengths)]
    w = data[0][1]
    dev = {k: t.to(DEV).contiguous() for k, t in w.items()}
    want = [plain_delta(proj, w, H, G, d, e, 1e-5) for proj, _ in data]
    got = [torch.zeros(n, H * e, dtype=torch.float64) for n in lengths]
    done, use_slots, step = [0, 0], [2, 0], 0
    while any(done[s] < lengths[s] for s in range(2)):
        batch = [(s, cuts[s][step]) for s in range(2) if step < len(cuts[s])]
        step += 1
        rows = torch.cat([data[s][0][done[s]:done[s] + n] for s, n in batch]).to(DEV).contiguous()
        positions = torch.cat([torch.arange(done[s], done[s] + n) for s, n in batch]).to(torch.int32).to(DEV)
        seq_of = torch.cat([torch.full((n,), b) for b, (s, n) in enumerate(batch)]).to(torch.int32).to(DEV)
        starts = [0]
        for _, n in batch:
            starts.append(starts[-1] + n)
        starts.append(starts[-1])                                                # a padding sequence without tokens
        q_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
        slot_of = torch.tensor([use_slots[s] for s, _ in batch] + [-1], dtype=torch.int32, device=DEV)
        if step == 3:
            before = state.clone()
            run_delta(rows, dev, state, H, G, d, e, taps, positions, seq_of, q_start, slot_of, 1e-5, write=False)
            assert torch.equal(state, before), "a step that keeps nothing wrote the state"
        out = run_delta(rows, dev, state, H, G, d, e, taps, positions, seq_of, q_start, slot_of, 1e-5)
        for b, (s, n) in enumerate(batch):
            got[s][done[s]:done[s] + n] = out[starts[b]:starts[b + 1]].double().cpu()
            done[s] += n
    for s in range(2):
        assert (got[s] - want[s]).abs().max() < 2e-4 * max(1.0, want[s].abs().max().item()), f"sequence {s}"
    assert (state[1] == 11.0).all(), "a slot that no sequence holds was written"
    rows = data[0][0][:9].to(DEV).contiguous()                                  # bfloat16 rows out of the same float32 recurrence
    out16 = run_delta(rows, dev, state, H, G, d, e, taps, torch.arange(9, dtype=torch.int32, device=DEV), torch.zeros(9, dtype=torch.int32, device=DEV),
                      torch.tensor([0, 9], dtype=torch.int32, device=DEV), torch.tensor([1], dtype=torch.int32, device=DEV), 1e-5, torch.bfloat16)
    assert (out16.double().cpu() - want[0][:9]).abs().max() < 8e-3 * max(1.0, want[0][:9].abs().max().item())


def test_delta_rule_long_portions_of_many_heads():
    """A long portion of many heads comes as more blocks than the GPU has multiprocessors and takes the recurrence kernel
    with fewer rows of S a thread; the short portion after it takes the usual one from the state that the long one left."""
    H, G, d, e, taps = 40, 8, 128, 64, 2
    length, cuts = 269, [262, 7]
    channels = 2 * G * d + H * e
    proj, w = delta_inputs(length, H, G, d, e, taps, 91)
    dev = {k: t.to(DEV).contiguous() for k, t in w.items()}
    want = plain_delta(proj, w, H, G, d, e, 1e-5)
    state = torch.full((2, (taps - 1) * channels + H * d * e), -7.0, device=DEV)
    got, done = torch.zeros(length, H * e, dtype=torch.float64), 0
    for n in cuts:
        rows = proj[done:done + n].to(DEV).contiguous()
        out = run_delta(rows, dev, state, H, G, d, e, taps, torch.arange(done, done + n, dtype=torch.int32, device=DEV),
                        torch.zeros(n, dtype=torch.int32, device=DEV), torch.tensor([0, n], dtype=torch.int32, device=DEV),
                        torch.tensor([1], dtype=torch.int32, device=DEV), 1e-5)
        got[done:done + n] = out.double().cpu()
        done += n
    assert (got - want).abs().max() < 2e-4 * max(1.0, want.abs().max().item())
    assert (state[0] == -7.0).all()


def test_delta_rule_keeps_a_far_token_and_corrects_it():
    """A head that hardly forgets carries one early token's value over hundreds of single-token steps in its float32 state;
    a later token with the same key and beta 1 replaces it, and the very last token reads the replacement."""
    H, G, d, e, taps, T_ = 1, 1, 8, 4, 1, 400
    channels = 2 * G * d + H * e
    proj = torch.zeros(T_, channels + 2 * H + H * e, dtype=torch.float64)
    key = torch.zeros(d, dtype=torch.float64)
    key[2] = 9.0                                           # silu(9) is all but 9; the unit norm makes it a unit vector
    for t, value in ((5, [1.0, 2.0, 3.0, 4.0]), (200, [-4.0, 3.0, -2.0, 1.0])):
        proj[t, d:2 * d] = key
        proj[t, 2 * d:2 * d + e] = torch.tensor(value, dtype=torch.float64)
    proj[:, channels] = 30.0                               # beta 1
    proj[:, channels + 1] = -30.0                          # a decay of all but 1
    proj[:, channels + 2:] = 1.0
    w = dict(conv=torch.ones(channels, 1, dtype=torch.float64), a_log=torch.full((H,), -4.0, dtype=torch.float64),
             dt_bias=torch.zeros(H, dtype=torch.float64), norm=torch.ones(e, dtype=torch.float64))
    for read_at, remembered in ((150, 5), (T_ - 1, 200)):
        p = proj[:read_at + 1].clone()
        p[read_at, :d] = key                               # the query that asks for the key
        want = plain_delta(p, w, H, G, d, e, 1e-5)
        direction = P.silu(p[remembered, 2 * d:2 * d + e])
        assert torch.nn.functional.cosine_similarity(want[read_at], direction * P.silu(torch.tensor(1.0, dtype=torch.float64)), dim=0) > 0.9999
        dev = {k: t.float().to(DEV).contiguous() for k, t in w.items()}
        state = torch.full((2, H * d * e), 5.0, device=DEV)
        got = torch.zeros(read_at + 1, H * e, dtype=torch.float64)
        for t in range(read_at + 1):
            got[t] = run_delta(p[t:t + 1].float().to(DEV), dev, state, H, G, d, e, taps, torch.tensor([t], dtype=torch.int32, device=DEV),
                               torch.zeros(1, dtype=torch.int32, device=DEV), torch.tensor([0, 1], dtype=torch.int32, device=DEV),
                               torch.tensor([1], dtype=torch.int32, device=DEV), 1e-5)[0].double().cpu()
        assert (got - want).abs().max() < 2e-4 * max(1.0, want.abs().max().item())
        assert (state[0] == 5.0).all()


# ----------------------------------------------------------------------------------------------------------------
# the engine's own entry point and scheduler
# ----------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["X", "Y"])
def test_greedy_generation_through_the_engine(folders, name, dtype):
    """Prompts of unequal lengths, more requests than run at a time (state slots are used again), prompt portions under a small
    token budget beside decoded tokens, 40 generated tokens each (the chunks begin anew among decoded tokens): every token
    is the plain implementation's arg-max, or within rounding of it."""
    from mini_rsglang_b200 import RuntimeConfig, SamplingParams
    from mini_rsglang_b200.engine import EngineHandle

    folder = folders[name]
    config, weights = load_plain(folder)
    prompts = [T.requests_for(config["vocab"], [n], seed=500 + n)["r0"] for n in (3, 50, 1, 77, 20, 31)]
    engine = EngineHandle.load(folder, 0, config=RuntimeConfig(max_seq_len=160, prefill_budget=24, max_running=3, page_size=SHAPES[name][1]),
                               dtype=dtype, num_pages=120 if name == "X" else 40)
    results = engine.generate_many(prompts, SamplingParams(max_tokens=40, ignore_eos=True))
    engine.shutdown()
    for prompt, result in zip(prompts, results):
        assert len(result.token_ids) == 40
        tokens = list(prompt)
        for token in result.token_ids:
            logits = P.forward(config, weights, tokens)[-1]
            best = int(logits.argmax())
            gap = (logits[best] - logits[token]).item()
            limit = 2e-5 * max(1.0, logits.abs().max().item()) if dtype == "float32" else 0.02 * logits.abs().max().item()
            assert token == best or gap <= limit, f"{dtype}: engine chose {token}, plain {best}, gap {gap}"
            tokens.append(token)


def test_command_line_generates_the_plain_tokens(folders):
    """`bin/mini-rsglang generate` on a Nubipel folder: the architecture is found by config.json, prefix sharing (on by
    default on the command line) is switched off with a note because the model keeps windows of keys and recurrent states,
    and the tokens are the plain implementation's."""
    import subprocess
    import sys

    folder = folders["X"]
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
        logits = P.forward(config, weights, sequence)[-1]
        best = int(logits.argmax())
        assert token == best or (logits[best] - logits[token]).item() <= 2e-5 * max(1.0, logits.abs().max().item()), (token, best)
        sequence.append(token)
