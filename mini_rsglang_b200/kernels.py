"""Python face of the engine's CUDA kernels.

Every function checks its tensors (device, dtype, contiguity, sizes) on the host and then
calls one `extern "C"` launcher of the in-tree kernel library with raw pointers and the
current CUDA stream.  There is no other implementation behind these names: without a GPU,
or without the compiled library, they raise `BackendError`."""
from __future__ import annotations

import ctypes
import math
import os

import torch

from .csrc.build import kernel_library, specialised_kernel_library
from .errors import BackendError, InvalidRequest

_c_int, _c_vp, _c_float = ctypes.c_int, ctypes.c_void_p, ctypes.c_float

_SIGNATURES = {
    "mrs_embed": [_c_int, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_float, _c_vp],
    "mrs_patch_tokens": [_c_vp, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_vp],
    "mrs_add_rmsnorm": [_c_int, _c_vp, _c_vp, _c_vp, _c_float, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_vp],
    "mrs_rmsnorm": [_c_int, _c_vp, _c_vp, _c_float, _c_vp, _c_int, _c_int, _c_vp],
    "mrs_qk_norm_rope_store": [_c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_float, _c_vp, _c_vp,
                               _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_vp],
    "mrs_rotation_table": [_c_vp, _c_vp, _c_int, _c_int, _c_vp, _c_vp],
    "mrs_silu_mul": [_c_int, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_vp],
    "mrs_attention_simt": [_c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_int,
                           _c_int, _c_int, _c_float, _c_int, _c_vp],
    "mrs_gemm_f32": [_c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_vp],
    "mrs_argmax": [_c_vp, _c_vp, _c_int, _c_int, _c_vp],
    "mrs_sample": [_c_vp, _c_int, _c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp],
}

_lib = None
_error_readers: list[tuple] = []
launch_count = 0   # launches of the engine's own kernels since import (read by the benchmark)


def library() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device: the engine has no CPU path")
        lib = kernel_library()
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = _c_int
        lib.mrs_error_string.argtypes = [_c_int]
        lib.mrs_error_string.restype = ctypes.c_char_p
        _lib = lib
    return _lib


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)      # the current stream without building an object for it


def _stream() -> int:
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _check(code: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if code != 0:
        raise BackendError(f"{what}: {library().mrs_error_string(code).decode()} (code {code})")


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, dtype, what: str, shape: tuple | None = None) -> None:
    if t.is_cuda and (dtype is None or t.dtype == dtype) and t.is_contiguous() and (shape is None or t.shape == shape):
        return                 # the usual case, in one line: this runs a hundred times a step
    if not t.is_cuda:
        raise BackendError(f"{what}: tensor is not on a CUDA device")
    if dtype is not None and t.dtype != dtype:
        raise InvalidRequest(f"{what}: dtype {t.dtype}, expected {dtype}")
    if not t.is_contiguous():
        raise InvalidRequest(f"{what}: tensor is not contiguous")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise InvalidRequest(f"{what}: shape {tuple(t.shape)}, expected {tuple(shape)}")


_sm_counts: dict[int, int] = {}


def sm_count(device=None) -> int:
    """Multiprocessors of the device (asked once): what launch plans fill."""
    index = torch.device(device).index if device is not None else None
    if index is None:
        index = torch.cuda.current_device()
    if index not in _sm_counts:
        _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _sm_counts[index]


def check_rotation(head_dim: int, rotary_dim: int, pairing: str, magnitude: float) -> None:
    """Refuses a rotation that the kernels do not compute.  They rotate every element of a head, element j
    with element j + head_dim / 2, by angles position * frequency, cosines and sines unscaled."""
    if pairing != "split_half":
        raise InvalidRequest(f"rotation pairing {pairing!r} is not built; the kernels pair element j with j + head_dim / 2 (\"split_half\")")
    if int(rotary_dim) != int(head_dim):
        raise InvalidRequest(f"a rotation of {rotary_dim} of a head's {head_dim} elements is not built; the kernels rotate whole heads")
    if float(magnitude) != 1.0:
        raise InvalidRequest(f"a rotation whose cosines and sines are scaled by {magnitude} is not built")


def _is_bf16(dtype: torch.dtype) -> int:
    if dtype is torch.bfloat16:
        return 1
    if dtype is torch.float32:
        return 0
    raise InvalidRequest(f"activations must be bfloat16 or float32, got {dtype}")


def embed(table: torch.Tensor, ids: torch.Tensor, residual: torch.Tensor, scale: float = 1.0) -> None:
    """residual[t, :] = float32(table[ids[t], :]) * scale."""
    tokens, width = residual.shape
    _need(table, None, "embed table")
    _need(ids, torch.int32, "embed ids", (tokens,))
    _need(residual, torch.float32, "embed output")
    if table.shape[1] != width:
        raise InvalidRequest("embed: width mismatch")
    _check(library().mrs_embed(_is_bf16(table.dtype), table.data_ptr(), ids.data_ptr(), residual.data_ptr(),
                               tokens, width, float(scale), _stream()), "embed")


def patch_tokens(ids: torch.Tensor, rows: torch.Tensor, index: torch.Tensor, sampled: torch.Tensor, vocab: int) -> None:
    """ids[rows[i]] = sampled[index[i]]: the tokens that the step before sampled go into this step's ids on the
    device, before the host has read them."""
    global launch_count
    n = rows.shape[0]
    _need(ids, torch.int32, "token ids")
    _need(rows, torch.int32, "rows", (n,))
    _need(index, torch.int32, "index", (n,))
    _need(sampled, torch.int32, "sampled tokens")
    launch_count += 1
    _check(library().mrs_patch_tokens(ids.data_ptr(), rows.data_ptr(), index.data_ptr(), sampled.data_ptr(), n, int(vocab),
                                      _stream()), "patch_tokens")


def add_rmsnorm(residual: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: torch.Tensor | None = None, write_back: bool = True) -> None:
    """v = residual (+ delta); residual = v when write_back; out = norm(v) * weight.
    With `rows`, out[i] comes from source row rows[i]."""
    n_rows, width = out.shape
    _need(residual, torch.float32, "add_rmsnorm residual")
    _need(weight, torch.float32, "add_rmsnorm weight", (width,))
    _need(out, None, "add_rmsnorm out")
    if residual.shape[1] != width:
        raise InvalidRequest("add_rmsnorm: width mismatch")
    if delta is not None:
        _need(delta, out.dtype, "add_rmsnorm delta", tuple(residual.shape))
    if rows is not None:
        _need(rows, torch.int32, "add_rmsnorm rows", (n_rows,))
    elif residual.shape[0] != n_rows:
        raise InvalidRequest("add_rmsnorm: row count mismatch")
    _check(library().mrs_add_rmsnorm(_is_bf16(out.dtype), residual.data_ptr(), _ptr(delta), weight.data_ptr(),
                                     float(eps), out.data_ptr(), _ptr(rows), n_rows, width, int(write_back),
                                     _stream()), "add_rmsnorm")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    width = x.shape[-1]
    _need(x, out.dtype, "rmsnorm input", tuple(out.shape))
    _need(weight, torch.float32, "rmsnorm weight", (width,))
    _need(out, None, "rmsnorm out")
    _check(library().mrs_rmsnorm(_is_bf16(x.dtype), x.data_ptr(), weight.data_ptr(), float(eps), out.data_ptr(),
                                 x.numel() // width, width, _stream()), "rmsnorm")


def rotation_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """[tokens, d / 2, 2] float32: (cos, sin) of position * inv_freq, computed once a step for every layer that
    rotates by the same frequencies."""
    tokens, half = positions.shape[0], inv_freq.shape[0]
    _need(positions, torch.int32, "positions", (tokens,))
    _need(inv_freq, torch.float32, "inv_freq", (half,))
    out = torch.empty((tokens, half, 2), dtype=torch.float32, device=positions.device)
    _check(library().mrs_rotation_table(positions.data_ptr(), inv_freq.data_ptr(), tokens, half, out.data_ptr(), _stream()),
           "rotation_table")
    return out


def qk_norm_rope_store(qkv: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor | None,
                       v_cache: torch.Tensor | None, positions: torch.Tensor, slots: torch.Tensor | None,
                       q_norm: torch.Tensor | None, k_norm: torch.Tensor | None, eps: float,
                       inv_freq: torch.Tensor | None, nq: int, nkv: int, d: int, page_size: int,
                       rotations: torch.Tensor | None = None) -> None:
    """Per-head norm of q and k, rotary of q and k, q to `q_out`, k and v into the paged cache
    ([pages, nkv, page_size, d]) at `slots`.  Without caches only q is produced.  `rotations`: the step's
    `rotation_table` for these positions and frequencies, if the caller has one; heads of 64, 128 and 256
    elements read their cosines and sines from it (and get one made here otherwise)."""
    tokens = qkv.shape[0]
    write_kv = k_cache is not None
    _need(qkv, None, "qkv", (tokens, (nq + 2 * nkv) * d))
    _need(q_out, qkv.dtype, "q_out", (tokens, nq * d))
    _need(positions, torch.int32, "positions", (tokens,))
    if write_kv:
        _need(k_cache, qkv.dtype, "k cache")
        _need(v_cache, qkv.dtype, "v cache", tuple(k_cache.shape))
        if tuple(k_cache.shape[1:]) != (nkv, page_size, d):
            raise InvalidRequest(f"cache shape {tuple(k_cache.shape)} does not match heads/page/head_dim")
        _need(slots, torch.int32, "slots", (tokens,))
    for w, name in ((q_norm, "q_norm"), (k_norm, "k_norm")):
        if w is not None:
            _need(w, torch.float32, name, (d,))
    if inv_freq is not None:
        _need(inv_freq, torch.float32, "inv_freq", (d // 2,))
        if d in (64, 128, 256):
            if rotations is None:
                rotations = rotation_table(positions, inv_freq)
            _need(rotations, torch.float32, "rotations", (tokens, d // 2, 2))
        else:
            rotations = None
    else:
        rotations = None
    _check(library().mrs_qk_norm_rope_store(_is_bf16(qkv.dtype), qkv.data_ptr(), q_out.data_ptr(), _ptr(k_cache),
                                            _ptr(v_cache), positions.data_ptr(), _ptr(slots), _ptr(q_norm),
                                            _ptr(k_norm), float(eps), _ptr(inv_freq), _ptr(rotations), tokens, nq, nkv, d,
                                            page_size, int(write_kv), _stream()), "qk_norm_rope_store")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, block: int = 0) -> None:
    """out = silu(gate) * up.  `gate_up` holds all gate columns and then all up columns (block 0), or
    alternating blocks of `block` gate columns and the `block` matching up columns."""
    tokens, inter = out.shape
    _need(gate_up, out.dtype, "gate_up", (tokens, 2 * inter))
    _need(out, None, "silu_mul out")
    if block < 0 or (block and inter % block):
        raise InvalidRequest("silu_mul: the width is no multiple of the block")
    _check(library().mrs_silu_mul(_is_bf16(out.dtype), gate_up.data_ptr(), out.data_ptr(), tokens, inter, int(block),
                                  _stream()), "silu_mul")


def attention_simt(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, positions: torch.Tensor,
                   seq_of_token: torch.Tensor, block_table: torch.Tensor, out: torch.Tensor, nq: int, nkv: int,
                   d: int, window: int = 0, scale: float | None = None) -> None:
    """Causal paged attention; one warp per (token, head); any sizes; float32 or bfloat16."""
    tokens = q.shape[0]
    _need(q, None, "q", (tokens, nq * d))
    _need(k_cache, q.dtype, "k cache")
    _need(v_cache, q.dtype, "v cache", tuple(k_cache.shape))
    _need(out, q.dtype, "attention out", (tokens, nq * d))
    _need(positions, torch.int32, "positions", (tokens,))
    _need(seq_of_token, torch.int32, "seq_of_token", (tokens,))
    _need(block_table, torch.int32, "block_table")
    page_size = k_cache.shape[2]
    if tuple(k_cache.shape[1:]) != (nkv, page_size, d):
        raise InvalidRequest("attention: cache shape does not match heads/head_dim")
    _check(library().mrs_attention_simt(_is_bf16(q.dtype), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                        positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(),
                                        out.data_ptr(), tokens, nq, nkv, d, page_size, block_table.shape[1],
                                        float(scale if scale is not None else 1.0 / math.sqrt(d)), int(window),
                                        _stream()), "attention_simt")


def gemm_f32(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = x[M, K] . weight[N, K]^T in true float32 (CUDA-core FMA)."""
    m, k = x.shape
    n = weight.shape[0]
    _need(x, torch.float32, "gemm input")
    _need(weight, torch.float32, "gemm weight", (n, k))
    _need(out, torch.float32, "gemm out", (m, n))
    _check(library().mrs_gemm_f32(x.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k, _stream()), "gemm_f32")


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    rows, vocab = logits.shape
    _need(logits, torch.float32, "logits")
    _need(out, torch.int32, "argmax out", (rows,))
    _check(library().mrs_argmax(logits.data_ptr(), out.data_ptr(), rows, vocab, _stream()), "argmax")


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           seed: torch.Tensor, draw_index: torch.Tensor, out: torch.Tensor) -> None:
    rows, vocab = logits.shape
    _need(logits, torch.float32, "logits")
    _need(temperature, torch.float32, "temperature", (rows,))
    _need(top_k, torch.int32, "top_k", (rows,))
    _need(top_p, torch.float32, "top_p", (rows,))
    _need(seed, torch.int64, "seed", (rows,))
    _need(draw_index, torch.int32, "draw_index", (rows,))
    _need(out, torch.int32, "sample out", (rows,))
    _check(library().mrs_sample(logits.data_ptr(), rows, vocab, temperature.data_ptr(), top_k.data_ptr(),
                                top_p.data_ptr(), seed.data_ptr(), draw_index.data_ptr(), out.data_ptr(),
                                _stream()), "sample")


# ------------------------------------------------------------------------------------------------
# tensor-core attention, one library per head size
# ------------------------------------------------------------------------------------------------
_attention_libs: dict[int, ctypes.CDLL] = {}
_scratch: dict[torch.device, torch.Tensor] = {}

MMA_ROWS_WIDE, MMA_ROWS_NARROW = 64, 16


def attention_mma_supported(d: int, group: int) -> bool:
    return d % 16 == 0 and 16 <= d <= 256 and group <= MMA_ROWS_WIDE


def attention_mma_library(d: int) -> ctypes.CDLL:
    """The tensor-core attention compiled for head size `d` (built at first use)."""
    if d not in _attention_libs:
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device: the engine has no CPU path")
        lib = specialised_kernel_library("attention_mma.cu", {"MRS_HEAD_DIM": d})
        lib.mrs_attention_mma_rows_mode.argtypes = [_c_vp] * 5 + [_c_int, _c_vp, _c_int, _c_vp, _c_int, _c_int, _c_int,
                                                    _c_float, _c_int, _c_vp]
        lib.mrs_attention_mma_rows_mode.restype = _c_int
        lib.mrs_attention_mma_keys_mode.argtypes = [_c_vp] * 5 + [_c_int, _c_vp, _c_int, _c_vp, _c_vp, _c_int, _c_int,
                                                    _c_int, _c_float, _c_int, _c_int, _c_vp]
        lib.mrs_attention_mma_keys_mode.restype = _c_int
        lib.mrs_attention_mma_scratch_floats.argtypes = [_c_int, _c_int, _c_int]
        lib.mrs_attention_mma_scratch_floats.restype = ctypes.c_longlong
        _attention_libs[d] = lib
    return _attention_libs[d]


_retired: list[torch.Tensor] = []     # outgrown scratch buffers: recorded steps may still point at them


def attention_scratch(device: torch.device, floats: int, lane: int = 0) -> torch.Tensor:
    """Scratch memory for split attention, kept and grown per device.  A buffer that is outgrown
    is never freed: a step recorded earlier replays with its address.  `lane`: the attention for few rows
    (0) and the one for prompt portions (1) have buffers of their own, because a step that holds both runs
    them side by side."""
    have = _scratch.get((device, lane))
    if have is None or have.numel() < floats:
        if have is not None:
            _retired.append(have)
        have = torch.empty(max(2 * floats, 1 << 22), dtype=torch.float32, device=device)
        _scratch[(device, lane)] = have
    return have


_side_streams: dict[torch.device, torch.cuda.Stream] = {}


def side_stream(device: torch.device) -> torch.cuda.Stream:
    """A second stream of the device, for kernels of one step that do not depend on one another."""
    if device not in _side_streams:
        _side_streams[device] = torch.cuda.Stream(device=device)
    return _side_streams[device]


_counters: dict[torch.device, torch.Tensor] = {}


def attention_counters(device: torch.device, count: int) -> torch.Tensor:
    """Zeroed ints by which the CTAs of a split attention find out which of them is last; the
    kernel leaves them zero.  Outgrown buffers stay alive like the scratch."""
    have = _counters.get(device)
    if have is None or have.numel() < count:
        if have is not None:
            _retired.append(have)
        have = torch.zeros(max(2 * count, 4096), dtype=torch.int32, device=device)
        _counters[device] = have
    return have


def _attention_mma_checks(q, k_cache, v_cache, positions, block_table, tiles, out, nq, nkv, d):
    tokens = q.shape[0]
    _need(q, torch.bfloat16, "q", (tokens, nq * d))
    _need(k_cache, torch.bfloat16, "k cache")
    _need(v_cache, torch.bfloat16, "v cache", tuple(k_cache.shape))
    _need(out, torch.bfloat16, "attention out", (tokens, nq * d))
    _need(positions, torch.int32, "positions", (tokens,))
    _need(block_table, torch.int32, "block_table")
    _need(tiles, torch.int32, "tiles")
    if tiles.dim() != 2 or tiles.shape[1] != 4:
        raise InvalidRequest("attention tiles must be [n, 4] (sequence, first token, tokens, 0)")
    if tuple(k_cache.shape[1:]) != (nkv, k_cache.shape[2], d):
        raise InvalidRequest("attention: cache shape does not match heads/head_dim")


def attention_mma_rows(q, k_cache, v_cache, positions, block_table, tiles, out, nq: int, nkv: int, d: int,
                       window: int = 0, scale: float | None = None) -> None:
    """Tiles of up to 64 // (nq // nkv) tokens of one request each."""
    _attention_mma_checks(q, k_cache, v_cache, positions, block_table, tiles, out, nq, nkv, d)
    lib = attention_mma_library(d)
    _check(lib.mrs_attention_mma_rows_mode(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), positions.data_ptr(),
                                           block_table.data_ptr(), block_table.shape[1], tiles.data_ptr(),
                                           tiles.shape[0], out.data_ptr(), nq, nkv, k_cache.shape[2],
                                           float(scale if scale is not None else 1.0 / math.sqrt(d)), int(window),
                                           _stream()), "attention_mma_rows")


def attention_mma_keys(q, k_cache, v_cache, positions, block_table, tiles, out, nq: int, nkv: int, d: int,
                       window: int = 0, splits: int = 1, scale: float | None = None,
                       scratch: torch.Tensor | None = None) -> None:
    """Tiles of up to 16 // (nq // nkv) tokens each; `splits` CTAs share the keys of a tile."""
    global launch_count
    _attention_mma_checks(q, k_cache, v_cache, positions, block_table, tiles, out, nq, nkv, d)
    lib = attention_mma_library(d)
    if splits > 1:
        need = lib.mrs_attention_mma_scratch_floats(tiles.shape[0], nkv, splits)
        if scratch is None:
            scratch = attention_scratch(q.device, need)
        _need(scratch, torch.float32, "attention scratch")
        if scratch.numel() < need:
            raise InvalidRequest(f"attention scratch holds {scratch.numel()} floats, {need} are needed")
        launch_count += 1          # the combine kernel
    _check(lib.mrs_attention_mma_keys_mode(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), positions.data_ptr(),
                                           block_table.data_ptr(), block_table.shape[1], tiles.data_ptr(),
                                           tiles.shape[0], out.data_ptr(), _ptr(scratch) if splits > 1 else None,
                                           nq, nkv, k_cache.shape[2],
                                           float(scale if scale is not None else 1.0 / math.sqrt(d)), int(window),
                                           int(splits), _stream()), "attention_mma_keys")


# ------------------------------------------------------------------------------------------------
# decode attention fed by bulk tensor copies (TMA), one library per head size (multiples of 64)
# ------------------------------------------------------------------------------------------------
_decode_libs: dict[int, ctypes.CDLL] = {}
_tensor_maps: dict[tuple, tuple] = {}


def attention_decode_tma_supported(d: int, group: int, page_size: int) -> bool:
    return d % 64 == 0 and 64 <= d <= 256 and group <= MMA_ROWS_NARROW and page_size >= 8


def attention_decode_tma_library(d: int) -> ctypes.CDLL:
    if d not in _decode_libs:
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device: the engine has no CPU path")
        lib = specialised_kernel_library("attention_decode_tma.cu", {"MRS_HEAD_DIM": d})
        lib.mrs_attention_decode_tma_map.argtypes = [_c_vp, ctypes.c_longlong, _c_int, _c_int, _c_vp]
        lib.mrs_attention_decode_tma_map.restype = _c_int
        lib.mrs_attention_decode_tma.argtypes = [_c_vp] * 5 + [_c_int, _c_vp, _c_int, _c_vp, _c_vp, _c_vp, _c_int, _c_int,
                                                 _c_int, _c_float, _c_int, _c_int, _c_float, _c_vp]
        lib.mrs_attention_decode_tma.restype = _c_int
        lib.mrs_attention_decode_tma_scratch_floats.argtypes = [_c_int, _c_int, _c_int]
        lib.mrs_attention_decode_tma_scratch_floats.restype = ctypes.c_longlong
        lib.mrs_attention_decode_tma_resident_clusters.argtypes = [_c_int]
        lib.mrs_attention_decode_tma_resident_clusters.restype = _c_int
        lib.mrs_attention_decode_tma_take_error.argtypes = [ctypes.POINTER(ctypes.c_uint)]
        lib.mrs_attention_decode_tma_take_error.restype = _c_int
        lib.mrs_attention_decode_tma_error_string.argtypes = [_c_int]
        lib.mrs_attention_decode_tma_error_string.restype = ctypes.c_char_p
        _decode_libs[d] = lib
        _register_error_word(f"attention_decode_tma (head size {d})", lib, "mrs_attention_decode_tma")
    return _decode_libs[d]


_resident_clusters: dict[tuple, int] = {}


def attention_decode_tma_resident_clusters(d: int, splits: int, device) -> int:
    """Thread-block clusters of `splits` CTAs of the decode attention (head size d) that the GPU holds at once, as
    the driver states it (B200, head size 128: 148, 71, 33 and 14 clusters of 2, 4, 8 and 16); 0 where no such
    cluster runs."""
    key = (d, splits, torch.device(device).index or 0)
    if key not in _resident_clusters:
        with torch.cuda.device(device):
            _resident_clusters[key] = int(attention_decode_tma_library(d).mrs_attention_decode_tma_resident_clusters(splits))
    return _resident_clusters[key]


def _aligned_block(size: int, alignment: int):
    """Host memory for a descriptor: (object that keeps it alive, aligned address)."""
    raw = ctypes.create_string_buffer(size + alignment)
    address = (ctypes.addressof(raw) + alignment - 1) // alignment * alignment
    return raw, address


def kv_tensor_map(cache: torch.Tensor) -> int:
    """Address of the tensor map of one layer's key or value pages [pages, kv_heads, page_size, d]
    (made once per tensor)."""
    key = (cache.data_ptr(), tuple(cache.shape))
    if key not in _tensor_maps:
        pages, nkv, page_size, d = cache.shape
        lib = attention_decode_tma_library(d)
        keep, address = _aligned_block(128, 64)
        code = lib.mrs_attention_decode_tma_map(cache.data_ptr(), pages, nkv, page_size, address)
        if code != 0:
            raise BackendError(f"tensor map of the cache: {lib.mrs_attention_decode_tma_error_string(code).decode()}")
        _tensor_maps[key] = (keep, address)
    return _tensor_maps[key][1]


def attention_decode_tma(q, k_cache, v_cache, positions, block_table, tiles, out, nq: int, nkv: int, d: int,
                         window: int = 0, splits: int = 1, scale: float | None = None,
                         scratch: torch.Tensor | None = None, cap: float = 0.0) -> None:
    """Tiles of up to 16 // (nq // nkv) tokens each; keys and values come through bulk tensor copies.  `scale`: of the
    scores (None: 1 / sqrt(d)); `cap` > 0: the scaled scores are bent into (-cap, cap), cap * tanh(score / cap)."""
    global launch_count
    _attention_mma_checks(q, k_cache, v_cache, positions, block_table, tiles, out, nq, nkv, d)
    lib = attention_decode_tma_library(d)
    counters = None
    if splits > 1:
        need = lib.mrs_attention_decode_tma_scratch_floats(tiles.shape[0], nkv, splits)
        if scratch is None:
            scratch = attention_scratch(q.device, need)
        _need(scratch, torch.float32, "attention scratch")
        if scratch.numel() < need:
            raise InvalidRequest(f"attention scratch holds {scratch.numel()} floats, {need} are needed")
        counters = attention_counters(q.device, tiles.shape[0] * nkv)
    code = lib.mrs_attention_decode_tma(kv_tensor_map(k_cache), kv_tensor_map(v_cache), q.data_ptr(), positions.data_ptr(),
                                        block_table.data_ptr(), block_table.shape[1], tiles.data_ptr(), tiles.shape[0],
                                        out.data_ptr(), _ptr(scratch) if splits > 1 else None, _ptr(counters), nq, nkv,
                                        k_cache.shape[2],
                                        float(scale if scale is not None else 1.0 / math.sqrt(d)), int(window),
                                        int(splits), float(cap), _stream())
    launch_count += 1
    if code != 0:
        raise BackendError(f"attention_decode_tma: {lib.mrs_attention_decode_tma_error_string(code).decode()} (code {code})")


# ------------------------------------------------------------------------------------------------
# tcgen05 attention for prompt portions, one library per head size (64, 128)
# ------------------------------------------------------------------------------------------------
_prefill_libs: dict[int, ctypes.CDLL] = {}
_prefill_kv_maps: dict[tuple, tuple] = {}
_prefill_q_map: dict[torch.device, tuple] = {}
PREFILL_TC_ROWS = 256          # two tiles of 128 query rows a CTA
PREFILL_TC_TILES = 2           # a tile holds 128 // group tokens (a group that does not divide 128 leaves rows empty)


def attention_prefill_tc_supported(d: int, group: int, page_size: int) -> bool:
    return d in (64, 128) and 1 <= group <= PREFILL_TC_ROWS // PREFILL_TC_TILES and page_size >= 8


def attention_prefill_tc_key_block(d: int) -> int:
    """Keys of one block of the tcgen05 kernel for prompt portions (the unit of its shares of a long context)."""
    lib = attention_prefill_tc_library(d)
    lib.mrs_attention_prefill_tc_key_block.restype = _c_int
    return lib.mrs_attention_prefill_tc_key_block()


def attention_prefill_tc_library(d: int) -> ctypes.CDLL:
    if d not in _prefill_libs:
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device: the engine has no CPU path")
        lib = specialised_kernel_library("attention_prefill_tc.cu", {"MRS_HEAD_DIM": d})
        lib.mrs_attention_prefill_tc_kv_map.argtypes = [_c_vp, ctypes.c_longlong, _c_int, _c_int, _c_vp]
        lib.mrs_attention_prefill_tc_q_map.argtypes = [_c_vp, ctypes.c_longlong, _c_int, _c_int, _c_vp]
        lib.mrs_attention_prefill_tc.argtypes = [_c_vp] * 5 + [_c_int, _c_vp, _c_int, _c_vp, _c_int, _c_int, _c_int, _c_float,
                                                 _c_int, _c_vp, _c_int, _c_float, _c_vp]
        lib.mrs_attention_prefill_tc_partial_floats.argtypes = [_c_int, _c_int]
        lib.mrs_attention_prefill_tc_partial_floats.restype = ctypes.c_longlong
        for name in ("mrs_attention_prefill_tc_kv_map", "mrs_attention_prefill_tc_q_map", "mrs_attention_prefill_tc"):
            getattr(lib, name).restype = _c_int
        lib.mrs_attention_prefill_tc_take_error.argtypes = [ctypes.POINTER(ctypes.c_uint)]
        lib.mrs_attention_prefill_tc_take_error.restype = _c_int
        lib.mrs_attention_prefill_tc_error_string.argtypes = [_c_int]
        lib.mrs_attention_prefill_tc_error_string.restype = ctypes.c_char_p
        lib.mrs_attention_prefill_tc_rows.restype = _c_int
        if lib.mrs_attention_prefill_tc_rows() != PREFILL_TC_ROWS:
            raise BackendError(f"attention_prefill_tc takes {lib.mrs_attention_prefill_tc_rows()} rows a CTA, the planner expects {PREFILL_TC_ROWS}")
        _prefill_libs[d] = lib
        _register_error_word(f"attention_prefill_tc (head size {d})", lib, "mrs_attention_prefill_tc")
    return _prefill_libs[d]


def attention_prefill_tc(q, k_cache, v_cache, positions, block_table, tiles, out, nq: int, nkv: int, d: int,
                         window: int = 0, scale: float | None = None, shares: bool = False, cap: float = 0.0) -> None:
    """Work entries of up to 256 // (nq // nkv) tokens of one request each, on the tcgen05 tensor cores; `scale` of the
    scores (None: 1 / sqrt(d)), `cap` > 0: the scaled scores are bent into (-cap, cap), cap * tanh(score / cap).  The
    fourth number of an entry is 0, or index | count << 8 when `count` entries (one after the other in the list)
    walk one share of the keys each (`shares` says that the list has such entries, whose sums a second kernel
    merges), or gap << 16 when the entry's second tile of 128 // (nq // nkv) tokens starts `gap` tokens behind
    the end of its first (the entry's token count is that of both tiles)."""
    global launch_count
    _attention_mma_checks(q, k_cache, v_cache, positions, block_table, tiles, out, nq, nkv, d)
    lib = attention_prefill_tc_library(d)

    def fail(code, what):
        raise BackendError(f"{what}: {lib.mrs_attention_prefill_tc_error_string(code).decode()} (code {code})")

    maps = []
    for cache in (k_cache, v_cache):
        key = (cache.data_ptr(), tuple(cache.shape))
        if key not in _prefill_kv_maps:
            keep, address = _aligned_block(128, 64)
            code = lib.mrs_attention_prefill_tc_kv_map(cache.data_ptr(), cache.shape[0], nkv, cache.shape[2], address)
            if code != 0:
                fail(code, "tensor map of the cache")
            _prefill_kv_maps[key] = (keep, address)
        maps.append(_prefill_kv_maps[key][1])
    if q.device not in _prefill_q_map:
        _prefill_q_map[q.device] = _aligned_block(128, 64)
    q_map = _prefill_q_map[q.device][1]
    code = lib.mrs_attention_prefill_tc_q_map(q.data_ptr(), q.shape[0], nq, nq // nkv, q_map)
    if code != 0:
        fail(code, "tensor map of the queries")
    launch_count += 2 if shares else 1
    partials = attention_scratch(q.device, lib.mrs_attention_prefill_tc_partial_floats(tiles.shape[0], nkv), lane=1) if shares else None
    code = lib.mrs_attention_prefill_tc(q_map, maps[0], maps[1], positions.data_ptr(), block_table.data_ptr(),
                                        block_table.shape[1], tiles.data_ptr(), tiles.shape[0], out.data_ptr(), nq, nkv,
                                        k_cache.shape[2], float(scale if scale is not None else 1.0 / math.sqrt(d)),
                                        int(window), _ptr(partials), int(shares), float(cap), _stream())
    if code != 0:
        fail(code, "attention_prefill_tc")


# ------------------------------------------------------------------------------------------------
# tcgen05 matrix product for few rows (decoded tokens, short portions)
# ------------------------------------------------------------------------------------------------
_gemm_lib = None
_weight_maps: dict[tuple, tuple] = {}
_gemm_state: dict[torch.device, dict] = {}
GEMM_TC_MAX_ROWS = 128          # what the kernel takes
# Measured in the engine (decode steps at a context of 4,096, with the norms riding on the products), this kernel against
# the library's products: batch 8 9% faster; batch 16 5.13 against 5.22 ms a step at the 8B shape, 8.83 against 8.94 ms
# at the 14B shape (context 8,192), 2.36 against 2.46 ms at the 0.6B shape; batch 32 8.15 against 6.65 ms.  Its epilogue
# (a thread a weight row, looping over the rows) and the partial sums of the ranges of K grow with the rows.
GEMM_TC_BEST_ROWS = int(os.environ.get("MRS_GEMM_TC_BEST_ROWS", "16"))      # the variable: for measuring other crossovers


def gemm_tc_library() -> ctypes.CDLL:
    global _gemm_lib
    if _gemm_lib is None:
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device: the engine has no CPU path")
        lib = specialised_kernel_library("gemm_tc.cu", {})
        lib.mrs_gemm_tc_map.argtypes = [_c_vp, ctypes.c_longlong, ctypes.c_longlong, _c_int, _c_vp]
        lib.mrs_gemm_tc_map.restype = _c_int
        lib.mrs_gemm_tc_splits.argtypes = [_c_int, _c_int, _c_int]
        lib.mrs_gemm_tc_splits.restype = _c_int
        lib.mrs_gemm_tc_partial_floats.argtypes = [_c_int, _c_int, _c_int]
        lib.mrs_gemm_tc_partial_floats.restype = ctypes.c_longlong
        lib.mrs_gemm_tc_counters.argtypes = [_c_int]
        lib.mrs_gemm_tc_counters.restype = _c_int
        lib.mrs_gemm_tc_small_m.argtypes = [_c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_int,
                                            _c_int, _c_int, _c_vp, _c_vp]
        lib.mrs_gemm_tc_small_m.restype = _c_int
        lib.mrs_gemm_tc_qkv_heads.argtypes = [_c_vp] * 10 + [_c_float, _c_int, _c_int, _c_int, _c_vp, _c_vp, _c_int, _c_int,
                                              _c_int, _c_int, _c_int, _c_vp, _c_vp]
        lib.mrs_gemm_tc_qkv_heads.restype = _c_int
        lib.mrs_gemm_tc_take_error.argtypes = [ctypes.POINTER(ctypes.c_uint)]
        lib.mrs_gemm_tc_take_error.restype = _c_int
        lib.mrs_gemm_tc_error_string.argtypes = [_c_int]
        lib.mrs_gemm_tc_error_string.restype = ctypes.c_char_p
        _gemm_lib = lib
        _register_error_word("gemm_tc", lib, "mrs_gemm_tc")
    return _gemm_lib


def gemm_tc_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Few rows, bfloat16, rows of a multiple of 8 elements on 16-byte boundaries: what the bulk
    tensor copies need."""
    return (x.dtype is torch.bfloat16 and weight.dtype is torch.bfloat16 and 0 < x.shape[0] <= GEMM_TC_MAX_ROWS
            and x.shape[1] % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def _gemm_device_state(device: torch.device) -> dict:
    state = _gemm_state.get(device)
    if state is None:
        state = {"sms": sm_count(device),
                 "counters": torch.zeros(4096, dtype=torch.int32, device=device),
                 "partials": torch.empty(1 << 24, dtype=torch.float32, device=device),
                 "x_map": _aligned_block(128, 64)}
        _gemm_state[device] = state
    return state


class _NormLink(ctypes.Structure):
    """The product's ties to the norms around it (`NormLink` of csrc/kernels/gemm_tc.cu)."""

    _fields_ = [("in_square_sums", _c_vp), ("in_parts", _c_int), ("in_stride", _c_int), ("in_inv_width", _c_float),
                ("in_eps", _c_float), ("stream", _c_vp), ("next_weight", _c_vp), ("out_square_sums", _c_vp)]


def _gemm_tc_prepare(x: torch.Tensor, weight: torch.Tensor, splits: int | None, max_mpad: int = 128):
    """Tensor maps, ranges of K and scratch for a product x . weight^T; returns (lib, state, w_map, x_map, splits, mpad)."""
    m, k = x.shape
    n = weight.shape[0]
    lib = gemm_tc_library()
    state = _gemm_device_state(x.device)
    key = (weight.data_ptr(), n, k)
    if key not in _weight_maps:
        keep, address = _aligned_block(128, 64)
        code = lib.mrs_gemm_tc_map(weight.data_ptr(), n, k, 128, address)
        if code != 0:
            _gemm_fail(lib, code, "tensor map of a weight")
        _weight_maps[key] = (keep, address, lib.mrs_gemm_tc_splits(n, k, state["sms"]))
    _, w_map, planned = _weight_maps[key]
    splits = planned if splits is None else int(splits)      # another count only for measurements and tests
    mpad = 16 if m <= 16 else (32 if m <= 32 else (64 if m <= 64 else 128))
    if mpad > max_mpad:
        raise InvalidRequest(f"this product takes at most {max_mpad} rows, got {m}")
    x_map = state["x_map"][1]
    code = lib.mrs_gemm_tc_map(x.data_ptr(), m, k, mpad, x_map)
    if code != 0:
        _gemm_fail(lib, code, "tensor map of the activations")
    if splits > 1:
        need = lib.mrs_gemm_tc_partial_floats(m, n, splits)
        if state["partials"].numel() < need:       # outgrown buffers stay alive: recorded steps hold their addresses
            _retired.append(state["partials"])
            state["partials"] = torch.empty(2 * int(need), dtype=torch.float32, device=x.device)
        tiles = lib.mrs_gemm_tc_counters(n)
        if state["counters"].numel() < tiles:
            _retired.append(state["counters"])
            state["counters"] = torch.zeros(2 * tiles, dtype=torch.int32, device=x.device)
    return lib, state, w_map, x_map, splits, mpad


def _gemm_fail(lib, code, what):
    raise BackendError(f"{what}: {lib.mrs_gemm_tc_error_string(code).decode()} (code {code})")


def _norm_link(m: int, row_sums, stream=None, next_weight=None, out_sums=None):
    """The link structure of a product (or None): `row_sums` = (parts of the rows' sums of squares [parts, stride],
    the norm's width, its eps) of activations that are still to be divided by their root mean square."""
    if row_sums is None and stream is None:
        return None
    link = _NormLink()
    if row_sums is not None:
        sums, width, eps = row_sums
        _need(sums, torch.float32, "sums of squares")
        if sums.dim() != 2 or sums.shape[1] < m:
            raise InvalidRequest(f"sums of squares {tuple(sums.shape)} do not cover {m} rows")
        link.in_square_sums, link.in_parts, link.in_stride = sums.data_ptr(), sums.shape[0], sums.shape[1]
        link.in_inv_width, link.in_eps = 1.0 / float(width), float(eps)
    if stream is not None:
        link.stream, link.next_weight, link.out_square_sums = stream.data_ptr(), next_weight.data_ptr(), out_sums.data_ptr()
    return link


def gemm_tc(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, gated: bool = False,
            splits: int | None = None, row_sums: tuple | None = None, residual: tuple | None = None) -> torch.Tensor | None:
    """out[M, N] = x[M, K] . weight[N, K]^T for M <= 128; bfloat16 in, float32 sums, `out` bfloat16 or float32.
    With `gated`, `weight` holds, in every block of 128 rows, 64 gate rows and then the 64 matching up rows, and
    out[M, N / 2] = silu(x . gate^T) * (x . up^T) in bfloat16.

    The RMSNorms around a product can ride on it.  `row_sums` = (parts [P, >= M] float32, width, eps): x holds
    rows that were multiplied by a norm's weights but not yet divided by their root mean square; the product
    multiplies row i's sums by rsqrt(sum_p parts[p, i] / width + eps).  `residual` = (stream [M, N] float32,
    next_weight [N] float32), up to 32 rows: stream += bfloat16(x . weight^T), out = bfloat16(stream *
    next_weight), and the parts of the new rows' sums of squares are returned ([ceil(N / 128), 16 or 32])."""
    m, k = x.shape
    n = weight.shape[0]
    _need(x, torch.bfloat16, "gemm input")
    _need(weight, torch.bfloat16, "gemm weight", (n, k))
    if gated:
        if n % 128:
            raise InvalidRequest("a gated product needs whole blocks of 64 gate and 64 up rows")
        _need(out, torch.bfloat16, "gemm out", (m, n // 2))
    else:
        _need(out, None, "gemm out", (m, n))
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise InvalidRequest("gemm out must be bfloat16 or float32")
    if m > GEMM_TC_MAX_ROWS:
        raise InvalidRequest(f"gemm_tc takes at most {GEMM_TC_MAX_ROWS} rows, got {m}")
    lib, state, w_map, x_map, splits, mpad = _gemm_tc_prepare(x, weight, splits, 32 if residual is not None else 128)
    out_sums = None
    if residual is not None:
        stream, next_weight = residual
        if gated or out.dtype is not torch.bfloat16:
            raise InvalidRequest("the product that adds to the stream is plain and writes bfloat16")
        _need(stream, torch.float32, "stream", (m, n))
        _need(next_weight, torch.float32, "next norm's weight", (n,))
        out_sums = torch.empty(((n + 127) // 128, mpad), dtype=torch.float32, device=x.device)
        link = _norm_link(m, row_sums, stream, next_weight, out_sums)
    else:
        link = _norm_link(m, row_sums)
    global launch_count
    launch_count += 1
    code = lib.mrs_gemm_tc_small_m(w_map, x_map, out.data_ptr(), int(out.dtype is torch.float32), int(gated),
                                   state["partials"].data_ptr(), state["counters"].data_ptr(), m, n, k, splits, mpad,
                                   state["sms"], ctypes.byref(link) if link is not None else None, _stream())
    if code != 0:
        _gemm_fail(lib, code, "gemm_tc")
    return out_sums


_qkv_heads_limits: tuple[int, int] | None = None


def gemm_tc_qkv_heads_limits() -> tuple[int, int]:
    """(head size, most rows) of the fused q/k/v projection, as its library states them."""
    global _qkv_heads_limits
    if _qkv_heads_limits is None:
        lib = gemm_tc_library()
        lib.mrs_gemm_tc_qkv_head_dim.restype = lib.mrs_gemm_tc_qkv_max_rows.restype = _c_int
        _qkv_heads_limits = (lib.mrs_gemm_tc_qkv_head_dim(), lib.mrs_gemm_tc_qkv_max_rows())
    return _qkv_heads_limits


def gemm_tc_qkv_heads_supported(x: torch.Tensor, weight: torch.Tensor, head_dim: int) -> bool:
    """Whether the fused q/k/v projection (head norms, rotation and cache write in the product's epilogue) takes
    these rows: the head size that the library's tiles are made for, few enough rows, and what `gemm_tc` needs."""
    if not gemm_tc_supported(x, weight):
        return False
    d, rows = gemm_tc_qkv_heads_limits()
    return head_dim == d and x.shape[0] <= rows


def gemm_tc_qkv_heads(x: torch.Tensor, weight: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor | None,
                      v_cache: torch.Tensor | None, positions: torch.Tensor, slots: torch.Tensor | None,
                      q_norm: torch.Tensor | None, k_norm: torch.Tensor | None, eps: float,
                      inv_freq: torch.Tensor | None, nq: int, nkv: int, row_sums: tuple | None = None) -> None:
    """The fused q/k/v projection for up to 32 rows and heads of 128 elements, with the per-head norms, the
    rotation and the cache write in the product's epilogue (what `qk_norm_rope_store` does after a product).
    `row_sums`: as for `gemm_tc`."""
    m, k = x.shape
    d, most = gemm_tc_qkv_heads_limits()
    _need(x, torch.bfloat16, "qkv input")
    _need(weight, torch.bfloat16, "qkv weight", ((nq + 2 * nkv) * d, k))
    _need(q_out, torch.bfloat16, "q_out", (m, nq * d))
    _need(positions, torch.int32, "positions", (m,))
    if m > most:
        raise InvalidRequest(f"the fused projection takes at most {most} rows, got {m}")
    page_size = 1
    if slots is not None:
        _need(slots, torch.int32, "slots", (m,))
        _need(k_cache, torch.bfloat16, "k cache")
        _need(v_cache, torch.bfloat16, "v cache", tuple(k_cache.shape))
        if tuple(k_cache.shape[1:]) != (nkv, k_cache.shape[2], d):
            raise InvalidRequest(f"cache shape {tuple(k_cache.shape)} does not match heads/head_dim")
        page_size = k_cache.shape[2]
    for w, name in ((q_norm, "q_norm"), (k_norm, "k_norm")):
        if w is not None:
            _need(w, torch.float32, name, (d,))
    if inv_freq is not None:
        _need(inv_freq, torch.float32, "inv_freq", (d // 2,))
    lib, state, w_map, x_map, splits, mpad = _gemm_tc_prepare(x, weight, None, most)
    link = _norm_link(m, row_sums)
    global launch_count
    launch_count += 1
    code = lib.mrs_gemm_tc_qkv_heads(w_map, x_map, q_out.data_ptr(), _ptr(k_cache) if slots is not None else None,
                                     _ptr(v_cache) if slots is not None else None, positions.data_ptr(), _ptr(slots),
                                     _ptr(q_norm), _ptr(k_norm), _ptr(inv_freq), float(eps), nq, nkv, page_size,
                                     state["partials"].data_ptr(), state["counters"].data_ptr(), m, k, splits, mpad,
                                     state["sms"], ctypes.byref(link) if link is not None else None, _stream())
    if code != 0:
        _gemm_fail(lib, code, "gemm_tc_qkv_heads")


# ------------------------------------------------------------------------------------------------
# the tcgen05 gate/up product for many rows (prompt portions) with the activation in its epilogue
# ------------------------------------------------------------------------------------------------
_many_rows_lib = None
_many_rows_maps: dict[tuple, tuple] = {}
# Measured against the library's product followed by `silu_mul` (8B shape, K 4096, N 24576): 290 against 299 us at
# 2,048 rows, 418 against 429 us at 3,072, 550 against 646 us at 4,096; below 2,048 rows the library's pair is ahead
# (1,536: 221 against 217 us; 512: 90 against 83 us: the 128 x 256 tiles fill the SMs' last round badly).  At other
# shapes the order differs (prefill of 2,048 tokens: 14B shape, K 5120, N 34816: 58.2 ms with this kernel against
# 57.7 ms; 0.6B shape, K 1024, N 6144: 4.9 against 4.4 ms), so from GEMM_GATED_ROWS_MIN rows on the two are timed
# once per (N, K, thousand of rows) on the first such product and the faster one is kept (`gemm_gated_rows_wins`).
GEMM_GATED_ROWS_MIN = int(os.environ.get("MRS_GEMM_GATED_ROWS_MIN", "2048"))      # the variable: for measuring other crossovers
GEMM_GATED_MEASURE = "MRS_GEMM_GATED_ROWS_MIN" not in os.environ                  # False: the kernel from that many rows on
_gated_rows_choice: dict[tuple, bool] = {}


def gemm_gated_rows_wins(x: torch.Tensor, weight: torch.Tensor, gate: str = "silu") -> bool:
    """Whether the tcgen05 gate/up product with the activation in it is the faster way for these sizes on this
    device: at least GEMM_GATED_ROWS_MIN rows, and ahead of the library's product followed by `silu_mul` when the
    two were timed (three runs each after one, CUDA events, on buffers of their own; never while a step is being
    recorded: such steps have fewer rows anyway)."""
    rows = x.shape[0]
    if rows < GEMM_GATED_ROWS_MIN or not gemm_gated_rows_supported(x, weight):
        return False
    if not GEMM_GATED_MEASURE:
        return True
    n, k = weight.shape
    key = (x.device, n, k, gate, 1 << (rows - 1).bit_length() if rows <= 1024 else 1024 * min(-(-rows // 1024), 16))
    if torch.cuda.is_current_stream_capturing():         # a step being recorded ran once just before: the choice is made
        return _gated_rows_choice.get(key, False)
    if key not in _gated_rows_choice:
        act = torch.empty((rows, n // 2), dtype=torch.bfloat16, device=x.device)

        def own():
            gemm_gated_rows(x, weight, act, gate)

        def library():
            if gate == "silu":
                silu_mul(torch.mm(x, weight.t()), act, 64)
            else:
                gated_activation(torch.mm(x, weight.t()), act, gate, 64)

        times = []
        for run in (own, library):
            run()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(3):
                run()
            end.record()
            end.synchronize()
            times.append(start.elapsed_time(end))
        _gated_rows_choice[key] = times[0] <= times[1]
    return _gated_rows_choice[key]


def gemm_many_rows_library() -> ctypes.CDLL:
    global _many_rows_lib
    if _many_rows_lib is None:
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device: the engine has no CPU path")
        lib = specialised_kernel_library("gemm_many_rows.cu", {})
        lib.mrs_gemm_many_rows_map.argtypes = [_c_vp, ctypes.c_longlong, ctypes.c_longlong, _c_int, _c_vp]
        lib.mrs_gemm_many_rows_map.restype = _c_int
        lib.mrs_gemm_gated_rows.argtypes = [_c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_int, _c_int, _c_vp]
        lib.mrs_gemm_gated_rows.restype = _c_int
        lib.mrs_gemm_act_rows.argtypes = [_c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_int, _c_int, _c_vp]
        lib.mrs_gemm_act_rows.restype = _c_int
        lib.mrs_gemm_many_rows_take_error.argtypes = [ctypes.POINTER(ctypes.c_uint)]
        lib.mrs_gemm_many_rows_take_error.restype = _c_int
        lib.mrs_gemm_many_rows_error_string.argtypes = [_c_int]
        lib.mrs_gemm_many_rows_error_string.restype = ctypes.c_char_p
        _many_rows_lib = lib
        _register_error_word("gemm_many_rows", lib, "mrs_gemm_many_rows")
    return _many_rows_lib


def _many_rows_maps_of(lib, x: torch.Tensor, weight: torch.Tensor):
    """(keep-alive of the activations' map, its address, the weights' map's address)."""
    n, k = weight.shape
    key = (weight.data_ptr(), n, k)
    if key not in _many_rows_maps:
        keep, address = _aligned_block(128, 64)
        code = lib.mrs_gemm_many_rows_map(weight.data_ptr(), n, k, 256, address)
        if code != 0:
            raise BackendError(f"tensor map of a weight: {lib.mrs_gemm_many_rows_error_string(code).decode()} (code {code})")
        _many_rows_maps[key] = (keep, address)
    x_keep, x_map = _aligned_block(128, 64)
    code = lib.mrs_gemm_many_rows_map(x.data_ptr(), x.shape[0], k, 128, x_map)
    if code != 0:
        raise BackendError(f"tensor map of the activations: {lib.mrs_gemm_many_rows_error_string(code).decode()} (code {code})")
    return x_keep, x_map, _many_rows_maps[key][1]


def gemm_gated_rows_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """bfloat16, rows of a multiple of 8 elements on 16-byte boundaries, whole blocks of 64 gate and 64 up rows."""
    return (x.dtype is torch.bfloat16 and weight.dtype is torch.bfloat16 and x.shape[1] % 8 == 0 and weight.shape[0] % 128 == 0
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


GATE_ACTIVATIONS = ("silu", "relu")       # what the tcgen05 gate/up product applies to the gate in its epilogue


def gemm_gated_rows(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, gate: str = "silu") -> None:
    """out[T, N / 2] = act(x . gate^T) * (x . up^T) in bfloat16 for any number of rows, act "silu" or "relu"; `weight`
    [N, K] holds, in every block of 128 rows, 64 gate rows and then the 64 matching up rows (as the gated `gemm_tc`)."""
    if gate not in GATE_ACTIVATIONS:
        raise InvalidRequest(f"the gated product applies one of {GATE_ACTIVATIONS} to the gate, not {gate!r}")
    global launch_count
    t, k = x.shape
    n = weight.shape[0]
    _need(x, torch.bfloat16, "gated product input")
    _need(weight, torch.bfloat16, "gated product weight", (n, k))
    _need(out, torch.bfloat16, "gated product out", (t, n // 2))
    if not gemm_gated_rows_supported(x, weight):
        raise InvalidRequest("the gated product needs K a multiple of 8, whole blocks of 64 gate and 64 up rows and 16-byte alignment")
    lib = gemm_many_rows_library()
    x_keep, x_map, w_map = _many_rows_maps_of(lib, x, weight)
    launch_count += 1
    code = lib.mrs_gemm_gated_rows(x_map, w_map, out.data_ptr(), t, n, k, ACTIVATIONS[gate], sm_count(x.device), _stream())
    del x_keep
    if code != 0:
        raise BackendError(f"gemm_gated_rows: {lib.mrs_gemm_many_rows_error_string(code).decode()} (code {code})")


def gemm_act_rows_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """bfloat16, rows of a multiple of 8 elements on 16-byte boundaries, a multiple of 32 weight rows."""
    return (x.dtype is torch.bfloat16 and weight.dtype is torch.bfloat16 and x.shape[1] % 8 == 0 and weight.shape[0] % 32 == 0
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def gemm_act_rows(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, kind: str) -> None:
    """out[T, N] = act(x . weight^T) in bfloat16 for any number of rows, the activation (one of ACTIVATIONS, computed in
    float32 on the float32 sums) in the product's epilogue: the ungated counterpart of `gemm_gated_rows`."""
    global launch_count
    t, k = x.shape
    n = weight.shape[0]
    _need(x, torch.bfloat16, "activated product input")
    _need(weight, torch.bfloat16, "activated product weight", (n, k))
    _need(out, torch.bfloat16, "activated product out", (t, n))
    if kind not in ACTIVATIONS:
        raise InvalidRequest(f"activation {kind!r} is not built; known: {sorted(ACTIVATIONS)}")
    if not gemm_act_rows_supported(x, weight):
        raise InvalidRequest("the activated product needs K a multiple of 8, N a multiple of 32 and 16-byte alignment")
    lib = gemm_many_rows_library()
    x_keep, x_map, w_map = _many_rows_maps_of(lib, x, weight)
    launch_count += 1
    code = lib.mrs_gemm_act_rows(x_map, w_map, out.data_ptr(), t, n, k, ACTIVATIONS[kind], sm_count(x.device), _stream())
    del x_keep
    if code != 0:
        raise BackendError(f"gemm_act_rows: {lib.mrs_gemm_many_rows_error_string(code).decode()} (code {code})")


_act_rows_choice: dict[tuple, bool] = {}


def gemm_act_rows_wins(x: torch.Tensor, weight: torch.Tensor, kind: str) -> bool:
    """`gemm_gated_rows_wins` for the ungated product: at least GEMM_GATED_ROWS_MIN rows, and ahead of the library's
    product followed by `activation` when the two were timed for these sizes (once, outside a recording)."""
    rows = x.shape[0]
    if rows < GEMM_GATED_ROWS_MIN or not gemm_act_rows_supported(x, weight):
        return False
    if not GEMM_GATED_MEASURE:
        return True
    n, k = weight.shape
    key = (x.device, n, k, kind, 1024 * min(-(-rows // 1024), 16))
    if torch.cuda.is_current_stream_capturing():
        return _act_rows_choice.get(key, False)
    if key not in _act_rows_choice:
        act = torch.empty((rows, n), dtype=torch.bfloat16, device=x.device)

        def own():
            gemm_act_rows(x, weight, act, kind)

        def library():
            torch.mm(x, weight.t(), out=act)
            activation(act, act, kind)

        times = []
        for run in (own, library):
            run()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(3):
                run()
            end.record()
            end.synchronize()
            times.append(start.elapsed_time(end))
        _act_rows_choice[key] = times[0] <= times[1]
    return _act_rows_choice[key]


def wait_probe(limit_cycles: int = 1 << 16, device=None) -> bool:
    """Runs a one-warp kernel whose only act is a bounded wait on a barrier at which nobody arrives, with a limit
    of `limit_cycles` clocks (at most 2^24: milliseconds).  The wait gives up as every wait of the engine's
    kernels does when its time runs out: it raises the error word of its library and the kernel returns.
    Returns whether the wait gave up (it always does).  For the tests of the error path: `check_device_errors`
    raises afterwards, and the device is as usable as before."""
    lib = gemm_tc_library()
    lib.mrs_gemm_tc_wait_probe.argtypes = [ctypes.c_longlong, _c_vp, _c_vp]
    lib.mrs_gemm_tc_wait_probe.restype = _c_int
    flag = torch.zeros(1, dtype=torch.int32, device=device or torch.device("cuda", torch.cuda.current_device()))
    code = lib.mrs_gemm_tc_wait_probe(int(limit_cycles), flag.data_ptr(), _stream())
    if code != 0:
        _gemm_fail(lib, code, "wait_probe")
    torch.cuda.current_stream().synchronize()
    return bool(flag.item())


# ------------------------------------------------------------------------------------------------
# error words of the kernels that wait on barriers
# ------------------------------------------------------------------------------------------------
_mirror_view = None
_mirror = None          # pinned host words, one per library, that the kernels' error words are mirrored into


def _register_error_word(what: str, lib, prefix: str) -> None:
    """Keeps the library's reader and points its mirror at the next free pinned word."""
    global _mirror, _mirror_view
    if _mirror is None:
        _mirror = torch.zeros(16, dtype=torch.int32).pin_memory()
        _mirror_view = _mirror.numpy()
    index = len(_error_readers)
    reader = getattr(lib, f"{prefix}_take_error")
    _error_readers.append((what, reader))
    mirror = getattr(lib, f"{prefix}_mirror_errors")
    mirror.argtypes = [_c_vp]
    mirror.restype = _c_int
    if index < _mirror.numel():
        code = mirror(_mirror.data_ptr() + 4 * index)
        if code != 0:
            raise BackendError(f"{what}: cannot mirror the error word (CUDA error {code})")


def check_device_errors(certain: bool = False) -> None:
    """Raises when a kernel gave up a wait.  Called after a step, when the device is idle: the
    kernels mirror their error words into pinned host memory, so all is well as long as those
    words are zero; only then (or when `certain`) the words are read from the device and cleared."""
    if _mirror is not None and not certain and len(_error_readers) <= _mirror.numel() and not _mirror_view.any():
        return
    if _mirror is not None:
        _mirror.zero_()
    failed = []
    for what, reader in _error_readers:       # every word is read, and with that cleared
        word = ctypes.c_uint(0)
        code = reader(ctypes.byref(word))
        if code != 0:
            raise BackendError(f"{what}: reading the error word failed (CUDA error {code})")
        if word.value:
            failed.append(f"{what}: a kernel gave up waiting (error word {word.value:#x})")
    if failed:
        # a kernel that gave up may have left the arrival counters of its splits half counted: the next launch
        # that shares them must find zeros
        for counters in list(_counters.values()) + [state["counters"] for state in _gemm_state.values()]:
            counters.zero_()
        raise BackendError("; ".join(failed) + "; the step's result is invalid")


# ------------------------------------------------------------------------------------------------
# layers with a norm after each branch, biased and windowed attention, state-space recurrences
# ------------------------------------------------------------------------------------------------
_c_ll = ctypes.c_longlong
_HYBRID_SIGNATURES = {
    "mrs_postnorm_add_norm": [_c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_float, _c_float, _c_vp, _c_int, _c_int, _c_float, _c_vp],
    "mrs_glu_clamped": [_c_int, _c_vp, _c_vp, _c_int, _c_int, _c_float, _c_float, _c_vp],
    "mrs_qkv_bias_store": [_c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_int, _c_int,
                           _c_int, _c_int, _c_float, _c_int, _c_vp, _c_vp, _c_float, _c_vp],
    "mrs_gated_part_norm": [_c_int, _c_vp, _c_vp, _c_int, _c_vp, _c_float, _c_vp, _c_int, _c_int, _c_int, _c_vp],
    "mrs_causal_conv_silu": [_c_vp, _c_int, _c_int, _c_vp, _c_vp, _c_vp, _c_ll, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_int, _c_int,
                             _c_int, _c_int, _c_int, _c_vp],
    "mrs_ssm_scan": [_c_vp, _c_vp, _c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_ll, _c_vp, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int,
                     _c_int, _c_int, _c_int, _c_int, _c_int, _c_vp, _c_vp],
}
_hybrid_lib = None


def hybrid_library() -> ctypes.CDLL:
    global _hybrid_lib
    if _hybrid_lib is None:
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device: the engine has no CPU path")
        from .csrc.build import hybrid_kernel_library

        lib = hybrid_kernel_library()
        for name, argtypes in _HYBRID_SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = _c_int
        _hybrid_lib = lib
    return _hybrid_lib


def postnorm_add_norm(stream: torch.Tensor, branch: torch.Tensor, post_weight: torch.Tensor, post_eps: float,
                      next_weight: torch.Tensor | None, next_eps: float, out: torch.Tensor | None, mult: float = 1.0) -> None:
    """stream += mult * rmsnorm(branch) * post_weight; with `next_weight`, out = rmsnorm(stream) * next_weight.
    `branch` holds a product's float32 sums; the norms and the sum are float32."""
    rows, width = stream.shape
    _need(stream, torch.float32, "postnorm stream")
    _need(branch, torch.float32, "postnorm branch", (rows, width))
    _need(post_weight, torch.float32, "postnorm weight", (width,))
    if next_weight is not None:
        _need(next_weight, torch.float32, "next norm weight", (width,))
        _need(out, None, "postnorm out", (rows, width))
    _check(hybrid_library().mrs_postnorm_add_norm(_is_bf16(out.dtype) if out is not None else 0, stream.data_ptr(),
                                                  branch.data_ptr(), post_weight.data_ptr(), _ptr(next_weight), float(post_eps),
                                                  float(next_eps), _ptr(out), rows, width, float(mult), _stream()), "postnorm_add_norm")


def glu_clamped(gate_up: torch.Tensor, out: torch.Tensor, limit: float, alpha: float) -> None:
    """out = g * sigmoid(alpha * g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit); `gate_up` holds
    all gate columns and then all up columns."""
    tokens, inter = out.shape
    _need(gate_up, out.dtype, "gate_up", (tokens, 2 * inter))
    _need(out, None, "glu_clamped out")
    _check(hybrid_library().mrs_glu_clamped(_is_bf16(out.dtype), gate_up.data_ptr(), out.data_ptr(), tokens, inter, float(limit),
                                            float(alpha), _stream()), "glu_clamped")


def qkv_bias_store(proj: torch.Tensor, bias: torch.Tensor | None, q_out: torch.Tensor, k_cache: torch.Tensor | None,
                   v_cache: torch.Tensor | None, slots: torch.Tensor | None, nq: int, nkv: int, d: int, e: int,
                   v_first: torch.Tensor | None = None, mix_mode: int = 0, mix: float = 0.0,
                   gate_out: torch.Tensor | None = None, q_norm: torch.Tensor | None = None, k_norm: torch.Tensor | None = None,
                   norm_eps: float = 0.0) -> None:
    """After the fused projection q | k | v (| one gate column a query head), float32: biases added, q to `q_out`, k into
    the key pages [pages, nkv, page, d], v into the value pages [pages, nkv, page, e] at `slots`, sigmoid(gate) to
    `gate_out` [tokens, nq] float32.  `mix_mode` 1 leaves this layer's values in `v_first` [tokens, nkv * e] float32;
    2 stores (1 - mix) v + mix v_first instead of v.  `q_norm` / `k_norm` [d] float32: every query / key head is divided
    by its root mean square (`norm_eps` inside the root) and multiplied by the weight first (not together with blending)."""
    tokens = proj.shape[0]
    width = nq * d + nkv * d + nkv * e
    _need(proj, torch.float32, "qkv projection", (tokens, width + (nq if gate_out is not None else 0)))
    if bias is not None:
        _need(bias, torch.float32, "qkv bias", (width,))
    _need(q_out, None, "q_out", (tokens, nq * d))
    page_size = 1
    if k_cache is not None:
        page_size = k_cache.shape[2]
        _need(k_cache, q_out.dtype, "key pages")
        _need(v_cache, q_out.dtype, "value pages")
        if tuple(k_cache.shape[1:]) != (nkv, page_size, d) or tuple(v_cache.shape[1:]) != (nkv, page_size, e):
            raise InvalidRequest("qkv_bias_store: the pages do not match heads, page size and head sizes")
        _need(slots, torch.int32, "slots", (tokens,))
    if mix_mode:
        _need(v_first, torch.float32, "v_first", (tokens, nkv * e))
    if gate_out is not None:
        _need(gate_out, torch.float32, "gate", (tokens, nq))
    for w in (q_norm, k_norm):
        if w is not None:
            _need(w, torch.float32, "head norm weight", (d,))
    if (q_norm is not None or k_norm is not None) and mix_mode:
        raise InvalidRequest("qkv_bias_store: head norms together with blended values are not built")
    _check(hybrid_library().mrs_qkv_bias_store(_is_bf16(q_out.dtype), proj.data_ptr(), _ptr(bias), q_out.data_ptr(), _ptr(k_cache),
                                               _ptr(v_cache), _ptr(slots) if k_cache is not None else None, _ptr(v_first),
                                               _ptr(gate_out), tokens, nq, nkv, d, e, page_size, int(mix_mode), float(mix),
                                               int(gate_out is not None), _ptr(q_norm), _ptr(k_norm), float(norm_eps), _stream()),
           "qkv_bias_store")


def gated_part_norm(y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, parts: int) -> None:
    """out = (y * silu(z)), each of `parts` equal parts of a row divided by its own root mean square, times weight.
    `z` may be a column range of wider float32 rows."""
    tokens, inner = y.shape
    _need(y, torch.float32, "recurrence output")
    if not z.is_cuda or z.dtype != torch.float32 or tuple(z.shape) != (tokens, inner) or z.stride(1) != 1:
        raise InvalidRequest("gated_part_norm: the gate must be float32 [tokens, inner] with unit column stride")
    _need(weight, torch.float32, "part norm weight", (inner,))
    _need(out, None, "part norm out", (tokens, inner))
    if inner % parts:
        raise InvalidRequest("gated_part_norm: the row is no multiple of the parts")
    _check(hybrid_library().mrs_gated_part_norm(_is_bf16(out.dtype), y.data_ptr(), z.data_ptr(), z.stride(0), weight.data_ptr(),
                                                float(eps), out.data_ptr(), tokens, inner, int(parts), _stream()), "gated_part_norm")


_biased_simt_lib = None


def biased_attention_library() -> ctypes.CDLL:
    global _biased_simt_lib
    if _biased_simt_lib is None:
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device: the engine has no CPU path")
        from .csrc.build import biased_attention_library as build

        lib = build()
        lib.mrs_attention_biased_simt.argtypes = [_c_int] + [_c_vp] * 9 + [_c_int] * 7 + [_c_float, _c_float, _c_int, _c_int, _c_int,
                                                                                         _c_int, _c_vp, _c_int, _c_vp]
        lib.mrs_attention_biased_simt.restype = _c_int
        _biased_simt_lib = lib
    return _biased_simt_lib


def attention_biased_simt(q, k_cache, v_cache, positions, seq_of_token, block_table, out, nq: int, nkv: int, d: int, e: int,
                          scale: float, cap: float = 0.0, window: int = 0, keep_first: int = 0, bias: torch.Tensor | None = None,
                          gate: torch.Tensor | None = None, sink: bool = False, sink_logits: torch.Tensor | None = None,
                          chunk: int = 0) -> None:
    """Causal paged attention with a soft cap on the scores, a bias by distance (`bias` float32 [rows, nq], the last row
    for every larger distance), a window that keeps the first `keep_first` positions or (`chunk` > 0, no window) sight
    within the query's own chunk of positions, an optional sink in the softmax (its logit 0, or `sink_logits` [nq] float32)
    and an optional gate a (token, head); keys of d and values of e elements.  `v_cache` None: the values are the first
    e elements of the key rows.  One warp per (token, head)."""
    tokens = q.shape[0]
    _need(q, None, "q", (tokens, nq * d))
    _need(k_cache, q.dtype, "key pages")
    _need(out, q.dtype, "attention out", (tokens, nq * e))
    _need(positions, torch.int32, "positions", (tokens,))
    _need(seq_of_token, torch.int32, "seq_of_token", (tokens,))
    _need(block_table, torch.int32, "block_table")
    page_size = k_cache.shape[2]
    if tuple(k_cache.shape[1:]) != (nkv, page_size, d):
        raise InvalidRequest("attention: the pages do not match heads and head sizes")
    if v_cache is not None:
        _need(v_cache, q.dtype, "value pages")
        if tuple(v_cache.shape[1:]) != (nkv, page_size, e):
            raise InvalidRequest("attention: the pages do not match heads and head sizes")
    elif e > d:
        raise InvalidRequest("attention: values inside the key rows cannot be longer than the rows")
    if bias is not None:
        _need(bias, torch.float32, "distance bias")
        if bias.dim() != 2 or bias.shape[1] != nq:
            raise InvalidRequest("attention: the distance bias must be [rows, query heads]")
    if gate is not None:
        _need(gate, torch.float32, "attention gate", (tokens, nq))
    if sink_logits is not None:
        _need(sink_logits, torch.float32, "sink logits", (nq,))
    _check(biased_attention_library().mrs_attention_biased_simt(
        _is_bf16(q.dtype), q.data_ptr(), k_cache.data_ptr(), _ptr(v_cache), positions.data_ptr(), seq_of_token.data_ptr(),
        block_table.data_ptr(), _ptr(bias), _ptr(gate), out.data_ptr(), tokens, nq, nkv, d, e, page_size, block_table.shape[1],
        float(scale), float(cap), int(window), int(keep_first), bias.shape[0] if bias is not None else 0,
        int(sink or sink_logits is not None), _ptr(sink_logits), int(chunk), _stream()), "attention_biased_simt")


def causal_conv_silu(proj: torch.Tensor, offset: int, weight: torch.Tensor, bias: torch.Tensor | None, conv_state: torch.Tensor,
                     positions, seq_of_token, q_start, state_slots, out: torch.Tensor, update_state: bool = True) -> None:
    """out[t, c] = silu(bias[c] + sum_k weight[c, k] * in[t - (taps - 1 - k), c]) over the columns offset .. offset + channels
    of the float32 rows `proj`, zeros before a sequence's start, inputs of earlier steps from `conv_state`
    [slots, taps - 1, channels] (a view: rows of a wider per-slot state); afterwards the state holds the last taps - 1 inputs."""
    tokens = proj.shape[0]
    channels, taps = weight.shape
    _need(proj, torch.float32, "conv input")
    _need(weight, torch.float32, "conv weight")
    _need(out, torch.float32, "conv out", (tokens, channels))
    if bias is not None:
        _need(bias, torch.float32, "conv bias", (channels,))
    if conv_state.dtype != torch.float32 or conv_state.dim() != 3 or tuple(conv_state.shape[1:]) != (max(taps - 1, 0), channels) or \
            (taps > 1 and (conv_state.stride(2) != 1 or conv_state.stride(1) != channels)):
        raise InvalidRequest("causal_conv_silu: the state must be float32 [slots, taps - 1, channels], dense within a slot")
    if offset < 0 or offset + channels > proj.shape[1]:
        raise InvalidRequest("causal_conv_silu: the channels lie outside the rows")
    sequences = state_slots.shape[0]
    _check(hybrid_library().mrs_causal_conv_silu(proj.data_ptr(), proj.shape[1], int(offset), weight.data_ptr(), _ptr(bias),
                                                 conv_state.data_ptr(), conv_state.stride(0), positions.data_ptr(),
                                                 seq_of_token.data_ptr(), q_start.data_ptr(), state_slots.data_ptr(), out.data_ptr(),
                                                 tokens, sequences, channels, taps, int(update_state), _stream()), "causal_conv_silu")


def ssm_scan(xbc: torch.Tensor, dt: torch.Tensor, dt_bias, a_log, d_skip, ssm_state: torch.Tensor, positions, q_start, state_slots,
             y: torch.Tensor, heads: int, groups: int, n_state: int, head_dim: int, write_state: bool = True,
             chunk_len: int | None = None) -> None:
    """The recurrence S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t with dt_t =
    softplus(raw + dt_bias), per (sequence, head), token by token in float32.  `xbc` [tokens, heads * P + 2 * groups * N]
    float32 holds x | B | C; `dt` the raw step sizes (a column range of wider float32 rows); `ssm_state`
    [slots, heads, N, P] float32 (a view: dense within a slot); a sequence that starts at position 0 starts from zero.
    `chunk_len` 0: every sequence in one go; n > 0: chunks of n rows side by side in three passes (local states, the
    states at the chunks' starts, the outputs); None: chosen from the step's shapes, chunks where long portions of few
    sequences would leave most of the GPU idle."""
    global launch_count
    tokens = xbc.shape[0]
    inner = heads * head_dim
    _need(xbc, torch.float32, "x|B|C", (tokens, inner + 2 * groups * n_state))
    if dt.dtype != torch.float32 or tuple(dt.shape) != (tokens, heads) or dt.stride(1) != 1:
        raise InvalidRequest("ssm_scan: dt must be float32 [tokens, heads] with unit column stride")
    for t, name in ((dt_bias, "dt_bias"), (a_log, "A_log"), (d_skip, "D")):
        _need(t, torch.float32, name, (heads,))
    if ssm_state.dtype != torch.float32 or tuple(ssm_state.shape[1:]) != (heads, n_state, head_dim) or \
            ssm_state.stride(3) != 1 or ssm_state.stride(2) != head_dim or ssm_state.stride(1) != n_state * head_dim:
        raise InvalidRequest("ssm_scan: the state must be float32 [slots, heads, N, P], dense within a slot")
    _need(y, torch.float32, "recurrence output", (tokens, inner))
    sequences = state_slots.shape[0]
    if chunk_len is None:
        chunk_len = ssm_chunk_length(tokens, sequences, heads, n_state, head_dim, sm_count(xbc.device))
    scratch = None
    if chunk_len:
        chunks = -(-tokens // chunk_len)
        scratch = attention_scratch(xbc.device, sequences * heads * chunks * (n_state * head_dim + 1), lane=2)
        launch_count += 2
    _check(hybrid_library().mrs_ssm_scan(xbc.data_ptr(), dt.data_ptr(), dt.stride(0), dt_bias.data_ptr(), a_log.data_ptr(),
                                         d_skip.data_ptr(), ssm_state.data_ptr(), ssm_state.stride(0), positions.data_ptr(),
                                         q_start.data_ptr(), state_slots.data_ptr(), y.data_ptr(), tokens, sequences, heads, groups,
                                         n_state, head_dim, int(write_state), int(chunk_len), _ptr(scratch), _stream()), "ssm_scan")


def ssm_chunk_length(tokens: int, sequences: int, heads: int, n_state: int, head_dim: int, sms: int) -> int:
    """Rows of a chunk of the recurrence, 0 for none, from a step's shapes alone (a recorded step keeps its choice).
    A block (a head's slice of columns, 128 threads) walks its rows one after the other and waits most of the time, so
    long portions are cut into chunks that run side by side, at the price of walking every row twice: measured on a
    B200 with 64 heads of 64 columns and a state of 128 (256 blocks a sequence), 2,048 rows take 1,034 us in one go and
    847, 783, 680, 658 us in chunks of 1,024, 512, 256 and 128 rows (with 64 the pass between the two costs what they
    save).  So: about fourteen blocks an SM, chunks of at least 128 rows, only for portions of 512 rows and more."""
    if os.environ.get("MRS_SSM_CHUNK"):             # the variable: for measuring other chunk lengths
        return int(os.environ["MRS_SSM_CHUNK"]) if tokens >= 512 and tokens >= 128 * sequences else 0
    lanes = 1
    while lanes < 32 and -(-n_state // lanes) > 16:
        lanes *= 2
    slices = -(-head_dim // max(1, min(128 // lanes, head_dim)))
    blocks = sequences * heads * slices
    if tokens < 512 or tokens < 128 * sequences:
        return 0
    chunks = min(-(-14 * sms // blocks), tokens // 128)
    if chunks < 2:
        return 0
    rows = -(-tokens // chunks)
    return -(-rows // 64) * 64


_biased_mma_libs: dict[tuple, ctypes.CDLL] = {}


def attention_biased_mma_supported(d: int, e: int, group: int, page_size: int, values_in_keys: bool = False) -> bool:
    """Head sizes that are multiples of 16 (keys up to 256, or 640 with the values inside their rows; values up to 256),
    groups of up to 64 query heads, pages of a power of two."""
    return (d % 16 == 0 and e % 16 == 0 and 16 <= d <= (640 if values_in_keys else 256) and 16 <= e <= 256
            and (not values_in_keys or e <= d) and group <= MMA_ROWS_WIDE and page_size & (page_size - 1) == 0)


def attention_biased_mma_library(d: int, e: int, values_in_keys: bool = False) -> ctypes.CDLL:
    """The tensor-core biased attention compiled for key heads of `d` and value heads of `e` elements (at first use);
    `values_in_keys`: for caches without value pages, whose values are the first `e` elements of the key rows."""
    key = (d, e, bool(values_in_keys))
    if key not in _biased_mma_libs:
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device: the engine has no CPU path")
        defines = {"MRS_HEAD_DIM": d, "MRS_VALUE_DIM": e}
        if values_in_keys:
            defines["MRS_VALUES_IN_KEYS"] = 1
        lib = specialised_kernel_library("attention_biased_mma.cu", defines)
        lib.mrs_attention_biased_mma.argtypes = [_c_int] + [_c_vp] * 5 + [_c_int, _c_vp, _c_int, _c_vp, _c_vp, _c_int, _c_vp, _c_int,
                                                 _c_int, _c_int, _c_float, _c_float, _c_int, _c_int, _c_int, _c_int, _c_vp, _c_vp, _c_int, _c_vp]
        lib.mrs_attention_biased_mma.restype = _c_int
        lib.mrs_attention_biased_mma_scratch_floats.argtypes = [_c_int, _c_int, _c_int]
        lib.mrs_attention_biased_mma_scratch_floats.restype = ctypes.c_longlong
        _biased_mma_libs[key] = lib
    return _biased_mma_libs[key]


def attention_biased_mma(q, k_cache, v_cache, positions, block_table, tiles, out, nq: int, nkv: int, d: int, e: int, scale: float,
                         cap: float = 0.0, window: int = 0, keep_first: int = 0, bias: torch.Tensor | None = None,
                         gate: torch.Tensor | None = None, sink: bool = False, narrow: bool = False, splits: int = 1,
                         sink_logits: torch.Tensor | None = None, chunk: int = 0) -> None:
    """`attention_biased_simt`'s formulas on the tensor cores, bfloat16, over a list of tiles (sequence, first row, tokens, 0):
    `narrow` tiles hold up to 16 // (nq // nkv) tokens (decoded tokens, short portions), the others up to 64 // (nq // nkv).
    `splits` > 1 (narrow tiles): that many CTAs share a tile's key blocks and a second kernel merges them.
    `v_cache` None: the values are the first `e` elements of the key rows."""
    global launch_count
    tokens = q.shape[0]
    _need(q, torch.bfloat16, "q", (tokens, nq * d))
    _need(k_cache, torch.bfloat16, "key pages")
    if v_cache is not None:
        _need(v_cache, torch.bfloat16, "value pages")
    _need(out, torch.bfloat16, "attention out", (tokens, nq * e))
    _need(positions, torch.int32, "positions", (tokens,))
    _need(block_table, torch.int32, "block_table")
    _need(tiles, torch.int32, "tiles")
    page_size = k_cache.shape[2]
    if tiles.dim() != 2 or tiles.shape[1] != 4:
        raise InvalidRequest("attention tiles must be [n, 4] (sequence, first token, tokens, 0)")
    if tuple(k_cache.shape[1:]) != (nkv, page_size, d) or (v_cache is not None and tuple(v_cache.shape[1:]) != (nkv, page_size, e)):
        raise InvalidRequest("attention: the pages do not match heads and head sizes")
    if bias is not None:
        _need(bias, torch.float32, "distance bias")
        if bias.dim() != 2 or bias.shape[1] != nq:
            raise InvalidRequest("attention: the distance bias must be [rows, query heads]")
    if gate is not None:
        _need(gate, torch.float32, "attention gate", (tokens, nq))
    if sink_logits is not None:
        _need(sink_logits, torch.float32, "sink logits", (nq,))
    lib = attention_biased_mma_library(d, e, values_in_keys=v_cache is None)
    scratch = None
    if splits > 1:
        if not narrow:
            raise InvalidRequest("only tiles of 16 rows share their keys among CTAs")
        scratch = attention_scratch(q.device, lib.mrs_attention_biased_mma_scratch_floats(tiles.shape[0], nkv, splits))
        launch_count += 1
    _check(lib.mrs_attention_biased_mma(int(narrow), q.data_ptr(), k_cache.data_ptr(), _ptr(v_cache), positions.data_ptr(),
                                        block_table.data_ptr(), block_table.shape[1], tiles.data_ptr(), tiles.shape[0], out.data_ptr(),
                                        _ptr(bias), bias.shape[0] if bias is not None else 0, _ptr(gate), nq, nkv, page_size,
                                        float(scale), float(cap), int(window), int(keep_first), int(sink or sink_logits is not None),
                                        int(splits), _ptr(scratch), _ptr(sink_logits), int(chunk), _stream()),
           "attention_biased_mma")


# ------------------------------------------------------------------------------------------------
# layer norms with bias, latent attention, routed experts
# ------------------------------------------------------------------------------------------------
_LATENT_SIGNATURES = {
    "mrs_add_layernorm": [_c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_float, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_vp],
    "mrs_latent_prepare": [_c_int, _c_vp, _c_int, _c_vp, _c_float, _c_vp, _c_float, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp] +
                          [_c_int] * 8 + [_c_vp],
    "mrs_latent_norms": [_c_int, _c_vp, _c_int, _c_vp, _c_vp, _c_float, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_vp],
    "mrs_sigmoid_gate_mul": [_c_int, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_vp],
    "mrs_scale": [_c_vp, ctypes.c_longlong, _c_float, _c_vp],
}
_EXPERT_SIGNATURES = {
    "mrs_moe_route": [_c_vp, _c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_vp],
    "mrs_moe_align": [_c_vp, _c_int, _c_int, _c_int, _c_vp, _c_vp, _c_int, _c_vp],
    "mrs_moe_product_simt": [_c_int, _c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_vp],
    "mrs_moe_product_rows": [_c_int, _c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_vp],
    "mrs_moe_gather_rows": [_c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_vp],
    "mrs_moe_gather_scaled_rows": [_c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_vp],
    "mrs_moe_product_mma": [_c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_vp],
    "mrs_moe_combine": [_c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_int, _c_int, _c_vp],
}
_latent_lib = None
_expert_lib = None


def _typed(lib, signatures: dict):
    for name, argtypes in signatures.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = _c_int
    return lib


def latent_library() -> ctypes.CDLL:
    global _latent_lib
    if _latent_lib is None:
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device: the engine has no CPU path")
        from .csrc.build import latent_kernel_library

        _latent_lib = _typed(latent_kernel_library(), _LATENT_SIGNATURES)
    return _latent_lib


def expert_library() -> ctypes.CDLL:
    global _expert_lib
    if _expert_lib is None:
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device: the engine has no CPU path")
        from .csrc.build import expert_kernel_library

        lib = _typed(expert_kernel_library(), _EXPERT_SIGNATURES)
        lib.mrs_moe_capacity.argtypes = [_c_int, _c_int, _c_int]
        lib.mrs_moe_capacity.restype = ctypes.c_longlong
        for name in ("mrs_moe_simt_tile", "mrs_moe_mma_tile", "mrs_moe_rows_tile"):
            getattr(lib, name).argtypes = []
            getattr(lib, name).restype = _c_int
        _expert_lib = lib
    return _expert_lib


def add_layernorm(residual: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, bias: torch.Tensor, eps: float,
                  out: torch.Tensor, rows: torch.Tensor | None = None, write_back: bool = True) -> None:
    """v = residual (+ delta); residual = v when write_back; out = (v - mean) / sqrt(var + eps) * weight + bias.
    With `rows`, out[i] comes from source row rows[i]."""
    n_rows, width = out.shape
    _need(residual, torch.float32, "add_layernorm residual")
    _need(weight, torch.float32, "add_layernorm weight", (width,))
    _need(bias, torch.float32, "add_layernorm bias", (width,))
    _need(out, None, "add_layernorm out")
    if residual.shape[1] != width:
        raise InvalidRequest("add_layernorm: width mismatch")
    if delta is not None:
        _need(delta, out.dtype, "add_layernorm delta", tuple(residual.shape))
    if rows is not None:
        _need(rows, torch.int32, "add_layernorm rows", (n_rows,))
    elif residual.shape[0] != n_rows:
        raise InvalidRequest("add_layernorm: row count mismatch")
    _check(latent_library().mrs_add_layernorm(_is_bf16(out.dtype), residual.data_ptr(), _ptr(delta), weight.data_ptr(), bias.data_ptr(),
                                              float(eps), out.data_ptr(), _ptr(rows), n_rows, width, int(write_back), _stream()),
           "add_layernorm")


def scale_(x: torch.Tensor, factor: float) -> None:
    """x *= factor, float32, in place."""
    _need(x, torch.float32, "scaled tensor")
    _check(latent_library().mrs_scale(x.data_ptr(), x.numel(), float(factor), _stream()), "scale")


def latent_prepare(proj: torch.Tensor, latent_weight: torch.Tensor | None, eps: float, inv_freq: torch.Tensor | None, magnitude: float,
                   positions: torch.Tensor, slots: torch.Tensor | None, q_plain: torch.Tensor, q_rows: torch.Tensor,
                   cache: torch.Tensor | None, gate: torch.Tensor | None, heads: int, plain: int, rotated: int, latent: int,
                   rotary: int, has_latent: bool) -> None:
    """After the fused float32 projection q | (latent, rotated key part) | (one gate a head) of a latent attention:
    `q_plain` [heads, tokens, plain] gets the unrotated query parts, the last `rotated` columns of `q_rows`
    [tokens, heads, latent + rotated] the rotated ones; with `has_latent`, the latent over its root mean square times
    `latent_weight` and the rotated key part go into `cache` [pages, 1, page, latent + rotated] at `slots` (None, or a
    slot of -1: nowhere); `gate` [tokens, heads] float32 gets the sigmoids.  Of a rotated part the first `rotary`
    elements turn, element i with i + rotary / 2, by position * inv_freq[i], cosines and sines times `magnitude`."""
    tokens, width = proj.shape
    _need(proj, torch.float32, "latent projection")
    _need(q_plain, None, "q_plain", (heads, tokens, plain))
    _need(q_rows, q_plain.dtype, "q_rows", (tokens, heads, latent + rotated))
    _need(positions, torch.int32, "positions", (tokens,))
    if rotary:
        _need(inv_freq, torch.float32, "rotation frequencies", (rotary // 2,))
    if has_latent:
        _need(latent_weight, torch.float32, "latent norm weight", (latent,))
    if cache is not None:
        _need(cache, q_plain.dtype, "latent pages")
        if cache.dim() != 4 or cache.shape[1] != 1 or cache.shape[3] != latent + rotated:
            raise InvalidRequest("latent_prepare: the pages must be [pages, 1, page, latent + rotated]")
        _need(slots, torch.int32, "slots", (tokens,))
    if gate is not None:
        _need(gate, torch.float32, "gate", (tokens, heads))
    _check(latent_library().mrs_latent_prepare(
        _is_bf16(q_plain.dtype), proj.data_ptr(), width, _ptr(latent_weight), float(eps), _ptr(inv_freq), float(magnitude),
        positions.data_ptr(), _ptr(slots) if cache is not None else None, q_plain.data_ptr(), q_rows.data_ptr(), _ptr(cache), _ptr(gate),
        tokens, heads, plain, rotated, latent, rotary, int(has_latent), int(gate is not None), _stream()), "latent_prepare")


def latent_norms(proj: torch.Tensor, q_weight: torch.Tensor, latent_weight: torch.Tensor, eps: float, slots: torch.Tensor | None,
                 q_latent: torch.Tensor, cache: torch.Tensor | None) -> None:
    """After the fused float32 projection query latent | key/value latent | ... of a latent attention that rotates nothing:
    `q_latent` [tokens, q_rank] gets the first columns over their root mean square times `q_weight`; the next `latent`
    columns, normed likewise with `latent_weight`, go into `cache` [pages, 1, page, latent] at `slots` (None, or a slot of
    -1: nowhere)."""
    tokens, width = proj.shape
    q_rank, latent = q_weight.shape[0], latent_weight.shape[0]
    _need(proj, torch.float32, "latent projection")
    if width < q_rank + latent:
        raise InvalidRequest("latent_norms: the projection is narrower than the two latents")
    _need(q_weight, torch.float32, "query latent norm weight", (q_rank,))
    _need(latent_weight, torch.float32, "latent norm weight", (latent,))
    _need(q_latent, None, "query latent", (tokens, q_rank))
    if cache is not None:
        _need(cache, q_latent.dtype, "latent pages")
        if cache.dim() != 4 or cache.shape[1] != 1 or cache.shape[3] != latent:
            raise InvalidRequest("latent_norms: the pages must be [pages, 1, page, latent]")
        _need(slots, torch.int32, "slots", (tokens,))
    _check(latent_library().mrs_latent_norms(_is_bf16(q_latent.dtype), proj.data_ptr(), width, q_weight.data_ptr(), latent_weight.data_ptr(),
                                             float(eps), _ptr(slots) if cache is not None else None, q_latent.data_ptr(), _ptr(cache),
                                             tokens, q_rank, latent, _stream()), "latent_norms")


def sigmoid_gate_mul(x: torch.Tensor, gate: torch.Tensor) -> None:
    """x <- x * sigmoid(gate), element by element, in place; `gate` float32 of x's shape, may be a column range of wider rows."""
    tokens, width = x.shape
    _need(x, None, "gated rows")
    if not gate.is_cuda or gate.dtype != torch.float32 or tuple(gate.shape) != (tokens, width) or gate.stride(1) != 1:
        raise InvalidRequest("sigmoid_gate_mul: the gate must be float32 of the rows' shape with unit column stride")
    _check(latent_library().mrs_sigmoid_gate_mul(_is_bf16(x.dtype), x.data_ptr(), gate.data_ptr(), gate.stride(0), tokens, width,
                                                 _stream()), "sigmoid_gate_mul")


def moe_route(logits: torch.Tensor, correction: torch.Tensor | None, chosen: torch.Tensor, weights: torch.Tensor,
              shared_gate: torch.Tensor | None, experts: int, top: int, scale: float, sigmoid_scores: bool = False,
              normalize: bool = True) -> None:
    """Router logits float32 [tokens, experts (+ 1) or more] -> `chosen` [tokens, top] int32, the `top` experts with the
    largest score + correction, and `weights` [tokens, top] float32, score / (sum of the chosen + 1e-20) * scale; scores
    are the softmax (or the sigmoids) of the first `experts` columns.  With `shared_gate` [tokens] the column after them
    is one more gate, whose sigmoid it gets.  Further columns are not read.  `normalize` False: the weights are score * scale."""
    tokens = logits.shape[0]
    _need(logits, torch.float32, "router logits")
    if logits.dim() != 2 or logits.shape[1] < experts + (1 if shared_gate is not None else 0):
        raise InvalidRequest("moe_route: fewer logits a token than experts")
    if correction is not None:
        _need(correction, torch.float32, "router correction", (experts,))
    _need(chosen, torch.int32, "chosen experts", (tokens, top))
    _need(weights, torch.float32, "expert weights", (tokens, top))
    if shared_gate is not None:
        _need(shared_gate, torch.float32, "shared gate", (tokens,))
    _check(expert_library().mrs_moe_route(logits.data_ptr(), logits.shape[1], _ptr(correction), chosen.data_ptr(), weights.data_ptr(),
                                          _ptr(shared_gate), tokens, experts, top, float(scale), int(sigmoid_scores),
                                          int(shared_gate is not None), int(normalize), _stream()), "moe_route")


def moe_capacity(pairs: int, routed: int, tile: int) -> int:
    """Rows of the expert lists for `pairs` (token, choice) pairs: every expert's run filled up to whole tiles."""
    return int(expert_library().mrs_moe_capacity(pairs, routed, tile))


def moe_simt_tile() -> int:
    return int(expert_library().mrs_moe_simt_tile())


def moe_mma_tile() -> int:
    return int(expert_library().mrs_moe_mma_tile())


def moe_rows_tile() -> int:
    return int(expert_library().mrs_moe_rows_tile())


def moe_rows_supported(x: torch.Tensor, inner: int) -> bool:
    """Rows of a multiple of 16 bytes in both products."""
    piece = 16 // x.element_size()
    return x.shape[1] % piece == 0 and inner % piece == 0


def moe_mma_supported(x: torch.Tensor, inner: int) -> bool:
    """bfloat16 with rows on 16-byte boundaries in both products: the width and the experts' inner size multiples of 8."""
    return x.dtype is torch.bfloat16 and x.shape[1] % 8 == 0 and inner % 8 == 0


def moe_align(chosen: torch.Tensor, routed: int, tile: int, sorted_rows: torch.Tensor, tile_expert: torch.Tensor) -> None:
    """Lists the pairs of `chosen` [tokens, top] that name one of the first `routed` experts, expert by expert, every run
    filled up with -1 to whole tiles: `sorted_rows` [capacity] the pairs (token * top + choice), `tile_expert`
    [capacity / tile + 1] the expert of every tile (-1: unused) and, last, the number of tiles in use."""
    _need(chosen, torch.int32, "chosen experts")
    _need(sorted_rows, torch.int32, "sorted rows")
    _need(tile_expert, torch.int32, "tile experts", (sorted_rows.shape[0] // tile + 1,))
    _check(expert_library().mrs_moe_align(chosen.data_ptr(), chosen.numel(), routed, tile, sorted_rows.data_ptr(), tile_expert.data_ptr(),
                                          sorted_rows.shape[0], _stream()), "moe_align")


def moe_product(x: torch.Tensor, sorted_rows: torch.Tensor, tile_expert: torch.Tensor, weight: torch.Tensor, out: torch.Tensor,
                top: int, gated: bool, kernel: str = "simt", block: int = 0, activation: str | None = None) -> None:
    """One product of the experts over the lists of `moe_align`: `kernel` "simt" (CUDA cores, tiles of `moe_simt_tile()`
    rows, every size), "rows" (CUDA cores, few rows an expert: tiles of `moe_rows_tile()` rows, the weights streamed once;
    rows of a multiple of 16 bytes) or "mma" (mma.sync, bfloat16, k a multiple of 8, tiles of `moe_mma_tile()` rows).
    `gated`: x [tokens, k], weight [experts, 2 n, k] (all gate rows, then all up rows; with `block`, blocks of that many
    gate rows each followed by the matching up rows), out [capacity, n] = silu(gate) * up of every listed pair's token;
    else x [capacity, k], weight [experts, n, k], out [pairs, n] written at the pair; or, with `activation` (one of
    ACTIVATIONS; not gated), out [capacity, n] = activation(sums), written at the rows' places in the lists."""
    capacity = sorted_rows.shape[0]
    if activation is not None and (gated or activation not in ACTIVATIONS):
        raise InvalidRequest(f"moe_product: an activation {sorted(ACTIVATIONS)} goes with the ungated product only")
    act = ACTIVATIONS[activation] if activation is not None else -1
    k = x.shape[1]
    n = out.shape[1]
    _need(x, None, "expert input")
    _need(weight, x.dtype, "expert weights", (weight.shape[0], (2 if gated else 1) * n, k))
    _need(out, x.dtype, "expert output")
    if (out.shape[0] if gated else x.shape[0]) != capacity or (act >= 0 and out.shape[0] != capacity):
        raise InvalidRequest("moe_product: the listed rows do not match the lists")
    if kernel == "mma":
        _need(x, torch.bfloat16, "expert input")
        _check(expert_library().mrs_moe_product_mma(int(gated), x.data_ptr(), sorted_rows.data_ptr(), tile_expert.data_ptr(),
                                                    weight.data_ptr(), out.data_ptr(), capacity, n, k, top, int(block) if gated else 0,
                                                    act, _stream()), "moe_product_mma")
        return
    if kernel == "rows":
        _check(expert_library().mrs_moe_product_rows(_is_bf16(x.dtype), int(gated), x.data_ptr(), sorted_rows.data_ptr(),
                                                     tile_expert.data_ptr(), weight.data_ptr(), out.data_ptr(), capacity, n, k, top,
                                                     int(block) if gated else 0, act, _stream()), "moe_product_rows")
        return
    if kernel != "simt":
        raise InvalidRequest(f"moe_product: unknown kernel {kernel!r}")
    _check(expert_library().mrs_moe_product_simt(_is_bf16(x.dtype), int(gated), x.data_ptr(), sorted_rows.data_ptr(), tile_expert.data_ptr(),
                                                 weight.data_ptr(), out.data_ptr(), capacity, n, k, top, int(block) if gated else 0,
                                                 act, _stream()), "moe_product_simt")


MOE_TC_BLOCK = 64              # gate rows of a block in the layout of the product for many rows; the 64 matching up rows follow
MOE_TC_MIN_PAIRS = int(os.environ.get("MRS_MOE_TC_MIN_PAIRS", "1024"))      # the variables: for measuring other crossovers
MOE_ROWS_MAX_PAIRS = int(os.environ.get("MRS_MOE_ROWS_MAX_PAIRS", "128"))
_moe_tc_lib = None
_moe_tc_maps: dict[tuple, tuple] = {}


def moe_tc_library() -> ctypes.CDLL:
    global _moe_tc_lib
    if _moe_tc_lib is None:
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device: the engine has no CPU path")
        lib = specialised_kernel_library("experts_tc.cu", {})
        lib.mrs_moe_tc_map.argtypes = [_c_vp, ctypes.c_longlong, ctypes.c_longlong, _c_int, _c_vp]
        lib.mrs_moe_tc_map.restype = _c_int
        lib.mrs_moe_product_tc.argtypes = [_c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_int, _c_int, _c_vp]
        lib.mrs_moe_product_tc.restype = _c_int
        lib.mrs_moe_tc_tile.argtypes = []
        lib.mrs_moe_tc_tile.restype = _c_int
        lib.mrs_moe_tc_take_error.argtypes = [ctypes.POINTER(ctypes.c_uint)]
        lib.mrs_moe_tc_take_error.restype = _c_int
        lib.mrs_moe_tc_error_string.argtypes = [_c_int]
        lib.mrs_moe_tc_error_string.restype = ctypes.c_char_p
        _moe_tc_lib = lib
        _register_error_word("moe_product_tc", lib, "mrs_moe_tc")
    return _moe_tc_lib


def moe_tc_supported(x: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, block: int) -> bool:
    """bfloat16, gate and up rows in blocks of 64, a width of a multiple of 8, weights on 16-byte boundaries."""
    return (x.dtype is torch.bfloat16 and block == MOE_TC_BLOCK and x.shape[1] % 8 == 0 and down.shape[2] % MOE_TC_BLOCK == 0
            and gate_up.data_ptr() % 16 == 0 and down.data_ptr() % 16 == 0)


def _moe_tc_map(lib, t: torch.Tensor, rows: int, cols: int, box_rows: int, keep: bool):
    """The address of a tensor map over `t` as a matrix [rows, cols]; kept for weights, made anew for activations."""
    key = (t.data_ptr(), rows, cols, box_rows)
    if keep and key in _moe_tc_maps:
        return _moe_tc_maps[key]
    block, address = _aligned_block(128, 64)
    code = lib.mrs_moe_tc_map(t.data_ptr(), rows, cols, box_rows, address)
    if code != 0:
        raise BackendError(f"tensor map for the experts' product: {lib.mrs_moe_tc_error_string(code).decode()} (code {code})")
    if keep:
        _moe_tc_maps[key] = (block, address)
    return block, address


def moe_product_tc(x_rows: torch.Tensor, sorted_rows: torch.Tensor, tile_expert: torch.Tensor, weight: torch.Tensor, out: torch.Tensor,
                   gated: bool, activation: str | None = None) -> None:
    """One product of the experts on the tcgen05 tensor cores over lists in tiles of 128 rows.  `x_rows` [capacity, k]: the
    rows in the order of the lists.  `gated`: weight [experts, 2 n, k] in blocks of 64 gate and 64 up rows, out
    [capacity, n] = silu(gate) * up; else weight [experts, n, k], out [pairs, n] written at the rows' pairs, or with
    `activation` (one of ACTIVATIONS) out [capacity, n] = activation(sums) at the rows' places."""
    global launch_count
    if activation is not None and (gated or activation not in ACTIVATIONS):
        raise InvalidRequest(f"moe_product_tc: an activation {sorted(ACTIVATIONS)} goes with the ungated product only")
    capacity, k = x_rows.shape
    experts, rows_each = weight.shape[0], weight.shape[1]
    _need(x_rows, torch.bfloat16, "expert rows")
    _need(weight, torch.bfloat16, "expert weights", (experts, rows_each, k))
    _need(out, torch.bfloat16, "expert output")
    _need(sorted_rows, torch.int32, "sorted rows", (capacity,))
    _need(tile_expert, torch.int32, "tile experts", (capacity // 128 + 1,))
    lib = moe_tc_library()
    x_keep, x_map = _moe_tc_map(lib, x_rows, capacity, k, 128, keep=False)
    _, w_map = _moe_tc_map(lib, weight, experts * rows_each, k, 256, keep=True)
    launch_count += 1
    code = lib.mrs_moe_product_tc(int(gated), x_map, w_map, tile_expert.data_ptr(), sorted_rows.data_ptr(), out.data_ptr(), capacity,
                                  rows_each, k, ACTIVATIONS[activation] if activation is not None else -1, sm_count(x_rows.device), _stream())
    del x_keep
    if code != 0:
        raise BackendError(f"moe_product_tc: {lib.mrs_moe_tc_error_string(code).decode()} (code {code})")


def moe_gather_rows(x: torch.Tensor, sorted_rows: torch.Tensor, out: torch.Tensor, top: int) -> None:
    """out[place] = x[pair / top] for every listed pair, zeros where a run is filled up (bfloat16, rows of a multiple of 8)."""
    _need(x, torch.bfloat16, "expert input")
    _need(out, torch.bfloat16, "gathered rows", (sorted_rows.shape[0], x.shape[1]))
    _check(expert_library().mrs_moe_gather_rows(x.data_ptr(), sorted_rows.data_ptr(), out.data_ptr(), out.shape[0], x.shape[1], top,
                                                _stream()), "moe_gather_rows")


def moe_gather_scaled_rows(x: torch.Tensor, sorted_rows: torch.Tensor, weights: torch.Tensor, out: torch.Tensor, top: int) -> None:
    """out[place] = x[pair / top] * weights[pair] for every listed pair (float32 product, rounded once), zeros where a run
    is filled up; `weights` float32 [tokens, top]."""
    _need(x, None, "expert input")
    _need(out, x.dtype, "gathered rows", (sorted_rows.shape[0], x.shape[1]))
    _need(weights, torch.float32, "expert weights")
    _check(expert_library().mrs_moe_gather_scaled_rows(_is_bf16(x.dtype), x.data_ptr(), sorted_rows.data_ptr(), weights.data_ptr(),
                                                       out.data_ptr(), out.shape[0], x.shape[1], top, _stream()), "moe_gather_scaled_rows")


def moe_plain_experts(h: torch.Tensor, chosen: torch.Tensor, weights: torch.Tensor | None, up: torch.Tensor, down: torch.Tensor,
                      y: torch.Tensor, routed: int, activation: str, kernel: str | None = None) -> None:
    """Experts without a gate: y[token * top + choice] = W_down[e] act(W_up[e] x) with x = h[token] (* weights[token, choice]
    when `weights` are given: the weight multiplies what the expert reads) for every pair whose expert is one of the first
    `routed`.  `up` [routed, inner, width], `down` [routed, width, inner].  The listed pairs' rows are gathered (and
    weighted) first; the up product writes act(sums) at the rows' places, the down product at the pairs.  `kernel` as
    `moe_experts` (None: by the number of pairs)."""
    tokens, top = chosen.shape
    inner = down.shape[2]
    if kernel is None:
        if tokens * top <= MOE_ROWS_MAX_PAIRS and moe_rows_supported(h, inner):
            kernel = "rows"
        elif tokens * top >= MOE_TC_MIN_PAIRS and moe_plain_tc_supported(h, up, down):
            kernel = "tc"
        else:
            kernel = "mma" if moe_mma_supported(h, inner) else ("rows" if moe_rows_supported(h, inner) and tokens * top <= 4 * MOE_ROWS_MAX_PAIRS else "simt")
    tile = {"tc": 128, "mma": moe_mma_tile(), "simt": moe_simt_tile(), "rows": moe_rows_tile()}[kernel]
    capacity = moe_capacity(tokens * top, routed, tile)
    sorted_rows = torch.empty((capacity,), dtype=torch.int32, device=h.device)
    tile_expert = torch.empty((capacity // tile + 1,), dtype=torch.int32, device=h.device)
    moe_align(chosen, routed, tile, sorted_rows, tile_expert)
    rows = torch.empty((capacity, h.shape[1]), dtype=h.dtype, device=h.device)
    if weights is not None:
        moe_gather_scaled_rows(h, sorted_rows, weights, rows, top)
    elif h.dtype is torch.bfloat16 and h.shape[1] % 8 == 0:
        moe_gather_rows(h, sorted_rows, rows, top)
    else:
        moe_gather_scaled_rows(h, sorted_rows, torch.ones((tokens, top), dtype=torch.float32, device=h.device), rows, top)
    act = torch.empty((capacity, inner), dtype=h.dtype, device=h.device)
    if kernel == "tc":
        moe_product_tc(rows, sorted_rows, tile_expert, up, act, gated=False, activation=activation)
        moe_product_tc(act, sorted_rows, tile_expert, down, y, gated=False)
        return
    moe_product(rows, sorted_rows, tile_expert, up, act, top, gated=False, kernel=kernel, activation=activation)
    moe_product(act, sorted_rows, tile_expert, down, y, top, gated=False, kernel=kernel)


def moe_plain_tc_supported(x: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> bool:
    """bfloat16, a width and an inner size of a multiple of 8, weights on 16-byte boundaries."""
    return (x.dtype is torch.bfloat16 and x.shape[1] % 8 == 0 and down.shape[2] % 8 == 0 and up.data_ptr() % 16 == 0
            and down.data_ptr() % 16 == 0)


def moe_experts(h: torch.Tensor, chosen: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, y: torch.Tensor, routed: int,
                kernel: str | None = None, block: int = 0) -> None:
    """y[token * top + choice] = W_down[e] (silu(W_gate[e] h) * (W_up[e] h)) for every pair whose expert e = chosen[token,
    choice] is one of the first `routed`; the other rows of y are left as they are.  `gate_up` [routed, 2 inner, width]
    (all gate rows, then all up rows; with `block`, blocks of that many gate rows each followed by the matching up rows),
    `down` [routed, width, inner].  `kernel`: "simt" (CUDA cores, every size and both dtypes), "rows" (CUDA cores, few rows
    an expert, rows of a multiple of 16 bytes), "mma" (mma.sync, bfloat16, sizes of a multiple of 8), "tc" (tcgen05, bfloat16,
    blocks of 64); None: up to MOE_ROWS_MAX_PAIRS pairs "rows", from MOE_TC_MIN_PAIRS pairs on "tc", between them "mma",
    wherever they apply, else "simt"."""
    tokens, top = chosen.shape
    inner = down.shape[2]
    if kernel is None:
        if tokens * top <= MOE_ROWS_MAX_PAIRS and moe_rows_supported(h, inner):
            kernel = "rows"
        elif tokens * top >= MOE_TC_MIN_PAIRS and moe_tc_supported(h, gate_up, down, block):
            kernel = "tc"
        else:
            kernel = "mma" if moe_mma_supported(h, inner) else ("rows" if moe_rows_supported(h, inner) and tokens * top <= 4 * MOE_ROWS_MAX_PAIRS else "simt")
    tile = {"tc": 128, "mma": moe_mma_tile(), "simt": moe_simt_tile(), "rows": moe_rows_tile()}[kernel]
    capacity = moe_capacity(tokens * top, routed, tile)
    sorted_rows = torch.empty((capacity,), dtype=torch.int32, device=h.device)
    tile_expert = torch.empty((capacity // tile + 1,), dtype=torch.int32, device=h.device)
    moe_align(chosen, routed, tile, sorted_rows, tile_expert)
    act = torch.empty((capacity, inner), dtype=h.dtype, device=h.device)
    if kernel == "tc":
        if not moe_tc_supported(h, gate_up, down, block):
            raise InvalidRequest("the experts' product for many rows needs bfloat16, blocks of 64 gate and up rows and sizes of a multiple of 8")
        rows = torch.empty((capacity, h.shape[1]), dtype=h.dtype, device=h.device)
        moe_gather_rows(h, sorted_rows, rows, top)
        moe_product_tc(rows, sorted_rows, tile_expert, gate_up, act, gated=True)
        moe_product_tc(act, sorted_rows, tile_expert, down, y, gated=False)
        return
    moe_product(h, sorted_rows, tile_expert, gate_up, act, top, gated=True, kernel=kernel, block=block)
    moe_product(act, sorted_rows, tile_expert, down, y, top, gated=False, kernel=kernel)


def moe_combine(y: torch.Tensor | None, h: torch.Tensor, shared_out: torch.Tensor | None, chosen: torch.Tensor,
                weights: torch.Tensor | None, shared_gate: torch.Tensor | None, out: torch.Tensor, routed: int) -> None:
    """out[token] = sum over its choices of weight * (y[pair] for one of the first `routed` experts, else h[token])
    (+ shared_gate[token] * shared_out[token]).  `weights` None: every weight is 1 (they were applied to the experts' inputs);
    `shared_gate` None: the shared expert's output counts fully.  `out` has h's dtype, or float32 (the sums as they are)."""
    tokens, width = h.shape
    top = chosen.shape[1]
    _need(h, None, "expert input", (tokens, width))
    if y is not None:
        _need(y, h.dtype, "expert outputs", (tokens * top, width))
    elif routed > 0:
        raise InvalidRequest("moe_combine: experts with weights need their outputs")
    if out.dtype is not torch.float32:
        _need(out, h.dtype, "combined output", (tokens, width))
    _need(out, None, "combined output", (tokens, width))
    _need(chosen, torch.int32, "chosen experts", (tokens, top))
    if weights is not None:
        _need(weights, torch.float32, "expert weights", (tokens, top))
    if shared_out is not None:
        _need(shared_out, h.dtype, "shared expert output", (tokens, width))
        if shared_gate is not None:
            _need(shared_gate, torch.float32, "shared gate", (tokens,))
    _check(expert_library().mrs_moe_combine(_is_bf16(h.dtype), _ptr(y), h.data_ptr(), _ptr(shared_out), chosen.data_ptr(), _ptr(weights),
                                            _ptr(shared_gate), out.data_ptr(), tokens, width, top, routed,
                                            int(out.dtype is torch.float32), _stream()), "moe_combine")


# ------------------------------------------------------------------------------------------------
# branches side by side, plain feed-forwards, capped logits; the gated delta rule
# ------------------------------------------------------------------------------------------------
_PARALLEL_SIGNATURES = {
    "mrs_add_branches_norm": [_c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_float, _c_vp, _c_int, _c_int, _c_vp],
    "mrs_activation": [_c_int, _c_vp, _c_vp, ctypes.c_longlong, _c_int, _c_vp],
    "mrs_scale_softcap": [_c_vp, ctypes.c_longlong, _c_float, _c_float, _c_vp],
    "mrs_gated_activation": [_c_int, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_int, _c_vp],
}
_DELTA_SIGNATURES = {
    "mrs_delta_prepare": [_c_vp, _c_vp, _c_int, _c_int, _c_int, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                          _c_float, _c_vp],
    "mrs_delta_scan": [_c_vp, _c_vp, _c_vp, ctypes.c_longlong, _c_vp, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_int, _c_int,
                       _c_int, _c_int, _c_vp],
    "mrs_head_norm_gate": [_c_int, _c_vp, _c_vp, _c_int, _c_vp, _c_float, _c_vp, _c_int, _c_int, _c_int, _c_vp],
}
_parallel_lib = None
_delta_lib = None
ACTIVATIONS = {"gelu_erf": 0, "gelu_tanh": 1, "silu": 2, "relu": 3, "relu2": 4}      # relu2: the square of relu


def parallel_library() -> ctypes.CDLL:
    global _parallel_lib
    if _parallel_lib is None:
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device: the engine has no CPU path")
        from .csrc.build import parallel_kernel_library

        _parallel_lib = _typed(parallel_kernel_library(), _PARALLEL_SIGNATURES)
    return _parallel_lib


def delta_library() -> ctypes.CDLL:
    global _delta_lib
    if _delta_lib is None:
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device: the engine has no CPU path")
        from .csrc.build import delta_kernel_library

        _delta_lib = _typed(delta_kernel_library(), _DELTA_SIGNATURES)
    return _delta_lib


def add_branches_norm(stream: torch.Tensor, a: torch.Tensor, b: torch.Tensor | None, next_weight: torch.Tensor | None,
                      next_eps: float, out: torch.Tensor | None) -> None:
    """stream += a (+ b), all float32 [rows, width]; with `next_weight`, out = stream / sqrt(mean(stream^2) + eps) * next_weight
    in out's dtype."""
    rows, width = stream.shape
    _need(stream, torch.float32, "stream")
    _need(a, torch.float32, "branch", (rows, width))
    if b is not None:
        _need(b, torch.float32, "second branch", (rows, width))
    if next_weight is not None:
        _need(next_weight, torch.float32, "next norm weight", (width,))
        _need(out, None, "normed rows", (rows, width))
    _check(parallel_library().mrs_add_branches_norm(_is_bf16(out.dtype) if out is not None and next_weight is not None else 0,
                                                    stream.data_ptr(), a.data_ptr(), _ptr(b), _ptr(next_weight), float(next_eps),
                                                    _ptr(out) if next_weight is not None else None, rows, width, _stream()),
           "add_branches_norm")


def activation(x: torch.Tensor, out: torch.Tensor, kind: str) -> None:
    """out = act(x) element by element (float32 arithmetic): "gelu_erf" 0.5 z (1 + erf(z / sqrt 2)), "gelu_tanh"
    0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3))), "silu"."""
    if kind not in ACTIVATIONS:
        raise InvalidRequest(f"activation {kind!r} is not built; known: {sorted(ACTIVATIONS)}")
    _need(x, None, "activation input")
    _need(out, x.dtype, "activation output", tuple(x.shape))
    _check(parallel_library().mrs_activation(_is_bf16(x.dtype), x.data_ptr(), out.data_ptr(), x.numel(), ACTIVATIONS[kind], _stream()),
           "activation")


def gated_activation(gate_up: torch.Tensor, out: torch.Tensor, kind: str, block: int = 0) -> None:
    """out = act(gate) * up (float32 arithmetic), act one of ACTIVATIONS.  `gate_up` holds all gate columns and then all up
    columns (block 0), or alternating blocks of `block` gate columns and the `block` matching up columns."""
    if kind not in ACTIVATIONS:
        raise InvalidRequest(f"activation {kind!r} is not built; known: {sorted(ACTIVATIONS)}")
    tokens, inter = out.shape
    _need(gate_up, out.dtype, "gate_up", (tokens, 2 * inter))
    _need(out, None, "gated activation out")
    if block and inter % block:
        raise InvalidRequest("gated_activation: the inner size is no multiple of the block")
    _check(parallel_library().mrs_gated_activation(_is_bf16(out.dtype), gate_up.data_ptr(), out.data_ptr(), tokens, inter,
                                                   ACTIVATIONS[kind], int(block), _stream()), "gated_activation")


def scale_softcap_(x: torch.Tensor, scale: float, cap: float) -> None:
    """x <- cap * tanh(x * scale / cap), float32, in place."""
    _need(x, torch.float32, "capped tensor")
    if not cap > 0:
        raise InvalidRequest("a soft cap must be positive")
    _check(parallel_library().mrs_scale_softcap(x.data_ptr(), x.numel(), float(scale), float(cap), _stream()), "scale_softcap")


def delta_prepare(qkv: torch.Tensor, raw: torch.Tensor, b_offset: int, a_offset: int, a_log: torch.Tensor, dt_bias: torch.Tensor,
                  coef: torch.Tensor, groups: int, d: int, heads: int, e: int, unit_eps: float, q_factor: float) -> None:
    """Per token, in place on `qkv` [tokens, 2 * groups * d + heads * e] float32 (q of every group | k of every group | v of
    every head): every q and k becomes x / sqrt(sum x^2 + unit_eps), q also times `q_factor`; `coef` [tokens, 2 * heads]
    gets beta = sigmoid(b) and g = exp(-exp(A_log) * softplus(a + dt_bias)) of every head, b and a read at the columns
    `b_offset` and `a_offset` of the float32 rows `raw`."""
    tokens = qkv.shape[0]
    _need(qkv, torch.float32, "q|k|v", (tokens, 2 * groups * d + heads * e))
    _need(raw, torch.float32, "delta projection")
    if raw.shape[0] != tokens or min(b_offset, a_offset) < 0 or max(b_offset, a_offset) + heads > raw.shape[1]:
        raise InvalidRequest("delta_prepare: b and a lie outside the rows")
    _need(a_log, torch.float32, "A_log", (heads,))
    _need(dt_bias, torch.float32, "dt_bias", (heads,))
    _need(coef, torch.float32, "beta|g", (tokens, 2 * heads))
    _check(delta_library().mrs_delta_prepare(qkv.data_ptr(), raw.data_ptr(), raw.shape[1], int(b_offset), int(a_offset), a_log.data_ptr(),
                                             dt_bias.data_ptr(), coef.data_ptr(), tokens, groups, d, heads, e, float(unit_eps),
                                             float(q_factor), _stream()), "delta_prepare")


def delta_scan(qkv: torch.Tensor, coef: torch.Tensor, state: torch.Tensor, positions, q_start, state_slots, out: torch.Tensor,
               heads: int, groups: int, d: int, e: int, write_state: bool = True) -> None:
    """The gated delta rule token by token, float32, per (sequence, head): S <- g S; u = beta (v - S^T k); S <- S + k u^T;
    o = S^T q.  `qkv` as `delta_prepare` leaves it, `coef` its beta | g; `state` [slots, heads, d, e] float32 (a view: dense
    within a slot); a sequence that starts at position 0 starts from zero; `out` [tokens, heads * e] float32."""
    tokens = qkv.shape[0]
    _need(qkv, torch.float32, "q|k|v", (tokens, 2 * groups * d + heads * e))
    _need(coef, torch.float32, "beta|g", (tokens, 2 * heads))
    if state.dtype != torch.float32 or tuple(state.shape[1:]) != (heads, d, e) or state.stride(3) != 1 or state.stride(2) != e or \
            state.stride(1) != d * e:
        raise InvalidRequest("delta_scan: the state must be float32 [slots, heads, d, e], dense within a slot")
    _need(out, torch.float32, "recurrence output", (tokens, heads * e))
    sequences = state_slots.shape[0]
    _check(delta_library().mrs_delta_scan(qkv.data_ptr(), coef.data_ptr(), state.data_ptr(), state.stride(0), positions.data_ptr(),
                                          q_start.data_ptr(), state_slots.data_ptr(), out.data_ptr(), tokens, sequences, heads, groups,
                                          d, e, int(write_state), _stream()), "delta_scan")


def head_norm_gate(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, heads: int) -> None:
    """out = o / sqrt(mean over a head of o^2 + eps) * weight * silu(gate): `o` float32 [tokens, heads * e], `weight` [e]
    float32 shared by the heads, `gate` float32 of o's shape (may be a column range of wider rows)."""
    tokens, inner = o.shape
    e = inner // heads
    _need(o, torch.float32, "recurrence output")
    if not gate.is_cuda or gate.dtype != torch.float32 or tuple(gate.shape) != (tokens, inner) or gate.stride(1) != 1:
        raise InvalidRequest("head_norm_gate: the gate must be float32 [tokens, heads * e] with unit column stride")
    _need(weight, torch.float32, "head norm weight", (e,))
    _need(out, None, "head norm out", (tokens, inner))
    _check(delta_library().mrs_head_norm_gate(_is_bf16(out.dtype), o.data_ptr(), gate.data_ptr(), gate.stride(0), weight.data_ptr(),
                                              float(eps), out.data_ptr(), tokens, heads, e, _stream()), "head_norm_gate")


# ------------------------------------------------------------------------------------------------
# rotated and normed heads with values of their own or taken from the keys; embeddings with a table of token pairs;
# a stream joined with another
# ------------------------------------------------------------------------------------------------
_ROTARY_SIGNATURES = {
    "mrs_qkv_rotary_store": [_c_int, _c_vp, _c_int, _c_vp, _c_vp, _c_int, _c_float, _c_vp, _c_int, _c_int, _c_vp, _c_vp, _c_vp, _c_vp,
                             _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_vp],
    "mrs_embed_pairs": [_c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_float, _c_int,
                        _c_ll, _c_ll, _c_int, _c_vp],
    "mrs_concat_rows": [_c_int, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_vp],
}
_rotary_lib = None
HEAD_NORM_PLACES = {None: 0, "before_rotation": 1, "after_rotation": 2}
ROTARY_MAX_HEAD = 256


def rotary_library() -> ctypes.CDLL:
    global _rotary_lib
    if _rotary_lib is None:
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device: the engine has no CPU path")
        from .csrc.build import rotary_kernel_library

        _rotary_lib = _typed(rotary_kernel_library(), _ROTARY_SIGNATURES)
    return _rotary_lib


def qkv_rotary_store(proj: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor | None, v_cache: torch.Tensor | None,
                     slots: torch.Tensor | None, nq: int, nkv: int, d: int, e: int, rotations: torch.Tensor | None = None,
                     rotary_dim: int = 0, pairing: str = "split_half", norm_place: str | None = None, q_norm: torch.Tensor | None = None,
                     k_norm: torch.Tensor | None = None, norm_eps: float = 0.0, values_from_keys: bool = False) -> None:
    """After a fused projection whose float32 rows start with q | k (| v): the first `rotary_dim` elements of every query and
    key head turn by the token's position (`rotations` [tokens, rotary_dim / 2, 2] float32 cosines and sines; `pairing`
    "split_half": element i with i + rotary_dim / 2, "interleaved": 2 i with 2 i + 1), the heads pass an RMS norm over all
    their elements `norm_place` the rotation ("before_rotation", "after_rotation", None: no norm) with `q_norm` / `k_norm`
    [d] float32 or, where one is None, without a weight; q goes to `q_out`, k into the key pages [pages, nkv, page, d], v
    into the value pages [pages, nkv, page, e] at `slots`.  `values_from_keys`: the rows have no value columns, a value is
    its key head as projected (e = d).  Columns behind these are not read."""
    tokens = proj.shape[0]
    need = nq * d + nkv * d + (0 if values_from_keys else nkv * e)
    _need(proj, torch.float32, "projection")
    if proj.dim() != 2 or proj.shape[1] < need:
        raise InvalidRequest("qkv_rotary_store: the projection's rows are shorter than q, k and v")
    if norm_place not in HEAD_NORM_PLACES:
        raise InvalidRequest(f"qkv_rotary_store: a head norm stands {sorted(k for k in HEAD_NORM_PLACES if k)} or nowhere")
    if pairing not in ("split_half", "interleaved"):
        raise InvalidRequest(f"qkv_rotary_store: unknown pairing {pairing!r}")
    if d > ROTARY_MAX_HEAD or rotary_dim > d or rotary_dim % 2 or (values_from_keys and e != d):
        raise InvalidRequest("qkv_rotary_store: heads of up to 256 elements, an even rotated part, values from keys of equal size")
    _need(q_out, None, "q_out", (tokens, nq * d))
    page_size = 1
    if k_cache is not None:
        page_size = k_cache.shape[2]
        _need(k_cache, q_out.dtype, "key pages")
        _need(v_cache, q_out.dtype, "value pages")
        if tuple(k_cache.shape[1:]) != (nkv, page_size, d) or tuple(v_cache.shape[1:]) != (nkv, page_size, e):
            raise InvalidRequest("qkv_rotary_store: the pages do not match heads, page size and head sizes")
        _need(slots, torch.int32, "slots", (tokens,))
    if rotary_dim:
        _need(rotations, torch.float32, "rotations", (tokens, rotary_dim // 2, 2))
    for w in (q_norm, k_norm):
        if w is not None:
            _need(w, torch.float32, "head norm weight", (d,))
    _check(rotary_library().mrs_qkv_rotary_store(
        _is_bf16(q_out.dtype), proj.data_ptr(), proj.shape[1], _ptr(q_norm), _ptr(k_norm), HEAD_NORM_PLACES[norm_place], float(norm_eps),
        _ptr(rotations) if rotary_dim else None, int(rotary_dim), int(pairing == "interleaved"), q_out.data_ptr(), _ptr(k_cache),
        _ptr(v_cache), _ptr(slots) if k_cache is not None else None, tokens, nq, nkv, d, e, page_size, int(values_from_keys), _stream()),
        "qkv_rotary_store")


def embed_pairs(table: torch.Tensor, pair_table: torch.Tensor, ctx, last_token: torch.Tensor, stream: torch.Tensor, scale: float,
                buckets: int, mul_prev: int, mul_cur: int, write_state: bool = True) -> None:
    """stream[t] = table[id] * scale + pair_table[(previous id * mul_prev + id * mul_cur) mod buckets], the table's row
    number `buckets` for a sequence's first token.  The token before a portion's first one is `last_token[slot]` (int32
    [slots]) of the sequence's state slot, which then gets the portion's last token unless `write_state` is False.  `ctx`
    gives the step's ids, positions, sequences, first rows and state slots."""
    tokens, width = stream.shape
    vocab = table.shape[0]
    _need(table, None, "embedding table", (vocab, width))
    _need(pair_table, table.dtype, "pair table", (buckets + 1, width))
    _need(stream, torch.float32, "stream")
    _need(last_token, torch.int32, "last tokens")
    _need(ctx.token_ids, torch.int32, "ids", (tokens,))
    _check(rotary_library().mrs_embed_pairs(_is_bf16(table.dtype), table.data_ptr(), pair_table.data_ptr(), ctx.token_ids.data_ptr(),
                                            ctx.positions.data_ptr(), ctx.seq_of_token.data_ptr(), ctx.q_start.data_ptr(),
                                            ctx.state_slots.data_ptr(), last_token.data_ptr(), stream.data_ptr(), tokens, width, vocab,
                                            float(scale), int(buckets), int(mul_prev), int(mul_cur), int(write_state), _stream()),
           "embed_pairs")


def concat_rows(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = [a[t] ; b[t]] in out's dtype; a and b float32 [rows, width]."""
    rows, width = a.shape
    _need(a, torch.float32, "first rows")
    _need(b, torch.float32, "second rows", (rows, width))
    _need(out, None, "joined rows", (rows, 2 * width))
    _check(rotary_library().mrs_concat_rows(_is_bf16(out.dtype), a.data_ptr(), b.data_ptr(), out.data_ptr(), rows, width, _stream()),
           "concat_rows")
