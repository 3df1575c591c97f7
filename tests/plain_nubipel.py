"""A plain, slow implementation of the Nubipel design: one function per mechanism, written from the design's
equations with torch on the CPU (float64 unless told otherwise).  It is the oracle of the tests and shares no
code with the engine: it reads the configuration as a plain dict and the weights as a dict of tensors under
their checkpoint names, runs one whole sequence at a time and keeps nothing between calls.

Notation: T tokens, W width, H heads, G key/value (or query/key) heads, d the query/key size of a head, e the
value size of a head, R the latent of keys and values, Q the latent of the queries, C the taps of a convolution."""
from __future__ import annotations

import math

import torch


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last dimension (weight None: no weight)."""
    y = x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def silu(z):
    return z * torch.sigmoid(z)


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def chunk_mask(T: int, size: int | None):
    """seen[i, j]: j <= i, and with a chunk size also floor(i / size) == floor(j / size), chunks counted from 0."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if size:
        seen = seen & (torch.div(i, size, rounding_mode="floor") == torch.div(j, size, rounding_mode="floor"))
    return seen


def softmax_with_sink(scores, seen, sink):
    """Rows of weights over the seen keys whose denominator also holds exp(sink): the sink has neither key nor value, so
    a row sums to less than one.  `sink` None: the ordinary softmax."""
    s = torch.where(seen, scores, torch.tensor(-math.inf, dtype=scores.dtype))
    top = s.max(dim=-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, sink.to(scores.dtype))
    ex = torch.exp(s - top)
    den = ex.sum(dim=-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink.to(scores.dtype) - top)
    return ex / den


def chunked_attention(h, w, p, c, eps):
    """Grouped heads, each query and key head RMS-normed with one weight for all heads, no positions in the scores,
    sight within the query's chunk, a learned sink a head; then W_o."""
    T = h.shape[0]
    H, G, d, e = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = rms_norm((h @ w[p + "q"].T).view(T, H, d), w[p + "q.norm"], eps)
    k = rms_norm((h @ w[p + "k"].T).view(T, G, d), w[p + "k.norm"], eps)
    v = (h @ w[p + "v"].T).view(T, G, e)
    seen = chunk_mask(T, (c.get("mask") or {}).get("size"))
    out = torch.empty(T, H, e, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        weights = softmax_with_sink(q[:, head] @ k[:, g].T * c["scale"], seen, w[p + "sink"][head])
        out[:, head] = weights @ v[:, g]
    return out.reshape(T, H * e) @ w[p + "o"].T


def latent_attention(h, w, p, c, eps):
    """Queries through a normed latent of their own; keys and values of every head from one normed latent; causal,
    ordinary softmax, no positions; every value element gated by a sigmoid of the layer's input; then W_o."""
    T = h.shape[0]
    H, d, e = c["heads"], c["dim"], c["vdim"]
    q = (rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps) @ w[p + "uq"].T).view(T, H, d)
    latent = rms_norm(h @ w[p + "dkv"].T, w[p + "dkv.norm"], eps)
    k = (latent @ w[p + "uk"].T).view(T, H, d)
    v = (latent @ w[p + "uv"].T).view(T, H, e)
    seen = chunk_mask(T, None)
    out = torch.empty(T, H, e, dtype=h.dtype)
    for head in range(H):
        out[:, head] = softmax_with_sink(q[:, head] @ k[:, head].T * c["scale"], seen, None) @ v[:, head]
    return (out.reshape(T, H * e) * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def causal_conv_silu(x, taps):
    """x [T, channels], taps [channels, C]: y_t = sum_c taps[:, c] x_(t - (C - 1) + c), zeros before the start; then silu."""
    T, channels = x.shape
    C = taps.shape[1]
    padded = torch.cat([torch.zeros(C - 1, channels, dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for c in range(C):
        y = y + padded[c:c + T] * taps[:, c]
    return silu(y)


def unit(x, eps=1e-6):
    return x / torch.sqrt(x.pow(2).sum(dim=-1, keepdim=True) + eps)


def delta_recurrence(q, k, v, beta, decay, state=None):
    """One head: q, k [T, d], v [T, e], beta, decay [T].  S <- decay S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.
    Returns (o [T, e], the last S [d, e])."""
    T, d = q.shape
    S = torch.zeros(d, v.shape[1], dtype=q.dtype) if state is None else state.clone()
    o = torch.empty(T, v.shape[1], dtype=q.dtype)
    for t in range(T):
        S = decay[t] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        o[t] = S.T @ q[t]
    return o, S


def gated_delta_rule(h, w, p, c, eps):
    T = h.shape[0]
    H, G, d, e = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = unit(causal_conv_silu(h @ w[p + "q"].T, w[p + "q.conv"]).view(T, G, d)) * d ** -0.5
    k = unit(causal_conv_silu(h @ w[p + "k"].T, w[p + "k.conv"]).view(T, G, d))
    v = causal_conv_silu(h @ w[p + "v"].T, w[p + "v.conv"]).view(T, H, e)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * torch.nn.functional.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    o = torch.empty(T, H, e, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        o[:, head], _ = delta_recurrence(q[:, g], k[:, g], v[:, head], beta[:, head], decay[:, head])
    o = rms_norm(o, w[p + "norm"], eps).reshape(T, H * e) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def dense_mlp(h, w, p):
    return gelu_erf(h @ w[p + "up"].T) @ w[p + "down"].T


MIXERS = {"attention": chunked_attention, "latent_attention": latent_attention, "delta": gated_delta_rule}


def logits_of(x, w, config):
    z = rms_norm(x, w["final.norm"], config["norm"]["eps"]) @ w["embed"].T * config.get("logit_scale", 1.0)
    cap = config.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z


def forward(config: dict, w: dict, tokens, dtype=torch.float64, layers_out: list | None = None):
    """Logits [T, vocab] of one sequence from position 0.  `layers_out`: a list that gets the residual stream
    after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * (config.get("embedding") or {}).get("scale", 1.0)
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps)
        y = MIXERS[layer["type"]](h, w, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            y = y + dense_mlp(h, w, p + "mlp.")
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    return logits_of(x, w, config)
