"""A plain, slow implementation of the Migenex design: one function per mechanism, written from the design's
equations with torch on the CPU (float64 unless told otherwise).  It is the oracle of the tests and shares no
code with the engine: it reads the configuration as a plain dict and the weights as a dict of tensors under
their checkpoint names, runs one whole sequence at a time and keeps nothing between calls.

Notation: T tokens, W width, H query heads, G key/value heads, d the query/key size of a head, e the value size
of a head, r the rotated elements of a head, E experts."""
from __future__ import annotations

import math

import torch


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last dimension (weight None: no weight)."""
    y = x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def embed(tokens, w, c):
    """embed[t] * scale + bigram[(previous * mul_prev + t * mul_cur) mod buckets]; the first token of a sequence takes
    the table's last row (row number `buckets`).  A model without a table of pairs adds nothing."""
    b = c.get("embedding", {}).get("bigram")
    x = w["embed"][tokens] * c.get("embedding", {}).get("scale", 1.0)
    if b is None:
        return x
    rows = []
    for i, t in enumerate(tokens.tolist()):
        rows.append(b["buckets"] if i == 0 else (int(tokens[i - 1]) * b["mul_prev"] + t * b["mul_cur"]) % b["buckets"])
    return x + w["bigram"][torch.tensor(rows)]


def rotate(x, base, dims, layout, start=0):
    """x [T, heads, d], rows at the positions start, start + 1, ...: the first `dims` elements of every head turn by
    position * base^(-2i/dims); pair i is (i, i + dims/2) ("half") or (2i, 2i + 1) ("interleaved");
    (u, v) -> (u cos - v sin, v cos + u sin)."""
    T = x.shape[0]
    half = dims // 2
    if half == 0:
        return x.clone()
    i = torch.arange(half, dtype=x.dtype)
    angle = torch.arange(start, start + T, dtype=x.dtype)[:, None] * base ** (-2.0 * i / dims)[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    out = x.clone()
    if layout == "half":
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * cos - v * sin
        out[..., half:dims] = v * cos + u * sin
    else:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    return out


def sight(T, window):
    """seen[i, j]: j <= i, and with a window also i - j < window."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window:
        seen = seen & (i - j < window)
    return seen


def attend(q, k, v, scale, cap, seen):
    """q [T, H, d], k [T, G, d], v [T, G, e]; query head h reads key/value head h // (H / G); the scaled scores may be
    capped, cap * tanh(score / cap); ordinary softmax over the seen keys.  -> [T, H * e]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        s = torch.where(seen, s, torch.tensor(-math.inf, dtype=s.dtype))
        out.append(torch.softmax(s, dim=-1) @ v[:, g])
    return torch.cat(out, dim=-1)


def attention(h, w, p, c, eps):
    """Normed, rotated, capped attention: q and k heads pass an RMS norm with a weight (one for all heads of a kind),
    then the rotation (half layout); every earlier position is seen."""
    T = h.shape[0]
    H, G, d, e = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = rms_norm((h @ w[p + "q"].T).view(T, H, d), w[p + "q.norm"], eps)
    k = rms_norm((h @ w[p + "k"].T).view(T, G, d), w[p + "k.norm"], eps)
    v = (h @ w[p + "v"].T).view(T, G, e)
    q = rotate(q, c["rot"]["base"], c["rot"]["dims"], "half")
    k = rotate(k, c["rot"]["base"], c["rot"]["dims"], "half")
    window = (c.get("mask") or {}).get("size", 0)
    return attend(q, k, v, c["scale"], c.get("softcap", 0.0), sight(T, window)) @ w[p + "o"].T


def attention_keys_as_values(h, w, p, c, eps):
    """The values are the keys as projected; q and k are rotated (interleaved layout) and then divided by their root
    mean square (no weight); a sliding window; the heads' outputs are gated element by element with sigmoid(W_g h)."""
    T = h.shape[0]
    H, G, d = c["heads"], c["kv_heads"], c["dim"]
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, G, d)
    v = k
    q = rms_norm(rotate(q, c["rot"]["base"], c["rot"]["dims"], "interleaved"), None, eps)
    k = rms_norm(rotate(k, c["rot"]["base"], c["rot"]["dims"], "interleaved"), None, eps)
    window = (c.get("mask") or {}).get("size", 0)
    o = attend(q, k, v, c["scale"], c.get("softcap", 0.0), sight(T, window))
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def dense_ff(h, w, p):
    """W_down (relu(W_gate h) * (W_up h))."""
    return (torch.relu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def small_ff(h, w, p):
    """W_down relu(W_up h)^2."""
    return torch.relu(h @ w[p + "up"].T).pow(2) @ w[p + "down"].T


def experts_ff(h, w, p, c):
    """Sigmoid scores a token and expert; the `top` largest are chosen; a chosen expert reads the token times its
    score (the score is neither renormalised nor applied to the output); a shared expert reads every token."""
    z = h @ w[p + "router"].T
    s = torch.sigmoid(z)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        order = sorted(range(s.shape[1]), key=lambda e: (-float(s[t, e]), e))[:c["router"]["top"]]
        for e in order:
            out[t] += small_ff((s[t, e] * h[t])[None], w, f"{p}e{e}.")[0]
    if c.get("shared"):
        out = out + small_ff(h, w, p + "shared.")
    return out


def layer(x, w, i, c, eps, mult):
    p = f"l{i}."
    h = rms_norm(x, w[p + "norm1"], eps)
    mix = attention if c["type"] == "attention" else attention_keys_as_values
    x = x + mult * rms_norm(mix(h, w, p + "mix.", c["mixer"], eps), w[p + "norm1b"], eps)
    if c["mlp"] is not None:
        h = rms_norm(x, w[p + "norm2"], eps)
        f = dense_ff(h, w, p + "mlp.") if c["mlp"]["kind"] == "dense" else experts_ff(h, w, p + "mlp.", c["mlp"])
        x = x + mult * rms_norm(f, w[p + "norm2b"], eps)
    return x


def run_order(c):
    """The layers in the order they run, with whether a run opens a pass of the loop."""
    loop = c.get("loop")
    n = len(c["layers"])
    if not loop:
        return [(i, False) for i in range(n)]
    out = [(i, False) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        out += [(i, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return out + [(i, False) for i in range(loop["stop"], n)]


def forward(tokens, w, c, dtype=torch.float64, streams=None):
    """Logits [T, vocab] of one whole sequence.  `streams`: a list that gets the residual stream after every layer run."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps, mult = c["norm"]["eps"], c.get("residual_mult", 1.0)
    x0 = embed(tokens, w, c)
    x = x0
    for i, opens in run_order(c):
        if opens:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T
        x = layer(x, w, i, c["layers"][i], eps, mult)
        if streams is not None:
            streams.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
