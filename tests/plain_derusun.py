"""A plain, slow Derusun: whole sequences, no cache, one function per mechanism.

It shares no code with the product path: it reads config.json and model.safetensors itself and computes with
ordinary tensor arithmetic, float64 by default so that it is the more exact side of every comparison. Notation:
T tokens, D model width, H query heads, G key/value heads, dk the size of a query or key head, dv the size of a
value head, R the latent size, dr the rotated size of a latent-attention head.

The design: X0 = table[id]. Layer i reads x (for i = 0: X0), x <- x + mixer(shift(norm1(x))), x <- x + ff(norm2(x))
(a layer may have no feed-forward); the result is X(i+1), and what the next layer (or the output) reads is the
weighted sum of X0 .. X(i+1) by the layer's depth weights. A norm divides each of ``groups`` equal stretches of the
row by its own root mean square and multiplies the row by a weight. The shift blends a row with the row of the token
before it, per channel. A mixer is the gated delta rule with a decay per key channel (short causal convolutions on q,
k and v, unit queries and keys, a low-rank decay and a low-rank output gate), attention over a compressed latent
(a shared rotated key part, a sink in the softmax), or windowed attention (biases, per-head norms of q and k, capped
scores, first tokens that stay visible, a sink, values blended with those of the first such layer). The feed-forward is
a clamped gated unit. The logits are head . norm(x).
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

# None, or a dtype that stored activations are rounded to (what a 16-bit engine keeps between its kernels), so that a
# test can measure how far such rounding alone moves the logits of a model
ROUND = None


def kept(x):
    return x if ROUND is None else x.to(ROUND).to(x.dtype)


_NP = {"F32": np.float32, "F64": np.float64, "F16": np.float16, "I32": np.int32, "I64": np.int64}


def read_folder(folder, dtype=torch.float64):
    """(config dict, {name: tensor}); floating tensors as ``dtype``, integer tables as int64."""
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    tensors = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        b, e = meta["data_offsets"]
        chunk = raw[8 + n + b:8 + n + e]
        if meta["dtype"] == "BF16":
            arr = (np.frombuffer(chunk, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
        else:
            arr = np.frombuffer(chunk, dtype=_NP[meta["dtype"]])
        t = torch.from_numpy(arr.copy()).reshape(meta["shape"])
        tensors[name] = t.to(dtype) if t.is_floating_point() else t.to(torch.int64)
    return config, tensors


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def grouped_norm(x, w, eps, groups):
    """The row in ``groups`` equal consecutive stretches, each divided by its own root mean square; then times w."""
    T, D = x.shape
    return rms(x.reshape(T, groups, D // groups), eps).reshape(T, D) * w


def token_shift(h, mu, before=None):
    """h[t] + (h[t-1] - h[t]) * mu, with h[-1] = ``before`` (zeros for the start of a sequence)."""
    first = torch.zeros_like(h[:1]) if before is None else before.reshape(1, -1)
    prev = torch.cat([first, h[:-1]], dim=0)
    return h + (prev - h) * mu


def short_convolution(x, taps, before=None):
    """x [T, C], taps [C, n]: y[t, c] = sum_j taps[c, j] * x[t - (n - 1 - j), c] (the last tap is the current token's);
    rows before the start are ``before`` [n - 1, C] (zeros for the start of a sequence)."""
    n = taps.shape[1]
    lead = torch.zeros((n - 1, x.shape[1]), dtype=x.dtype) if before is None else before
    padded = torch.cat([lead, x], dim=0)
    y = torch.zeros_like(x)
    for j in range(n):
        y = y + padded[j:j + x.shape[0]] * taps[:, j]
    return y


def silu(x):
    return x * torch.sigmoid(x)


def unit_vectors(x):
    """x / sqrt(sum(x^2) + 1e-6) over the last axis."""
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_rule(q, k, v, beta, decay, state=None):
    """q, k [T, H, dk], v [T, H, dv], beta [T, H], decay [T, H, dk] in (0, 1]. Per head, token by token:
    S <- decay[:, None] * S;  u = beta * (v - S^T k);  S <- S + k u^T;  o = S^T q  (S [dk, dv], from ``state`` or zero).
    Returns (o [T, H, dv], the last S [H, dk, dv])."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    S = torch.zeros((H, dk, dv), dtype=q.dtype) if state is None else state.clone()
    out = torch.zeros((T, H, dv), dtype=q.dtype)
    for t in range(T):
        S = S * decay[t][:, :, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
        S = S + torch.einsum("hk,hv->hkv", k[t], u)
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out, S


def channel_delta(h, w, p, m, eps):
    """The gated-delta mixer over a whole sequence. w: tensors, p: the prefix '<layer>.mix.', m: the mixer's sizes."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_convolution(kept(h @ w[p + "q"].T), w[p + "q.conv"])).reshape(T, G, dk)
    k = silu(short_convolution(kept(h @ w[p + "k"].T), w[p + "k.conv"])).reshape(T, G, dk)
    v = silu(short_convolution(kept(h @ w[p + "v"].T), w[p + "v.conv"])).reshape(T, H, dv)
    q = unit_vectors(q) * dk ** -0.5
    k = unit_vectors(k)
    share = H // G
    q, k = q.repeat_interleave(share, dim=1), k.repeat_interleave(share, dim=1)
    beta = torch.sigmoid(kept(h @ w[p + "b"].T))
    rate = torch.exp(w[p + "A_log"])[None, :, None]
    step = torch.nn.functional.softplus(kept(h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).reshape(T, H, dk)
    decay = torch.exp(-rate * step)
    o, _ = delta_rule(q, k, v, beta, decay)
    gate = torch.sigmoid(kept(h @ w[p + "g1"].T) @ w[p + "g2"].T).reshape(T, H, dv)
    o = kept(rms(o, eps) * w[p + "norm"] * gate)
    return o.reshape(T, H * dv) @ w[p + "o"].T


def rotate_neighbours(x, positions, n_rot, base):
    """x [T, heads, d]: of every head the first n_rot dimensions turn, dimension 2i with dimension 2i + 1:
    (a, b) -> (a cos - b sin, b cos + a sin) of the angle position * base^(-2i/n_rot); the others stay."""
    half = n_rot // 2
    f = float(base) ** (-2.0 * torch.arange(half, dtype=torch.float64) / n_rot)
    angle = positions.to(torch.float64)[:, None] * f[None, :]
    c, s = torch.cos(angle).to(x.dtype)[:, None, :], torch.sin(angle).to(x.dtype)[:, None, :]
    a, b = x[..., 0:n_rot:2], x[..., 1:n_rot:2]
    out = x.clone()
    out[..., 0:n_rot:2] = a * c - b * s
    out[..., 1:n_rot:2] = b * c + a * s
    return out


def visible(T, window=None, keep_first=0):
    """[T, T] bool: query i sees key j if j <= i and (no window, or i - j < window, or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    see = j <= i
    if window is not None:
        see = see & ((i - j < window) | (j < keep_first))
    return see


def softmax_with_sink(scores, see, sink):
    """scores [H, T, T], see [T, T] bool, sink [H] or None: weights exp(s) / (sum over seen keys of exp(s) + exp(sink))."""
    scores = scores.masked_fill(~see[None], -math.inf)
    top = scores.max(-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, sink[:, None, None])
    e = torch.exp(scores - top)
    total = e.sum(-1, keepdim=True)
    if sink is not None:
        total = total + torch.exp(sink[:, None, None] - top)
    return e / total


def latent_attention(h, w, p, m, eps):
    """Attention whose keys and values are projections of one small latent row per token; a rotated key part shared
    by all heads; a sink in the softmax; every earlier token is seen."""
    T = h.shape[0]
    H, dk, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = torch.arange(T)
    q = kept(h @ w[p + "q"].T).reshape(T, H, dk + dr)
    q_plain, q_turn = q[..., :dk], kept(rotate_neighbours(q[..., dk:], positions, m["rot"]["dims"], m["rot"]["base"]))
    down = kept(h @ w[p + "dkv"].T)
    latent = kept(rms(down[:, :R], eps) * w[p + "dkv.norm"])
    k_turn = kept(rotate_neighbours(down[:, None, R:], positions, m["rot"]["dims"], m["rot"]["base"])[:, 0])
    k_plain = (latent @ w[p + "uk"].T).reshape(T, H, dk)
    v = (latent @ w[p + "uv"].T).reshape(T, H, dv)
    scores = (torch.einsum("thd,shd->hts", q_plain, k_plain) + torch.einsum("thd,sd->hts", q_turn, k_turn)) * m["scale"]
    weights = softmax_with_sink(scores, visible(T), w[p + "sink"])
    o = kept(torch.einsum("hts,shd->thd", weights, v)).reshape(T, H * dv)
    return o @ w[p + "o"].T


def windowed_attention(h, w, p, m, eps, v_first=None):
    """Grouped attention with biases, per-head norms of q and k, capped scores, a window that keeps the first tokens, a
    sink, and values blended with ``v_first`` (None: this is the first such layer). Returns (output, its own values
    as they were attended to)."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = kept(h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, dk)
    k = kept(h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, dk)
    v = kept(h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
    q = kept(rms(q, eps) * w[p + "q.norm"])
    k = kept(rms(k, eps) * w[p + "k.norm"])
    if m.get("v_mix") and v_first is not None:
        lam = w[p + "vmix"]
        v = kept((1 - lam) * v + lam * v_first)
    share = H // G
    kk, vv = k.repeat_interleave(share, dim=1), v.repeat_interleave(share, dim=1)
    scores = torch.einsum("thd,shd->hts", q, kk) * m["scale"]
    cap = m.get("softcap")
    if cap:
        scores = cap * torch.tanh(scores / cap)
    mask = m.get("mask")
    see = visible(T, None if mask is None else mask["size"], 0 if mask is None else mask.get("keep_first", 0))
    weights = softmax_with_sink(scores, see, w[p + "sink"])
    o = kept(torch.einsum("hts,shd->thd", weights, vv)).reshape(T, H * dv)
    return o @ w[p + "o"].T, v


def clamped_unit(h, w, p, limit):
    """W_down (g * sigmoid(1.702 g) * (u + 1)) with g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit)."""
    g = torch.clamp(kept(h @ w[p + "gate"].T), max=limit)
    u = torch.clamp(kept(h @ w[p + "up"].T), min=-limit, max=limit)
    return kept(g * torch.sigmoid(1.702 * g) * (u + 1)) @ w[p + "down"].T


def forward(config, w, ids, return_layers=False):
    """Logits [T, vocab] of one whole sequence (ids: a list or tensor of token ids); with return_layers also what every
    layer hands on, [layers, T, D]."""
    ids = torch.as_tensor(ids, dtype=torch.int64)
    eps, groups = config["norm"]["eps"], config["norm"]["groups"]
    x = w["embed"][ids]
    results, handed = [x], []
    v_first = None
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = kept(token_shift(grouped_norm(x, w[p + "norm1"], eps, groups), w[p + "shift"]))
        if layer["type"] == "channel_delta":
            x = x + channel_delta(h, w, p + "mix.", m, eps)
        elif layer["type"] == "latent_attention":
            x = x + latent_attention(h, w, p + "mix.", m, eps)
        elif layer["type"] == "attention":
            mixed, v = windowed_attention(h, w, p + "mix.", m, eps, v_first)
            if m.get("v_mix") and v_first is None:
                v_first = v
            x = x + mixed
        else:
            raise ValueError(f"unknown layer type {layer['type']!r}")
        if layer["mlp"] is not None:
            x = x + clamped_unit(kept(grouped_norm(x, w[p + "norm2"], eps, groups)), w, p + "mlp.", layer["mlp"]["limit"])
        results.append(x)
        x = sum(w[p + "dwa"][j] * results[j] for j in range(i + 2))
        handed.append(x)
    logits = kept(grouped_norm(x, w["final.norm"], eps, groups)) @ w["head"].T
    return (logits, torch.stack(handed)) if return_layers else logits
