"""A plain, slow Tetitar: whole sequences, no cache, one function per mechanism.

It shares no code with the product path: it reads config.json and model.safetensors itself and computes with
ordinary tensor arithmetic, float64 by default so that it is the more exact side of every comparison. Notation:
T tokens, D model width, H query heads, G key/value heads, dk the size of a query or key head, dv the size of a
value head, N the state size of the state-space mixer.

The design: X0[t] = table[id[t]] + pairs[hash(id[t-1], id[t])] (the last row of ``pairs`` for t = 0). The layers
``loop.start`` .. ``loop.stop - 1`` run ``loop.times`` times in a row; before pass p > 0 X0 is added to the stream, and
before every pass row p of ``loop.step``. A layer is x <- x + mixer(n1(x)); x <- x + ff(n2(x)) (a layer may have no
feed-forward) with n(x) = tanh(alpha x) w + b. A mixer is full causal attention whose values are its unnormed, unrotated
keys (queries and keys normed over the whole projection, rotated with stretched frequencies, an element-wise sigmoid
gate on the output); or windowed attention with a unit term in the softmax's denominator beside a state-space mixer,
both outputs normed and averaged; or a gated linear recurrence per channel behind a short convolution. The
feed-forward is a silu gated unit. The logits are cap tanh(table . n(x) / cap).
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

_NP = {"F32": np.float32, "F64": np.float64, "F16": np.float16, "I32": np.int32, "I64": np.int64}

RECURRENCE_GAIN = 8.0         # the design fixes the factor in log a = -8 r softplus(lam)

# None, or a dtype that stored activations are rounded to (what a 16-bit engine keeps between its kernels), so that a
# test can measure how far such rounding alone moves the logits of a model
ROUND = None


def kept(x):
    return x if ROUND is None else x.to(ROUND).to(x.dtype)


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


# ---------------------------------------------------------------- small pieces

def rms(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def tanh_norm(x, w, p):
    return kept(torch.tanh(w[p + ".alpha"] * x) * w[p] + w[p + ".b"])


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def pair_rows(ids, m):
    """Row of the pair table per token: (previous * mul_prev + current * mul_cur) mod buckets; row ``buckets`` at t = 0."""
    ids = torch.as_tensor(ids, dtype=torch.int64)
    rows = torch.full_like(ids, m["buckets"])
    rows[1:] = (ids[:-1] * m["mul_prev"] + ids[1:] * m["mul_cur"]) % m["buckets"]
    return rows


def embedding(ids, w, config):
    x = w["embed"][torch.as_tensor(ids, dtype=torch.int64)]
    pair = (config.get("embedding") or {}).get("bigram")
    if pair is not None:
        x = x + w["bigram"][pair_rows(ids, pair)]
    return x


def frequencies(rot):
    """Rotary frequencies of dims / 2 pairs, float64; with ``scaling`` long wavelengths are stretched by ``factor``,
    short ones kept, those between blended linearly in original / wavelength."""
    dims = rot["dims"]
    f = float(rot["base"]) ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
    s = rot.get("scaling")
    if s is None:
        return f
    length = 2 * math.pi / f
    blend = (s["original"] / length - s["low"]) / (s["high"] - s["low"])
    mixed = (1 - blend) * f / s["factor"] + blend * f
    return torch.where(length < s["original"] / s["high"], f, torch.where(length > s["original"] / s["low"], f / s["factor"], mixed))


def rotate_halves(x, positions, rot):
    """x [T, heads, d]: dimension i < dims / 2 pairs with i + dims / 2; the rest of a head passes unchanged."""
    dims = rot["dims"]
    half = dims // 2
    angle = positions.to(torch.float64)[:, None] * frequencies(rot)[None, :]
    c, s = torch.cos(angle)[:, None, :].to(x.dtype), torch.sin(angle)[:, None, :].to(x.dtype)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def visible(T, window=None):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    see = j <= i
    if window is not None:
        see = see & (i - j < window)
    return see


def attend(q, k, v, scale, see, unit_term):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H * dv]. unit_term: one is added to the softmax's denominator."""
    T, H, _ = q.shape
    G = k.shape[1]
    group = torch.arange(H) // (H // G)
    scores = torch.einsum("thd,shd->hts", q, k[:, group]) * scale
    scores = scores.masked_fill(~see[None], float("-inf"))
    top = scores.max(-1, keepdim=True).values
    if unit_term:
        top = torch.clamp(top, min=0.0)
    e = torch.exp(scores - top)
    total = e.sum(-1, keepdim=True)
    if unit_term:
        total = total + torch.exp(-top)
    return torch.einsum("hts,shd->thd", e / total, v[:, group]).reshape(T, -1)


def causal_convolution(x, taps, bias):
    """x [T, C], taps [C, n] (the last column is the current token's), zeros before the start."""
    T, n = x.shape[0], taps.shape[1]
    padded = torch.cat([x.new_zeros(n - 1, x.shape[1]), x], dim=0)
    out = bias.expand(T, -1).clone()
    for j in range(n):
        out = out + padded[j:j + T] * taps[:, j]
    return out


# ---------------------------------------------------------------- mixers

def full_attention(h, w, p, m, eps):
    T = h.shape[0]
    H, G, dk = m["heads"], m["kv_heads"], m["dim"]
    positions = torch.arange(T)
    q, k = kept(h @ w[p + "q"].T), kept(h @ w[p + "k"].T)
    v = k.reshape(T, G, dk)
    q = (rms(q, eps) * w[p + "q.norm"]).reshape(T, H, dk)
    k = (rms(k, eps) * w[p + "k.norm"]).reshape(T, G, dk)
    q, k = kept(rotate_halves(q, positions, m["rot"])), kept(rotate_halves(k, positions, m["rot"]))
    mask = m.get("mask")
    o = attend(q, k, v, m["scale"], visible(T, None if mask is None else mask["size"]), False)
    return kept(kept(o) * torch.sigmoid(kept(h @ w[p + "g"].T))) @ w[p + "o"].T


def windowed_attention(h, w, p, m, eps):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = torch.arange(T)
    q = kept(h @ w[p + "q"].T).reshape(T, H, dk)
    k = kept(h @ w[p + "k"].T).reshape(T, G, dk)
    v = kept(h @ w[p + "v"].T).reshape(T, G, dv)
    q, k = rms(q, eps) * w[p + "q.norm"], rms(k, eps) * w[p + "k.norm"]
    q, k = kept(rotate_halves(q, positions, m["rot"])), kept(rotate_halves(k, positions, m["rot"]))
    mask = m.get("mask")
    return kept(attend(q, k, v, m["scale"], visible(T, None if mask is None else mask["size"]), True)) @ w[p + "o"].T


def state_space(h, w, p, m, eps):
    """Per head S <- exp(-exp(A) dt) S + dt B x^T, y = S^T C + D x, S [N, dv] from zero."""
    T = h.shape[0]
    H, dv, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * dv
    proj = kept(h @ w[p + "in"].T)
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_convolution(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, dv)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * dt)
    group = torch.arange(H) // (H // G)
    S = h.new_zeros(H, N, dv)
    y = h.new_zeros(T, H, dv)
    for t in range(T):
        S = decay[t][:, None, None] * S + dt[t][:, None, None] * B[t, group][:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnd,hn->hd", S, C[t, group]) + w[p + "D"][:, None] * x[t]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return kept(y) @ w[p + "o"].T


def side_by_side(h, w, p, m, eps):
    left = windowed_attention(h, w, p + "left.", m["left"], eps)
    right = state_space(h, w, p + "right.", m["right"], eps)
    return 0.5 * (rms(left, eps) * w[p + "left.out"] + rms(right, eps) * w[p + "right.out"])


def gated_recurrence(h, w, p, m, eps):
    """y = gelu(W_y h + b); u = conv(W_x h + b); per block of channels r = sigmoid(Ra u + b), i = sigmoid(Ri u + b);
    a = exp(-8 r softplus(lam)); S <- a S + sqrt(1 - a^2) i u from zero; out = W_o (S y)."""
    T = h.shape[0]
    width, blocks = m["width"], m["blocks"]
    y = gelu_tanh(kept(h @ w[p + "y"].T + w[p + "y.b"]))
    u = causal_convolution(kept(h @ w[p + "x"].T + w[p + "x.b"]), w[p + "conv"], w[p + "conv.b"])
    ub = u.reshape(T, blocks, width // blocks)
    r = torch.sigmoid(torch.einsum("boi,tbi->tbo", w[p + "ra"], ub) + w[p + "ra.b"]).reshape(T, width)
    i = torch.sigmoid(torch.einsum("boi,tbi->tbo", w[p + "ri"], ub) + w[p + "ri.b"]).reshape(T, width)
    a = torch.exp(-RECURRENCE_GAIN * r * softplus(w[p + "lam"]))
    drive = torch.sqrt(1.0 - a * a) * i * u
    S = h.new_zeros(width)
    out = h.new_zeros(T, width)
    for t in range(T):
        S = a[t] * S + drive[t]
        out[t] = S
    return kept(out * y) @ w[p + "o"].T


def silu_unit(h, w, p):
    return kept(silu(kept(h @ w[p + "gate"].T)) * kept(h @ w[p + "up"].T)) @ w[p + "down"].T


MIXERS = {"attention": full_attention, "parallel": side_by_side, "rglru": gated_recurrence}


def run_order(config):
    """[(layer, pass number or None, first of its pass)] in the order the layers run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if loop is None:
        return [(i, None, False) for i in range(n)]
    order = [(i, None, False) for i in range(loop["start"])]
    for p in range(loop["times"]):
        order += [(i, p, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None, False) for i in range(loop["stop"], n)]


def forward(config, w, ids, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer run)."""
    eps = config["norm"]["eps"]
    x0 = embedding(ids, w, config)
    x = x0
    streams = []
    for i, p, first in run_order(config):
        if first:
            if p > 0:
                x = x + x0
            x = x + w["loop.step"][p]
        layer, pre = config["layers"][i], f"l{i}."
        x = x + MIXERS[layer["type"]](tanh_norm(x, w, pre + "norm1"), w, pre + "mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            x = x + silu_unit(tanh_norm(x, w, pre + "norm2"), w, pre + "mlp.")
        streams.append(x)
    logits = tanh_norm(x, w, "final.norm") @ w["embed"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(streams)) if return_layers else logits
