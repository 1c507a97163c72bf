"""Single kernels at GPT-2 XL shapes, for timing and for profiler captures.

``python bench.py --kernel-case NAME [--case-iters N]`` builds the inputs of one case, runs the
kernel N times back to back (rotating through enough copies of the big operand that the 126 MB
L2 cannot hold them) and prints the time per launch from CUDA events. A profiler is pointed at
the same command with a small N.
"""
from __future__ import annotations

import torch

from damendaemon_b200 import kernels as K

H, D, PAGE = 25, 64, 16
SHAPES = {"qkv": (4800, 1600, "bias"), "proj": (1600, 1600, "residual"), "fc": (6400, 1600, "gelu"),
          "fc2": (1600, 6400, "residual"), "head": (50257, 1600, "none")}


def _gemm_case(name, tokens, dev):
    features, reduction, epilogue = SHAPES[name]
    copies = max(2, min(24, (300 << 20) // (features * reduction * 2)))
    weights = [torch.randn(features, reduction, device=dev).mul_(0.02).to(torch.bfloat16) for _ in range(copies)]
    bias = torch.randn(features, device=dev)
    x = torch.randn(tokens, reduction, device=dev).to(torch.bfloat16)
    stream = torch.zeros(tokens, features, device=dev)
    out16 = torch.empty(tokens, features, device=dev, dtype=torch.bfloat16)

    def run(i):
        w = weights[i % copies]
        if epilogue == "bias":
            K.gemm_tcgen05(x, w, bias, out=out16)
        elif epilogue == "gelu":
            K.gemm_tcgen05(x, w, bias, activation="gelu_new", out=out16)
        elif epilogue == "residual":
            K.gemm_tcgen05(x, w, bias, residual=stream, out_dtype=torch.float32, out=stream)
        else:
            K.gemm_tcgen05(x, w, out_dtype=torch.float32, out=stream)
    work = {"bytes": features * reduction * 2, "flops": 2 * tokens * features * reduction}
    return run, work


def _gemm32_case(name, tokens, dev):
    """The same products in true 32-bit on the CUDA cores (float32 weights, activations and stream)."""
    features, reduction, epilogue = SHAPES[name]
    copies = max(2, min(12, (300 << 20) // (features * reduction * 4)))
    weights = [torch.randn(features, reduction, device=dev).mul_(0.02) for _ in range(copies)]
    bias = torch.randn(features, device=dev)
    x = torch.randn(tokens, reduction, device=dev)
    stream = torch.zeros(tokens, features, device=dev)
    out = torch.empty(tokens, features, device=dev)

    def run(i):
        w = weights[i % copies]
        if epilogue == "residual":
            K.gemm_simt(x, w, bias, residual=stream, out=stream)
        else:
            K.gemm_simt(x, w, bias if epilogue != "none" else None, activation="gelu_new" if epilogue == "gelu" else None, out=out)
    return run, {"bytes": features * reduction * 4, "flops": 2 * tokens * features * reduction}


def _layernorm_case(rows, dev):
    """LayerNorm of `rows` rows of the float32 stream (width 1600) into bfloat16, as before every projection."""
    width = H * D
    copies = max(2, min(24, (300 << 20) // (rows * width * 4)))
    xs = [torch.randn(rows, width, device=dev) for _ in range(copies)]
    gamma, beta = torch.ones(width, device=dev), torch.zeros(width, device=dev)
    out = torch.empty(rows, width, device=dev, dtype=torch.bfloat16)
    run = lambda i: K.layernorm(xs[i % copies], gamma, beta, 1e-5, torch.bfloat16, out=out)
    return run, {"bytes": rows * width * 6, "flops": 8 * rows * width}


def _rmsnorm_case(rows, dev):
    """RMS norm (weight stored around zero) of `rows` rows of the float32 stream (width 1600) into bfloat16."""
    width = H * D
    copies = max(2, min(24, (300 << 20) // (rows * width * 4)))
    xs = [torch.randn(rows, width, device=dev) for _ in range(copies)]
    weight = torch.zeros(width, device=dev)
    out = torch.empty(rows, width, device=dev, dtype=torch.bfloat16)
    run = lambda i: K.rmsnorm(xs[i % copies], weight, 1e-6, torch.bfloat16, offset=1.0, out=out)
    return run, {"bytes": rows * width * 6, "flops": 4 * rows * width}


def _rotary_case(rows, dev):
    """Rotary positions on the queries and keys of `rows` tokens (25 + 25 heads of 64, all dimensions rotated)."""
    copies = max(2, min(24, (300 << 20) // (rows * 3 * H * D * 2)))
    bufs = [torch.randn(rows, 3 * H * D + 32, device=dev).to(torch.bfloat16) for _ in range(copies)]
    pos = torch.arange(rows, dtype=torch.int32, device=dev) % 1024
    freqs = (10000.0 ** (-torch.arange(D // 2, dtype=torch.float64) * 2 / D)).float().to(dev)
    run = lambda i: K.rotary(bufs[i % copies][:, :H * D], bufs[i % copies][:, H * D:2 * H * D], pos, freqs, 1.0, H, H, D)
    return run, {"bytes": rows * 2 * H * D * 4, "flops": 6 * rows * H * D}


def _head_norm_case(rows, dev):
    """The heads' RMS norm and the rotation of halves in one pass, on the queries and keys of `rows` tokens (25 + 25
    heads of 64, all dimensions rotated)."""
    copies = max(2, min(24, (300 << 20) // (rows * 3 * H * D * 2)))
    bufs = [torch.randn(rows, 3 * H * D + 32, device=dev).to(torch.bfloat16) for _ in range(copies)]
    pos = torch.arange(rows, dtype=torch.int32, device=dev) % 1024
    freqs = (10000.0 ** (-torch.arange(D // 2, dtype=torch.float64) * 2 / D)).float().to(dev)
    wq, wk = torch.ones(D, device=dev), torch.ones(D, device=dev)
    run = lambda i: K.head_norm_rotary(bufs[i % copies][:, :H * D], bufs[i % copies][:, H * D:2 * H * D], pos, wq, wk, 1e-6, H, H, D,
                                       freqs=freqs, interleaved=False)
    return run, {"bytes": rows * 2 * H * D * 4, "flops": 10 * rows * H * D}


def _retention_case(entries, length, dev, finish=False):
    """Retention of `entries` requests of `length` tokens each in one step (25 heads of 64 by 64, all dimensions
    rotated): the recurrence over float32 state, or (finish) the read-out's norm and gate. Its sums are float32 on the CUDA
    cores: 'fp32' tells the roofline to take that peak."""
    tokens = entries * length
    copies = max(2, min(24, (300 << 20) // max(1, tokens * 4 * H * D * 2 + entries * H * D * D * 4)))
    bufs = [torch.randn(tokens, 4 * H * D, device=dev).mul_(0.5).to(torch.bfloat16) for _ in range(copies)]
    states = [torch.zeros(entries, *K.retention_state_shape(H, D, D), device=dev) for _ in range(copies)]
    pos = (torch.arange(tokens, dtype=torch.int32, device=dev) % length) + (0 if length > 1 else 767)
    start = torch.arange(entries + 1, dtype=torch.int32, device=dev) * length
    slot = torch.arange(entries, dtype=torch.int32, device=dev)
    decay = torch.full((H,), 0.99, device=dev)
    freqs = (10000.0 ** (-torch.arange(D // 2, dtype=torch.float64) * 2 / D)).float().to(dev)
    o = torch.empty(tokens, H * D, device=dev)
    out = torch.empty(tokens, H * D, device=dev, dtype=torch.bfloat16)
    if finish:
        run = lambda i: K.retention_finish(o, bufs[i % copies][:, 3 * H * D:], H, 1e-6, torch.bfloat16, out=out)
        return run, {"bytes": tokens * H * D * 8, "flops": 8 * tokens * H * D}

    def run(i):
        b = bufs[i % copies]
        K.retention(b[:, :H * D], b[:, H * D:2 * H * D], b[:, 2 * H * D:3 * H * D], pos, start, slot, decay, D ** -0.5, states[i % copies],
                    D, D, freqs=freqs, interleaved=False, out=o)
    return run, {"bytes": entries * H * D * D * 8 + tokens * H * D * (6 + 4), "flops": 4 * tokens * H * D * D, "fp32": True}


def _group_norm_shift_case(rows, dev):
    """The RMS norm in two groups of `rows` rows of the float32 stream (width 1600), each blended with the normed row of
    the token before (requests of 256 tokens, or single tokens), into bfloat16."""
    width = H * D
    length = 256 if rows >= 256 else 1
    entries = rows // length
    copies = max(2, min(24, (300 << 20) // (rows * width * 4)))
    xs = [torch.randn(rows, width, device=dev) for _ in range(copies)]
    weight, shift = torch.ones(width, device=dev), torch.rand(width, device=dev)
    state = torch.zeros(entries, width, device=dev)
    entry = torch.arange(rows, dtype=torch.int32, device=dev) // length
    start = torch.arange(entries + 1, dtype=torch.int32, device=dev) * length
    slot = torch.arange(entries, dtype=torch.int32, device=dev)
    out = torch.empty(rows, width, device=dev, dtype=torch.bfloat16)
    run = lambda i: K.rmsnorm_shift(xs[i % copies], weight, 1e-5, torch.bfloat16, shift, state, entry, start, slot, groups=2, out=out)
    return run, {"bytes": rows * width * 6, "flops": 7 * rows * width}


def _depth_mix_case(rows, dev, planes=7):
    """The weighted sum of `planes` float32 streams of `rows` rows (width 1600): what a layer in the middle of a model of
    twelve layers hands on."""
    width = H * D
    copies = max(2, min(12, (300 << 20) // (rows * width * 4 * (planes + 1))))
    stacks = [torch.randn(planes + 1, rows, width, device=dev) for _ in range(copies)]
    w = torch.rand(planes, device=dev)
    run = lambda i: K.weighted_sum(stacks[i % copies], w, planes, stacks[i % copies][planes])
    return run, {"bytes": rows * width * 4 * (planes + 1), "flops": 2 * planes * rows * width}


def _delta_case(entries, length, dev, which="rule", taps=4):
    """The gated delta rule of `entries` requests of `length` tokens each in one step (25 heads of 64 by 64, every head
    its own keys): 'rule' the recurrence over float32 state, 'prepare' its operands (convolutions of four taps with silu,
    unit vectors, decay, beta), 'finish' the read-out's norm and gate. Float32 sums on the CUDA cores."""
    tokens = entries * length
    qk = vw = H * D
    channels = 2 * qk + vw
    copies = max(2, min(24, (300 << 20) // max(1, tokens * (2 * qk + vw + H * D + H) * 4 + entries * H * D * D * 4)))
    start = torch.arange(entries + 1, dtype=torch.int32, device=dev) * length
    slot = torch.arange(entries, dtype=torch.int32, device=dev)
    entry = torch.arange(tokens, dtype=torch.int32, device=dev) // length
    if which == "prepare":
        projs = [torch.randn(tokens, channels + 64 + 64 + 32, device=dev).mul_(0.5).to(torch.bfloat16) for _ in range(copies)]
        step_in = torch.randn(tokens, H * D, device=dev)
        conv_w = torch.randn(channels, taps, device=dev) * 0.5
        conv_state = torch.zeros(entries, taps - 1, channels, device=dev)
        a_log, dt_bias = torch.full((H,), -1.0, device=dev), torch.zeros(H * D, device=dev)

        def run(i):
            p = projs[i % copies]
            K.delta_prepare(p, p[:, channels + 128:channels + 128 + H], step_in, conv_w, conv_state, a_log, dt_bias, entry, start, slot,
                            H, H, D, D)
        return run, {"bytes": tokens * (channels * 2 + H * D * 4 + (channels + H * D + H) * 4), "flops": tokens * (channels * (2 * taps + 8) + 12 * H * D),
                     "fp32": True}
    if which == "finish":
        os_ = [torch.randn(tokens, vw, device=dev) for _ in range(copies)]
        gate = torch.randn(tokens, vw, device=dev)
        weight = torch.ones(D, device=dev)
        out = torch.empty(tokens, vw, device=dev, dtype=torch.bfloat16)
        run = lambda i: K.delta_finish(os_[i % copies], gate, weight, H, 1e-5, torch.bfloat16, out=out)
        return run, {"bytes": tokens * vw * 10, "flops": 12 * tokens * vw}
    unit = lambda x: x / x.view(tokens, H, D).norm(dim=-1, keepdim=True).repeat_interleave(D, -1).view(tokens, H * D)
    ops = []
    for _ in range(copies):
        q, k = unit(torch.randn(tokens, qk, device=dev)) * D ** -0.5, unit(torch.randn(tokens, qk, device=dev))
        ops.append((q, k, torch.randn(tokens, vw, device=dev), torch.rand(tokens, H * D, device=dev) * 0.1 + 0.9,
                    torch.rand(tokens, H, device=dev)))
    states = [torch.zeros(entries, *K.delta_state_shape(H, D, D), device=dev) for _ in range(copies)]
    o = torch.empty(tokens, vw, device=dev)
    run = lambda i: K.delta_rule(*ops[i % copies], start, slot, states[i % copies], H, H, D, D, out=o)
    return run, {"bytes": entries * H * D * D * 8 + tokens * (2 * qk + vw + H * D + H + vw) * 4, "flops": 7 * tokens * H * D * D, "fp32": True}


RANK, ROT = 256, 64        # the latent row of the latent-attention cases: 256 + 64 rotated, heads of 64 + 64, values of 64


def _latent_cache(batch, context, dev, copies):
    row = RANK + ROT
    n_pages = batch * ((context + PAGE - 1) // PAGE)
    caches = [torch.randn(n_pages, PAGE * row, device=dev).mul_(0.3).to(torch.bfloat16) for _ in range(copies)]
    table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(batch, -1)
    return caches, table


def _latent_attention_case(batch, length, dev, decode, kernel="tensor"):
    """Attention of 25 heads over cached latent rows of 256 + 64 (one row a token is every head's key, its first 256
    elements every head's value): `batch` prompts of `length` tokens, or (decode) `batch` single tokens behind `length`
    keys each; through the tensor-core kernel or ('rows') the general one."""
    row = RANK + ROT
    context = length
    tokens = batch if decode else batch * length
    copies = max(2, min(12, (300 << 20) // (batch * context * row * 2)))
    caches, table = _latent_cache(batch, context, dev, copies)
    q = torch.randn(tokens, H * row, device=dev).mul_(0.3).to(torch.bfloat16)
    if decode:
        ent = torch.arange(batch, dtype=torch.int32, device=dev)
        pos = torch.full((batch,), context - 1, dtype=torch.int32, device=dev)
        splits = max(1, min(-(-(K.sm_count(dev) * 2) // (batch * H)), (context + 127) // 128, 32))
        keys = batch * context
    else:
        ent = torch.arange(tokens, dtype=torch.int32, device=dev) // length
        pos = torch.arange(tokens, dtype=torch.int32, device=dev) % length
        splits = 1
        keys = batch * (length * (length + 1) // 2)
    sink = torch.zeros(H, device=dev)
    if kernel == "tensor":
        start = torch.arange(batch + 1, dtype=torch.int32, device=dev) * (1 if decode else length)
        pos0 = torch.full((batch,), context - 1 if decode else 0, dtype=torch.int32, device=dev)
        if decode:
            splits = K.attention_latent_splits(batch, batch, H, context, dev)
        run = lambda i: K.attention_latent(q, caches[i % copies], start, pos0, table, H, RANK, 0.1, n_splits=splits, sink=sink)
    else:
        run = lambda i: K.attention_rows(q, caches[i % copies], ent, pos, table, H, 0.1, n_splits=splits, kv_heads=1, v_dim=RANK,
                                         sink=sink, values_in_keys=True)
    return run, {"bytes": batch * context * row * 2 + tokens * H * (row + RANK) * 2, "flops": 2 * keys * H * (row + RANK)}


def _latent_prepare_case(rows, dev):
    """A step's latent rows normed, their shared key part and the queries' rotated parts rotated, the rows written into
    their pages (25 heads of 64 + 64, latent 256 + 64)."""
    row, qw = RANK + ROT, H * (D + ROT)
    copies = max(2, min(24, (300 << 20) // (rows * (qw + row) * 2)))
    bufs = [torch.randn(rows, qw + row, device=dev).to(torch.bfloat16) for _ in range(copies)]
    caches, table = _latent_cache(max(1, rows // 256), min(rows, 256), dev, 1)
    length = min(rows, 256)
    ent = torch.arange(rows, dtype=torch.int32, device=dev) // length
    pos = torch.arange(rows, dtype=torch.int32, device=dev) % length
    weight = torch.ones(RANK, device=dev)
    freqs = (10000.0 ** (-torch.arange(ROT // 2, dtype=torch.float64) * 2 / ROT)).float().to(dev)

    def run(i):
        b = bufs[i % copies]
        K.latent_prepare(b[:, :qw], b[:, qw:], weight, 1e-5, freqs, ent, pos, table, caches[0], H, D, ROT, RANK)
    return run, {"bytes": rows * (H * ROT * 4 + row * 4), "flops": rows * (6 * H * ROT + 5 * row)}


def _per_head_case(rows, dev, up, kernel=None):
    """Every head's piece of a row times the head's own matrix (25 heads): the plain queries of 64 through the transposed
    key matrices to 256 (with the rotated 64 carried along), or (up) the attended latent rows of 256 to values of 64."""
    if up:
        x = torch.randn(rows, H * RANK, device=dev).to(torch.bfloat16)
        w = torch.randn(H, D, RANK, device=dev).mul_(0.05).to(torch.bfloat16)
        run = lambda i: K.per_head_linear(x, w, RANK, kernel=kernel)
        return run, {"bytes": rows * H * (RANK + D) * 2 + w.numel() * 2, "flops": 2 * rows * H * D * RANK}
    x = torch.randn(rows, H * (D + ROT), device=dev).to(torch.bfloat16)
    w = torch.randn(H, RANK, D, device=dev).mul_(0.1).to(torch.bfloat16)
    run = lambda i: K.per_head_linear(x, w, D + ROT, tail=ROT, kernel=kernel)
    return run, {"bytes": rows * H * (D + ROT + RANK + ROT) * 2 + w.numel() * 2, "flops": 2 * rows * H * D * RANK}


def _sinks_case(batch, length, dev, decode, kernel, unit_only=False):
    """Attention with a window that keeps the first keys, capped scores and a sink (25 heads of 64): prompts through the
    mma.sync kernel or single tokens through the row decode kernel ('tensor'), or either through the general kernel
    ('rows'). The window holds the whole context, so the same keys are read as in the plain cases."""
    context = length
    tokens = batch if decode else batch * length
    copies = max(2, min(12, (300 << 20) // (batch * context * H * D * 4)))
    caches, table = _cache_case(batch, context, dev, copies)
    q = torch.randn(tokens, H * D, device=dev).to(torch.bfloat16)
    kw = dict(window=1024 * ((context + 1023) // 1024), keep_first=4, softcap=30.0, sink=torch.zeros(H, device=dev))
    exact = True
    if unit_only:        # a window and one added to the softmax's denominator, nothing else
        kw, exact = dict(window=kw["window"], sink=kw["sink"]), False
    if decode:
        ent = torch.arange(batch, dtype=torch.int32, device=dev)
        pos = torch.full((batch,), context - 1, dtype=torch.int32, device=dev)
        splits = max(1, min(-(-(K.sm_count(dev) * 2) // (batch * H)), (context + 127) // 128, 32))
        work = {"bytes": batch * context * H * D * 4, "flops": 4 * batch * context * H * D}
        if kernel == "tensor":
            run = lambda i: K.attention_decode(q, caches[i % copies], ent, pos, table, H, D ** -0.5, n_splits=splits, exact_weights=exact, **kw)
        else:
            run = lambda i: K.attention_rows(q, caches[i % copies], ent, pos, table, H, D ** -0.5, n_splits=splits, **kw)
        return run, work
    start = torch.arange(batch + 1, dtype=torch.int32, device=dev) * length
    pos0 = torch.zeros(batch, dtype=torch.int32, device=dev)
    work = {"bytes": batch * length * H * D * 6, "flops": batch * 4 * (length * (length + 1) // 2) * H * D}
    if kernel == "tensor" and unit_only:
        # the tcgen05 prompt kernel takes a sink alone; keys and values of the step as the fused projection leaves them
        qkv = torch.randn(tokens, 3 * H * D, device=dev).to(torch.bfloat16)
        run = lambda i: K.attention_prefill(qkv[:, :H * D], caches[i % copies], start, pos0, table, H, D ** -0.5, kernel="tcgen05",
                                            k_new=qkv[:, H * D:2 * H * D], v_new=qkv[:, 2 * H * D:], **kw)
    elif kernel == "tensor":
        run = lambda i: K.attention_prefill(q, caches[i % copies], start, pos0, table, H, D ** -0.5, exact_weights=exact, **kw)
    else:
        ent = torch.arange(tokens, dtype=torch.int32, device=dev) // length
        pos = torch.arange(tokens, dtype=torch.int32, device=dev) % length
        run = lambda i: K.attention_rows(q, caches[i % copies], ent, pos, table, H, D ** -0.5, **kw)
    return run, work


def _entries(entries, length, dev):
    tokens = entries * length
    ent = torch.arange(tokens, dtype=torch.int32, device=dev) // length
    start = torch.arange(entries + 1, dtype=torch.int32, device=dev) * length
    return tokens, ent, start, torch.arange(entries, dtype=torch.int32, device=dev)


def _tanh_norm_case(rows, dev):
    """The norm without statistics, tanh(alpha x) w + b, of `rows` rows of the float32 stream (width 1600) into bfloat16."""
    width = 1600
    copies = max(2, min(24, (300 << 20) // (rows * width * 4)))
    xs = [torch.randn(rows, width, device=dev) for _ in range(copies)]
    alpha, w, b = torch.full((1,), 0.5, device=dev), torch.ones(width, device=dev), torch.zeros(width, device=dev)
    out = torch.empty(rows, width, device=dev, dtype=torch.bfloat16)
    run = lambda i: K.tanh_norm(xs[i % copies], alpha, w, b, torch.bfloat16, out=out)
    return run, {"bytes": rows * width * 6, "flops": 10 * rows * width}


def _wide_norm_case(rows, dev):
    """Queries and keys of `rows` tokens (25 + 25 heads of 64) normed over the whole projection and rotated in halves."""
    copies = max(2, min(24, (300 << 20) // (rows * 3 * H * D * 2)))
    bufs = [torch.randn(rows, 3 * H * D + 32, device=dev).to(torch.bfloat16) for _ in range(copies)]
    pos = torch.arange(rows, dtype=torch.int32, device=dev) % 1024
    freqs = (10000.0 ** (-torch.arange(D // 2, dtype=torch.float64) * 2 / D)).float().to(dev)
    wq, wk = torch.ones(H * D, device=dev), torch.ones(H * D, device=dev)
    run = lambda i: K.wide_norm_rotary(bufs[i % copies][:, :H * D], bufs[i % copies][:, H * D:2 * H * D], pos, wq, wk, 1e-6, H, H, D,
                                       freqs=freqs, interleaved=False)
    return run, {"bytes": rows * 2 * H * D * 4, "flops": 10 * rows * H * D}


STATE = 64          # rows of the state-space mixer's state: 25 heads of 64 by 64, the size of a retention head


def _state_space_case(entries, length, dev, which):
    """The state-space mixer of `entries` requests of `length` tokens each in one step (25 heads with values of 64 and a
    state of 64 rows, one group, four taps): 'conv' the convolution with silu over [x | B | C], 'scan' the recurrence over
    the float32 state, 'finish' the gate, the norm and the weight of the read-out."""
    tokens, ent, start, slot = _entries(entries, length, dev)
    inner, channels = H * D, H * D + 2 * STATE
    copies = max(2, min(24, (300 << 20) // max(1, tokens * (2 * inner + channels) * 2 + entries * H * D * STATE * 4)))
    bufs = [torch.randn(tokens, inner + channels + H + 7, device=dev).mul_(0.5).to(torch.bfloat16) for _ in range(copies)]
    if which == "conv":
        taps, bias = torch.randn(channels, 4, device=dev) * 0.5, torch.zeros(channels, device=dev)
        state = torch.zeros(entries, 3, channels, device=dev)
        out = torch.empty(tokens, channels, device=dev)
        run = lambda i: K.conv_channels(bufs[i % copies][:, inner:inner + channels], taps, bias, state, ent, start, slot, activation="silu", out=out)
        return run, {"bytes": tokens * channels * 6, "flops": 12 * tokens * channels}
    if which == "finish":
        y, w = torch.randn(tokens, inner, device=dev), torch.ones(inner, device=dev)
        out = torch.empty(tokens, inner, device=dev, dtype=torch.bfloat16)
        run = lambda i: K.gated_group_norm(y, bufs[i % copies][:, :inner], w, 1, 1e-6, torch.bfloat16, out=out)
        return run, {"bytes": tokens * inner * 8, "flops": 8 * tokens * inner}
    xbc = [torch.randn(tokens, channels, device=dev).mul_(0.5) for _ in range(min(copies, 6))]
    states = [torch.zeros(entries, *K.state_space_state_shape(H, STATE, D), device=dev) for _ in range(copies)]
    dt_bias, a_log, skip = torch.zeros(H, device=dev), torch.full((H,), -3.0, device=dev), torch.ones(H, device=dev)
    out = torch.empty(tokens, inner, device=dev)

    def run(i):
        K.state_space_scan(xbc[i % len(xbc)], bufs[i % copies][:, inner + channels:inner + channels + H], dt_bias, a_log, skip, start, slot,
                           states[i % copies], H, 1, STATE, D, out=out)
    return run, {"bytes": entries * H * D * STATE * 8 + tokens * (channels * 4 + inner * 4), "flops": 4 * tokens * H * D * STATE, "fp32": True}


def _recurrence_case(entries, length, dev, which):
    """The gated linear recurrence of `entries` requests of `length` tokens (1,600 channels in ten parts of 160): 'gates' the
    two float32 products of every part with their sigmoids, the decay and the drive; 'scan' the walk over the tokens with the
    tanh-gelu branch multiplied in."""
    tokens, ent, start, slot = _entries(entries, length, dev)
    width, blocks = 1600, 10
    part = width // blocks
    copies = max(2, min(24, (300 << 20) // (tokens * width * 8)))
    us = [torch.randn(tokens, width, device=dev) for _ in range(copies)]
    if which == "gates":
        wa, wi = (torch.randn(blocks, part, part, device=dev) / part ** 0.5 for _ in range(2))
        ba, bi, lam = torch.zeros(width, device=dev), torch.zeros(width, device=dev), torch.full((width,), -2.0, device=dev)
        run = lambda i: K.recurrence_gates(us[i % copies], wa, ba, wi, bi, lam, 8.0)
        return run, {"bytes": tokens * width * 12 + 2 * width * part * 4, "flops": 4 * tokens * width * part, "fp32": True}
    fade, y = torch.rand(tokens, width, device=dev) * 0.1, torch.randn(tokens, width + 8, device=dev).to(torch.bfloat16)
    state = torch.zeros(entries, width, device=dev)
    out = torch.empty(tokens, width, device=dev, dtype=torch.bfloat16)
    run = lambda i: K.linear_scan(fade, us[i % copies], y[:, :width], start, slot, state, activation="gelu_tanh", out=out)
    return run, {"bytes": tokens * width * 12 + entries * width * 8, "flops": 12 * tokens * width, "fp32": True}


def _row_ops_case(which, rows, dev):
    """'gate': the attended rows (25 heads of 64) times the sigmoid of a gate per element; 'pairnorm': two float32 results of
    width 1600, each RMS-normed and weighted, averaged into the stream; 'embedpairs': the token's row plus the row of its
    pair with the token before, into the float32 stream."""
    width = 1600
    copies = max(2, min(24, (300 << 20) // (rows * width * 8)))
    if which == "gate":
        bufs = [torch.randn(rows, 2 * H * D, device=dev).to(torch.bfloat16) for _ in range(copies)]
        run = lambda i: K.sigmoid_gate(bufs[i % copies][:, :H * D], bufs[i % copies][:, H * D:])
        return run, {"bytes": rows * H * D * 6, "flops": 6 * rows * H * D}
    if which == "pairnorm":
        both = [torch.randn(2, rows, width, device=dev) for _ in range(copies)]
        x, wl, wr = torch.zeros(rows, width, device=dev), torch.ones(width, device=dev), torch.ones(width, device=dev)
        run = lambda i: K.norm_pair_add(x, both[i % copies][0], both[i % copies][1], wl, wr, 1e-6, 0.5)
        return run, {"bytes": rows * width * 16, "flops": 10 * rows * width}
    vocab, buckets = 50257, 99991
    table, pairs = torch.randn(vocab, width, device=dev).to(torch.bfloat16), torch.randn(buckets + 1, width, device=dev).to(torch.bfloat16)
    ids = torch.randint(0, vocab, (rows,), dtype=torch.int32, device=dev)
    n = max(1, rows // 1024) if rows >= 1024 else rows
    tokens, ent, start, slot = _entries(n, rows // n, dev)
    pos = torch.arange(rows, dtype=torch.int32, device=dev) % (rows // n) + 1
    last = torch.zeros(n, dtype=torch.int32, device=dev)
    out = torch.empty(rows, width, device=dev)
    run = lambda i: K.embed_pairs(ids, pos, ent, start, slot, table, pairs, last, 1009, 613, out=out)
    return run, {"bytes": rows * width * 8, "flops": 2 * rows * width}


def _gated_act_case(rows, dev):
    """The dense gated unit between its two products: rows of [gate | up] halves (2 x 6400) -> tanh-gelu(gate) * up."""
    inner = 6400
    copies = max(2, min(24, (300 << 20) // (rows * 2 * inner * 2)))
    bufs = [torch.randn(rows, 2 * inner, device=dev).to(torch.bfloat16) for _ in range(copies)]
    out = torch.empty(rows, inner, device=dev, dtype=torch.bfloat16)
    run = lambda i: K.gated_unit(bufs[i % copies], 0.0, 1.0, out=out, form="gelu_tanh")
    return run, {"bytes": rows * inner * 6, "flops": 12 * rows * inner}


EXPERTS, TOP, INNER = 16, 2, 1600       # sixteen experts of a quarter of the dense inner width, two per token


def _grouped_case(which, tokens, dev):
    """The experts' products of a step of `tokens` tokens (width 1600): 'up' = gate and up with the gated unit fused,
    'down' = the down projection into float32 rows; 'route' = sorting the pairs, gathering the rows and the weighted sum."""
    width = H * D
    g = torch.Generator().manual_seed(0)
    table = torch.rand((50257, EXPERTS), generator=g).argsort(dim=1)[:, :TOP].to(torch.int32).contiguous().to(dev)
    ids = torch.randint(0, 50257, (tokens,), generator=g).to(torch.int32).to(dev)
    from damendaemon_b200.parts.linear import grouped_tile
    x = torch.randn(tokens, width, device=dev).to(torch.bfloat16)
    tile = grouped_tile(True, tokens * TOP, EXPERTS)
    pair_row, row_token, tile_group = K.route_by_table(ids, table, EXPERTS, tile)
    rows = K.gather_rows(x, row_token)
    used = int(torch.unique(tile_group[tile_group >= 0]).numel())      # experts whose matrices this step streams
    if which == "score":
        # the router's logits and the choice within groups (one kernel), then sorting, gathering and the weighted sum
        router = torch.randn(EXPERTS + 1, width, device=dev).mul_(0.05).to(torch.bfloat16)
        stream = torch.zeros(tokens, width, device=dev)
        y = torch.zeros(rows.shape[0], width, device=dev)

        def run(i):
            chosen, weight, _ = K.route_by_score(x, router, EXPERTS, TOP, 4, 2, 2.5, shared_gate=True)
            pr, rt, tg = K.route_by_table(None, chosen, EXPERTS, tile)
            K.gather_rows(x, rt)
            K.combine_rows(y, pr, stream, TOP, 1.0, pair_weight=weight.view(-1))
        return run, {"bytes": tokens * TOP * width * (2 + 2 + 4) + tokens * width * 10, "flops": tokens * (TOP + 2 * EXPERTS) * width}
    if which == "route":
        stream = torch.zeros(tokens, width, device=dev)
        y = torch.zeros(rows.shape[0], width, device=dev)

        def run(i):
            pr, rt, tg = K.route_by_table(ids, table, EXPERTS, tile)
            K.gather_rows(x, rt)
            K.combine_rows(y, pr, stream, TOP, 1.0 / TOP)
        return run, {"bytes": tokens * TOP * width * (2 + 2 + 4) + tokens * width * 8, "flops": tokens * TOP * width}
    if which in ("up", "upsilu"):
        copies = max(2, min(8, (300 << 20) // (EXPERTS * 2 * INNER * width * 2)))
        weights = [torch.randn(EXPERTS, 2 * INNER, width, device=dev).mul_(0.02).to(torch.bfloat16) for _ in range(copies)]
        gated = (0.0, 1.0, "silu") if which == "upsilu" else (7.0, 1.702)
        run = lambda i: K.gemm_grouped_tcgen05(rows, weights[i % copies], tile_group, tile, gated=gated)
        return run, {"bytes": used * 2 * INNER * width * 2, "flops": 2 * tokens * TOP * 2 * INNER * width}
    hidden = torch.randn(rows.shape[0], INNER, device=dev).to(torch.bfloat16)
    copies = max(2, min(8, (300 << 20) // (EXPERTS * INNER * width * 2)))
    weights = [torch.randn(EXPERTS, width, INNER, device=dev).mul_(0.02).to(torch.bfloat16) for _ in range(copies)]
    run = lambda i: K.gemm_grouped_tcgen05(hidden, weights[i % copies], tile_group, tile, out_dtype=torch.float32)
    return run, {"bytes": used * INNER * width * 2, "flops": 2 * tokens * TOP * INNER * width}


def _cache_case(batch, context, dev, copies):
    n_pages = batch * ((context + PAGE - 1) // PAGE)
    caches = [torch.randn(n_pages, 2, H, PAGE, D, device=dev).to(torch.bfloat16) for _ in range(copies)]
    table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(batch, -1)
    return caches, table


def _decode_case(batch, context, dev, kernel="pages", masked=False):
    copies = max(2, min(12, (300 << 20) // (batch * context * H * D * 4)))
    caches, table = _cache_case(batch, context, dev, copies)
    ent = torch.arange(batch, dtype=torch.int32, device=dev)
    pos = torch.full((batch,), context - 1, dtype=torch.int32, device=dev)
    q = torch.randn(batch, H * D, device=dev).to(torch.bfloat16)
    if kernel == "pages":
        splits = K.attention_decode_pages_splits(batch, H, PAGE, context, dev)
    else:
        splits = max(1, min(-(-(K.sm_count(dev) * 2) // (batch * H)), (context + 127) // 128, 32))
    # masked: a chunked mask whose chunk holds the whole context (the same keys are read) and a gate on every head
    more = dict(chunk=1024 * ((context + 1023) // 1024), gate=torch.randn(batch, H, device=dev).to(torch.bfloat16)) if masked else {}
    run = lambda i: K.attention_decode(q, caches[i % copies], ent, pos, table, H, D ** -0.5, None, n_splits=splits, kernel=kernel, **more)
    return run, {"bytes": batch * context * H * D * 4, "flops": 4 * batch * context * H * D}


def _prefill_case(prompts, length, dev, kernel="tcgen05", store=False, masked=False):
    caches, table = _cache_case(prompts, length, dev, 4)
    start = torch.arange(prompts + 1, dtype=torch.int32, device=dev) * length
    pos0 = torch.zeros(prompts, dtype=torch.int32, device=dev)
    qkv = torch.randn(prompts * length, 3 * H * D, device=dev).to(torch.bfloat16)      # as the fused projection leaves them
    q, k, v = qkv[:, :H * D], qkv[:, H * D:2 * H * D], qkv[:, 2 * H * D:]
    new = {"k_new": k, "v_new": v, "store_new": store} if kernel == "tcgen05" else {}
    if masked:
        new.update(chunk=1024 * ((length + 1023) // 1024), gate=torch.randn(prompts * length, H, device=dev).to(torch.bfloat16))
    run = lambda i: K.attention_prefill(q, caches[i % 4], start, pos0, table, H, D ** -0.5, None, kernel=kernel, **new)
    return run, {"bytes": prompts * length * H * D * 6, "flops": prompts * 4 * (length * (length + 1) // 2) * H * D}


def build(name, device="cuda:0"):
    """name: gemm_<qkv|proj|fc|fc2|head>_m<tokens> | gemm32_<...>_m<tokens> (float32, CUDA cores) | attn_decode_b<batch>[_c<context>] (page streaming) | attn_decode_rows_b<batch>[_c<context>] | attn_prefill_p<prompts>_t<tokens> | attn_prefill | attn_prefill_store (the kernel writes the cache too) | attn_prefill_mma |
    attn_prefill_long (one prompt of 4,096 tokens) | layernorm_m<rows> | rmsnorm_m<rows> | rotary_m<rows> |
    grouped_<up|upsilu|down|route|score>_m<tokens> (sixteen experts, two per token; upsilu: the silu form of the unit;
    score: routing by a router's scores) | headnorm_m<rows> | gatedact_m<rows> | retention_p<requests>_t<tokens> |
    retfinish_p<requests>_t<tokens> | groupnorm_m<rows> | depthmix_m<rows> | delta_p<requests>_t<tokens> | deltaprep_p.._t.. |
    deltafinish_p.._t.. | latent_prefill_p<prompts>_t<tokens> | latent_decode_b<batch>_c<context> | latentprep_m<rows> |
    perhead_m<rows> | perheadup_m<rows> | sinks_prefill_p<prompts>_t<tokens> | sinks_decode_b<batch>_c<context> (and
    sinks_prefillrows_.., sinks_decoderows_..: through the general kernel) | tanhnorm_m<rows> | widenorm_m<rows> |
    ssmconv_p<requests>_t<tokens> | ssmscan_p.._t.. | ssmfinish_p.._t.. | rglrugates_p.._t.. | rglruscan_p.._t.. |
    sigmoidgate_m<rows> | pairnorm_m<rows> | embedpairs_m<rows> | unitsink_prefill_p<prompts>_t<tokens> |
    unitsink_decode_b<batch>_c<context>; attention cases take the suffix _masked (a chunked mask and a gate on every head's
    output)"""
    K.library("core"), K.library("tensor")
    masked = name.endswith("_masked")          # attention cases: with a chunked mask and an output gate
    if masked:
        name = name[:-len("_masked")]
    parts = name.split("_")
    if name.startswith("tanhnorm_m"):
        return _tanh_norm_case(int(name[len("tanhnorm_m"):]), device)
    if name.startswith("widenorm_m"):
        return _wide_norm_case(int(name[len("widenorm_m"):]), device)
    if parts[0] in ("ssmconv", "ssmscan", "ssmfinish", "rglrugates", "rglruscan") and "_p" in name:
        # ssmconv_p<requests>_t<tokens of each> | ssmscan_.. | ssmfinish_.. | rglrugates_.. | rglruscan_..
        entries, tokens = name.split("_p")[1].split("_t")
        if parts[0].startswith("ssm"):
            return _state_space_case(int(entries), int(tokens), device, parts[0][3:])
        return _recurrence_case(int(entries), int(tokens), device, parts[0][5:])
    if parts[0] in ("sigmoidgate", "pairnorm", "embedpairs") and len(parts) == 2 and parts[1][0] == "m":
        return _row_ops_case({"sigmoidgate": "gate"}.get(parts[0], parts[0]), int(parts[1][1:]), device)
    if parts[0] == "unitsink" and parts[1] in ("prefill", "decode"):
        # unitsink_prefill_p<prompts>_t<tokens> | unitsink_decode_b<batch>_c<context>: a window and a unit term in the softmax
        a, b = name.split("_", 2)[2][1:].replace("_t", " ").replace("_c", " ").split()
        return _sinks_case(int(a), int(b), device, parts[1] == "decode", "tensor", unit_only=True)
    if name.startswith("groupnorm_m"):
        return _group_norm_shift_case(int(name[len("groupnorm_m"):]), device)
    if name.startswith("depthmix_m"):
        return _depth_mix_case(int(name[len("depthmix_m"):]), device)
    if parts[0] in ("delta", "deltaprep", "deltafinish") and "_p" in name:
        entries, tokens = name.split("_p")[1].split("_t")
        return _delta_case(int(entries), int(tokens), device, {"delta": "rule", "deltaprep": "prepare", "deltafinish": "finish"}[parts[0]])
    if parts[0] == "latent" and parts[1] in ("prefill", "decode", "prefillrows", "decoderows"):
        # latent_prefill_p<prompts>_t<tokens> | latent_decode_b<batch>_c<context>; ...rows: through the general kernel
        a, b = name.split("_", 2)[2][1:].replace("_t", " ").replace("_c", " ").split()
        return _latent_attention_case(int(a), int(b), device, parts[1].startswith("decode"), "rows" if parts[1].endswith("rows") else "tensor")
    if name.startswith("latentprep_m"):
        return _latent_prepare_case(int(name[len("latentprep_m"):]), device)
    if parts[0] in ("perhead", "perheadup", "perheadplain", "perheadupplain"):
        # perhead_m<rows> | perheadup_m<rows>; ...plain: the kernel without tensor cores
        return _per_head_case(int(name.split("_m")[1]), device, parts[0].startswith("perheadup"), "plain" if parts[0].endswith("plain") else None)
    if parts[0] == "sinks" and parts[1] in ("prefill", "decode", "prefillrows", "decoderows"):
        # sinks_prefill_p<prompts>_t<tokens> | sinks_decode_b<batch>_c<context>; ...rows: through the general kernel
        a, b = name.split("_", 2)[2][1:].replace("_t", " ").replace("_c", " ").split()
        return _sinks_case(int(a), int(b), device, parts[1].startswith("decode"), "rows" if parts[1].endswith("rows") else "tensor")
    if name.startswith("rmsnorm_m"):
        return _rmsnorm_case(int(name[len("rmsnorm_m"):]), device)
    if name.startswith("rotary_m"):
        return _rotary_case(int(name[len("rotary_m"):]), device)
    if name.startswith("headnorm_m"):
        return _head_norm_case(int(name[len("headnorm_m"):]), device)
    if name.startswith("gatedact_m"):
        return _gated_act_case(int(name[len("gatedact_m"):]), device)
    if name.startswith("retention_p") or name.startswith("retfinish_p"):
        # retention_p<requests>_t<tokens of each>: prompts; _t1: a decode step of that many requests
        entries, tokens = name.split("_p")[1].split("_t")
        return _retention_case(int(entries), int(tokens), device, finish=name.startswith("retfinish"))
    if parts[0] == "grouped" and len(parts) == 3 and parts[1] in ("up", "upsilu", "down", "route", "score") and parts[2][0] == "m":
        return _grouped_case(parts[1], int(parts[2][1:]), device)
    if parts[0] == "gemm" and len(parts) == 3 and parts[1] in SHAPES and parts[2][0] == "m":
        return _gemm_case(parts[1], int(parts[2][1:]), device)
    if parts[0] == "gemm32" and len(parts) == 3 and parts[1] in SHAPES and parts[2][0] == "m":
        return _gemm32_case(parts[1], int(parts[2][1:]), device)
    if name.startswith("layernorm_m"):
        return _layernorm_case(int(name[len("layernorm_m"):]), device)
    if name.startswith("attn_decode_rows_b") or name.startswith("attn_decode_b"):
        # attn_decode[_rows]_b<batch>[_c<context>]: the context is 768 keys unless it is given
        rows = name.startswith("attn_decode_rows_b")
        numbers = name[len("attn_decode_rows_b" if rows else "attn_decode_b"):].split("_c")
        return _decode_case(int(numbers[0]), int(numbers[1]) if len(numbers) > 1 else 768, device, kernel="rows" if rows else "pages",
                            masked=masked)
    if name.startswith("attn_prefill_p"):
        # attn_prefill_p<prompts>_t<tokens>: whole prompts of that many tokens
        prompts, tokens = name[len("attn_prefill_p"):].split("_t")
        return _prefill_case(int(prompts), int(tokens), device, masked=masked)
    if name == "attn_prefill":
        return _prefill_case(2, 1024, device)
    if name == "attn_prefill_store":
        return _prefill_case(2, 1024, device, store=True)
    if name == "attn_prefill_mma":
        return _prefill_case(2, 1024, device, kernel="mma")
    if name == "attn_prefill_long":
        return _prefill_case(1, 4096, device)
    if name == "attn_prefill_long_mma":
        return _prefill_case(1, 4096, device, kernel="mma")
    raise ValueError(f"unknown kernel case {name!r}")


def time_case(name, iters=50, device="cuda:0", graph=False):
    """graph: the launches are captured into one CUDA graph and replayed, so that the host's time per launch (a
    few microseconds of Python) does not stand between two kernels, as it does not in a captured decode step."""
    run, work = build(name, device)
    for i in range(3):
        run(i)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        captured = torch.cuda.CUDAGraph()
        with torch.cuda.graph(captured):
            for i in range(iters):
                run(i)
        captured.replay()
        torch.cuda.synchronize()
        start.record()
        captured.replay()
        stop.record()
    else:
        start.record()
        for i in range(iters):
            run(i)
        stop.record()
    torch.cuda.synchronize()
    us = start.elapsed_time(stop) * 1000.0 / iters
    return {"case": name, "us_per_launch": round(us, 2), "GB_per_s": round(work["bytes"] / us / 1e3, 1),
            "TFLOP_per_s": round(work["flops"] / us / 1e6, 1), "iters": iters, "graph": bool(graph),
            "float32_on_cuda_cores": bool(work.get("fp32", False))}
