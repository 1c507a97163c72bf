"""Each mechanism of Derusun alone: the kernel or part against the plain function of the same name."""
import math

import pytest
import torch

import plain_derusun as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


def layout(lengths):
    """(entry_start, token_entry) of entries of these lengths laid side by side."""
    starts, entry = [0], []
    for e, n in enumerate(lengths):
        starts.append(starts[-1] + n)
        entry += [e] * n
    return starts, entry


# ------------------------------------------------------------------ the norm in groups, the blend with the token before

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,groups", [(64, 4), (48, 1), (100, 5), (256, 8), (2048, 2), (6, 6), (4100, 2)])
def test_norm_in_groups(width, groups, dtype):
    from damendaemon_b200 import kernels
    x, w = rnd(9, width, seed=1, scale=3.0), 1.0 + rnd(width, seed=2, scale=0.2)
    x[3] *= 1e-3                                            # a row so small that eps matters
    want = plain.grouped_norm(x.double(), w.double(), 1e-5, groups)
    got = kernels.rmsnorm(x.to(DEV), w.to(DEV), 1e-5, dtype, groups=groups).cpu().double()
    assert (got - want).abs().max() < (1e-5 if dtype == torch.float32 else 0.03)
    rows = i32([7, 0, 7, 2])
    picked = kernels.rmsnorm(x.to(DEV), w.to(DEV), 1e-5, torch.float32, row_index=rows, groups=groups).cpu().double()
    assert (picked - want[[7, 0, 7, 2]]).abs().max() < 1e-5


@pytest.mark.parametrize("width,groups", [(64, 4), (48, 1), (100, 5), (1024, 2)])
def test_norm_blended_with_the_token_before_over_steps_and_slots(width, groups):
    """Three requests in shuffled slots, run in steps of unequal portions (one request left out of a step, portions of one
    and two tokens): every row equals the plain shift over the whole sequence, so the state carried the last normed row;
    and the rows have the same bits however the sequence was cut."""
    from damendaemon_b200 import kernels
    total, slots = [37, 12, 25], [3, 0, 2]
    xs = [rnd(n, width, seed=40 + i, scale=2.0) for i, n in enumerate(total)]
    w, mu = 1.0 + rnd(width, seed=3, scale=0.2), torch.rand(width, generator=torch.Generator().manual_seed(4))
    mu[0], mu[1] = 0.0, 1.0
    want = [plain.token_shift(plain.grouped_norm(x.double(), w.double(), 1e-5, groups), mu.double()) for x in xs]

    def run(steps):
        state = torch.full((5, width), float("nan"), device=DEV)
        for s in slots:
            state[s].zero_()
        at, rows = [0, 0, 0], [[], [], []]
        for lengths in steps:
            live = [i for i, n in enumerate(lengths) if n]
            x = torch.cat([xs[i][at[i]:at[i] + lengths[i]] for i in live]).to(DEV)
            starts, entry = layout([lengths[i] for i in live])
            out = kernels.rmsnorm_shift(x, w.to(DEV), 1e-5, torch.float32, mu.to(DEV), state, i32(entry), i32(starts),
                                        i32([slots[i] for i in live]), groups=groups).cpu()
            for j, i in enumerate(live):
                rows[i].append(out[starts[j]:starts[j + 1]])
                at[i] += lengths[i]
        assert at == total and torch.isnan(state[1]).all() and torch.isnan(state[4]).all()
        return [torch.cat(r) for r in rows]
    cut = run([[5, 1, 2], [1, 0, 1], [2, 2, 0], [16, 8, 20], [13, 1, 2]])
    whole = run([total])
    for got, other, ref in zip(cut, whole, want):
        assert (got.double() - ref).abs().max() < 1e-5
        assert torch.equal(got, other)


# ------------------------------------------------------------------ streams mixed over depth, values blended

@pytest.mark.parametrize("count", [64 * 7, 101])
def test_weighted_sum_of_streams_and_blend_of_rows(count):
    from damendaemon_b200 import kernels
    stack = rnd(6, count, seed=5).to(DEV)
    w = rnd(5, seed=6).to(DEV)
    for n in (1, 2, 5):
        before = stack.clone()
        kernels.weighted_sum(stack, w, n, stack[5])
        want = (before[:n].double() * w[:n].double()[:, None]).sum(0)
        assert (stack[5].double() - want).abs().max() < 1e-5 and torch.equal(stack[:5], before[:5])
    for dtype in (torch.float32, torch.bfloat16):
        buf, other = rnd(7, 40, seed=7).to(dtype).to(DEV), rnd(7, 24, seed=8).to(dtype).to(DEV)
        v, src, lam = buf[:, 8:20], other[:, 3:15], torch.tensor(0.3, device=DEV)
        want = 0.7 * v.double() + 0.3 * src.double()
        kept = buf.clone()
        kernels.blend_rows(v, src, lam)
        assert (buf[:, 8:20].double() - want).abs().max() < (1e-6 if dtype == torch.float32 else 0.02)
        assert torch.equal(buf[:, :8], kept[:, :8]) and torch.equal(buf[:, 20:], kept[:, 20:])


# ------------------------------------------------------------------ the gated delta rule

def delta_operands(n, H, G, dk, dv, seed, sharp=1.0):
    q = plain.unit_vectors(rnd(n, G, dk, seed=seed).double()) * dk ** -0.5
    k = plain.unit_vectors(rnd(n, G, dk, seed=seed + 1).double())
    v = rnd(n, H, dv, seed=seed + 2).double()
    beta = torch.sigmoid(rnd(n, H, seed=seed + 3).double() * sharp)
    decay = torch.exp(-torch.exp(rnd(n, H, dk, seed=seed + 4).double() - 2.0))
    return q, k, v, beta, decay


def run_delta(ops, lengths, slots, state, H, G, dk, dv):
    from damendaemon_b200 import kernels
    starts, _ = layout(lengths)
    q, k, v, beta, decay = (t.float().reshape(t.shape[0], -1).contiguous().to(DEV) for t in ops)
    out = kernels.delta_rule(q, k, v, decay, beta, i32(starts), i32(slots), state, H, G, dk, dv)
    return out.cpu().double(), starts


@pytest.mark.parametrize("H,G,dk,dv", [(4, 2, 16, 24), (3, 3, 20, 12), (4, 4, 64, 64), (6, 2, 24, 10), (2, 1, 128, 64), (1, 1, 256, 40),
                                       (1, 1, 1, 1), (2, 2, 8, 130)])
def test_delta_rule_in_portions_against_the_recurrence(H, G, dk, dv):
    """Four requests of unequal length in shuffled slots: a first step of portions, then more portions down to two tokens
    and single tokens, a request left out of a step; every output equals the plain recurrence over the whole sequence."""
    from damendaemon_b200 import kernels
    n_slots, total, slots = 6, [60, 9, 40, 58], [4, 0, 5, 2]
    seqs = [delta_operands(n, H, G, dk, dv, 100 * i) for i, n in enumerate(total)]
    share = H // G
    want = [plain.delta_rule(q.repeat_interleave(share, 1), k.repeat_interleave(share, 1), v, b, d)[0].reshape(n, H * dv)
            for (q, k, v, b, d), n in zip(seqs, total)]
    state = torch.full((n_slots, *kernels.delta_state_shape(H, dk, dv)), float("nan"), device=DEV)
    for s in slots:
        state[s].zero_()
    at = [0] * 4
    for lengths in [[1, 5, 17, 40], [2, 1, 16, 1], [33, 1, 0, 2], [1, 2, 7, 1], [23, 0, 0, 14]]:
        live = [i for i, n in enumerate(lengths) if n]
        ops = [torch.cat([seqs[i][j][at[i]:at[i] + lengths[i]] for i in live]) for j in range(5)]
        out, starts = run_delta(ops, [lengths[i] for i in live], [slots[i] for i in live], state, H, G, dk, dv)
        for j, i in enumerate(live):
            ref = want[i][at[i]:at[i] + lengths[i]]
            assert (out[starts[j]:starts[j + 1]] - ref).abs().max() < 2e-5 * max(1.0, ref.abs().max().item()), (i, at[i])
            at[i] += lengths[i]
    assert at == total and torch.isnan(state[1]).all() and torch.isnan(state[3]).all()


def test_a_prompt_equals_its_tokens_one_by_one_and_a_far_token_is_read_through_the_state():
    """Bit equality of a prompt against single-token steps; and a value written 700 tokens back under a key that nothing
    else touches, with no decay on that key's channel, is read back exactly by a query along that key."""
    from damendaemon_b200 import kernels
    H, G, dk, dv, n = 2, 1, 32, 48, 760
    q, k, v, beta, decay = delta_operands(n, H, G, dk, dv, 7)
    k[:, :, 5] = 0.0                                       # channel 5 belongs to the marked token alone
    k[30] = 0.0
    k[30, :, 5] = 1.0
    beta[30] = 1.0
    decay[:, :, 5] = 1.0
    q[730] = 0.0
    q[730, :, 5] = 1.0
    ops = (q, k, v, beta, decay)
    state = torch.zeros((2, *kernels.delta_state_shape(H, dk, dv)), device=DEV)
    whole, _ = run_delta(ops, [n], [0], state, H, G, dk, dv)
    assert (whole[730].reshape(H, dv) - v[30]).abs().max() < 1e-5
    ref = plain.delta_rule(q.repeat_interleave(2, 1), k.repeat_interleave(2, 1), v, beta, decay)[0].reshape(n, -1)
    assert (whole - ref).abs().max() < 5e-5
    rows = [run_delta([t[:700] for t in ops], [700], [1], state, H, G, dk, dv)[0]]
    for t in range(700, n):
        rows.append(run_delta([x[t:t + 1] for x in ops], [1], [1], state, H, G, dk, dv)[0])
    assert torch.equal(torch.cat(rows), whole) and torch.equal(state[0], state[1])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,taps", [(4, 2, 16, 24, 3), (3, 3, 20, 12, 1), (2, 1, 64, 32, 4), (1, 1, 40, 36, 2), (2, 2, 8, 8, 6)])
def test_delta_operands_convolution_state_and_finish(H, G, dk, dv, taps, dtype):
    """The prepare kernel over steps of portions (down to one token, shorter than the taps) against the plain pieces over
    the whole sequence: convolution through the carried inputs, silu, unit vectors, decay and beta; then the read-out's
    norm and gate."""
    from damendaemon_b200 import kernels
    total, slots = [23, 7], [2, 0]
    C = 2 * G * dk + H * dv
    taps_w = rnd(C, taps, seed=9)
    a_log, dt_bias = rnd(H, seed=10) - 1.0, rnd(H * dk, seed=11)
    seqs, want = [], []
    for i, n in enumerate(total):
        proj = rnd(n, C + H + 3, seed=60 + i).to(dtype)                  # q | k | v | beta | something behind
        step = rnd(n, H * dk, seed=70 + i)
        seqs.append((proj, step))
        act = plain.silu(plain.short_convolution(proj[:, :C].double(), taps_w.double()))
        q = plain.unit_vectors(act[:, :G * dk].reshape(n, G, dk)) * dk ** -0.5
        k = plain.unit_vectors(act[:, G * dk:2 * G * dk].reshape(n, G, dk))
        decay = torch.exp(-torch.exp(a_log.double())[None, :, None] *
                          torch.nn.functional.softplus(step.double() + dt_bias.double()).reshape(n, H, dk))
        want.append((q.reshape(n, -1), k.reshape(n, -1), act[:, 2 * G * dk:], decay.reshape(n, -1), torch.sigmoid(proj[:, C:C + H].double())))
    conv_state = torch.full((3, taps - 1, C), float("nan"), device=DEV)
    for s in slots:
        conv_state[s].zero_()
    at = [0, 0]
    for lengths in [[1, 2], [1, 0], [2, 1], [12, 3], [7, 1]]:
        live = [i for i, n in enumerate(lengths) if n]
        proj = torch.cat([seqs[i][0][at[i]:at[i] + lengths[i]] for i in live]).to(DEV)
        step = torch.cat([seqs[i][1][at[i]:at[i] + lengths[i]] for i in live]).to(DEV)
        starts, entry = layout([lengths[i] for i in live])
        es, sl = i32(starts), i32([slots[i] for i in live])
        got = kernels.delta_prepare(proj, proj[:, C:C + H], step, taps_w.to(DEV), conv_state, a_log.to(DEV), dt_bias.to(DEV), i32(entry),
                                    es, sl, H, G, dk, dv)
        if taps > 1:
            kernels.conv_state_update(proj, conv_state, es, sl)
        for j, i in enumerate(live):
            for g, w in zip(got, want[i]):
                ref = w[at[i]:at[i] + lengths[i]]
                assert (g[starts[j]:starts[j + 1]].cpu().double() - ref).abs().max() < 2e-5, (i, at[i])
            at[i] += lengths[i]
    assert at == total and (taps == 1 or torch.isnan(conv_state[1]).all())
    o, gate, w = rnd(11, H * dv, seed=12, scale=3.0), rnd(11, H * dv, seed=13), 1.0 + rnd(dv, seed=14, scale=0.2)
    ref = (plain.rms(o.double().reshape(11, H, dv), 1e-5) * w.double() * torch.sigmoid(gate.double().reshape(11, H, dv))).reshape(11, -1)
    got = kernels.delta_finish(o.to(DEV), gate.to(DEV), w.to(DEV), H, 1e-5, dtype).cpu().double()
    assert (got - ref).abs().max() < (1e-5 if dtype == torch.float32 else 0.03)


# ------------------------------------------------------------------ attention: window with kept first keys, cap, sink

def paged(k, v, page_size, n_pages, seed, dtype, shuffle=True):
    """A cache [pages, ...] holding keys k [T, G, dk] and values v [T, G, dv] of one request in shuffled pages; pages that
    hold no token are filled with NaN. Returns (cache, block table row)."""
    T, G, dk = k.shape
    dv = v.shape[2]
    blocks = -(-T // page_size)
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed))[:blocks].tolist() if shuffle else list(range(blocks))
    cache = torch.full((n_pages, G * page_size * (dk + dv)), float("nan"), dtype=dtype)
    for b, page in enumerate(order):
        rows = slice(b * page_size, min(T, (b + 1) * page_size))
        n = rows.stop - rows.start
        keys = torch.full((G, page_size, dk), float("nan"), dtype=dtype)
        vals = torch.full((G, page_size, dv), float("nan"), dtype=dtype)
        keys[:, :n] = k[rows].transpose(0, 1).to(dtype)
        vals[:, :n] = v[rows].transpose(0, 1).to(dtype)
        cache[page] = torch.cat([keys.reshape(-1), vals.reshape(-1)])
    if dk == dv:
        cache = cache.view(n_pages, 2, G, page_size, dk)
    return cache.to(DEV), order


def plain_attention(q, k, v, scale, window, keep_first, cap, sink):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H, dv] with the plain pieces."""
    T, H, _ = q.shape
    share = H // k.shape[1]
    scores = torch.einsum("thd,shd->hts", q, k.repeat_interleave(share, 1)) * scale
    if cap:
        scores = cap * torch.tanh(scores / cap)
    w = plain.softmax_with_sink(scores, plain.visible(T, window, keep_first), sink)
    return torch.einsum("hts,shd->thd", w, v.repeat_interleave(share, 1))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,window,keep,cap,sinks,splits", [
    (4, 2, 16, 16, 24, 5, 8.0, True, 1), (3, 3, 12, 20, 7, 9, None, True, 3), (4, 1, 64, 64, 100, 33, 20.0, True, 4),
    (3, 1, 20, 12, 33, 0, 50.0, False, 2), (2, 2, 32, 32, None, 0, None, True, 5), (2, 1, 48, 40, 40, 20, 30.0, True, 1),
    (1, 1, 8, 8, 1, 1, None, True, 1), (2, 2, 128, 128, 70, 70, 3.0, False, 2)])
def test_attention_with_kept_first_keys_cap_and_sink(H, G, dk, dv, window, keep, cap, sinks, splits, dtype):
    """Every position of a sequence of 150 as a query in one launch (a prompt), and the last 50 again as single-token
    launches, over shuffled pages, with and without a split of the keys."""
    from damendaemon_b200 import kernels
    T, P = 150, 16
    q, k, v = (rnd(T, h, d, seed=s).to(dtype) for h, d, s in ((H, dk, 1), (G, dk, 2), (G, dv, 3)))
    sink = rnd(H, seed=4) if sinks else None
    scale = 2.0 * dk ** -0.5
    want = plain_attention(q.double(), k.double(), v.double(), scale, window, keep, cap, None if sink is None else sink.double())
    cache, order = paged(k, v, P, 14, 5, dtype)
    table = i32([order + [-1] * 3])
    kw = dict(window=window, keep_first=keep, softcap=cap, sink=None if sink is None else sink.to(DEV), kv_heads=G, v_dim=dv)
    tol = 2e-5 if dtype == torch.float32 else 0.03
    qd = q.reshape(T, H * dk).to(DEV)
    got = kernels.attention_rows(qd, cache, i32([0] * T), i32(list(range(T))), table, H, scale, n_splits=1, **kw)
    assert (got.cpu().double().view(T, H, dv) - want).abs().max() < tol
    for t in range(100, T):
        one = kernels.attention_rows(qd[t:t + 1], cache, i32([0]), i32([t]), table, H, scale, n_splits=splits, **kw)
        assert (one.cpu().double().view(H, dv) - want[t]).abs().max() < tol, t
    assert kernels.read_error_flag(DEV) == 0


@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("window,keep", [(40, 20), (16, 3), (7, 9), (33, 0)])
def test_a_marked_key_at_every_edge_decides_the_output(window, keep, decode):
    """One key that the query matches a hundred times better than the rest, with a value of its own: the output is that
    value when the key is just inside the window, or among the kept first keys, and not when it is just outside either;
    the same for the query's own position and for position zero. Pages of 8 so that the edges fall on page borders and
    beside them."""
    from damendaemon_b200 import kernels
    H, dk, dv, P = 2, 16, 8, 8
    for pos in (window + keep + 30, 199, 64):
        edges = {pos - window + 1: True, pos - window: pos - window < keep, pos: True, 0: keep > 0 or pos < window,
                 keep - 1: keep > 0, keep: pos - keep < window, pos - window + 2: True, 63: pos - 63 < window or 63 < keep}
        for marked, seen in edges.items():
            if not 0 <= marked <= pos:
                continue
            T = pos + 1
            k, v = rnd(T, 1, dk, seed=1) * 0.1, rnd(T, 1, dv, seed=2) * 0.1
            q = rnd(T, H, dk, seed=3) * 0.1
            k[marked, 0] = 0.0
            k[marked, 0, 3] = 30.0
            q[pos] = 0.0
            q[pos, :, 3] = 30.0
            v[marked, 0] = torch.arange(dv) + 5.0
            cache, order = paged(k, v, P, 40, marked, torch.float32)
            table = i32([order + [-1] * 2])
            qd = q.reshape(T, H * dk).to(DEV)
            kw = dict(window=window, keep_first=keep, sink=torch.zeros(H, device=DEV), kv_heads=1, v_dim=dv)
            if decode:
                out = kernels.attention_rows(qd[pos:], cache, i32([0]), i32([pos]), table, H, 1.0, n_splits=3, **kw)[0]
            else:
                out = kernels.attention_rows(qd, cache, i32([0] * T), i32(list(range(T))), table, H, 1.0, **kw)[pos]
            hit = (out.cpu().view(H, dv) - v[marked, 0]).abs().max().item() < 1e-3
            assert hit == bool(seen), (pos, marked, seen)


@pytest.mark.parametrize("exact", [False, True])
@pytest.mark.parametrize("H,G,d,window,keep,cap,sinks", [
    (4, 2, 64, 100, 33, 20.0, True), (3, 3, 64, 70, 9, None, True), (2, 1, 128, 130, 70, 3.0, False), (4, 4, 64, None, 0, None, True),
    (2, 2, 128, 64, 64, 10.0, True), (6, 2, 64, 65, 130, None, True), (2, 2, 64, 1, 1, 5.0, True)])
def test_tensor_core_attention_with_kept_first_keys_cap_and_sink(H, G, d, window, keep, cap, sinks, exact):
    """The mma.sync prompt kernel (whole prompt; portions that start anywhere; single tokens) and, where every head has
    keys of its own, the row decode kernel (with and without a split of the keys, the token's own key and value taken
    from the projection's rows and written by the kernel) against the plain pieces."""
    from damendaemon_b200 import kernels
    T, P = 330, 16
    dtype = torch.bfloat16
    q, k, v = (rnd(T, h, d, seed=s).to(dtype) for h, s in ((H, 1), (G, 2), (G, 3)))
    sink = rnd(H, seed=4) if sinks else None
    scale = 2.0 * d ** -0.5
    want = plain_attention(q.double(), k.double(), v.double(), scale, window, keep, cap, None if sink is None else sink.double())
    cache, order = paged(k, v, P, 26, 5, dtype)
    table = i32([order + [-1] * 3])
    kw = dict(window=window, keep_first=keep, softcap=cap, sink=None if sink is None else sink.to(DEV), exact_weights=exact)
    assert kernels.attention_prefill_supported(H, G, d, dtype)
    qd = q.reshape(T, H * d).to(DEV)
    tol = 0.012 if exact else 0.03
    got = kernels.attention_prefill(qd, cache, i32([0, T]), i32([0]), table, H, scale, **kw)
    assert (got.cpu().double().view(T, H, d) - want).abs().max() < tol
    for first, n in ((0, 1), (1, 2), (63, 66), (64, 64), (129, 201), (T - 1, 1), (200, 65)):
        part = kernels.attention_prefill(qd[first:first + n], cache, i32([0, n]), i32([first]), table, H, scale, **kw)
        assert (part.cpu().double().view(n, H, d) - want[first:first + n]).abs().max() < tol, (first, n)
    if exact:
        # the weights' second term takes the error below what rounding them to bfloat16 costs: against the general
        # kernel, whose weights are float32 over the same bfloat16 cache
        rows = kernels.attention_rows(qd, cache, i32([0] * T), i32(list(range(T))), table, H, scale, window=window, keep_first=keep,
                                      softcap=cap, sink=kw["sink"])
        assert (got.float() - rows.float()).abs().max() <= 2.0 ** -7 * max(1.0, rows.float().abs().max().item())
    if H == G and kernels.attention_decode_supported(H, G, d, dtype):
        for t in (0, 1, 15, 16, 17, 63, 64, 65, 100, 199, 200, 201, T - 1):
            for splits in (1, 3):
                one = kernels.attention_decode(qd[t:t + 1], cache, i32([0]), i32([t]), table, H, scale, n_splits=splits, **kw)
                assert (one.cpu().double().view(H, d) - want[t]).abs().max() < tol, (t, splits)
        # the token's own key and value from the projection's rows, into a page that held something else
        t = 205
        rows = torch.cat([q[t].reshape(-1), k[t].reshape(-1), v[t].reshape(-1)]).view(1, -1).to(DEV)
        qr, kr, vr = rows[:, :H * d], rows[:, H * d:2 * H * d], rows[:, 2 * H * d:]
        spoiled = cache.clone()
        spoiled[order[t // P], :, :, t % P] = 7.0
        one = kernels.attention_decode(qr, spoiled, None, i32([t]), table, H, scale, n_splits=2, k_new=kr, v_new=vr, **kw)
        assert (one.cpu().double().view(H, d) - want[t]).abs().max() < tol
        assert torch.equal(spoiled[order[t // P]], cache[order[t // P]])
    assert kernels.read_error_flag(DEV) == 0


@pytest.mark.parametrize("kernel", ["prompt", "decode"])
@pytest.mark.parametrize("window,keep", [(40, 20), (16, 3), (7, 9), (33, 0), (64, 64), (65, 130)])
def test_a_marked_key_at_every_edge_decides_the_output_of_the_tensor_core_kernels(window, keep, kernel):
    """As above for the mma.sync prompt kernel (the query is the last row of a portion of 70) and the row decode kernel."""
    from damendaemon_b200 import kernels
    H, d, P = 2, 64, 16
    for pos in (window + keep + 30, 199, 64, 300):
        edges = {pos - window + 1: True, pos - window: pos - window < keep, pos: True, 0: keep > 0 or pos < window,
                 keep - 1: keep > 0, keep: pos - keep < window, pos - window + 2: True, 63: pos - 63 < window or 63 < keep,
                 64: pos - 64 < window or 64 < keep, 127: pos - 127 < window or 127 < keep}
        for marked, seen in edges.items():
            if not 0 <= marked <= pos:
                continue
            T = pos + 1
            k, v = rnd(T, H, d, seed=1) * 0.1, rnd(T, H, d, seed=2) * 0.1
            q = rnd(T, H, d, seed=3) * 0.1
            k[marked] = 0.0
            k[marked, :, 3] = 30.0
            q[pos] = 0.0
            q[pos, :, 3] = 30.0
            v[marked] = torch.arange(d) + 5.0
            cache, order = paged(k, v, P, 30, marked, torch.bfloat16)
            table = i32([order + [-1] * 2])
            qd = q.reshape(T, H * d).to(torch.bfloat16).to(DEV)
            kw = dict(window=window, keep_first=keep, sink=torch.zeros(H, device=DEV), exact_weights=True)
            if kernel == "decode":
                out = kernels.attention_decode(qd[pos:], cache, i32([0]), i32([pos]), table, H, 1.0, n_splits=3, **kw)[0]
            else:
                first = max(0, pos - 69)
                out = kernels.attention_prefill(qd[first:], cache, i32([0, T - first]), i32([first]), table, H, 1.0, **kw)[-1]
            hit = (out.float().cpu().view(H, d) - v[marked]).abs().max().item() < 0.3
            assert hit == bool(seen), (pos, marked, seen)


# ------------------------------------------------------------------ attention over latent rows

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dk,dr,dv,R,dims", [(3, 16, 8, 20, 40, 8), (2, 24, 16, 12, 32, 8), (4, 64, 32, 64, 128, 32), (5, 12, 12, 20, 36, 6),
                                               (3, 48, 64, 80, 192, 64), (1, 8, 4, 8, 24, 4), (2, 10, 6, 7, 13, 6)])
def test_latent_rows_per_head_products_and_attention_against_the_plain_mixer(H, dk, dr, dv, R, dims, dtype):
    """The latent mixer's kernels in the order the part runs them, from given projections: prepare (norm, rotation, cache
    row), the queries through the transposed key matrices, attention over the rows with a sink, the values through W_uv.
    A prompt of 130 in two portions, then 20 single tokens, pages shuffled. The plain side computes keys and values of
    every head explicitly."""
    from damendaemon_b200 import kernels
    T, P, base, eps = 150, 16, 300.0, 1e-5
    Qw = H * (dk + dr)
    proj = rnd(T, Qw + R + dr + 5, seed=1).to(dtype)
    proj[:, :Qw] *= 3.0
    wn, uk, uv, sink = 1.0 + rnd(R, seed=2, scale=0.2), rnd(H * dk, R, seed=3).to(dtype) / math.sqrt(R), rnd(H * dv, R, seed=4).to(dtype) / math.sqrt(R), rnd(H, seed=5)
    scale = (dk + dr) ** -0.5
    # the plain side, as the mixer's function does it after the projections
    pos = torch.arange(T)
    q = proj[:, :Qw].double().view(T, H, dk + dr)
    q_plain, q_turn = q[..., :dk], plain.rotate_neighbours(q[..., dk:], pos, dims, base)
    down = proj[:, Qw:Qw + R + dr].double()
    latent_rows = plain.rms(down[:, :R], eps) * wn.double()
    k_turn = plain.rotate_neighbours(down[:, None, R:], pos, dims, base)[:, 0]
    keys = (latent_rows @ uk.double().T).view(T, H, dk)
    vals = (latent_rows @ uv.double().T).view(T, H, dv)
    scores = (torch.einsum("thd,shd->hts", q_plain, keys) + torch.einsum("thd,sd->hts", q_turn, k_turn)) * scale
    want = torch.einsum("hts,shd->thd", plain.softmax_with_sink(scores, plain.visible(T), sink.double()), vals)
    # the kernels
    n_pages = 12
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(6))[:-(-T // P)].tolist()
    cache = torch.full((n_pages, P * (R + dr)), float("nan"), dtype=dtype, device=DEV)
    table = i32([order + [-1]])
    freqs = (base ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)).float().to(DEV)
    key_t = uk.view(H, dk, R).transpose(1, 2).contiguous().to(DEV)
    value_up = uv.view(H, dv, R).contiguous().to(DEV)
    dev = proj.to(DEV)
    got = []
    for lo, hi, splits in [(0, 77, 1), (77, 130, 1)] + [(t, t + 1, 1 + t % 3) for t in range(130, T)]:
        n = hi - lo
        rows = dev[lo:hi]
        qv, dn = rows[:, :Qw], rows[:, Qw:Qw + R + dr]
        positions = i32(list(range(lo, hi)))
        kernels.latent_prepare(qv, dn, wn.to(DEV), eps, freqs, i32([0] * n), positions, table, cache, H, dk, dr, R)
        q_rows = kernels.per_head_linear(qv, key_t, dk + dr, tail=dr)
        mixed = kernels.attention_rows(q_rows, cache, i32([0] * n), positions, table, H, scale, n_splits=splits, kv_heads=1,
                                       v_dim=R, sink=sink.to(DEV), values_in_keys=True)
        got.append(kernels.per_head_linear(mixed, value_up, R).cpu().double().view(n, H, dv))
    assert kernels.read_error_flag(DEV) == 0
    err = (torch.cat(got) - want).abs().max().item()
    assert err < (5e-5 if dtype == torch.float32 else 0.06), err
    assert torch.equal(dev[:, Qw + R + dr:].cpu(), proj[:, Qw + R + dr:])          # what lies behind is untouched


def test_a_far_latent_row_among_hundreds_is_found():
    """900 rows; the query's rotated part matches the shared key part of one row far back (at a page border) at the right
    relative angle only, a hundred times better than any other: the output is that row's value."""
    from damendaemon_b200 import kernels
    H, dk, dr, dv, R, P, T = 2, 8, 8, 6, 16, 16, 900
    Qw = H * (dk + dr)
    for marked in (16 * 13, 16 * 13 - 1, 0, 898):
        proj = rnd(T, Qw + R + dr, seed=marked + 1) * 0.05
        proj[marked, Qw:Qw + R] = rnd(R, seed=2) * 4.0                 # a latent of its own (the norm rescales it)
        proj[marked, Qw + R:] = 0.0
        proj[marked, Qw + R] = 40.0                                    # shared key part: along the first pair's axis
        proj[T - 1, :Qw] = 0.0
        for h in range(H):
            proj[T - 1, h * (dk + dr) + dk] = 40.0                     # the query's rotated part likewise
        wn, uk, uv = torch.ones(R), rnd(H * dk, R, seed=3) * 0.01, rnd(H * dv, R, seed=4)
        # one pair turns at one radian a token: the two meet only if both are rotated by their own positions
        freqs = torch.tensor([1.0, 0.0, 0.0, 0.0], device=DEV)
        latent_row = plain.rms(proj[marked, Qw:Qw + R].double(), 1e-5)
        want = (uv.double() @ latent_row).view(H, dv)
        cache = torch.full((60, P * (R + dr)), float("nan"), device=DEV)
        order = torch.randperm(60, generator=torch.Generator().manual_seed(9))[:57].tolist()
        table = i32([order])
        dev = proj.to(DEV)
        positions = i32(list(range(T)))
        kernels.latent_prepare(dev[:, :Qw], dev[:, Qw:], wn.to(DEV), 1e-5, freqs, i32([0] * T), positions, table, cache, H, dk, dr, R)
        q_rows = kernels.per_head_linear(dev[T - 1:, :Qw], uk.view(H, dk, R).transpose(1, 2).contiguous().to(DEV), dk + dr, tail=dr)
        mixed = kernels.attention_rows(q_rows, cache, i32([0]), i32([T - 1]), table, H, 1.0, n_splits=4, kv_heads=1, v_dim=R,
                                       sink=torch.zeros(H, device=DEV), values_in_keys=True)
        got = kernels.per_head_linear(mixed, uv.view(H, dv, R).contiguous().to(DEV), R).cpu().double().view(H, dv)
        assert (got - want).abs().max() < 2e-2, marked


@pytest.mark.parametrize("H,R,dr,splits", [(5, 48, 16, 1), (25, 256, 64, 1), (3, 320, 32, 3), (7, 448, 64, 2), (2, 16, 16, 4), (16, 80, 48, 1), (40, 64, 16, 2), (33, 144, 32, 3)])
def test_tensor_core_attention_over_latent_rows_against_the_general_kernel(H, R, dr, splits):
    """Three requests side by side on shuffled pages: a portion that starts inside a page behind 70 cached rows, a prompt
    from its start, and a single token behind 200 rows; then the same single token with its keys cut into splits."""
    from damendaemon_b200 import kernels
    P, row = 16, R + dr
    held, new = [70, 0, 200], [45, 130, 1]
    n_pages = sum(-(-(a + b) // P) for a, b in zip(held, new)) + 3
    pages = torch.randperm(n_pages, generator=torch.Generator().manual_seed(3)).tolist()
    cache = torch.full((n_pages, P * row), float("nan"), dtype=torch.bfloat16, device=DEV)
    width = max(-(-(a + b) // P) for a, b in zip(held, new)) + 1
    table = []
    for e, (a, b) in enumerate(zip(held, new)):
        mine = [pages.pop() for _ in range(-(-(a + b) // P))]
        table.append(mine + [-1] * (width - len(mine)))
        rows = (rnd(a + b, row, seed=10 + e) * 0.7).to(torch.bfloat16).to(DEV)
        for t in range(a + b):
            cache[mine[t // P], (t % P) * row:(t % P + 1) * row] = rows[t]
    table = i32(table)
    starts, entry = layout(new)
    positions = [a + t for a, b in zip(held, new) for t in range(b)]
    q = (rnd(sum(new), H * row, seed=4) * 1.5).to(torch.bfloat16).to(DEV)
    sink = rnd(H, seed=5).to(DEV)
    scale = row ** -0.5
    want = kernels.attention_rows(q, cache, i32(entry), i32(positions), table, H, scale, kv_heads=1, v_dim=R, sink=sink,
                                  values_in_keys=True).float()
    got = kernels.attention_latent(q, cache, i32(starts), i32(held), table, H, R, scale, sink=sink).float()
    assert kernels.read_error_flag(DEV) == 0
    assert (got - want).abs().max().item() < 0.02, (got - want).abs().max().item()
    one = kernels.attention_latent(q[-1:], cache, i32([0, 1]), i32(held[2:]), table[2:], H, R, scale, n_splits=splits, sink=sink).float()
    assert (one - want[-1:]).abs().max().item() < 0.02
    none = kernels.attention_latent(q[-1:], cache, i32([0, 1]), i32(held[2:]), table[2:], H, R, scale, n_splits=splits).float()
    plain_one = kernels.attention_rows(q[-1:], cache, i32([0]), i32(positions[-1:]), table[2:], H, scale, kv_heads=1, v_dim=R,
                                       values_in_keys=True).float()
    assert (none - plain_one).abs().max().item() < 0.02


@pytest.mark.parametrize("decode", [False, True])
def test_a_marked_latent_row_decides_the_output_of_the_tensor_core_kernel(decode):
    """600 rows of noise and one whose last element answers the query a hundred times better, placed at the first row, at
    page and tile borders, and at the query's own place: the output is that row's first elements. One place later than
    the query it is not seen."""
    from damendaemon_b200 import kernels
    H, R, dr, P, T = 3, 32, 16, 16, 600
    row = R + dr
    for marked in (0, 63, 64, 16 * 17 - 1, 16 * 17, T - 2, T - 1):
        for at in (T - 1, marked, marked - 1):
            if at < 0:
                continue
            rows = (rnd(T, row, seed=marked + 1) * 0.05).to(torch.bfloat16)
            rows[marked, :R] = torch.arange(R) / 8.0 - 2.0
            rows[marked, row - 1] = 6.0
            cache = rows.view(-1).clone()
            cache = torch.cat([cache, torch.zeros((-T % P) * row, dtype=torch.bfloat16)]).view(-1, P * row).to(DEV)
            table = i32([list(range(cache.shape[0]))])
            q = torch.zeros(T, H * row, dtype=torch.bfloat16)
            q.view(T, H, row)[:, :, row - 1] = 6.0
            q = q.to(DEV)
            if decode:
                out = kernels.attention_latent(q[at:at + 1], cache, i32([0, 1]), i32([at]), table, H, R, 1.0, n_splits=3)[0]
            else:
                out = kernels.attention_latent(q[:at + 1], cache, i32([0, at + 1]), i32([0]), table, H, R, 1.0)[at]
            out = out.float().cpu().view(H, R)
            if at >= marked:
                assert (out - rows[marked, :R].float()).abs().max() < 0.02, (marked, at)
            else:
                assert out.abs().max() < 0.2, (marked, at)


@pytest.mark.parametrize("n,H,I,J,tail,stride_pad", [(130, 3, 48, 40, 8, 0), (1, 25, 64, 256, 64, 0), (77, 2, 256, 130, 0, 24), (9, 5, 40, 6, 8, 8),
                                                     (64, 1, 512, 128, 0, 0)])
def test_per_head_products_on_the_tensor_cores(n, H, I, J, tail, stride_pad):
    from damendaemon_b200 import kernels
    x = rnd(n, H * (I + tail) + stride_pad, seed=1).to(torch.bfloat16).to(DEV)
    w = (rnd(H, J, I, seed=2) / math.sqrt(I)).to(torch.bfloat16).to(DEV)
    got = kernels.per_head_linear(x[:, :H * (I + tail)], w, I + tail, tail=tail, kernel="mma").float().view(n, H, J + tail)
    heads = x[:, :H * (I + tail)].float().view(n, H, I + tail)
    want = torch.einsum("nhi,hji->nhj", heads[..., :I].double(), w.double())
    assert (got[..., :J].double() - want).abs().max().item() < 0.03
    assert torch.equal(got[..., J:], heads[..., I:])
    plain_kernel = kernels.per_head_linear(x[:, :H * (I + tail)], w, I + tail, tail=tail, kernel="plain").float().view(n, H, J + tail)
    assert (got - plain_kernel).abs().max().item() < 0.03


# ------------------------------------------------------------------ the clamped gated unit through the feed-forward part

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_clamped_unit_of_the_feed_forward(dtype):
    from damendaemon_b200.parts import Runtime
    from damendaemon_b200.parts.feed_forward import GatedFeedForward
    from damendaemon_b200.parts.spec import GatedFeedForwardSpec, GatedUnitSpec
    from damendaemon_b200 import kernels
    kernels.library("core")
    t = getattr(torch, dtype)
    width, ff, limit = 64, 88, 0.8
    w = {"g": rnd(ff, width, seed=1).to(t) * 0.3, "u": rnd(ff, width, seed=2).to(t) * 0.3, "d": rnd(width, ff, seed=3).to(t) * 0.1}
    spec = GatedFeedForwardSpec("gated", width, GatedUnitSpec(ff, limit, "g", "u", "d", alpha=1.702, activation="clamped_swish"))
    placed = {}
    for d in GatedFeedForward.tensor_decls(spec):
        placed[d.name] = torch.cat([w[n] for n, _ in d.pieces]).to(DEV) if d.pieces else w[d.name].to(DEV)
    part = GatedFeedForward(spec, placed, Runtime(dtype=t, device=torch.device(DEV)))
    y = rnd(13, width, seed=4, scale=3.0).to(t)
    stream = rnd(13, width, seed=5)
    want = stream.double() + plain.clamped_unit(y.double(), {"p.gate": w["g"].double(), "p.up": w["u"].double(), "p.down": w["d"].double()}, "p.", limit)
    got = part.forward(y.to(DEV), stream.to(DEV), None).cpu().double()
    assert (got - want).abs().max() < (1e-4 if dtype == "float32" else 0.05)
