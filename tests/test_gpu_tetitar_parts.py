"""Tetitar's kernels and parts, each alone against the plain implementation's function for the same mechanism."""
import math

import pytest
import torch

import plain_tetitar as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def gen(seed):
    return torch.Generator().manual_seed(seed)


def randn(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=gen(seed)) * scale


def entries_meta(lengths, slots):
    """Device arrays of a step whose entries bring ``lengths`` tokens: token_entry, entry_start, entry_slot."""
    ent = torch.tensor([e for e, n in enumerate(lengths) for _ in range(n)], dtype=torch.int32, device=DEV)
    start = torch.tensor([sum(lengths[:i]) for i in range(len(lengths) + 1)], dtype=torch.int32, device=DEV)
    return ent, start, torch.tensor(slots, dtype=torch.int32, device=DEV)


def cuts(total, sizes):
    out, at, i = [], 0, 0
    while at < total:
        n = min(sizes[i % len(sizes)], total - at)
        out.append((at, at + n))
        at, i = at + n, i + 1
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pair_embedding_keeps_the_token_before_per_request(dtype):
    """Two requests fed in portions through shuffled slots, another request's steps between them: every row equals the plain
    embedding of the whole sequence; multipliers whose product with an id does not fit 32 bits."""
    from damendaemon_b200 import kernels
    vocab, width, m = 97, 40, {"buckets": 1000003, "mul_prev": 2000000011, "mul_cur": 1999999973}
    m_small = {"buckets": 13, "mul_prev": 5, "mul_cur": 3}
    for pair in (m_small, m):
        rows = min(pair["buckets"], 5000) + 1
        pair = dict(pair, buckets=rows - 1)
        table, pairs = randn(vocab, width, seed=1).to(dtype), randn(rows, width, seed=2).to(dtype)
        w = {"embed": table.double(), "bigram": pairs.double()}
        config = {"embedding": {"bigram": pair}}
        seqs = {0: torch.randint(0, vocab, (23,), generator=gen(3)).tolist(), 1: torch.randint(0, vocab, (9,), generator=gen(4)).tolist()}
        want = {r: plain.embedding(s, w, config) for r, s in seqs.items()}
        last = torch.full((4,), 12345, dtype=torch.int32, device=DEV)
        slot = {0: 3, 1: 1}
        last[3] = last[1] = 0                       # what taking a slot does
        at = {0: 0, 1: 0}
        for sizes in ((5, 1), (1, 3), (2, 2), (7, 1), (8, 2)):
            lengths = [min(n, len(seqs[r]) - at[r]) for r, n in enumerate(sizes)]
            order = [r for r in (1, 0) if lengths[r] > 0]
            ids = torch.tensor([t for r in order for t in seqs[r][at[r]:at[r] + lengths[r]]], dtype=torch.int32, device=DEV)
            pos = torch.tensor([p for r in order for p in range(at[r], at[r] + lengths[r])], dtype=torch.int32, device=DEV)
            ent, start, slots = entries_meta([lengths[r] for r in order], [slot[r] for r in order])
            x = kernels.embed_pairs(ids, pos, ent, start, slots, table.to(DEV), pairs.to(DEV), last, pair["mul_prev"], pair["mul_cur"]).cpu()
            row = 0
            for r in order:
                n = lengths[r]
                assert torch.allclose(x[row:row + n].double(), want[r][at[r]:at[r] + n], atol=1e-6), (pair, r, at[r])
                row, at[r] = row + n, at[r] + n
        assert at == {0: 23, 1: 9} and last[0].item() == 12345 and last[3].item() == seqs[0][-1]


def test_tanh_norm_and_small_row_operations():
    from damendaemon_b200 import kernels
    for width in (40, 100, 1028):
        x = randn(7, width, seed=1, scale=3.0)
        w = {"n": randn(width, seed=2).double(), "n.b": randn(width, seed=3).double(), "n.alpha": torch.tensor(0.37, dtype=torch.float64)}
        want = plain.tanh_norm(x.double(), w, "n")
        args = (torch.tensor([0.37], device=DEV), w["n"].float().to(DEV), w["n.b"].float().to(DEV))
        got = kernels.tanh_norm(x.to(DEV), *args, torch.float32)
        assert torch.allclose(got.cpu().double(), want, atol=2e-6)
        rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
        assert torch.equal(kernels.tanh_norm(x.to(DEV), *args, torch.float32, rows), got[[5, 0, 5]])
        assert torch.allclose(kernels.tanh_norm(x.to(DEV), *args, torch.bfloat16).float().cpu().double(), want, atol=3e-2)
        # x += other + vec
        y, other, vec = x.to(DEV).clone(), randn(7, width, seed=4).to(DEV), randn(width, seed=5).to(DEV)
        assert torch.allclose(kernels.add_rows(y.clone(), other, vec), y + other + vec, atol=1e-6)
        assert torch.allclose(kernels.add_rows(y.clone(), None, vec), y + vec, atol=1e-6)
        # two results normed and averaged into the stream
        l, r = randn(7, width, seed=6, scale=5.0), randn(7, width, seed=7, scale=0.01)
        wl, wr = randn(width, seed=8), randn(width, seed=9)
        want = x.double() + 0.5 * (plain.rms(l.double(), 1e-5) * wl.double() + plain.rms(r.double(), 1e-5) * wr.double())
        got = kernels.norm_pair_add(x.to(DEV).clone(), l.to(DEV), r.to(DEV), wl.to(DEV), wr.to(DEV), 1e-5, 0.5)
        assert torch.allclose(got.cpu().double(), want, atol=1e-5)
        # the cap and the element-wise gate
        z = randn(5, width, seed=10, scale=20.0)
        assert torch.allclose(kernels.tanh_cap(z.to(DEV).clone(), 11.0).cpu(), 11.0 * torch.tanh(z / 11.0), atol=1e-5)
        buffer = randn(5, 2 * width, seed=11).to(DEV)
        o = randn(5, width, seed=12).to(DEV)
        want = o * torch.sigmoid(buffer[:, width:])
        assert torch.allclose(kernels.sigmoid_gate(o.clone(), buffer[:, width:]), want, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, kv_heads, d, dims, scaling", [(4, 2, 16, 8, (4.0, 1.0, 4.0, 64)), (1, 1, 32, 32, None),
                                                               (6, 2, 12, 2, (8.0, 0.5, 2.0, 32)), (4, 4, 64, 48, (8.0, 1.0, 4.0, 512))])
def test_norm_over_the_whole_projection_with_rotation(dtype, heads, kv_heads, d, dims, scaling):
    """q and k normed over all their heads at once and rotated in halves at positions up to 5,000, against the plain
    functions; the frequencies are the plain ones (stretched or not)."""
    from damendaemon_b200 import kernels
    from damendaemon_b200.parts.positions import rotary_frequencies
    from damendaemon_b200.parts.spec import RotarySpec, WavelengthStretch
    rot = {"dims": dims, "base": 100.0}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    spec = RotarySpec("rotary", d, dims, 100.0, interleaved=False, blend=WavelengthStretch(*scaling) if scaling else None)
    freqs = rotary_frequencies(spec)[0].float().to(DEV)
    n = 9
    positions = torch.tensor([0, 1, 2, 17, 100, 1023, 1024, 4999, 3], dtype=torch.int32)
    qw, kw = 1 + randn(heads * d, seed=1, scale=0.2), 1 + randn(kv_heads * d, seed=2, scale=0.2)
    buffer = randn(n, (heads + kv_heads) * d + 8, seed=3, scale=2.0).to(dtype)
    q, k = buffer[:, :heads * d], buffer[:, heads * d:(heads + kv_heads) * d]
    want_q = plain.rotate_halves((plain.rms(q.double(), 1e-5) * qw.double()).reshape(n, heads, d), positions, rot).reshape(n, -1)
    want_k = plain.rotate_halves((plain.rms(k.double(), 1e-5) * kw.double()).reshape(n, kv_heads, d), positions, rot).reshape(n, -1)
    dev = buffer.to(DEV)
    kernels.wide_norm_rotary(dev[:, :heads * d], dev[:, heads * d:(heads + kv_heads) * d], positions.to(DEV), qw.to(DEV), kw.to(DEV),
                             1e-5, heads, kv_heads, d, freqs=freqs, interleaved=False)
    # float32: a frequency is rounded to 32 bits and so is its product with the position, so the angle at position p is off
    # by up to p * 1.2e-7, and an element (at most 8 here) by that times its size
    tol = torch.full((n, 1), 3e-2, dtype=torch.float64) if dtype == torch.bfloat16 else 2e-5 + positions.double()[:, None] * 1.2e-7 * 8
    got = dev.cpu().double()
    assert ((got[:, :heads * d] - want_q).abs() <= tol).all() and ((got[:, heads * d:(heads + kv_heads) * d] - want_k).abs() <= tol).all()
    assert torch.equal(got[:, (heads + kv_heads) * d:], buffer[:, (heads + kv_heads) * d:].double())     # the rest is untouched


@pytest.mark.parametrize("taps", [1, 2, 4])
def test_convolution_in_portions_continues_from_the_state(taps):
    from damendaemon_b200 import kernels
    C, total = 70, 41
    for dtype in (torch.float32, torch.bfloat16):
        x = {r: randn(total - 7 * r, C + 5, seed=r).to(dtype) for r in range(2)}
        w, b = randn(C, taps, seed=5), randn(C, seed=6)
        state = torch.full((3, taps - 1, C), float("nan"), device=DEV)
        slot = {0: 2, 1: 0}
        for s in slot.values():
            state[s] = 0
        for act, f in ((None, lambda v: v), ("silu", plain.silu)):
            for s in slot.values():
                state[s] = 0
            want = {r: f(plain.causal_convolution(x[r][:, :C].double(), w.double(), b.double())) for r in x}
            parts = {0: cuts(total, (1, 2, 5, 1, 1, 11)), 1: cuts(total - 7, (3, 1, 9))}
            for i in range(max(len(p) for p in parts.values())):
                live = [r for r in (1, 0) if i < len(parts[r])]
                rows = torch.cat([x[r][parts[r][i][0]:parts[r][i][1]] for r in live]).to(DEV)
                ent, start, slots = entries_meta([parts[r][i][1] - parts[r][i][0] for r in live], [slot[r] for r in live])
                got = kernels.conv_channels(rows[:, :C], w.to(DEV), b.to(DEV), state, ent, start, slots, activation=act).cpu().double()
                if taps > 1:
                    kernels.conv_state_update(rows[:, :C], state, start, slots)
                at = 0
                for r in live:
                    a, e = parts[r][i]
                    assert torch.allclose(got[at:at + e - a], want[r][a:e], atol=1e-5), (taps, act, r, a)
                    at += e - a


def plain_state_space_core(xbc, dt_raw, dt_bias, a_log, skip, H, G, N, dv):
    """The recurrence alone, float64: xbc [T, H dv + 2 G N] after the convolution, dt_raw [T, H]."""
    T, inner = xbc.shape[0], H * dv
    x, B, C = xbc[:, :inner].reshape(T, H, dv), xbc[:, inner:inner + G * N].reshape(T, G, N), xbc[:, inner + G * N:].reshape(T, G, N)
    dt = plain.softplus(dt_raw + dt_bias)
    decay = torch.exp(-torch.exp(a_log) * dt)
    group = torch.arange(H) // (H // G)
    S = xbc.new_zeros(H, N, dv)
    y = xbc.new_zeros(T, H, dv)
    for t in range(T):
        S = decay[t][:, None, None] * S + dt[t][:, None, None] * B[t, group][:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnd,hn->hd", S, C[t, group]) + skip[:, None] * x[t]
    return y.reshape(T, inner)


@pytest.mark.parametrize("H, G, N, dv", [(4, 2, 48, 16), (2, 1, 16, 8), (6, 3, 20, 10), (1, 1, 8, 12), (4, 4, 128, 32), (2, 1, 24, 64), (3, 3, 1, 5)])
def test_state_space_scan_in_portions_with_shuffled_slots(H, G, N, dv):
    """Two requests in portions down to one token beside each other, in slots that are not in order, against the plain
    recurrence; a prompt cut anywhere gives the same bits as the prompt whole."""
    from damendaemon_b200 import kernels
    inner, total = H * dv, 57
    seqs = {r: (randn(total - 9 * r, inner + 2 * G * N, seed=r), randn(total - 9 * r, H + 3, seed=10 + r)) for r in range(2)}
    dt_bias, a_log, skip = randn(H, seed=20) - 1.0, randn(H, seed=21) * 0.7 - 0.5, 1 + randn(H, seed=22) * 0.1
    want = {r: plain_state_space_core(x.double(), d[:, :H].double(), dt_bias.double(), a_log.double(), skip.double(), H, G, N, dv)
            for r, (x, d) in seqs.items()}
    shape = kernels.state_space_state_shape(H, N, dv)
    params = (dt_bias.to(DEV), a_log.to(DEV), skip.to(DEV))

    def run(parts):
        state = torch.full((4, *shape), float("nan"), device=DEV)
        slot = {0: 3, 1: 1}
        for s in slot.values():
            state[s] = 0
        out = {r: [] for r in seqs}
        for i in range(max(len(p) for p in parts.values())):
            live = [r for r in (1, 0) if i < len(parts[r])]
            x = torch.cat([seqs[r][0][parts[r][i][0]:parts[r][i][1]] for r in live]).to(DEV)
            d = torch.cat([seqs[r][1][parts[r][i][0]:parts[r][i][1]] for r in live]).to(DEV)
            _, start, slots = entries_meta([parts[r][i][1] - parts[r][i][0] for r in live], [slot[r] for r in live])
            y = kernels.state_space_scan(x, d[:, :H], *params, start, slots, state, H, G, N, dv).cpu()
            at = 0
            for r in live:
                n = parts[r][i][1] - parts[r][i][0]
                out[r].append(y[at:at + n])
                at += n
        return {r: torch.cat(v) for r, v in out.items()}
    whole = run({0: [(0, total)], 1: [(0, total - 9)]})
    cut = run({0: cuts(total, (1, 2, 7, 1, 1, 16)), 1: cuts(total - 9, (5, 1, 1, 30))})
    for r in seqs:
        scale = want[r].abs().max().item()
        assert torch.allclose(whole[r].double(), want[r], atol=2e-5 * max(1.0, scale)), (r, (whole[r].double() - want[r]).abs().max())
        assert torch.equal(whole[r], cut[r])


def test_a_token_far_back_reaches_the_read_out_through_a_slow_state():
    """A head that hardly decays carries one marked token over 3,000 steps: the read-out of the last token is that token's
    value to a relative 1e-4 although the decay per step differs from one by 1e-5 only (a decay rounded to float32 would be
    off by up to 6e-8 of one a step, 2e-4 over the distance)."""
    from damendaemon_b200 import kernels
    H, G, N, dv, T = 1, 1, 8, 4, 3000
    xbc = torch.zeros(T, dv + 2 * N)
    xbc[0, :dv] = torch.tensor([1.0, -2.0, 3.0, 0.5])
    xbc[0, dv] = 1.0                                  # B of the marked token
    xbc[:, dv + N] = 1.0                              # every token reads row 0
    dt = torch.zeros(T, 1)
    a_log = torch.tensor([math.log(1.4427e-5)])       # decay = exp(-1.4427e-5 * softplus(0)) = exp(-1e-5)
    args = (torch.zeros(1), a_log, torch.zeros(1))
    want = plain_state_space_core(xbc.double(), dt.double(), *(a.double() for a in args), H, G, N, dv)
    state = torch.zeros((1, *kernels.state_space_state_shape(H, N, dv)), device=DEV)
    _, start, slots = entries_meta([T], [0])
    got = kernels.state_space_scan(xbc.to(DEV), dt.to(DEV), *(a.to(DEV) for a in args), start, slots, state, H, G, N, dv).cpu().double()
    assert want[-1].abs().max() > 0.3 and torch.allclose(got[-1], want[-1], rtol=1e-5, atol=0)


def test_gated_group_norm():
    from damendaemon_b200 import kernels
    for inner, groups in ((128, 2), (60, 3), (96, 1), (512, 4)):
        for dtype in (torch.float32, torch.bfloat16):
            y, buffer, w = randn(6, inner, seed=1, scale=4.0), randn(6, inner + 16, seed=2).to(dtype), 1 + randn(inner, seed=3) * 0.1
            z = buffer[:, 8:8 + inner]
            gated = y.double() * plain.silu(z.double())
            want = plain.rms(gated.reshape(6, groups, -1), 1e-5).reshape(6, inner) * w.double()
            got = kernels.gated_group_norm(y.to(DEV), buffer.to(DEV)[:, 8:8 + inner], w.to(DEV), groups, 1e-5, dtype).float().cpu().double()
            assert torch.allclose(got, want, atol=1e-5 if dtype == torch.float32 else 3e-2)


@pytest.mark.parametrize("width, blocks", [(192, 4), (48, 3), (40, 1), (60, 5), (300, 2), (7, 7)])
def test_gated_linear_recurrence_in_portions(width, blocks):
    """Gates and scan against the plain recurrence (its branches given), two requests in portions with shuffled slots; cut
    anywhere the bits are those of the whole prompt."""
    from damendaemon_b200 import kernels
    part, total = width // blocks, 45
    wts = {"ra": randn(blocks, part, part, seed=1) / math.sqrt(part), "ra.b": randn(blocks, part, seed=2) * 0.1,
           "ri": randn(blocks, part, part, seed=3) / math.sqrt(part), "ri.b": randn(blocks, part, seed=4) * 0.1,
           "lam": randn(width, seed=5) * 1.5 - 2.0}
    seqs = {r: (randn(total - 6 * r, width, seed=10 + r), randn(total - 6 * r, width + 4, seed=20 + r)) for r in range(2)}

    def plain_core(u, y):
        T = u.shape[0]
        ub = u.reshape(T, blocks, part)
        r = torch.sigmoid(torch.einsum("boi,tbi->tbo", wts["ra"].double(), ub) + wts["ra.b"].double()).reshape(T, width)
        i = torch.sigmoid(torch.einsum("boi,tbi->tbo", wts["ri"].double(), ub) + wts["ri.b"].double()).reshape(T, width)
        a = torch.exp(-8.0 * r * plain.softplus(wts["lam"].double()))
        S, out = u.new_zeros(width), u.new_zeros(T, width)
        for t in range(T):
            S = a[t] * S + torch.sqrt(1 - a[t] ** 2) * i[t] * u[t]
            out[t] = S * plain.gelu_tanh(y[t])
        return out
    want = {r: plain_core(u.double(), y[:, :width].double()) for r, (u, y) in seqs.items()}
    dev = {k: v.to(DEV) for k, v in wts.items()}

    def run(parts):
        state = torch.full((4, width), float("nan"), device=DEV)
        slot = {0: 2, 1: 3}
        for s in slot.values():
            state[s] = 0
        out = {r: [] for r in seqs}
        for i in range(max(len(p) for p in parts.values())):
            live = [r for r in (1, 0) if i < len(parts[r])]
            u = torch.cat([seqs[r][0][parts[r][i][0]:parts[r][i][1]] for r in live]).to(DEV)
            y = torch.cat([seqs[r][1][parts[r][i][0]:parts[r][i][1]] for r in live]).to(DEV)
            _, start, slots = entries_meta([parts[r][i][1] - parts[r][i][0] for r in live], [slot[r] for r in live])
            fade, drive = kernels.recurrence_gates(u, dev["ra"], dev["ra.b"].reshape(-1), dev["ri"], dev["ri.b"].reshape(-1), dev["lam"], 8.0)
            o = kernels.linear_scan(fade, drive, y[:, :width], start, slots, state, activation="gelu_tanh").cpu()
            at = 0
            for r in live:
                n = parts[r][i][1] - parts[r][i][0]
                out[r].append(o[at:at + n])
                at += n
        return {r: torch.cat(v) for r, v in out.items()}
    whole = run({0: [(0, total)], 1: [(0, total - 6)]})
    cut = run({0: cuts(total, (1, 2, 17, 1, 1, 5)), 1: cuts(total - 6, (4, 1, 1, 20))})
    for r in seqs:
        assert torch.allclose(whole[r].double(), want[r], atol=1e-5), (r, (whole[r].double() - want[r]).abs().max())
        assert torch.equal(whole[r], cut[r])


def test_a_slow_channel_keeps_its_distance_from_one():
    """A channel whose decay differs from one by 4e-6 a step, driven for 4,000 steps, against float64: the relative error stays
    below 5e-6 (with the decay itself rounded to float32, whose neighbours near one lie 6e-8 apart, it would be 1.4e-5)."""
    from damendaemon_b200 import kernels
    T = 4000
    u = 0.5 + torch.rand(T, 1, generator=gen(0))
    zero = torch.zeros(1, 1, 1)
    lam = torch.tensor([math.log(math.expm1(1e-6))])              # softplus(lam) = 1e-6; r = 1/2: log a = -4e-6
    a = math.exp(-4e-6)
    S, want = 0.0, []
    for _ in range(T):
        S = a * S + math.sqrt(1 - a * a) * 0.5 * float(u[len(want), 0])
        want.append(S)
    fade, drive = kernels.recurrence_gates(u.to(DEV), zero.to(DEV), torch.zeros(1, device=DEV), zero.to(DEV), torch.zeros(1, device=DEV),
                                           lam.to(DEV), 8.0)
    state = torch.zeros(1, 1, device=DEV)
    _, start, slots = entries_meta([T], [0])
    got = kernels.linear_scan(fade, drive, torch.ones(T, 1, device=DEV), start, slots, state).cpu().double().reshape(-1)
    assert torch.allclose(got, torch.tensor(want, dtype=torch.float64), rtol=5e-6, atol=0)


def _paged(seq_k, seq_v, page_size, order_seed):
    """Keys and values of one sequence written into shuffled pages by the framework's own cache write."""
    from damendaemon_b200 import kernels
    T, G, dk = seq_k.shape
    dv = seq_v.shape[2]
    n_pages = -(-T // page_size) + 3
    pages = torch.randperm(n_pages, generator=gen(order_seed))[:-(-T // page_size)].to(torch.int32)
    table = torch.full((1, n_pages), -1, dtype=torch.int32)
    table[0, :pages.numel()] = pages
    shape = (n_pages, 2, G, page_size, dk) if dk == dv else (n_pages, G * page_size * (dk + dv))
    cache = torch.full(shape, float("nan"), dtype=seq_k.dtype, device=DEV)
    buffer = torch.cat([seq_k.reshape(T, -1), seq_v.reshape(T, -1)], dim=1).to(DEV)
    k, v = buffer[:, :G * dk], buffer[:, G * dk:]
    ent = torch.zeros(T, dtype=torch.int32, device=DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    extra = {} if dk == dv else dict(kv_heads=G, head_dim=dk, v_dim=dv)
    kernels.kv_store(k, v, ent, pos, table.to(DEV), cache, **extra)
    return cache, table.to(DEV), extra


@pytest.mark.parametrize("dk, dv, window", [(16, 8, 20), (96, 40, 72), (64, 64, 33), (24, 24, None)])
def test_a_marked_key_at_every_edge_of_the_window_with_the_unit_term(dk, dv, window):
    """One key's score stands out (its key and the queries are scaled along one direction): queries for which that key is the
    window's oldest key, the first one outside, the query's own place, a page border, and far away, in a prompt and alone,
    against the plain attention with one added to the denominator."""
    from damendaemon_b200 import kernels
    H, G, T, page = 4, 2, 700, 16
    q, k, v = randn(T, H, dk, seed=1) * 0.3, randn(T, G, dk, seed=2) * 0.3, randn(T, G, dv, seed=3)
    marked = 311
    k[marked, :, 0] = 10.0
    q[:, :, 0] = 5.0
    v[marked] = 9.0
    see = plain.visible(T, window)
    want = plain.attend(q.double(), k.double(), v.double(), 0.2, see, True)
    edge = marked + (window or 300)
    rows = sorted({marked - 1, marked, marked + 1, marked + 15, marked + 16, marked + 17, edge - 2, edge - 1, edge, edge + 1, T - 1})
    cache, table, extra = _paged(k, v, page, 5)
    sink = torch.zeros(H, device=DEV)
    common = dict(n_heads=H, scale=0.2, window=window, sink=sink, **({} if dk == dv else dict(kv_heads=G, v_dim=dv)))
    # a portion of the prompt: all rows at once
    qd = q.reshape(T, -1).to(DEV)
    ent, pos = torch.zeros(len(rows), dtype=torch.int32, device=DEV), torch.tensor(rows, dtype=torch.int32, device=DEV)
    got = kernels.attention_rows(qd[rows], cache, ent, pos, table, **common).cpu().double()
    assert torch.allclose(got, want[rows], atol=2e-4), (got - want[rows]).abs().max()
    seen = (want[rows].reshape(len(rows), H, dv)[:, 0, 0] > 4.0).tolist()
    inside = [marked <= r and (window is None or r - marked < window) for r in rows]
    assert seen == inside                        # the marked key decides the output exactly where the mask lets it through
    # single tokens, with the keys cut into splits
    for r in rows:
        one = kernels.attention_rows(qd[r:r + 1], cache, ent[:1], pos.new_tensor([r]), table, n_splits=3, **common).cpu().double()
        assert torch.allclose(one, want[r:r + 1], atol=2e-4), r


@pytest.mark.parametrize("G, window, sink_value", [(4, 100, 0.0), (2, None, 0.0), (4, 33, 1.5), (1, 300, -2.0)])
def test_the_tcgen05_prompt_kernel_with_a_term_in_the_denominator(G, window, sink_value):
    """Heads of 64 in bfloat16: a portion that starts in the middle of a prompt (and of a key block), through the tcgen05
    prompt kernel with a sink, against the plain attention with that term in the denominator (one for a sink of 0); queries
    whose window holds one key only lose most of their weight to the term."""
    from damendaemon_b200 import kernels
    H, d, T, page = 4, 64, 333, 16
    if not kernels.attention_prefill_tcgen05_supported(H, G, d, page, torch.bfloat16):
        pytest.skip("sizes the tcgen05 prompt kernel does not take")
    r = lambda t: t.bfloat16().double()
    q, k, v = randn(T, H, d, seed=1) * 0.4, randn(T, G, d, seed=2) * 0.4, randn(T, G, d, seed=3)
    see = plain.visible(T, window)
    # the plain attention's unit term is exp(0); a sink s is the same as scores shifted by -s with a unit term: by hand
    scores = torch.einsum("thd,shd->hts", r(q), r(k)[:, torch.arange(H) // (H // G)]) * 0.125
    scores = scores.masked_fill(~see[None], float("-inf"))
    e = torch.exp(scores)
    weights = e / (e.sum(-1, keepdim=True) + math.exp(sink_value))
    want = torch.einsum("hts,shd->thd", weights, r(v)[:, torch.arange(H) // (H // G)]).reshape(T, -1)
    if sink_value == 0.0:
        assert torch.allclose(want, plain.attend(r(q), r(k), r(v), 0.125, see, True), atol=1e-12)
    cache, table, _ = _paged(k.bfloat16(), v.bfloat16(), page, 7)
    sink = torch.full((H,), sink_value, device=DEV)
    first = 77
    start = torch.tensor([0, T - first], dtype=torch.int32, device=DEV)
    pos0 = torch.tensor([first], dtype=torch.int32, device=DEV)
    qd = q[first:].reshape(T - first, -1).bfloat16().to(DEV)
    got = kernels.attention_prefill(qd, cache, start, pos0, table, H, 0.125, window, kernel="tcgen05", sink=sink).cpu().double()
    assert kernels.read_error_flag(DEV) == 0
    assert (got - want[first:]).abs().max() < 0.03
    general = kernels.attention_rows(qd, cache, torch.zeros(T - first, dtype=torch.int32, device=DEV),
                                     torch.arange(first, T, dtype=torch.int32, device=DEV), table, H, 0.125, window, sink=sink).cpu().double()
    assert (got - general).abs().max() < 0.03
    if (window or T) < 50 or sink_value > 1.0:
        # without the term the rows differ where it is a good part of the denominator: it is not idle
        bare = kernels.attention_prefill(qd, cache, start, pos0, table, H, 0.125, window, kernel="tcgen05").cpu().double()
        assert (bare - got).abs().max() > 0.05
