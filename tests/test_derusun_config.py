"""Derusun on the CPU: configuration, the spec it becomes, tensor names, what the cache keeps, and the plain
implementation's own pieces (which the GPU tests then trust)."""
import copy

import pytest
import torch

import plain_derusun as plain
from derusun_tools import CONFIGS, TINY_P, TINY_Q, TINY_R, make_tensors, plain_config, plain_tensors

from damendaemon_b200.cache import CacheManager
from damendaemon_b200.config import ConfigError
from damendaemon_b200.parts import cache_needs, tensor_decls
from damendaemon_b200.registry import architecture_of


def spec_of(config):
    arch = architecture_of(config)
    return arch, arch.parse_config(config), arch.build_spec(arch.parse_config(config))


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_configuration_round_trip_and_tensor_names(name):
    config = CONFIGS[name]
    arch, typed, spec = spec_of(config)
    assert arch.name == "Derusun"
    assert arch.parse_config(typed.to_dict()) == typed
    random = arch.random_tensors(typed, 0)
    declared, shapes = set(), {}
    for d in tensor_decls(spec):
        declared |= {n for n, _ in d.pieces} if d.pieces else {d.name}
        shapes.update({n: tuple(s) for n, s in d.pieces} if d.pieces else {d.name: tuple(d.shape)})
    # the first blending layer's weight is in the checkpoint but nothing reads it
    unread = {n for n in random if any(__import__("re").fullmatch(p, n) for p in spec.ignored_tensors)}
    assert declared == set(random) - unread and len(unread) <= 1
    for n, t in random.items():
        if n not in unread:
            assert tuple(t.shape) == shapes[n], n


def test_the_ranks_come_from_the_tensors_shapes():
    arch = architecture_of(TINY_Q)
    bare = arch.parse_config(plain_config(TINY_Q))
    assert bare.layers[1].mixer.decay_rank is None
    with pytest.raises(ValueError):
        arch.build_spec(bare)
    shapes = {n: tuple(t.shape) for n, t in arch.random_tensors(arch.parse_config(TINY_Q), 0).items()}
    filled = arch.sizes_from_shapes(bare, shapes)
    assert filled == arch.parse_config(TINY_Q)
    assert (filled.layers[1].mixer.decay_rank, filled.layers[1].mixer.gate_rank) == (5, 11)
    with pytest.raises(ConfigError):
        arch.sizes_from_shapes(bare, {})
    wrong = dict(shapes)
    wrong["l1.mix.a1"] = (6, 48)
    with pytest.raises(ConfigError):
        arch.sizes_from_shapes(arch.parse_config(TINY_Q), wrong)


def test_the_constants_of_the_design_reach_the_specs():
    _, typed, spec = spec_of(TINY_P)
    assert spec.depth_mix == tuple(f"l{i}.dwa" for i in range(8)) and spec.max_positions is None
    assert all(l.arrangement == "pre_norm_shift" and l.shift_weight == f"l{i}.shift" for i, l in enumerate(spec.layers))
    assert [len(l.norms) for l in spec.layers] == [1, 2, 2, 1, 2, 2, 1, 2] and spec.layers[0].norms[0].groups == 4
    assert spec.head.norm.groups == 4
    d, la, a = spec.layers[0].mixer, spec.layers[1].mixer, spec.layers[2].mixer
    assert (d.kind, d.n_heads, d.n_kv_heads, d.head_dim, d.value_dim, d.conv_taps) == ("gated_delta", 4, 2, 16, 24, 3)
    assert (la.kind, la.rank, la.rot_dim, la.rotary.dims, la.rotary.interleaved, la.sink) == ("latent_attention", 40, 8, 8, True, "l1.mix.sink")
    assert (a.window, a.keep_first, a.softcap, a.sink, a.value_dim) == (24, 5, 8.0, "l2.mix.sink", 16)
    assert a.qkv_bias == ("l2.mix.q.b", "l2.mix.k.b", "l2.mix.v.b") and a.rotary is None and a.head_norm_eps == 1e-5
    # values: the first blending layer leaves them, the later ones blend, a layer that does not blend does neither
    roles = [(l.mixer.value_mix_source, l.mixer.value_mix) for l in spec.layers if l.mixer.kind == "attention"]
    assert roles == [(True, None), (False, "l3.mix.vmix"), (False, "l4.mix.vmix"), (False, None)]
    f = spec.layers[2].feed_forward
    assert (f.kind, f.unit.activation, f.unit.limit, f.unit.alpha, f.unit.inner) == ("gated", "clamped_swish", 1.5, 1.702, 80)
    last = spec.layers[7].mixer
    assert last.window is None and last.keep_first == 0 and last.softcap is None


def test_what_the_cache_keeps():
    _, _, spec = spec_of(TINY_R)
    needs = cache_needs(spec)
    kv = needs[0][0]
    assert (kv.kv_heads, kv.head_dim, kv.window, kv.keep_first) == (2, 64, 100, 33)
    assert [n.name for n in needs[0][1:]] == ["shift"] and needs[0][1].shape == (256,)
    state, conv, shift = needs[1]
    assert state.name == "" and state.shape == (4, 64, 64) and (conv.name, conv.shape) == ("conv", (4, 3 * 4 * 64)) and shift.name == "shift"
    assert type(needs[2][0]).__name__ == "PagedRows" and needs[2][0].width == 160 and needs[2][0].window is None
    # one tap: no convolution state
    assert [n.name for n in cache_needs(spec_of(TINY_Q)[2])[1]] == ["", "shift"]
    # the window's pages come back, the kept first keys' pages never do
    manager = CacheManager([[kv]], kv_tokens=400, page_size=8, max_requests=2, max_context=400)
    manager.admit("a")
    for length in (40, 170, 300):
        manager.extend([("a", length)])
        manager.advance("a", length)
    table = manager.groups[0].tables["a"]
    first_needed = (300 - 100 + 1) // 8
    assert all(p >= 0 for p in table[:5]) and all(p < 0 for p in table[5:first_needed]) and all(p >= 0 for p in table[first_needed:])
    manager.check()
    manager.release("a")
    assert manager.used_tokens == 0


def test_bad_fields_are_named():
    for path, value in ((("norm", "groups"), 5), (("layers", 0, "type"), "conv"), (("layers", 2, "mixer", "mask", "keep_first"), -1),
                        (("layers", 1, "mixer", "rot", "dims"), 7), (("layers", 1, "mixer", "rot", "dims"), 64),
                        (("layers", 0, "mixer", "kv_heads"), 3), (("layers", 1, "mlp", "kind"), "moe"), (("layers", 2, "mixer", "v_mix"), 1)):
        config = copy.deepcopy(TINY_P)
        at = config
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(ConfigError):
            architecture_of(config).parse_config(config)
    config = copy.deepcopy(TINY_P)
    del config["layers"][1]["mlp"]["limit"]
    with pytest.raises(ConfigError):
        architecture_of(config).parse_config(config)


# ------------------------------------------------------------------ the plain implementation's own pieces

def test_the_plain_delta_rule_against_its_closed_form_and_in_portions():
    """With beta = 1, no decay and orthonormal keys the rule stores each value under its key exactly; and a sequence run in
    two portions from the carried state equals the whole."""
    torch.manual_seed(0)
    T, H, dk, dv = 6, 2, 8, 5
    keys = torch.linalg.qr(torch.randn(H, dk, dk, dtype=torch.float64))[0][:, :T].transpose(0, 1)      # [T, H, dk]
    v = torch.randn(T, H, dv, dtype=torch.float64)
    ones = torch.ones(T, H, dtype=torch.float64)
    o, S = plain.delta_rule(keys, keys, v, ones, torch.ones(T, H, dk, dtype=torch.float64))
    assert (o - v).abs().max() < 1e-12                                 # a token reads its own write
    for t in range(T):
        assert (torch.einsum("hkv,hk->hv", S, keys[t]) - v[t]).abs().max() < 1e-12
    q, k = torch.randn(9, H, dk, dtype=torch.float64), torch.randn(9, H, dk, dtype=torch.float64)
    vv, beta, decay = torch.randn(9, H, dv, dtype=torch.float64), torch.rand(9, H, dtype=torch.float64), torch.rand(9, H, dk, dtype=torch.float64)
    whole, last = plain.delta_rule(q, k, vv, beta, decay)
    a, mid = plain.delta_rule(q[:4], k[:4], vv[:4], beta[:4], decay[:4])
    b, end = plain.delta_rule(q[4:], k[4:], vv[4:], beta[4:], decay[4:], state=mid)
    assert (torch.cat([a, b]) - whole).abs().max() < 1e-12 and (end - last).abs().max() < 1e-12


def test_the_plain_pieces():
    x = torch.arange(12, dtype=torch.float64).reshape(2, 6) + 1
    n = plain.grouped_norm(x, torch.ones(6, dtype=torch.float64), 0.0, 3)
    assert torch.allclose((n.reshape(2, 3, 2) ** 2).mean(-1), torch.ones(2, 3, dtype=torch.float64))
    h = torch.randn(5, 4, dtype=torch.float64)
    mu = torch.tensor([0.0, 1.0, 0.5, 0.25], dtype=torch.float64)
    s = plain.token_shift(h, mu)
    assert torch.equal(s[:, 0], h[:, 0]) and torch.allclose(s[1:, 1], h[:-1, 1]) and abs(s[0, 1]) < 1e-15
    again = torch.cat([plain.token_shift(h[:2], mu), plain.token_shift(h[2:], mu, before=h[1])])
    assert torch.allclose(again, s)
    taps = torch.randn(4, 3, dtype=torch.float64)
    y = plain.short_convolution(h, taps)
    assert torch.allclose(y[2], taps[:, 0] * h[0] + taps[:, 1] * h[1] + taps[:, 2] * h[2]) and torch.allclose(y[0], taps[:, 2] * h[0])
    cut = torch.cat([plain.short_convolution(h[:3], taps), plain.short_convolution(h[3:], taps, before=h[1:3])])
    assert torch.allclose(cut, y)
    see = plain.visible(12, 4, 2)
    assert see[9].tolist() == [True, True] + [False] * 4 + [True] * 4 + [False, False] and see[3].tolist() == [True] * 4 + [False] * 8
    w = plain.softmax_with_sink(torch.zeros(1, 3, 3, dtype=torch.float64), plain.visible(3), torch.zeros(1, dtype=torch.float64))
    assert torch.allclose(w[0, 2], torch.full((3,), 0.25, dtype=torch.float64)) and torch.allclose(w[0, 0, 0], torch.tensor(0.5, dtype=torch.float64))
    p = torch.randn(4, 1, 6, dtype=torch.float64)
    r = plain.rotate_neighbours(p, torch.arange(4), 4, 10.0)
    assert torch.equal(r[..., 4:], p[..., 4:]) and torch.equal(r[0], p[0])
    assert torch.allclose(r[..., :4].norm(dim=-1), p[..., :4].norm(dim=-1))


@pytest.mark.parametrize("name", ["P", "Q"])
def test_every_mechanism_moves_the_logits_when_it_is_left_out(name):
    """So that a test which compares logits notices each of them."""
    config = CONFIGS[name]
    tensors = plain_tensors(make_tensors(config, 2))
    ids = torch.randint(0, config["vocab"], (60,), generator=torch.Generator().manual_seed(1)).tolist()
    base = plain.forward(config, tensors, ids)

    def moved(change_config=None, change_tensors=None):
        c, t = copy.deepcopy(config), dict(tensors)
        if change_config:
            change_config(c)
        if change_tensors:
            change_tensors(t)
        return (plain.forward(c, t, ids) - base)[40:].abs().max().item()

    attention = [i for i, l in enumerate(config["layers"]) if l["type"] == "attention" and "mask" in l["mixer"]]
    i = attention[0]
    assert moved(lambda c: c["norm"].update(groups=1 if c["norm"]["groups"] > 1 else 2)) > 1e-3
    assert moved(None, lambda t: t.update({f"l{i}.shift": torch.zeros_like(t[f"l{i}.shift"])})) > 1e-3
    assert moved(lambda c: c["layers"][i]["mixer"]["mask"].update(keep_first=0)) > 1e-4
    assert moved(lambda c: c["layers"][i]["mixer"]["mask"].update(size=c["layers"][i]["mixer"]["mask"]["size"] + 1)) > 1e-4
    assert moved(None, lambda t: t.update({f"l{i}.mix.sink": t[f"l{i}.mix.sink"] - 30.0})) > 1e-3
    assert moved(None, lambda t: t.update({"l0.dwa": torch.tensor([0.0, 1.0], dtype=torch.float64)})) > 1e-3
    capped = [j for j in attention if "softcap" in config["layers"][j]["mixer"]]
    if capped:
        assert moved(lambda c: c["layers"][capped[0]]["mixer"].pop("softcap")) > 1e-5
    blending = [j for j in attention if config["layers"][j]["mixer"].get("v_mix")]
    if len(blending) > 1:
        assert moved(None, lambda t: t.update({f"l{blending[1]}.mix.vmix": torch.zeros((), dtype=torch.float64)})) > 1e-4
    d = next(j for j, l in enumerate(config["layers"]) if l["type"] == "channel_delta")
    assert moved(None, lambda t: t.update({f"l{d}.mix.A_log": t[f"l{d}.mix.A_log"] + 2.0})) > 1e-4
    assert moved(None, lambda t: t.update({f"l{d}.mix.b": t[f"l{d}.mix.b"] * 0.0})) > 1e-4
    la = next(j for j, l in enumerate(config["layers"]) if l["type"] == "latent_attention")
    assert moved(lambda c: c["layers"][la]["mixer"]["rot"].update(base=c["layers"][la]["mixer"]["rot"]["base"] * 3)) > 1e-4
    assert moved(None, lambda t: t.update({f"l{la}.mix.sink": t[f"l{la}.mix.sink"] - 30.0})) > 1e-4
