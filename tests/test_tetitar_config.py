"""Tetitar's configuration, its description in parts, and the plain implementation's own pieces (CPU)."""
import copy
import math

import pytest
import torch

import plain_tetitar as plain
from tetitar_tools import CONFIGS, TINY_A, TINY_B, TINY_C, TINY_D, make_tensors, plain_tensors

from damendaemon_b200.config.reader import ConfigError
from damendaemon_b200.parts import cache_needs, tensor_decls
from damendaemon_b200.parts.positions import rotary_frequencies
from damendaemon_b200.registry import architecture_of


def spec_of(config):
    arch = architecture_of(config)
    typed = arch.parse_config(config)
    return arch, typed, arch.build_spec(typed)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_a_configuration_round_trips_and_names_its_tensors(name):
    config = CONFIGS[name]
    arch, typed, spec = spec_of(config)
    assert typed.to_dict() == config
    assert arch.parse_config(typed.to_dict()) == typed
    wanted = set()
    for d in tensor_decls(spec):
        wanted |= {n for n, _ in d.pieces} if d.pieces else {d.name}
    tensors = arch.random_tensors(typed, 1)
    assert wanted == set(tensors)
    for d in tensor_decls(spec):
        for n, shape in (d.pieces or ((d.name, d.shape),)):
            assert tuple(tensors[n].shape) == tuple(shape), n


def test_the_run_order_repeats_the_loop_with_a_cache_for_every_pass():
    _, _, spec = spec_of(TINY_A)
    assert [(e.layer, e.add_embedding, e.add_vector) for e in spec.run_order] == \
        [(0, False, 0), (1, False, None), (0, True, 1), (1, False, None), (0, True, 2), (1, False, None), (2, False, None)]
    needs = cache_needs(spec)
    assert len(needs) == len(spec.run_order) + 1 and needs[-1][0].name == "last_id"      # the embedding's own site
    assert needs[1][0].window == 20 and needs[1][0].value_dim == 12 and [n.name for n in needs[1][1:]] == ["", "conv"]
    _, _, once = spec_of(TINY_C)
    assert [(e.layer, e.add_embedding, e.add_vector) for e in once.run_order] == \
        [(0, False, None), (1, False, 0), (2, False, None), (3, False, None)]
    _, _, plain_order = spec_of(TINY_B)
    assert [e.layer for e in plain_order.run_order] == [0, 1, 2, 3] and plain_order.pass_vectors is None
    assert plain.run_order(TINY_A) == [(0, 0, True), (1, 0, False), (0, 1, True), (1, 1, False), (0, 2, True), (1, 2, False), (2, None, False)]
    # one tap: no convolution state; no table of pairs: no site for the embedding
    assert [n.name for n in cache_needs(plain_order)[2]] == [""]
    assert len(cache_needs(spec_of(TINY_D)[2])) == len(spec_of(TINY_D)[2].run_order)


@pytest.mark.parametrize("change, message", [
    (lambda c: c.update(architecture="Other"), "architecture"),
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "share"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=8), "keys' size"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(groups=3), "groups"),
    (lambda c: c["layers"][2]["mixer"].update(blocks=5), "equal parts"),
    (lambda c: c["loop"].update(stop=9), "run of the model"),
    (lambda c: c["layers"][2]["mlp"].update(kind="experts"), "dense"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_bad_fields_are_refused(change, message):
    config = copy.deepcopy(TINY_A)
    change(config)
    with pytest.raises(ConfigError, match=message):
        architecture_of(config).parse_config(config)


def test_stretched_frequencies_equal_the_plain_ones():
    for config in CONFIGS.values():
        _, _, spec = spec_of(config)
        for layer, raw in zip(spec.layers, config["layers"]):
            mixer, m = (layer.mixer, raw["mixer"]) if raw["type"] == "attention" else \
                ((layer.mixer.left, raw["mixer"]["left"]) if raw["type"] == "parallel" else (None, None))
            if mixer is None:
                continue
            f, magnitude = rotary_frequencies(mixer.rotary)
            assert magnitude == 1.0 and torch.allclose(f, plain.frequencies(m["rot"]), rtol=1e-14, atol=0)
    # the three stretches of the rule, by hand: base 100 over 8 dimensions gives wavelengths 2 pi * (1, 3.16, 10, 31.6)
    f = plain.frequencies({"dims": 8, "base": 100.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}})
    plain_f = 100.0 ** (-torch.arange(4, dtype=torch.float64) / 4)
    assert f[0] == plain_f[0] and f[3] == plain_f[3] / 4 and plain_f[2] / 4 < f[2] < plain_f[2]
    s = (64 / (2 * math.pi / plain_f[1]) - 1.0) / 3.0
    assert torch.isclose(f[1], (1 - s) * plain_f[1] / 4 + s * plain_f[1])


def test_pair_rows_by_hand():
    m = {"buckets": 13, "mul_prev": 5, "mul_cur": 3}
    assert plain.pair_rows([4, 7, 7, 0], m).tolist() == [13, (4 * 5 + 7 * 3) % 13, (7 * 5 + 7 * 3) % 13, (7 * 5) % 13]
    big = TINY_B["embedding"]["bigram"]
    assert plain.pair_rows([96, 95], big).tolist() == [big["buckets"], (96 * big["mul_prev"] + 95 * big["mul_cur"]) % big["buckets"]]


def test_the_plain_recurrences_equal_their_explicit_sums():
    torch.manual_seed(0)
    config = TINY_D
    w = plain_tensors(make_tensors(config, 3))
    h = torch.randn(9, 100, dtype=torch.float64)
    # gated linear recurrence: S_t = sum_k (prod_{j>k} a_j) drive_k
    m, p = config["layers"][1]["mixer"], "l1.mix."
    out = plain.gated_recurrence(h, w, p, m, 1e-5)
    y = plain.gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    u = plain.causal_convolution(h @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    ub = u.reshape(9, 5, 12)
    r = torch.sigmoid(torch.einsum("boi,tbi->tbo", w[p + "ra"], ub) + w[p + "ra.b"]).reshape(9, 60)
    i = torch.sigmoid(torch.einsum("boi,tbi->tbo", w[p + "ri"], ub) + w[p + "ri.b"]).reshape(9, 60)
    a = torch.exp(-8.0 * r * torch.nn.functional.softplus(w[p + "lam"]))
    S = sum(torch.prod(a[k + 1:9], dim=0) * torch.sqrt(1 - a[k] ** 2) * i[k] * u[k] for k in range(9))
    assert torch.allclose(out[8], (S * y[8]) @ w[p + "o"].T, rtol=1e-10, atol=1e-12)
    # the convolution's first outputs see zeros before the start
    x = torch.randn(5, 3, dtype=torch.float64)
    taps, bias = torch.randn(3, 4, dtype=torch.float64), torch.randn(3, dtype=torch.float64)
    c = plain.causal_convolution(x, taps, bias)
    assert torch.allclose(c[0], bias + taps[:, 3] * x[0]) and torch.allclose(c[1], bias + taps[:, 3] * x[1] + taps[:, 2] * x[0])


def test_every_mechanism_moves_the_logits():
    """Leaving a mechanism out of the plain model changes its logits: none of them is idle in the test configurations."""
    config = TINY_A
    w = plain_tensors(make_tensors(config, 5))
    ids = torch.randint(0, config["vocab"], (40,), generator=torch.Generator().manual_seed(1)).tolist()
    base = plain.forward(config, w, ids)

    def moved(new_config=None, **new_w):
        out = plain.forward(new_config or config, {**w, **new_w}, ids)
        return (out - base).abs().max().item()
    assert moved(bigram=torch.zeros_like(w["bigram"])) > 1e-3
    assert moved(**{"loop.step": torch.zeros_like(w["loop.step"])}) > 1e-3
    no_cap = copy.deepcopy(config); no_cap.pop("logit_softcap")
    assert moved(no_cap) > 1e-4
    one_pass = copy.deepcopy(config); one_pass["loop"]["times"] = 2
    assert moved(one_pass) > 1e-3
    no_window = copy.deepcopy(config); no_window["layers"][1]["mixer"]["left"].pop("mask")
    assert moved(no_window) > 1e-4
    no_stretch = copy.deepcopy(config); no_stretch["layers"][0]["mixer"]["rot"].pop("scaling")
    assert moved(no_stretch) > 1e-4
    assert moved(**{"l0.mix.g": torch.zeros_like(w["l0.mix.g"])}) > 1e-3
    assert moved(**{"l1.mix.right.D": torch.zeros_like(w["l1.mix.right.D"])}) > 1e-5
    assert moved(**{"l2.mix.lam": w["l2.mix.lam"] + 1.0}) > 1e-4
    # the unit term: without it a lone first key would get all the weight
    q = torch.randn(1, 1, 4, dtype=torch.float64)
    o = plain.attend(q, q, torch.ones(1, 1, 2, dtype=torch.float64), 1.0, plain.visible(1), True)
    s = float((q * q).sum())
    assert torch.allclose(o, torch.full((1, 2), math.exp(s) / (1 + math.exp(s)), dtype=torch.float64))
