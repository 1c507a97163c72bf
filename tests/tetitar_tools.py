"""Small Tetitar configurations and random models for the tests; nothing here touches the disk unless asked."""
import copy

import torch

from damendaemon_b200.registry import architecture_of


def rot(dims, base=10000.0, scaling=None):
    out = {"dims": dims, "base": base}
    if scaling is not None:
        out["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return out


def attention(heads, kv_heads, dim, rotation, mask=None, scale=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale if scale is not None else dim ** -0.5,
           "rot": rotation}
    if mask is not None:
        out["mask"] = {"size": mask}
    return "attention", out


def parallel(heads, kv_heads, dim, vdim, rotation, mask, ss_heads, ss_vdim, state, groups, conv, norm_groups, scale=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5,
            "rot": rotation}
    if mask is not None:
        left["mask"] = {"size": mask}
    right = {"heads": ss_heads, "vdim": ss_vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}
    return "parallel", {"left": left, "right": right}


def rglru(width, blocks, conv):
    return "rglru", {"width": width, "blocks": blocks, "conv": conv}


def layer(mixer, ff):
    return {"type": mixer[0], "mixer": copy.deepcopy(mixer[1]), "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def model(vocab, width, layers, loop=None, pairs=(97, 7, 3), cap=None, eps=1e-5):
    out = {"architecture": "Tetitar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if pairs is not None:
        out["embedding"] = {"bigram": {"buckets": pairs[0], "mul_prev": pairs[1], "mul_cur": pairs[2]}}
    if loop is not None:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    if cap is not None:
        out["logit_softcap"] = cap
    return out


# A: the first two layers run three times; part of a head rotated with stretched frequencies (wavelengths on both sides of the
# blend and inside it); a window of 20 (no multiple of a page) on one key/value head with values smaller than keys; a state
# of 16 in one group, four taps; a recurrence in three parts with two taps; a layer without a feed-forward
TINY_A = model(211, 64, [layer(attention(4, 2, 16, rot(8, 100.0, (4.0, 1.0, 4.0, 64))), 96),
                         layer(parallel(2, 1, 24, 12, rot(24, 5000.0), 20, 2, 8, 16, 1, 4, 1), None),
                         layer(rglru(48, 3, 2), 80)], loop=(0, 2, 3), cap=12.0)
# B: no loop, no cap; every head its own keys, one head; windows smaller than a page (7) and on the full-attention mixer
# too (40); convolutions of one tap (no convolution state); a recurrence in one part; multipliers that overflow 32 bits
# when multiplied by a token id; a first layer that is the parallel one
TINY_B = model(97, 48, [layer(parallel(3, 3, 8, 16, rot(4, 30.0), 7, 1, 12, 8, 1, 1, 2), 40),
                        layer(attention(1, 1, 32, rot(32, 77.0), mask=40), None),
                        layer(rglru(40, 1, 1), 56),
                        layer(attention(2, 2, 8, rot(2, 10.0, (8.0, 0.5, 2.0, 32))), 40)], pairs=(1000003, 2000000011, 1999999973), eps=1e-6)
# C: heads of 64 (what the tensor-core attention kernels take, were it not for the unit term of the windowed one), a width
# of 256; the loop runs once (only its vector is added); a state of 128 and one of 24 (no power of two), as many groups as
# heads; a window of 100; a recurrence with parts of 128
TINY_C = model(300, 256, [layer(rglru(256, 2, 4), 256),
                          layer(attention(4, 4, 64, rot(64, 10000.0, (8.0, 1.0, 4.0, 512))), 512),
                          layer(parallel(4, 2, 64, 64, rot(16, 200000.0), 100, 4, 32, 128, 4, 3, 4), 256),
                          layer(parallel(2, 2, 64, 64, rot(64, 100.0), 33, 2, 64, 24, 1, 2, 1), None)], loop=(1, 3, 1), cap=30.0)
# D: awkward sizes: a width of 100, a vocabulary of 131, all layers in the loop, twice; three query heads on one key/value
# head with keys of 20 and values of 12, a window of 33; six state-space heads in three groups, values of 10, a state of 20,
# normed in three parts; a recurrence of 60 channels in five parts of 12, three taps; no table of pairs
TINY_D = model(131, 100, [layer(parallel(3, 1, 20, 12, rot(6, 50.0), 33, 6, 10, 20, 3, 3, 3), 52),
                          layer(rglru(60, 5, 3), None),
                          layer(attention(6, 2, 12, rot(12, 1000.0)), 30)], loop=(0, 3, 2), pairs=None)

# E: grouped heads at the sizes the tensor-core prompt kernels take: four query heads of 64 on two key/value heads whose
# values are the keys; four heads of 128 on one key/value head with a window of 50 and the unit term; only the first layer
# is repeated; a pair table of 31 buckets with both multipliers one
TINY_E = model(150, 128, [layer(attention(4, 2, 64, rot(32, 1000.0)), 128),
                          layer(parallel(4, 1, 128, 128, rot(64, 300.0), 50, 2, 16, 32, 2, 2, 1), 64)], loop=(0, 1, 2), pairs=(31, 1, 1))

CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}


def make_tensors(config, seed, sharpen=3.0, dtype=torch.float32):
    """Random weights with the queries' norm weights scaled up, so that attention is peaky and a key that is wrongly seen or
    missed moves the logits; matrices rounded to ``dtype`` (the values a bfloat16 folder would hold)."""
    arch = architecture_of(config)
    tensors = arch.random_tensors(arch.parse_config(config), seed, torch.float32)
    for name in tensors:
        if name.endswith("q.norm"):
            tensors[name] = tensors[name] * sharpen
        t = tensors[name]
        if t.dim() == 2 and t.is_floating_point() and not name.endswith((".conv", ".b", "loop.step")):
            tensors[name] = t.to(dtype).to(torch.float32)
    return tensors


def plain_tensors(tensors):
    return {k: (v.double() if v.is_floating_point() else v.long()) for k, v in tensors.items()}


def random_requests(config, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, config["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}
