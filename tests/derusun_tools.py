"""Small Derusun configurations and random models for the tests; nothing here touches the disk unless asked."""
import copy

import torch

from damendaemon_b200.registry import architecture_of


def delta(heads, kv_heads, dim, vdim, conv, decay_rank=8, gate_rank=8):
    return "channel_delta", {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
                             "decay_rank": decay_rank, "gate_rank": gate_rank}


def latent(heads, dim, rot_dim, vdim, rank, rot_dims=None, base=10000.0, scale=None):
    return "latent_attention", {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
                                "scale": scale if scale is not None else (dim + rot_dim) ** -0.5,
                                "rot": {"dims": rot_dims if rot_dims is not None else rot_dim, "base": base}}


def attention(heads, kv_heads, dim, vdim, mask=None, keep_first=0, softcap=None, v_mix=False, scale=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if mask is not None:
        out["mask"] = {"size": mask, "keep_first": keep_first}
    if softcap is not None:
        out["softcap"] = softcap
    if v_mix:
        out["v_mix"] = True
    return "attention", out


def dense(ff, limit=2.0):
    return {"kind": "dense", "ff": ff, "limit": limit}


def layer(mixer, mlp):
    return {"type": mixer[0], "mixer": copy.deepcopy(mixer[1]), "mlp": copy.deepcopy(mlp)}


def model(vocab, width, layers, groups=2, eps=1e-5):
    return {"architecture": "Derusun", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups}, "layers": layers}


# P: every mixer twice. Four delta heads on two query/key heads, value heads larger than key heads, three taps; a latent of
# 40 with a rotated part of 8; a window of 24 (no multiple of a page) that keeps 5 first keys, capped scores, values blended
# over three layers (the first of them only leaves its values); a last attention layer without mask, cap or blending
_PD = delta(4, 2, 16, 24, 3)
_PA = attention(4, 2, 16, 16, mask=24, keep_first=5, softcap=8.0, v_mix=True)
TINY_P = model(211, 64, [layer(_PD, None), layer(latent(3, 16, 8, 20, 40, base=500.0), dense(96)), layer(_PA, dense(80, limit=1.5)),
                         layer(_PA, None), layer(attention(2, 2, 32, 16, mask=24, keep_first=5, v_mix=True), dense(64)),
                         layer(_PD, dense(72)), layer(latent(2, 24, 16, 12, 32, rot_dims=8, base=77.0), None),
                         layer(attention(4, 4, 16, 8), dense(48, limit=0.7))], groups=4)
# Q: one group in the norm (an ordinary RMS norm), one tap (no convolution state), sizes that are no multiples of 8: delta
# heads of 20 by 12, every head its own keys; a window of 7 (smaller than a page) that keeps more first keys (9) than it is
# wide; a layer that only leaves its values and no layer that blends; an attention layer first, a delta layer last
_QA = attention(3, 3, 12, 20, mask=7, keep_first=9, v_mix=True)
TINY_Q = model(97, 48, [layer(_QA, dense(40, limit=3.0)), layer(delta(3, 3, 20, 12, 1, decay_rank=5, gate_rank=11), None),
                        layer(latent(3, 8, 4, 8, 24, base=30.0), dense(56)), layer(attention(1, 1, 16, 16, mask=16, softcap=5.0), None),
                        layer(delta(1, 1, 40, 36, 2, decay_rank=16, gate_rank=4), dense(40))], groups=1, eps=1e-6)
# R: heads of 64 (what the tensor-core attention kernels would take, were it not for the sink), a width of 256 in eight
# groups, a window of 100 that keeps 33 (neither a multiple of a page), delta heads of 64 with five taps, a latent of 128 + 32
_RA = attention(4, 2, 64, 64, mask=100, keep_first=33, softcap=20.0, v_mix=True)
TINY_R = model(300, 256, [layer(_RA, dense(512, limit=1.0)), layer(delta(4, 4, 64, 64, 5, decay_rank=32, gate_rank=16), dense(256)),
                          layer(latent(4, 64, 32, 64, 128), dense(256)), layer(_RA, None)], groups=8)
# S: awkward sizes: a width of 100 in five groups, a vocabulary of 131, three query heads on one key/value head with keys of
# 20 and values of 12, a window of 33 without kept keys, six delta heads on two key heads (dim 24, vdim 10), four taps,
# a latent of 36 + 12 of which 6 dimensions turn
_SA = attention(3, 1, 20, 12, mask=33, softcap=50.0, v_mix=True)
TINY_S = model(131, 100, [layer(latent(5, 12, 12, 20, 36, rot_dims=6, base=50.0), dense(52)), layer(_SA, dense(30)),
                          layer(delta(6, 2, 24, 10, 4, decay_rank=12, gate_rank=20), None), layer(_SA, dense(52, limit=5.0))], groups=5)
# T: large heads: delta keys of 128 and 256, values of 64 and 40; attention heads of 128 on one key/value head with a
# window of 70 keeping 70; a latent of 192 + 64; one layer each
TINY_T = model(150, 192, [layer(delta(2, 1, 128, 64, 4, decay_rank=24, gate_rank=24), dense(200)),
                          layer(attention(4, 1, 128, 128, mask=70, keep_first=70, softcap=30.0), None),
                          layer(latent(3, 48, 64, 80, 192, base=300.0), dense(128)),
                          layer(delta(1, 1, 256, 40, 2, decay_rank=8, gate_rank=8), None)], groups=3)

CONFIGS = {"P": TINY_P, "Q": TINY_Q, "R": TINY_R, "S": TINY_S, "T": TINY_T}


def make_tensors(config, seed, sharpen=3.0, dtype=torch.float32):
    """Random weights with the query heads' norm weights and the latent layers' query matrices scaled up, so that
    attention is peaky and a key that is wrongly seen or missed moves the logits; matrices rounded to ``dtype`` (the
    values a bfloat16 folder would hold)."""
    arch = architecture_of(config)
    tensors = arch.random_tensors(arch.parse_config(config), seed, torch.float32)
    for i, l in enumerate(config["layers"]):
        if l["type"] == "attention":
            tensors[f"l{i}.mix.q.norm"] = tensors[f"l{i}.mix.q.norm"] * sharpen
        elif l["type"] == "latent_attention":
            tensors[f"l{i}.mix.q"] = tensors[f"l{i}.mix.q"] * sharpen
    for name in tensors:
        if tensors[name].dim() == 2 and tensors[name].is_floating_point() and not name.endswith(".conv"):
            tensors[name] = tensors[name].to(dtype).to(torch.float32)
    return tensors


def plain_tensors(tensors):
    return {k: (v.double() if v.is_floating_point() else v.long()) for k, v in tensors.items()}


def plain_config(config):
    """The configuration as config.json would hold it: without the ranks that only the tensors' shapes give."""
    out = copy.deepcopy(config)
    for l in out["layers"]:
        l["mixer"].pop("decay_rank", None)
        l["mixer"].pop("gate_rank", None)
    return out


def random_requests(config, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, config["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}
