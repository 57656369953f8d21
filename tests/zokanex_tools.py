"""Small Zokanex configurations and random models for the tests; nothing here touches the disk unless asked."""
import copy

import torch

from damendaemon_b200.registry import architecture_of


def attention(heads, kv_heads, dim, vdim, mask=None, rot_dims=None, base=10000.0, scale=None, kv_from=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if rot_dims is not None:
        out["rot"] = {"dims": rot_dims, "base": base}
    if mask is not None:
        out["mask"] = {"size": mask}
    if kv_from is not None:
        out["kv_from"] = kv_from
    return "attention", out


def retention(heads, dim, vdim, decay, rot_dims=None, base=10000.0):
    out = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot_dims is not None:
        out["rot"] = {"dims": rot_dims, "base": base}
    return "retention", out


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, groups=None, scale=1.0, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "router": router, "expert": {"ff": ff}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def layer(mixer, mlp):
    return {"type": mixer[0], "mixer": copy.deepcopy(mixer[1]), "mlp": copy.deepcopy(mlp)}


def model(vocab, width, layers, scale=None, eps=1e-6):
    return {"architecture": "Zokanex", "vocab": vocab, "width": width, "embedding": {"scale": scale or width ** 0.5},
            "norm": {"eps": eps}, "layers": layers}


# P: two key/value heads for four query heads, value heads smaller than key heads, half of a head rotated, a window of 24
# (no multiple of a page); the second layer reads the first one's keys through a WIDER window (40); experts in four
# groups of which two stay, two of eight a token, a shared one; retention with two heads, value heads larger than keys
_PA = attention(4, 2, 32, 16, mask=24, rot_dims=16, base=500.0)
_PR = retention(2, 16, 24, [0.9, 0.97], rot_dims=8, base=300.0)
_PE = moe(8, 2, 24, groups=(4, 2), scale=2.5, shared=40)
TINY_P = model(211, 64, [layer(_PA, dense(96)), layer(attention(4, 2, 32, 16, mask=40, rot_dims=16, base=500.0, kv_from=0), _PE),
                         layer(_PR, dense(80)), layer(_PR, _PE), layer(_PA, dense(96))])
# Q: retention first, a layer without a feed-forward, decays at both ends (1: nothing fades; 0: only the token itself)
# and no rotation; every head its own key/value head, value heads larger than key heads, whole heads rotated, a window of
# 7 (smaller than a page); one expert of five a token, no groups, no shared one; a layer that sees every key (no mask) and
# is not rotated, and one that reads its keys through a window of 9; an embedding scale that is not the root of the width
_QA = attention(3, 3, 16, 40, mask=7, rot_dims=16)
_QF = attention(3, 3, 16, 40)
TINY_Q = model(97, 48, [layer(retention(3, 8, 8, [1.0, 0.5, 0.0]), None), layer(_QA, moe(5, 1, 16, scale=0.7)),
                        layer(_QF, dense(72)), layer(attention(3, 3, 16, 40, mask=9, kv_from=2), None),
                        layer(retention(1, 32, 16, [0.95], rot_dims=32), dense(40))], scale=3.0, eps=1e-5)
# R: equal head sizes of 64 with a key/value head each (what every tensor-core attention kernel takes, decode
# included), a window of 100 (no multiple of a key block of 128 nor of a page), a reader with a narrower window, retention
# with heads of 64, three experts of three (every token uses all) in one group
_RA = attention(4, 4, 64, 64, mask=100, rot_dims=64)
TINY_R = model(300, 256, [layer(_RA, moe(3, 3, 32, groups=(1, 1), scale=1.0, shared=16)),
                          layer(attention(4, 4, 64, 64, mask=50, rot_dims=64, kv_from=0), dense(512)),
                          layer(retention(4, 64, 64, [0.99, 0.995, 0.999, 0.9], rot_dims=32), dense(256))])
# S: awkward sizes: a width (100), head sizes (20 and 12), an expert width (30) and a vocabulary (131) that are no
# multiples of 8, five rotated pairs, three heads on one key/value head, a window of 33; retention heads of 40 by 36 (no
# multiples of 32), six experts in three groups of which one stays
_SA = attention(3, 1, 20, 12, mask=33, rot_dims=10, base=77.0)
TINY_S = model(131, 100, [layer(_SA, moe(6, 2, 30, groups=(3, 1), scale=1.5, shared=12)),
                          layer(retention(2, 40, 36, [0.98, 0.8], rot_dims=20, base=50.0), dense(52)),
                          layer(attention(3, 1, 20, 12, mask=33, rot_dims=10, base=77.0, kv_from=0), dense(52))], scale=2.5)
# T: heads of 128 (the mma.sync prompt kernel in bfloat16), four query heads on one key/value head, a window of 70,
# half of every head rotated; retention heads of 128 by 64; one expert of four a token, two groups both kept
_TA = attention(4, 1, 128, 128, mask=70, rot_dims=64, base=300.0)
TINY_T = model(150, 192, [layer(_TA, moe(4, 1, 48, groups=(2, 2), scale=0.5)), layer(retention(2, 128, 64, [0.97, 0.999], rot_dims=128), dense(200)),
                          layer(attention(4, 1, 128, 128, mask=70, rot_dims=64, base=300.0, kv_from=0), None)], scale=4.0)

CONFIGS = {"P": TINY_P, "Q": TINY_Q, "R": TINY_R, "S": TINY_S, "T": TINY_T}


def make_tensors(config, seed, sharpen=3.0, dtype=torch.float32):
    """Random weights with the weights of the query heads' norm scaled up, so that attention is peaky and a key that is
    wrongly seen or missed moves the logits; matrices rounded to ``dtype`` (the values a bfloat16 folder would hold)."""
    arch = architecture_of(config)
    tensors = arch.random_tensors(arch.parse_config(config), seed, torch.float32)
    for name in tensors:
        if name.endswith("mix.q.norm"):
            tensors[name] = tensors[name] * sharpen
        if tensors[name].dim() == 2 and tensors[name].is_floating_point():
            tensors[name] = tensors[name].to(dtype).to(torch.float32)
    return tensors


def plain_tensors(tensors):
    return {k: (v.double() if v.is_floating_point() else v.long()) for k, v in tensors.items()}


def random_requests(config, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, config["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}
