"""Small Bonatar configurations and random models for the tests; nothing here touches the disk unless asked."""
import copy

import torch

from damendaemon_b200.registry import architecture_of


def mixer(heads, kv_heads, dim, vdim, mask=None, rot_dims=None, base=10000.0, scaling=None, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5,
            "rot": None if rot_dims is None else {"dims": rot_dims, "base": base, "scaling": scaling},
            "mask": None if mask is None else {"size": mask}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def layer(mix, mlp, weights_of=None):
    out = {"type": "attention", "mixer": copy.deepcopy(mix), "mlp": copy.deepcopy(mlp)}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def model(vocab, width, layers, scale=None, eps=1e-6):
    return {"architecture": "Bonatar", "vocab": vocab, "width": width, "embedding": {"scale": scale or width ** 0.5},
            "norm": {"eps": eps}, "layers": layers}


YARN = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}

# P: grouped heads, value heads smaller than key heads, part of a head rotated with blended frequencies, chunks of 24
# (no multiple of a page), a dense layer, an expert layer run three times (two of them on the first one's tensors)
_PM = mixer(4, 2, 32, 16, mask=24, rot_dims=16, base=500.0, scaling=YARN)
_PE = moe(4, 2, 24, 1.5, shared=(40, 2.5))
TINY_P = model(211, 64, [layer(_PM, dense(96)), layer(_PM, _PE), layer(_PM, _PE, 1), layer(_PM, _PE, 1)])
# Q: every head its own key/value head, value heads larger than key heads, whole heads rotated without blending,
# chunks of 7 (smaller than a page), one expert per token and no shared one, a layer without a feed-forward, an
# embedding scale that is not the root of the width, another eps
_QM = mixer(3, 3, 16, 40, mask=7, rot_dims=16, base=10000.0)
TINY_Q = model(97, 48, [layer(_QM, moe(5, 1, 16, 0.75)), layer(_QM, None), layer(_QM, dense(72)), layer(_QM, None, 1)],
               scale=3.0, eps=1e-5)
# R: one key/value head for all, equal head sizes of 64 (what the tensor-core kernels take), no mask at all, no rotation
# in the first layer, three experts per token of three (every token uses all), chunks of 128 in the second layer
_RM0 = mixer(2, 1, 64, 64)
_RM1 = mixer(2, 2, 64, 64, mask=128, rot_dims=32, base=100.0, scaling={"factor": 2.0, "original": 32, "fast": 4.0, "slow": 1.0})
TINY_R = model(300, 128, [layer(_RM0, moe(3, 3, 32, 2.0, shared=(16, 1.0))), layer(_RM1, dense(128))], eps=1e-6)

# S: heads of 64 with a key/value head each (what every tensor-core attention kernel takes, decode included), chunks of
# 100 (no multiple of a key block of 128 nor of a page), eight experts of which a token uses two
_SM = mixer(4, 4, 64, 64, mask=100, rot_dims=64, base=10000.0, scaling={"factor": 8.0, "original": 128, "fast": 16.0, "slow": 1.0})
TINY_S = model(400, 256, [layer(_SM, moe(8, 2, 64, 3.0, shared=(64, 3.0))), layer(_SM, dense(512)), layer(_SM, dense(512), 1)])

# T: awkward sizes: a width (100), head sizes (20 and 12), an expert width (30) and a vocabulary (131) that are no
# multiples of 8, five rotated pairs, three heads on one key/value head, chunks of 33
_TM = mixer(3, 1, 20, 12, mask=33, rot_dims=10, base=77.0, scaling={"factor": 1.5, "original": 40, "fast": 4.0, "slow": 1.0})
TINY_T = model(131, 100, [layer(_TM, moe(5, 2, 30, 1.0, shared=(12, 0.5))), layer(_TM, dense(52))], scale=2.5)

# U: heads of 128 with a key/value head each (the mma.sync prompt kernel and the row decode kernel in bfloat16), chunks
# of 70, half of every head rotated, one expert of four a token
_UM = mixer(2, 2, 128, 128, mask=70, rot_dims=64, base=300.0)
TINY_U = model(150, 192, [layer(_UM, moe(4, 1, 48, 4.0)), layer(_UM, dense(200))], scale=4.0)

CONFIGS = {"P": TINY_P, "Q": TINY_Q, "R": TINY_R, "S": TINY_S, "T": TINY_T, "U": TINY_U}


def make_tensors(config, seed, sharpen=3.0, dtype=torch.float32):
    """Random weights with the query and key projections scaled up, so that attention is peaky and a key that is
    wrongly seen or missed moves the logits; matrices rounded to ``dtype`` (the values a bfloat16 folder would hold)."""
    arch = architecture_of(config)
    tensors = arch.random_tensors(arch.parse_config(config), seed, torch.float32)
    for name in tensors:
        if name.endswith(("mix.q", "mix.k")):
            tensors[name] = tensors[name] * sharpen
        if tensors[name].dim() == 2 and tensors[name].is_floating_point():
            tensors[name] = tensors[name].to(dtype).to(torch.float32)
    return tensors


def plain_tensors(tensors):
    return {k: (v.double() if v.is_floating_point() else v.long()) for k, v in tensors.items()}


def random_requests(config, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, config["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}
