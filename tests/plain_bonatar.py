"""A plain, slow Bonatar: whole sequences, no cache, one function per mechanism.

It shares no code with the product path: it reads config.json and model.safetensors itself and
computes with ordinary tensor arithmetic, float64 by default so that it is the more exact side of
every comparison. Notation: T tokens, D model width, H query heads, G key/value heads, dk the
size of a query or key head, dv the size of a value head, E experts of which a token uses K.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

# None, or a dtype that stored activations are rounded to (what a 16-bit engine keeps between its kernels), so that a
# test can measure how far such rounding alone moves the logits of a model
ROUND = None


def kept(x):
    return x if ROUND is None else x.to(ROUND).to(x.dtype)


_NP = {"F32": np.float32, "F64": np.float64, "F16": np.float16, "I32": np.int32, "I64": np.int64}


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


def embed(ids, table, scale):
    """x[t] = table[ids[t]] * scale."""
    return table[ids] * scale


def rms_norm_offset(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * (1 + w): the weight is stored as its distance from one."""
    return kept(x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * (1.0 + w))


def rotary_frequencies(n_rot, base, scaling=None):
    """(frequencies [n_rot/2], factor on cos and sin) in float64.

    Plain: f_i = base^(-2i/n_rot). With YaRN-style scaling {factor s, original length L, fast, slow}: the pair
    whose wavelength makes t turns over L tokens is d(t) = n_rot ln(L / (2 pi t)) / (2 ln base); pairs below
    lo = max(floor(d(fast)), 0) keep f_i, pairs above hi = min(ceil(d(slow)), n_rot - 1) get f_i / s, those
    between are blended linearly, r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1); cos and sin are scaled by
    0.1 ln s + 1.
    """
    i = torch.arange(n_rot // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / n_rot)
    if not scaling:
        return f, 1.0
    s, length = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns):
        return n_rot * math.log(length / (2 * math.pi * turns)) / (2 * math.log(base))
    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), n_rot - 1)
    r = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / s * r + f * (1.0 - r), 0.1 * math.log(s) + 1.0


def rotate_pairs(x, positions, freqs, magnitude):
    """x: [T, heads, d]; the first 2 * len(freqs) dimensions of every head are rotated, neighbours (2i, 2i+1)
    forming a pair: (a, b) -> (a c - b s, b c + a s) with c, s = magnitude * cos / sin (position * f_i)."""
    n = 2 * freqs.numel()
    angle = positions.to(freqs.dtype)[:, None] * freqs[None, :]
    c = (torch.cos(angle) * magnitude).to(x.dtype)[:, None, :]
    s = (torch.sin(angle) * magnitude).to(x.dtype)[:, None, :]
    a, b = x[..., 0:n:2], x[..., 1:n:2]
    out = x.clone()
    out[..., 0:n:2] = a * c - b * s
    out[..., 1:n:2] = b * c + a * s
    return out


def visible(n_tokens, chunk=None):
    """[T, T] bool: query i sees key j <= i, and with chunks only if i // chunk == j // chunk."""
    i = torch.arange(n_tokens)[:, None]
    j = torch.arange(n_tokens)[None, :]
    see = j <= i
    if chunk:
        see = see & (i // chunk == j // chunk)
    return see


def grouped_attention(q, k, v, scale, see):
    """q [T,H,dk], k [T,G,dk], v [T,G,dv] -> [T,H,dv]; query head h reads key/value head h // (H/G);
    softmax over the visible keys of (q . k) * scale."""
    H, G = q.shape[1], k.shape[1]
    k = k.repeat_interleave(H // G, dim=1)
    v = v.repeat_interleave(H // G, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    scores = scores.masked_fill(~see[None], float("-inf"))
    return torch.einsum("hij,jhd->ihd", torch.softmax(scores, dim=-1), v)


def attention_mixer(h, w, m, positions):
    """The whole mixer on its normed input h [T, D]; w: the mixer's tensors by short name; m: its config."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = kept(h @ w["q"].T).view(T, H, dk)
    k = kept(h @ w["k"].T).view(T, G, dk)
    v = kept(h @ w["v"].T).view(T, G, dv)
    rot = m.get("rot")
    if rot:
        freqs, magnitude = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        freqs = freqs.to(h.dtype)
        q, k = kept(rotate_pairs(q, positions, freqs, magnitude)), kept(rotate_pairs(k, positions, freqs, magnitude))
    mask = m.get("mask")
    out = grouped_attention(q, k, v, m["scale"], visible(T, mask["size"] if mask else None))
    gate = torch.sigmoid(kept(h @ w["g"].T))                 # [T, H]: one number per head
    out = kept(out * gate[:, :, None])
    return out.reshape(T, H * dv) @ w["o"].T


def dense_ff(h, w):
    """down(relu(up h)^2)."""
    return kept(torch.relu(h @ w["up"].T) ** 2) @ w["down"].T


def clamped_glu_expert(h, w, limit):
    """g = min(gate h, limit), u = clamp(up h, -limit, limit); down(g sigmoid(1.702 g) (u + 1))."""
    g = kept(h @ w["gate"].T).clamp(max=limit)
    u = kept(h @ w["up"].T).clamp(-limit, limit)
    return kept(g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].T


def table_routed_experts(h, ids, w, c):
    """Each token's experts are row ids[t] of an integer table [vocab, K]; every chosen expert weighs 1/K; a shared
    expert, if the layer has one, runs for every token and is added."""
    table = w["table"]
    K = table.shape[1]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in table[ids[t]].tolist():
            ew = {n: w[f"e{e}.{n}"] for n in ("gate", "up", "down")}
            out[t] += clamped_glu_expert(h[t:t + 1], ew, c["expert"]["limit"])[0] / K
    if c.get("shared"):
        out = out + clamped_glu_expert(h, {n: w[f"shared.{n}"] for n in ("gate", "up", "down")}, c["shared"]["limit"])
    return out


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, ids, streams=None):
    """Logits [T, vocab] of one whole sequence. streams: a list that receives the residual stream after each layer."""
    ids = torch.as_tensor(ids, dtype=torch.int64)
    positions = torch.arange(len(ids))
    eps = config["norm"]["eps"]
    x = embed(ids, tensors["embed"], config["embedding"]["scale"])
    for i, layer in enumerate(config["layers"]):
        if layer["type"] != "attention":
            raise ValueError(f"layer {i}: unknown type {layer['type']!r}")
        w = sub(tensors, f"l{layer.get('weights_of', i)}.")
        x = x + attention_mixer(rms_norm_offset(x, w["norm1"], eps), sub(w, "mix."), layer["mixer"], positions)
        mlp = layer.get("mlp")
        if mlp:
            h = rms_norm_offset(x, w["norm2"], eps)
            if mlp["kind"] == "dense":
                x = x + dense_ff(h, sub(w, "mlp."))
            elif mlp["kind"] == "moe":
                x = x + table_routed_experts(h, ids, sub(w, "mlp."), mlp)
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp['kind']!r}")
        if streams is not None:
            streams.append(x.clone())
    return rms_norm_offset(x, tensors["final.norm"], eps) @ tensors["head"].T
