"""A plain, slow Zokanex: whole sequences, no cache, one function per mechanism.

It shares no code with the product path: it reads config.json and model.safetensors itself and computes with
ordinary tensor arithmetic, float64 by default so that it is the more exact side of every comparison. Notation:
T tokens, D model width, H query heads, G key/value heads, dk the size of a query or key head, dv the size of a
value head, E experts of which a token uses K, in C groups of which B stay eligible.

The design: x0 = table[id] * scale; every layer is parallel, x <- x + mixer(n) + ff(n) with n = rms(x) * w; the mixer
is softmax attention (grouped heads, per-head RMS norm of queries and keys before a half-split rotation, a sliding
window, optionally the keys and values of an earlier layer) or retention (a per-head decaying outer-product state,
rotated queries and keys, a weightless per-head RMS norm of the read-out and a silu gate); the feed-forward is a
gated unit (tanh-gelu), or experts (silu) chosen by sigmoid scores within the best groups plus a shared expert behind
a sigmoid gate, or absent; the logits are head . (rms(x) * w).
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


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis; w None: no weight."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def rotate_halves(x, positions, n_rot, base):
    """x [T, heads, d]: of every head the first n_rot dimensions turn, dimension i with dimension i + n_rot/2:
    (a, b) -> (a cos - b sin, b cos + a sin) of the angle position * base^(-2i/n_rot); the others stay."""
    half = n_rot // 2
    f = float(base) ** (-2.0 * torch.arange(half, dtype=torch.float64) / n_rot)
    angle = positions.to(torch.float64)[:, None] * f[None, :]
    c, s = torch.cos(angle).to(x.dtype)[:, None, :], torch.sin(angle).to(x.dtype)[:, None, :]
    a, b = x[..., :half], x[..., half:n_rot]
    out = x.clone()
    out[..., :half] = a * c - b * s
    out[..., half:n_rot] = b * c + a * s
    return out


def window_visible(n_tokens, size=None):
    """[T, T] bool: query i sees key j when 0 <= i - j < size (no size: every j <= i)."""
    i = torch.arange(n_tokens)[:, None]
    j = torch.arange(n_tokens)[None, :]
    see = j <= i
    if size:
        see = see & (i - j < size)
    return see


def grouped_softmax_attention(q, k, v, scale, see):
    """q [T,H,dk], k [T,G,dk], v [T,G,dv] -> [T,H,dv]; query head h reads key/value head h // (H/G);
    softmax over the visible keys of (q . k) * scale."""
    H, G = q.shape[1], k.shape[1]
    k = k.repeat_interleave(H // G, dim=1)
    v = v.repeat_interleave(H // G, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    scores = scores.masked_fill(~see[None], float("-inf"))
    return torch.einsum("hij,jhd->ihd", torch.softmax(scores, dim=-1), v)


def attention_keys_values(h, w, m, positions, eps):
    """What an attention layer caches: keys after their norm and rotation [T,G,dk], values [T,G,dv]."""
    T, G, dk, dv = h.shape[0], m["kv_heads"], m["dim"], m["vdim"]
    k = kept(h @ w["k"].T).view(T, G, dk)
    k = rms_norm(k, w["k.norm"], eps)
    if m.get("rot"):
        k = rotate_halves(k, positions, m["rot"]["dims"], m["rot"]["base"])
    return kept(k), kept(h @ w["v"].T).view(T, G, dv)


def attention_mixer(h, w, m, positions, eps, keys_values):
    """Softmax attention of the normed input h [T, D] over keys_values = (k, v), the layer's own or another's."""
    T, H, dk, dv = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q = kept(h @ w["q"].T).view(T, H, dk)
    q = rms_norm(q, w["q.norm"], eps)
    if m.get("rot"):
        q = rotate_halves(q, positions, m["rot"]["dims"], m["rot"]["base"])
    k, v = keys_values
    mask = m.get("mask")
    out = grouped_softmax_attention(kept(q), k, v, m["scale"], window_visible(T, mask["size"] if mask else None))
    return kept(out).reshape(T, H * dv) @ w["o"].T


def retention_recurrence(q, k, v, decay, state=None):
    """Token by token, per head: S <- decay * S + k_t v_t^T, o_t = S^T q_t. q, k [T,H,dk], v [T,H,dv], decay [H],
    S [H,dk,dv] from zero (or ``state``). Returns (o [T,H,dv], S)."""
    T, H, dk = q.shape
    S = torch.zeros(H, dk, v.shape[2], dtype=q.dtype) if state is None else state.clone()
    out = []
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hkv,hk->hv", S, q[t]))
    return torch.stack(out), S


def retention_mixer(h, w, m, positions, eps):
    """Retention of the normed input h [T, D]: rotated queries and keys, keys times dk^-1/2 after the rotation, the
    recurrence, every head's read-out divided by its root mean square, times silu(gate), projected."""
    T, H, dk, dv = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q = kept(h @ w["q"].T).view(T, H, dk)
    k = kept(h @ w["k"].T).view(T, H, dk)
    v = kept(h @ w["v"].T).view(T, H, dv)
    if m.get("rot"):
        q = rotate_halves(q, positions, m["rot"]["dims"], m["rot"]["base"])
        k = rotate_halves(k, positions, m["rot"]["dims"], m["rot"]["base"])
    k = k * dk ** -0.5
    o, _ = retention_recurrence(q, k, v, torch.tensor(m["decay"], dtype=h.dtype))
    o = rms_norm(o, None, eps).reshape(T, H * dv)
    gate = kept(h @ w["g"].T)
    return kept(o * (gate * torch.sigmoid(gate))) @ w["o"].T


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def gated_ff(h, w, act):
    """down(act(gate h) * (up h))."""
    return kept(act(kept(h @ w["gate"].T)) * kept(h @ w["up"].T)) @ w["down"].T


def choose_experts(scores, top, n_groups, keep):
    """scores [T, E] -> chosen [T, top] (by falling score). The E experts form n_groups runs of neighbours; a run's
    worth is the sum of its two best scores (of its one, if a run is a single expert); only the ``keep`` worthiest
    runs stay eligible."""
    T, E = scores.shape
    per = E // n_groups
    runs = scores.view(T, n_groups, per)
    worth = runs.topk(min(2, per), dim=-1).values.sum(-1)
    best = worth.topk(keep, dim=-1).indices
    open_run = torch.zeros(T, n_groups, dtype=torch.bool)
    open_run.scatter_(1, best, True)
    eligible = open_run[:, :, None].expand(T, n_groups, per).reshape(T, E)
    return scores.masked_fill(~eligible, float("-inf")).topk(top, dim=-1).indices


def routed_experts(h, w, c):
    """Experts by score: s = sigmoid(router h); the chosen experts' outputs weighted by s * router scale (not
    renormalised); the shared expert, if any, times sigmoid(sg . h), is added."""
    r = c["router"]
    scores = torch.sigmoid(h @ w["router"].T)
    groups = r.get("groups") or {"count": 1, "keep": 1}
    chosen = choose_experts(scores, r["top"], groups["count"], groups["keep"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            ew = {n: w[f"e{e}.{n}"] for n in ("gate", "up", "down")}
            out[t] += gated_ff(h[t:t + 1], ew, silu)[0] * scores[t, e] * r["scale"]
    if c.get("shared"):
        shared = gated_ff(h, {n: w[f"shared.{n}"] for n in ("gate", "up", "down")}, silu)
        out = out + shared * torch.sigmoid(h @ w["shared.sg"].T)
    return out


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, ids, streams=None):
    """Logits [T, vocab] of one whole sequence. streams: a list that receives the residual stream after each layer."""
    ids = torch.as_tensor(ids, dtype=torch.int64)
    positions = torch.arange(len(ids))
    eps = config["norm"]["eps"]
    x = embed(ids, tensors["embed"], config["embedding"]["scale"])
    cached = {}
    for i, layer in enumerate(config["layers"]):
        w = sub(tensors, f"l{i}.")
        mix, m = sub(w, "mix."), layer["mixer"]
        h = kept(rms_norm(x, w["norm1"], eps))
        if layer["type"] == "attention":
            source = m.get("kv_from")
            if source is None:
                cached[i] = attention_keys_values(h, mix, m, positions, eps)
                source = i
            mixed = attention_mixer(h, mix, m, positions, eps, cached[source])
        elif layer["type"] == "retention":
            mixed = retention_mixer(h, mix, m, positions, eps)
        else:
            raise ValueError(f"layer {i}: unknown type {layer['type']!r}")
        mlp = layer.get("mlp")
        fed = 0.0
        if mlp:
            if mlp["kind"] == "dense":
                fed = gated_ff(h, sub(w, "mlp."), gelu_tanh)
            elif mlp["kind"] == "moe":
                fed = routed_experts(h, sub(w, "mlp."), mlp)
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp['kind']!r}")
        x = x + (mixed + fed)
        if streams is not None:
            streams.append(x.clone())
    return kept(rms_norm(x, tensors["final.norm"], eps)) @ tensors["head"].T
