"""Plain, slow statement of the Namesun design: one function per mechanism, token by token where
the design is a recurrence, whole-sequence where it is attention.  It shares no code with the
package; the tests compare the engine with it.

Notation: h is a sublayer's input [T, width]; weights are [out, in]; positions count from 0.
A layer adds to the stream x the NORMED output of each sublayer, which reads x itself:
    x <- x + m * ls1 * (w1 * N(mixer(x)));   x <- x + m * ls2 * (w2 * N(ff(x)))
with N(y) = y / sqrt(mean(y^2) + eps), w the norm's weight, ls the layer-scale vector, m one number.
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch
import torch.nn.functional as F


# ------------------------------------------------------------------ small pieces
def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def rotate_half(x, positions, dims, base):
    """x [T, heads, D]: coordinate i of the first `dims` is paired with i + dims/2 and the pair is turned by
    p * base^(-2i/dims); coordinates from `dims` on pass unchanged."""
    out = x.clone()
    half = dims // 2
    for i in range(half):
        ang = positions.to(x.dtype) * (base ** (-2.0 * i / dims))
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


# ------------------------------------------------------------------ mixers
def chunked_sink_attention(h, w, pre, m, eps, v_first=None):
    """Softmax attention without positions: q and k are unit-RMS vectors per head, a query at i sees j <= i of its own
    block of `mask.size` positions (blocks counted from position 0), and the softmax has one more term of score 0
    that carries no value.  v_first (values of an earlier layer for the same tokens) is blended into v if given.
    Returns (output [T, width], the values this layer used [T, G, vdim])."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms((h @ w[pre + "q"].T).view(T, H, D), eps)
    k = rms((h @ w[pre + "k"].T).view(T, G, D), eps)
    v = (h @ w[pre + "v"].T).view(T, G, V)
    if v_first is not None:
        lam = w[pre + "vmix"].to(h.dtype)
        v = (1 - lam) * v + lam * v_first
    size = (m.get("mask") or {}).get("size")
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for i in range(T):
        lo = 0 if not size else (i // size) * size
        for hd in range(H):
            g = hd // (H // G)
            s = (k[lo:i + 1, g] @ q[i, hd]) * m["scale"]
            e = torch.exp(s)
            p = e / (1.0 + e.sum())
            out[i, hd] = p @ v[lo:i + 1, g]
    return out.reshape(T, H * V) @ w[pre + "o"].T, v


def retention(h, w, pre, m, eps):
    """Per head S_t = decay * S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; q, k rotated, k also / sqrt(dim); each head's o made
    unit-RMS, then gated by silu(W_g h)."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rotate_half((h @ w[pre + "q"].T).view(T, H, D), pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_half((h @ w[pre + "k"].T).view(T, H, D), pos, m["rot"]["dims"], m["rot"]["base"]) * D ** -0.5
    v = (h @ w[pre + "v"].T).view(T, H, V)
    S = torch.zeros(H, D, V, dtype=h.dtype)
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    o = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(o, eps).reshape(T, H * V) * F.silu(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T


# ------------------------------------------------------------------ feed-forwards
def dense_ff(h, w, pre):
    return (F.silu(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def clamped_expert(h, w, pre, limit):
    g = torch.clamp(h @ w[pre + "gate"].T, max=limit)
    u = torch.clamp(h @ w[pre + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ w[pre + "down"].T


def route(h, w, pre, r):
    """(chosen experts [T, top], their weights [T, top]): softmax scores; the choice adds the correction and is confined
    to the `keep` groups of neighbouring experts whose best choice score is largest; the weights are the plain scores."""
    E, top = r["experts"], r["top"]
    s = torch.softmax(h @ w[pre + "router"].to(h.dtype).T, dim=-1)
    choice = s + w[pre + "correction"].to(h.dtype)
    groups = r.get("groups")
    if groups:
        per = E // groups["count"]
        best = choice.view(-1, groups["count"], per).max(-1).values
        kept = best.topk(groups["keep"], dim=-1).indices
        allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True).repeat_interleave(per, dim=1)
        choice = choice.masked_fill(~allowed, float("-inf"))
    idx = choice.topk(top, dim=-1).indices
    return idx, s.gather(1, idx)


def moe_ff(h, w, pre, mlp):
    idx, wt = route(h, w, pre, mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            out[t] += wt[t, j] * clamped_expert(h[t:t + 1], w, f"{pre}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        out = out + clamped_expert(h, w, pre + "shared.", mlp["shared"]["limit"])
    return out


# ------------------------------------------------------------------ the model
def forward_layers(cfg, w, token_ids, dtype=torch.float64):
    """The residual stream after every layer [layers, T, width] and the logits [T, vocab]."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x = w["embed"][torch.as_tensor(token_ids, dtype=torch.long)]
    v_first, streams = None, []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "attention":
            mixes = bool(m.get("v_mix"))
            y, v = chunked_sink_attention(x, w, p + "mix.", m, eps, v_first if mixes else None)
            if mixes and v_first is None:
                v_first = v
        elif layer["type"] == "retention":
            y = retention(x, w, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + mult * w[p + "ls1"] * (rms(y, eps) * w[p + "norm1"])
        mlp = layer.get("mlp")
        if mlp is not None:
            y = dense_ff(x, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(x, w, p + "mlp.", mlp)
            x = x + mult * w[p + "ls2"] * (rms(y, eps) * w[p + "norm2"])
        streams.append(x)
    logits = (rms(x, eps) * w["final.norm"]) @ w["head"].T
    return torch.stack(streams), logits


def forward_logits(cfg, w, token_ids, dtype=torch.float64):
    return forward_layers(cfg, w, token_ids, dtype)[1]


# ------------------------------------------------------------------ reading a model folder
_DT = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32, "F16": torch.float16, "I64": torch.int64}


def load_model_dir(path):
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(path, "model.safetensors"), "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        blob = f.read()
    w = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        a, b = e["data_offsets"]
        t = torch.frombuffer(bytearray(blob[a:b]), dtype=_DT[e["dtype"]]) if b > a else torch.zeros(0, dtype=_DT[e["dtype"]])
        w[name] = t.reshape(e["shape"]).clone()
    return cfg, w
