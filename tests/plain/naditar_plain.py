"""Plain, slow statement of the Naditar design: one function per mechanism, token by token
where the design is a recurrence, whole-sequence where it is attention.  It shares no code
with the package; the tests compare the engine with it.

Notation: h is a mixer's input [T, width]; weights are [out, in]; positions count from 0.
"""
from __future__ import annotations

import json
import os
import struct

import torch
import torch.nn.functional as F


# ------------------------------------------------------------------ small pieces
def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    return rms(x, eps) * g


def polynorm(z, coef, eps):
    a, b, c, e = [float(v) for v in coef]
    return a * rms(z, eps) + b * rms(z * z, eps) + c * rms(z * z * z, eps) + e


def dense_ff(h, w, pre, eps):
    return polynorm(h @ w[pre + "up"].T, w[pre + "act"], eps) @ w[pre + "down"].T


def causal_conv(x, taps_w):
    """x [T, C], taps_w [C, taps]: out[t] = sum_j taps_w[:, j] * x[t - (taps - 1 - j)], terms with a negative index left out."""
    T, C = x.shape
    taps = taps_w.shape[1]
    out = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1 - j)
            if src >= 0:
                out[t] += taps_w[:, j] * x[src]
    return out


def rotate_interleaved(x, positions, dims, base):
    """x [T, ..., D]: pairs (2i, 2i+1) of the first `dims` coordinates are turned by p * base^(-2i/dims)."""
    out = x.clone()
    for i in range(dims // 2):
        ang = positions.to(x.dtype) * (base ** (-2.0 * i / dims))
        shape = [-1] + [1] * (x.dim() - 2)
        c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


# ------------------------------------------------------------------ mixers
def lightning(h, w, pre, m, eps):
    H, D, V = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = F.silu(h @ w[pre + "q"].T).view(T, H, D)
    k = F.silu(h @ w[pre + "k"].T).view(T, H, D)
    v = F.silu(h @ w[pre + "v"].T).view(T, H, V)
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    S = torch.zeros(H, D, V, dtype=h.dtype)
    o = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(o.reshape(T, H * V), eps) * w[pre + "norm"]
    o = o * torch.sigmoid(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T


def channel_delta(h, w, pre, m, eps):
    H, KV, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = F.silu(causal_conv(h @ w[pre + "q"].T, w[pre + "q.conv"])).view(T, KV, D)
    k = F.silu(causal_conv(h @ w[pre + "k"].T, w[pre + "k.conv"])).view(T, KV, D)
    v = F.silu(causal_conv(h @ w[pre + "v"].T, w[pre + "v.conv"])).view(T, H, V)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[pre + "b"].T)                                        # [T, H]
    a = (h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "dt_bias"]
    g = torch.exp(-torch.exp(w[pre + "A_log"])[None, :, None] * F.softplus(a).view(T, H, D))
    S = torch.zeros(H, D, V, dtype=h.dtype)
    o = torch.zeros(T, H, V, dtype=h.dtype)
    rep = H // KV
    for t in range(T):
        for hd in range(H):
            kt, qt = k[t, hd // rep], q[t, hd // rep]
            S[hd] = g[t, hd][:, None] * S[hd]
            u = beta[t, hd] * (v[t, hd] - S[hd].T @ kt)
            S[hd] = S[hd] + kt[:, None] * u[None, :]
            o[t, hd] = S[hd].T @ qt
    o = rms(o, eps) * w[pre + "norm"]
    gate = torch.sigmoid((h @ w[pre + "g1"].T) @ w[pre + "g2"].T).view(T, H, V)
    return (o * gate).reshape(T, H * V) @ w[pre + "o"].T


def latent_attention(h, w, pre, m, eps):
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    pos = torch.arange(T)
    q = (h @ w[pre + "q"].T).view(T, H, D + R)
    qu, qr = q[..., :D], rotate_interleaved(q[..., D:], pos, m["rot"]["dims"], m["rot"]["base"])
    dkv = h @ w[pre + "dkv"].T
    c = rms(dkv[:, :C], eps) * w[pre + "dkv.norm"]
    kr = rotate_interleaved(dkv[:, C:], pos, m["rot"]["dims"], m["rot"]["base"])    # [T, R], shared by the heads
    ku = (c @ w[pre + "uk"].T).view(T, H, D)
    val = (c @ w[pre + "uv"].T).view(T, H, V)
    sc = (torch.einsum("ihd,jhd->hij", qu, ku) + torch.einsum("ihr,jr->hij", qr, kr)) * m["scale"]
    sc = sc.masked_fill(pos[None, :, None] < pos[None, None, :], float("-inf"))
    o = torch.einsum("hij,jhv->ihv", torch.softmax(sc, dim=-1), val)
    o = o * torch.sigmoid(h @ w[pre + "g"].T)[:, :, None]
    return o.reshape(T, H * V) @ w[pre + "o"].T


MIXERS = {"lightning": lightning, "channel_delta": channel_delta, "latent_attention": latent_attention}


# ------------------------------------------------------------------ the model
def layer_order(cfg):
    """[(layer index, pass number or None)] in the order the layers run; the pass number is given at a pass's first layer."""
    L = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(L)]
    a, b, n = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(a)]
    for t in range(n):
        order += [(i, t if i == a else None) for i in range(a, b)]
    return order + [(i, None) for i in range(b, L)]


def forward(cfg, w, token_ids, layers_out=None):
    """Logits [T, vocab] for one sequence from position 0.  layers_out: a list that receives the residual stream after each layer run."""
    eps = cfg["norm"]["eps"]
    x = scalar_norm(w["embed"][torch.as_tensor(token_ids)], w["embed.norm"], eps)
    for li, pass_no in layer_order(cfg):
        layer, pre = cfg["layers"][li], f"l{li}."
        if pass_no is not None:
            x = x + w["loop.step"][pass_no]
        x = x + MIXERS[layer["type"]](scalar_norm(x, w[pre + "norm1"], eps), w, pre + "mix.", layer["mixer"], eps)
        if layer.get("mlp"):
            x = x + dense_ff(scalar_norm(x, w[pre + "norm2"], eps), w, pre + "mlp.", eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return scalar_norm(x, w["final.norm"], eps) @ w["head"].T


# ------------------------------------------------------------------ reading a model folder (own reader)
_DT = {"BF16": (torch.bfloat16, 2), "F32": (torch.float32, 4), "I32": (torch.int32, 4), "F64": (torch.float64, 8)}


def load_dir(model_dir, dtype=torch.float64):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    w = {}
    for name, h in header.items():
        if name == "__metadata__":
            continue
        dt, _ = _DT[h["dtype"]]
        a, b = h["data_offsets"]
        t = torch.frombuffer(bytearray(data[a:b]), dtype=dt).reshape(h["shape"]) if b > a else torch.empty(h["shape"], dtype=dt)
        w[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, w
