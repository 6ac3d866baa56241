"""Govopel, written out plainly: float64, whole sequences, one function per mechanism, explicit
loops over tokens and heads where that keeps the formula visible.  It shares no code with the
package; the tests hold the engine against it.

A model is (config dictionary as config.json gives it, {tensor name: float64 tensor}).
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def rotary_frequencies(rot):
    """(f [dims/2], m): frequency of pair i and the multiplier of cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=F64), 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return torch.tensor(out, dtype=F64), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot):
    """x [T, heads, d]: the first rot.dims entries of each head are turned, pair (i, i + dims/2) by
    the angle position * f_i; the rest pass."""
    dims = int(rot["dims"])
    half = dims // 2
    f, m = rotary_frequencies(rot)
    out = x.clone()
    for t in range(x.shape[0]):
        a = float(positions[t]) * f
        c, s = torch.cos(a) * m, torch.sin(a) * m
        u, v = x[t, :, :half], x[t, :, half:dims]
        out[t, :, :half] = u * c - v * s
        out[t, :, half:dims] = v * c + u * s
    return out


def softmax_rows(scores, visible):
    """scores [T, T]; visible [T, T] bool.  Ordinary softmax over the visible keys of each row."""
    s = scores.masked_fill(~visible, float("-inf"))
    s = s - s.max(-1, keepdim=True).values
    e = torch.exp(s)
    return e / e.sum(-1, keepdim=True)


def chunk_mask(T, size):
    """Position i sees j <= i within the same run of `size` positions counted from 0 (size 0: all j <= i)."""
    vis = torch.zeros((T, T), dtype=torch.bool)
    for i in range(T):
        for j in range(i + 1):
            vis[i, j] = (size <= 0) or (i // size == j // size)
    return vis


def attention_mixer(h, mx, w, eps):
    """Grouped heads, the values are the keys as projected, rotation then unit norm, capped scores,
    chunked mask.  h [T, width]; w: q, k, o."""
    T = h.shape[0]
    H, G, d = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"])
    q = (h @ w["q"].T).view(T, H, d)
    k = (h @ w["k"].T).view(T, G, d)
    v = k.clone()
    pos = list(range(T))
    q, k = rotate(q, pos, mx["rot"]), rotate(k, pos, mx["rot"])
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    size = int((mx.get("mask") or {}).get("size", 0) or 0)
    vis = chunk_mask(T, size)
    cap = float(mx.get("softcap", 0.0) or 0.0)
    outs = []
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * float(mx["scale"])
        if cap:
            s = cap * torch.tanh(s / cap)
        outs.append(softmax_rows(s, vis) @ v[:, g])
    return torch.cat(outs, -1) @ w["o"].T


def latent_attention_mixer(h, mx, w, eps):
    """Queries and keys/values through low-rank latents; one rotated key part shared by the heads.
    w: dq, dq.norm, uq, dkv, dkv.norm, uk, uv, o."""
    T = h.shape[0]
    H, d, r, dv, rank = int(mx["heads"]), int(mx["dim"]), int(mx["rot_dim"]), int(mx["vdim"]), int(mx["kv_rank"])
    cq = rms_norm(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).view(T, H, d + r)
    q_plain, q_rot = q[..., :d], q[..., d:]
    low = h @ w["dkv"].T
    c = rms_norm(low[:, :rank], w["dkv.norm"], eps)
    k_rot = low[:, rank:rank + r].reshape(T, 1, r)
    pos = list(range(T))
    rot = dict(mx["rot"], dims=r)
    q_rot, k_rot = rotate(q_rot, pos, rot), rotate(k_rot, pos, rot)
    k_plain = (c @ w["uk"].T).view(T, H, d)
    v = (c @ w["uv"].T).view(T, H, dv)
    vis = chunk_mask(T, 0)
    outs = []
    for head in range(H):
        s = (q_plain[:, head] @ k_plain[:, head].T + q_rot[:, head] @ k_rot[:, 0].T) * float(mx["scale"])
        outs.append(softmax_rows(s, vis) @ v[:, head])
    return torch.cat(outs, -1) @ w["o"].T


def dense_ff(h, mlp, w):
    """g = min(gate, limit), u = clamp(up, -limit, limit), y = g sigmoid(1.702 g) (u + 1), down."""
    limit = float(mlp["limit"])
    g = torch.clamp(h @ w["gate"].T, max=limit)
    u = torch.clamp(h @ w["up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w["down"].T


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence from position 0.  `layers_out`: a list that receives the
    stream after every layer."""
    eps = float(config["norm"]["eps"])
    tensors = {k: v.to(F64) for k, v in tensors.items()}
    x = rms_norm(tensors["embed"][torch.tensor(list(tokens))], tensors["embed.norm"], eps)
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        mixer = {"attention": attention_mixer, "latent_attention": latent_attention_mixer}[layer["type"]]
        x = x + rms_norm(mixer(x, layer["mixer"], sub(tensors, p + "mix."), eps), tensors[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + rms_norm(dense_ff(x, layer["mlp"], sub(tensors, p + "mlp.")), tensors[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    logits = rms_norm(x, tensors["final.norm"], eps) @ tensors["embed"].T
    cap = float(config.get("logit_softcap", 0.0) or 0.0)
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits
