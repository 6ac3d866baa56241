"""Plain, slow implementation of the Falalix decoder, the oracle of the tests.

Whole sequences, no cache, no batching, one function per mechanism, torch on the CPU only.  It
shares no code with ``rllm_b200``: it takes a config dict and a dict of tensors (as stored, names
as in the weight file) and computes everything in one floating-point type (float64 by default)
with explicit loops over tokens wherever the definition is a recurrence.

Notation: T tokens, d model width, rows of a [T, d] tensor are tokens.  Linear weights are
[out, in]; ``lin(W, a)`` is ``a @ W.T``.
"""
from __future__ import annotations

import math

import torch


def lin(W, a, b=None):
    y = a @ W.T
    return y if b is None else y + b


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


# ---------------------------------------------------------------- feed-forward

def relu2_ffn(h, W_up, W_down):
    """down(relu(up(h))^2)."""
    a = torch.relu(lin(W_up, h))
    return lin(W_down, a * a)


# ---------------------------------------------------------------- attention with a window and kept first tokens

def visible(T, size, keep_first):
    """[T, T] boolean: query i sees key j iff j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def gated_window_attention(h, t, p, c, eps):
    """`t`: tensors, `p`: prefix of this mixer's tensors, `c`: its config entry.
    Biased q/k/v projections, RMS norm over the whole q and k rows, no position encoding,
    softmax over the visible keys, sigmoid output gate read from `h`, output projection."""
    T = h.shape[0]
    H, G, dk, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = lin(t[p + "q"], h, t[p + "q.b"])
    k = lin(t[p + "k"], h, t[p + "k.b"])
    v = lin(t[p + "v"], h, t[p + "v.b"])
    q = rms_norm(q, t[p + "q.norm"], eps).reshape(T, H, dk)
    k = rms_norm(k, t[p + "k.norm"], eps).reshape(T, G, dk)
    v = v.reshape(T, G, dv)
    see = visible(T, c["mask"]["size"], c["mask"]["keep_first"])
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    per = H // G
    for head in range(H):
        g = head // per
        s = (q[:, head] @ k[:, g].T) * c["scale"]
        s = s.masked_fill(~see, -math.inf)
        out[:, head] = torch.softmax(s, -1) @ v[:, g]
    gate = torch.sigmoid(lin(t[p + "g"], h))
    return lin(t[p + "o"], out.reshape(T, H * dv) * gate)


# ---------------------------------------------------------------- RWKV-style time mixing

def rwkv_time_mix(h, t, p, c, eps):
    """Token shift with one mixing vector per stream, data-dependent decay through a small
    tanh bottleneck, a [dim, dim] state per head with a bonus for the current token, unit RMS per
    head, norm weight, silu gate, output projection."""
    T, d = h.shape
    H, D = c["heads"], c["dim"]
    prev = torch.cat([torch.zeros(1, d, dtype=h.dtype), h[:-1]], 0)
    mix = {s: h + (prev - h) * t[p + "mu." + s] for s in "rkvgw"}
    r = lin(t[p + "r"], mix["r"]).reshape(T, H, D)
    k = lin(t[p + "k"], mix["k"]).reshape(T, H, D)
    v = lin(t[p + "v"], mix["v"]).reshape(T, H, D)
    gate = silu(lin(t[p + "g"], mix["g"]))
    w = torch.exp(-torch.exp(lin(t[p + "w2"], torch.tanh(lin(t[p + "w1"], mix["w"]))) + t[p + "w0"])).reshape(T, H, D)
    u = t[p + "u"]
    S = torch.zeros(H, D, D, dtype=h.dtype)            # [head, key channel, value channel]
    o = torch.zeros(T, H, D, dtype=h.dtype)
    for i in range(T):
        kv = k[i][:, :, None] * v[i][:, None, :]
        o[i] = torch.einsum("hk,hkv->hv", r[i], S + u[:, :, None] * kv)
        S = w[i][:, :, None] * S + kv
    o = rms_unit(o, eps).reshape(T, H * D) * t[p + "norm"] * gate
    return lin(t[p + "o"], o)


def parallel_mixer(h, t, p, c, eps):
    left = gated_window_attention(h, t, p + "left.", c["left"], eps)
    right = rwkv_time_mix(h, t, p + "right.", c["right"], eps)
    return c["left_scale"] * left + c["right_scale"] * right


# ---------------------------------------------------------------- Mamba (selective scan)

def mamba1(h, t, p, c):
    T = h.shape[0]
    inner, N, R, taps = c["inner"], c["state"], c["dt_rank"], c["conv"]
    xz = lin(t[p + "in"], h)
    x, z = xz[:, :inner], xz[:, inner:]
    pad = torch.cat([torch.zeros(taps - 1, inner, dtype=h.dtype), x], 0)
    conv = torch.zeros(T, inner, dtype=h.dtype)
    for j in range(taps):                              # the last column weighs the current token
        conv = conv + pad[j:j + T] * t[p + "conv"][:, j]
    x = silu(conv + t[p + "conv.b"])
    low = lin(t[p + "x"], x)
    dt, B, C = low[:, :R], low[:, R:R + N], low[:, R + N:R + 2 * N]
    dt = softplus(lin(t[p + "dt"], dt, t[p + "dt.b"]))
    A = -torch.exp(t[p + "A_log"])
    S = torch.zeros(inner, N, dtype=h.dtype)
    y = torch.zeros(T, inner, dtype=h.dtype)
    for i in range(T):
        S = torch.exp(dt[i][:, None] * A) * S + (dt[i] * x[i])[:, None] * B[i][None, :]
        y[i] = S @ C[i] + t[p + "D"] * x[i]
    return lin(t[p + "o"], y * silu(z))


# ---------------------------------------------------------------- the model

def run_order(cfg):
    """[(layer index, pass number or None when the layer opens no pass)]."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            order.append((i, t if i == loop["start"] else None))
    order += [(i, None) for i in range(loop["stop"], n)]
    return order


def forward(cfg, tensors, tokens, dtype=torch.float64, return_layers=False):
    """Logits [T, vocab] of one sequence (and the residual stream after every layer run)."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    x = t["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x0 = x
    after = []
    for i, opens in run_order(cfg):
        if opens is not None:
            x = lin(t["loop.in"], torch.cat([x, x0], -1)) + t["loop.step"][opens]
        layer, p = cfg["layers"][i], f"l{i}."
        h = rms_norm(x, t[p + "norm1"], eps)
        if layer["type"] == "parallel":
            a = parallel_mixer(h, t, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "mamba1":
            a = mamba1(h, t, p + "mix.", layer["mixer"])
        else:
            raise ValueError(layer["type"])
        x = x + m * a
        if layer.get("mlp") is not None:
            assert layer["mlp"]["kind"] == "dense"
            x = x + m * relu2_ffn(rms_norm(x, t[p + "norm2"], eps), t[p + "mlp.up"], t[p + "mlp.down"])
        after.append(x)
    logits = lin(t["head"], rms_norm(x, t["final.norm"], eps))
    return (logits, torch.stack(after)) if return_layers else logits
