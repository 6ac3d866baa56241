"""RWKV-style time mixing with a data-dependent decay.

For normed input rows h [n, d] of one request in order, prev(t) the row before t (zeros before
the first token), H heads of size D:

    x_s  = h + (prev - h) * mu_s                       for the five streams s in r, k, v, g, w
    r, k, v = x_r Wr^T, x_k Wk^T, x_v Wv^T             ([H, D] each);   gate = silu(x_g Wg^T)
    w    = exp(-exp(tanh(x_w W1^T) W2^T + w0))         decay per head and key channel, in (0, 1)
    per head, S [D keys, D values] starting at zero:
        o_t = (S + diag(u) k_t v_t^T)^T r_t            u: bonus of the current token only
        S  <- diag(w_t) S + k_t v_t^T
    out  = ((o / rms(o) per head, eps inside the root) * norm * gate) Wo^T

State per request (float32): S of every head (in the WKV kernel's own order, padded to its tile)
and the last row of h, kept from step to step.
Parameters: hidden_size, num_heads, head_dim, eps.  Tensors under <prefix>: mu.r, mu.k, mu.v,
mu.g, mu.w [d]; r, k, v, g [H*D, d]; w1 [low, d], w2 [H*D, low] (low = decay_rank, or what the file has), w0 [H*D]; u [H, D]; norm [H*D];
o [d, H*D].  The decay, its exponentials, the gate, the unit norm and the state are float32.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, PartError, StateNeed, register_part

STREAMS = "rkvgw"


@register_part("mixer", "rwkv_time_mix")
class RWKVTimeMix(Mixer):
    CAPTURE_SAFE = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.hidden_size = int(params["hidden_size"])
        self.H, self.D = int(params["num_heads"]), int(params["head_dim"])
        # the width of the decay's bottleneck; None: whatever the weight file's w1 and w2 have
        self.low = int(params["decay_rank"]) if params.get("decay_rank") else None
        self.eps = float(params.get("eps", 1e-6))
        if self.D > 256:
            raise PartError("rwkv_time_mix: head sizes up to 256")
        self.prev_off = ops.wkv_state_floats(self.H, self.D)      # the heads' states first, then the previous row

    def cache_need(self):
        return StateNeed((self.prev_off + self.hidden_size,), torch.float32)

    def expected_tensors(self):
        d, HD, p = self.hidden_size, self.H * self.D, self.prefix
        t = {p + "mu." + s: ((d,), "mix") for s in STREAMS}
        t.update({p + s: ((HD, d), "matrix") for s in "rkvg"})
        t.update({p + "w1": ((self.low, d), "matrix"), p + "w2": ((HD, self.low), "matrix"), p + "w0": ((HD,), "bias"),
                  p + "u": ((self.H, self.D), "bias"), p + "norm": ((HD,), "norm"), p + "o": ((d, HD), "matrix")})
        return t

    def load(self, tensors):
        p, f32 = self.prefix, torch.float32
        self.mu = self._to_device(torch.stack([tensors[p + "mu." + s].to(f32) for s in STREAMS], 0), f32)
        self.w_r, self.w_k, self.w_v, self.w_g = (self._to_device(tensors[p + s]) for s in "rkvg")
        self.w_1, self.w_2, self.w_o = (self._to_device(tensors[p + s]) for s in ("w1", "w2", "o"))
        if self.w_1.shape[0] != self.w_2.shape[1]:
            raise PartError(f"{p}w1 {tuple(self.w_1.shape)} and {p}w2 {tuple(self.w_2.shape)} do not fit together")
        self.low = int(self.w_1.shape[0])
        self.w0 = self._to_device(tensors[p + "w0"], f32)
        self.u = self._to_device(tensors[p + "u"], f32)
        self.norm_w = self._to_device(tensors[p + "norm"], f32)

    def forward(self, h, ctx, cache, position=None, residual=None):
        n, dt, dev, HD = h.shape[0], self.runtime.dtype, h.device, self.H * self.D
        mixed = torch.empty((len(STREAMS), n, self.hidden_size), dtype=dt, device=dev)
        ops.token_shift(h, self.mu, cache.state, self.prev_off, ctx.seq_ids, ctx.cu_q, cache.slots, mixed)
        proj = torch.empty((5, n, HD), dtype=torch.float32, device=dev)           # r, k, v, gate, decay (raw)
        for i, w in enumerate((self.w_r, self.w_k, self.w_v, self.w_g)):
            ops.linear(mixed[i], w, out=proj[i])
        low = ops.linear(mixed[4], self.w_1, out_dtype=torch.float32)
        low_t = torch.empty((n, self.low), dtype=dt, device=dev)
        ops.rows_act(low, low_t, act="tanh")
        ops.linear(low_t, self.w_2, out=proj[4])
        out = torch.empty((n, HD), dtype=dt, device=dev)
        ops.wkv(proj[0], proj[1], proj[2], proj[4], proj[3], self.w0, self.u.view(-1), self.norm_w, self.eps,
                cache.state, self.prev_off, h, ctx.cu_q, cache.slots, out, ctx.n_requests, self.H, self.D,
                segments=ops.time_segments(ctx, dev))
        return ops.linear(out, self.w_o, out_dtype=torch.float32)
