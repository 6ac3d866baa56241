"""Mamba (selective state-space) mixer.

For normed input rows h [n, d] of one request in order, `inner` channels, N state entries per
channel, a convolution of `conv` taps:

    [x | z] = h Win^T                                   (inner each)
    x  <- silu(conv_b + sum_j conv[:, j] * x(t - (conv-1) + j))    causal per channel, zeros before the start,
                                                                   the last tap weighs the current token
    [dt | B | C] = x Wx^T                               (dt_rank, N, N)
    dt <- softplus(dt Wdt^T + dt_b)                     one step size per channel
    A  = -exp(A_log)                                    [inner, N]
    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;   y_c = sum_n S[c, n] C_n + D_c x_c
    out = (y * silu(z)) Wo^T

State per request (float32): S and the last conv-1 inputs of the convolution.  Parameters:
hidden_size, inner, state, dt_rank, conv.  Tensors under <prefix>: in [2*inner, d], conv [inner,
conv], conv.b, x [dt_rank + 2N, inner], dt [inner, dt_rank], dt.b, A_log [inner, N], D, o [d,
inner].  Step sizes, decays, their exponentials and the state are float32 in every mode.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, PartError, StateNeed, register_part


@register_part("mixer", "mamba1")
class Mamba1(Mixer):
    CAPTURE_SAFE = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.hidden_size = int(params["hidden_size"])
        self.inner, self.N = int(params["inner"]), int(params["state"])
        self.R, self.taps = int(params["dt_rank"]), int(params["conv"])
        if self.N > 256:
            raise PartError("mamba1: at most 256 state entries per channel")
        if self.taps < 1:
            raise PartError("mamba1: the convolution needs at least one tap")
        self.conv_off = self.inner * self.N

    def cache_need(self):
        return StateNeed((self.conv_off + self.inner * (self.taps - 1),), torch.float32)

    def expected_tensors(self):
        d, I, N, R, p = self.hidden_size, self.inner, self.N, self.R, self.prefix
        return {p + "in": ((2 * I, d), "matrix"), p + "conv": ((I, self.taps), "conv"), p + "conv.b": ((I,), "bias"),
                p + "x": ((R + 2 * N, I), "matrix"), p + "dt": ((I, R), "matrix"), p + "dt.b": ((I,), "bias"),
                p + "A_log": ((I, N), "bias"), p + "D": ((I,), "norm"), p + "o": ((d, I), "matrix")}

    def load(self, tensors):
        p, f32 = self.prefix, torch.float32
        self.w_in, self.w_x, self.w_dt, self.w_o = (self._to_device(tensors[p + s]) for s in ("in", "x", "dt", "o"))
        self.conv_w = self._to_device(tensors[p + "conv"], f32)
        self.conv_b = self._to_device(tensors[p + "conv.b"], f32)
        self.dt_b = self._to_device(tensors[p + "dt.b"], f32)
        self.A = self._to_device(-torch.exp(tensors[p + "A_log"].to(f32)), f32)
        self.Dp = self._to_device(tensors[p + "D"], f32)

    def forward(self, h, ctx, cache, position=None, residual=None):
        n, dt, dev, I, N, R = h.shape[0], self.runtime.dtype, h.device, self.inner, self.N, self.R
        xz = ops.linear(h, self.w_in, out_dtype=torch.float32)
        x = torch.empty((n, I), dtype=dt, device=dev)
        ops.conv_silu(xz, self.conv_w, self.conv_b, cache.state, self.conv_off, ctx.seq_ids, ctx.cu_q, cache.slots,
                      x, I)
        low = ops.linear(x, self.w_x, out_dtype=torch.float32)
        step_in = torch.empty((n, R), dtype=dt, device=dev)
        ops.rows_act(low[:, :R], step_in)
        dtr = ops.linear(step_in, self.w_dt, out_dtype=torch.float32)
        y = torch.empty((n, I), dtype=dt, device=dev)
        ops.selective_scan(x, xz, low, R, R + N, dtr, self.dt_b, self.A, self.Dp, cache.state, self.conv_off,
                           ctx.cu_q, cache.slots, y, ctx.n_requests, I, N, self.taps,
                           segments=ops.time_segments(ctx, dev))
        return ops.linear(y, self.w_o, out_dtype=torch.float32)
