"""Junctions: parts between two run entries that rewrite the residual stream.

``loop_input``: where a pass through a repeated run of layers begins, the stream is mixed with the
embedding output x0 of the same tokens and shifted by a vector of the pass:

    x <- [x | x0] Win^T + step[pass]            Win [d, 2d] (the stream's columns first), step [passes, d]

Parameters: hidden_size, passes, `in` and `step` (tensor names).
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Junction, register_part


@register_part("junction", "loop_input")
class LoopInput(Junction):
    CAPTURE_SAFE = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.d, self.passes = int(params["hidden_size"]), int(params["passes"])
        self.in_name, self.step_name = params["in"], params["step"]
        self.w_in = self.step = None

    def expected_tensors(self):
        return {self.in_name: ((self.d, 2 * self.d), "matrix"), self.step_name: ((self.passes, self.d), "bias")}

    def load(self, tensors):
        self.w_in = self._to_device(tensors[self.in_name])
        self.step = self._to_device(tensors[self.step_name], torch.float32)

    def forward(self, x, x0, delta, delta_scale, arg):
        n = x.shape[0]
        both = torch.empty((n, 2 * self.d), dtype=self.runtime.dtype, device=x.device)
        ops.cat2_cast(x, x0, both, delta=delta, delta_scale=delta_scale)
        out = ops.linear(both, self.w_in, out_dtype=torch.float32)
        return ops.rows_act(out, out, bias=self.step[arg])
