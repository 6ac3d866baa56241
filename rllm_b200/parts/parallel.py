"""Two mixers side by side on the same input: out = left_scale * left(h) + right_scale * right(h).

Parameters: left, right (PartSpec of registered mixer kinds, with their own prefixes), left_scale,
right_scale.  Each side keeps what it needs in the cache under its own need; this part's need is
the tuple of both and its cache view the tuple of their views.
"""
from __future__ import annotations

from ..csrc import ops
from .base import Mixer, build_part, register_part


@register_part("mixer", "parallel")
class ParallelMixer(Mixer):
    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        self.left = build_part("mixer", params["left"], runtime)
        self.right = build_part("mixer", params["right"], runtime)
        self.left_scale, self.right_scale = float(params["left_scale"]), float(params["right_scale"])
        self.CAPTURE_SAFE = bool(getattr(self.left, "CAPTURE_SAFE", False) and getattr(self.right, "CAPTURE_SAFE", False))

    def cache_need(self):
        return (self.left.cache_need(), self.right.cache_need())

    def expected_tensors(self):
        return {**self.left.expected_tensors(), **self.right.expected_tensors()}

    def load(self, tensors):
        self.left.load(tensors)
        self.right.load(tensors)

    def forward(self, h, ctx, cache, position=None, residual=None):
        a = self.left.forward(h, ctx, cache[0], position)
        b = self.right.forward(h, ctx, cache[1], position)
        return ops.axpby(self.left_scale, a, self.right_scale, b, a)
