"""Grouped-query attention whose queries and keys are rotated first and normed afterwards, with
capped scores, a chunked mask, and (optionally) the keys as values.

For input rows h [n, d] (H query heads, G key/value heads of size dk; query head i uses key/value
head floor(i / (H / G))):

    q = h Wq^T,  k = h Wk^T,  v = k as projected (`tie_values`), or h Wv^T
    q, k <- rotary on their first rot.dims entries (the position part), then each head divided by
          its root mean square over dk, eps inside the root, no weight (`qk_norm: "unit"`)
    s = (q . k) * scale;  s <- softcap * tanh(s / softcap)               (`softcap` > 0)
    query at position i sees key j iff j <= i and floor(i / chunk) = floor(j / chunk)   (`chunk` > 0;
          runs are counted from position 0 of the sequence, wherever a prompt was cut)
    p = softmax over the visible keys;  out = (heads side by side) Wo^T

Parameters: hidden_size, num_heads, num_kv_heads, head_dim, scale, softcap, chunk, eps, qk_norm
("unit" or None), tie_values.  Tensors <prefix>q, k, o (and v unless the values are tied).  q and k
(and v) are one stacked product.  The cache holds the rotated, normed keys and, as values, the
key heads as projected.  Scores, softmax, angles and norms are float32 in every mode.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Mixer, PagedKVNeed, PartError, register_part


@register_part("mixer", "chunked_attention")
class ChunkedAttention(Mixer):
    CAPTURE_SAFE = True

    def __init__(self, params, prefix, runtime):
        super().__init__(params, prefix, runtime)
        p = params
        self.hidden_size = int(p["hidden_size"])
        self.H, self.G, self.dk = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        self.scale = float(p["scale"])
        self.softcap = float(p.get("softcap", 0.0) or 0.0)
        self.chunk = int(p.get("chunk", 0) or 0)
        self.eps = float(p.get("eps", 1e-6))
        self.qk_norm = p.get("qk_norm")
        self.tie_values = bool(p.get("tie_values", False))
        if self.H % self.G:
            raise PartError(f"chunked_attention: {self.H} heads are not a multiple of {self.G} key/value heads")
        if self.qk_norm not in (None, "unit"):
            raise PartError(f"chunked_attention: qk_norm {self.qk_norm!r} is not supported ('unit' or none)")
        if self.dk > 512:
            raise PartError("chunked_attention: head sizes up to 512")
        self.w_qkv = self.w_o = None

    def cache_need(self):
        return PagedKVNeed(self.G, self.dk)

    def expected_tensors(self):
        d, p = self.hidden_size, self.prefix
        t = {p + "q": ((self.H * self.dk, d), "matrix"), p + "k": ((self.G * self.dk, d), "matrix"),
             p + "o": ((d, self.H * self.dk), "matrix")}
        if not self.tie_values:
            t[p + "v"] = ((self.G * self.dk, d), "matrix")
        return t

    def load(self, tensors):
        p, dt = self.prefix, self.runtime.dtype
        names = "qk" if self.tie_values else "qkv"
        self.w_qkv = self._to_device(torch.cat([tensors[p + n].to(dt) for n in names], 0))
        self.w_o = self._to_device(tensors[p + "o"])

    def forward(self, h, ctx, cache, position=None, residual=None):
        n, dt, dev = h.shape[0], self.runtime.dtype, h.device
        rows = ops.linear(h, self.w_qkv, out_dtype=torch.float32)               # [q | k (| v)]
        q = torch.empty((n, self.H * self.dk), dtype=dt, device=dev)
        rot = min(position.dims, self.dk) if position is not None else 0
        ops.rope_unitnorm_store(rows, position.angles(ctx) if rot else None, rot, position.mult if rot else 1.0,
                                cache.slots, q, cache.k, cache.v, self.H, self.G, self.dk, cache.block_size, self.eps,
                                unit_norm=self.qk_norm == "unit", v_tied=self.tie_values, write_kv=cache.write)
        attn = torch.empty_like(q)
        ops.paged_attention(q, cache.k, cache.v, attn, ctx, cache.block_table, self.H, self.G, self.dk,
                            cache.block_size, self.scale, chunk=self.chunk, softcap=self.softcap)
        return ops.linear(attn, self.w_o, out_dtype=torch.float32)
