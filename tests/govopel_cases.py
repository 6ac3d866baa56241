"""Small Govopel configurations and random weights for the tests, made here (not by the package's
random-weights mode), and the glue that runs a schedule through the engine and the plain
implementation (tests/plain_govopel.py).  The configurations differ from one another in every size;
between them they cover one query head per key/value head and several, rotation over a part of the
head and over all of it, with and without frequency scaling, runs of 1 position, runs longer than
the sequence and no mask at all, with and without capped scores and logits, layers without a
feed-forward, either mixer first, sizes that are no multiple of 8, and head sizes of 64 and 128.
"""
from __future__ import annotations

import copy
import math

import torch

import plain_govopel


def rot(dims, base=10000.0, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def att(heads, kv, dim, rdims, size, scale=None, softcap=None, base=10000.0, scaling=None, ff=None, limit=1.5):
    mx = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "rot": rot(rdims, base, scaling),
          "scale": scale if scale is not None else 3.0 / math.sqrt(dim)}
    if size:
        mx["mask"] = {"size": size}
    if softcap:
        mx["softcap"] = softcap
    return {"type": "attention", "mixer": mx, "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


def lat(heads, dim, rdim, vdim, kv_rank, q_rank, scale=None, base=5000.0, scaling=None, ff=None, limit=2.5):
    mx = {"heads": heads, "dim": dim, "rot_dim": rdim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
          "rot": rot(rdim, base, scaling), "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rdim)}
    return {"type": "latent_attention", "mixer": mx,
            "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


def config(layers, width, vocab, eps=1e-5, logit_softcap=None):
    c = {"architecture": "Govopel", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps}}
    if logit_softcap:
        c["logit_softcap"] = logit_softcap
    return c


CASES = {
    # one mechanism at a time
    "chunked": config([att(3, 3, 16, 8, 7, softcap=5.0, ff=56)], width=40, vocab=83, logit_softcap=20.0),
    "chunked_scaled": config([att(4, 2, 24, 24, 13, scaling=(4.0, 16, 8.0, 2.0))], width=36, vocab=71, eps=3e-6),
    "runs_of_one": config([att(2, 1, 12, 4, 1, ff=20, limit=0.7)], width=20, vocab=53),
    "no_mask": config([att(6, 2, 10, 6, 0, softcap=30.0, ff=44)], width=28, vocab=61, logit_softcap=8.0),
    "latent": config([lat(3, 8, 4, 12, 20, 24, ff=48)], width=32, vocab=67),
    "latent_scaled": config([lat(2, 40, 16, 24, 56, 40, scaling=(8.0, 32, 16.0, 1.0))], width=48, vocab=97,
                            logit_softcap=15.0),
    "latent_odd": config([lat(5, 6, 2, 5, 9, 7, ff=30)], width=22, vocab=59, eps=1e-6),
    # head sizes 64 and 128 (the tensor-core attention kernels in bfloat16)
    "heads64": config([att(8, 2, 64, 48, 19, softcap=40.0, ff=72)], width=64, vocab=113, logit_softcap=25.0),
    "heads128": config([att(2, 2, 128, 64, 37, scaling=(2.0, 64, 16.0, 1.0)), lat(2, 16, 8, 16, 32, 24, ff=40)],
                       width=48, vocab=103),
    # everything together, either mixer first
    "stack": config([lat(4, 16, 8, 24, 40, 48, ff=96), att(6, 2, 32, 16, 11, softcap=12.0, ff=80),
                     att(2, 2, 16, 16, 29, scaling=(2.0, 24, 8.0, 1.0)), lat(2, 24, 12, 8, 16, 32, ff=64, limit=1.0)],
                    width=64, vocab=131, logit_softcap=30.0),
    "stack_attention_first": config([att(4, 4, 8, 2, 5, ff=40), lat(3, 12, 6, 10, 24, 16),
                                     att(3, 1, 20, 10, 64, softcap=50.0, ff=36)], width=40, vocab=89),
}


def tensor_shapes(cfg):
    """name -> (shape, kind) from the configuration alone, written out from the model's description."""
    d = cfg["width"]
    out = {"embed": ((cfg["vocab"], d), "embed"), "embed.norm": ((d,), "norm"), "final.norm": ((d,), "norm")}
    for i, layer in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = ((d,), "norm")
        if layer["type"] == "attention":
            out.update({p + "mix.q": ((mx["heads"] * mx["dim"], d), "matrix"),
                        p + "mix.k": ((mx["kv_heads"] * mx["dim"], d), "matrix"),
                        p + "mix.o": ((d, mx["heads"] * mx["dim"]), "matrix")})
        else:
            H, dq, r, dv, rank, qr = (mx[k] for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"))
            out.update({p + "mix.dq": ((qr, d), "matrix"), p + "mix.dq.norm": ((qr,), "norm"),
                        p + "mix.uq": ((H * (dq + r), qr), "matrix"), p + "mix.dkv": ((rank + r, d), "matrix"),
                        p + "mix.dkv.norm": ((rank,), "norm"), p + "mix.uk": ((H * dq, rank), "matrix"),
                        p + "mix.uv": ((H * dv, rank), "matrix"), p + "mix.o": ((d, H * dv), "matrix")})
        if layer.get("mlp"):
            F = layer["mlp"]["ff"]
            out.update({p + "norm2": ((d,), "norm"), p + "mlp.gate": ((F, d), "matrix"),
                        p + "mlp.up": ((F, d), "matrix"), p + "mlp.down": ((d, F), "matrix")})
    return out


def make_weights(cfg, seed, dtype=torch.float32, gain=1.3):
    """Random tensors at which every mechanism moves the output (activations of order 1, so that the
    clamps of the feed-forward and the caps bite now and then).  Stored in `dtype`."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    out = {}
    for name, (shape, kind) in tensor_shapes(cfg).items():
        if kind == "matrix":
            t = rnd(*shape) * gain / math.sqrt(shape[1])
        elif kind == "embed":
            t = rnd(*shape)
        else:
            t = 1.0 + 0.2 * rnd(*shape)
        out[name] = t.to(dtype)
    return out


def oracle(cfg, weights, tokens, layers_out=None):
    """float64 logits [T, vocab] of the plain implementation from the weights as stored."""
    return plain_govopel.forward(cfg, weights, tokens, layers_out)


def sharpened(cfg, factor):
    cfg = copy.deepcopy(cfg)
    for layer in cfg["layers"]:
        layer["mixer"]["scale"] *= factor
    return cfg


def with_chunk(cfg, delta):
    """The same model with every run of the chunked mask `delta` positions longer."""
    cfg = copy.deepcopy(cfg)
    for layer in cfg["layers"]:
        if layer["type"] == "attention" and layer["mixer"].get("mask"):
            layer["mixer"]["mask"]["size"] += delta
    return cfg


def _normed_embedding(cfg, w, token):
    f = lambda n: w[n].double()
    return plain_govopel.rms_norm(f("embed")[token], f("embed.norm"), cfg["norm"]["eps"])


def _redirect(cfg, w, asker, target):
    """The map R on the stream with R x(asker) = x(target), identity across x(asker): a projection
    W R then gives the asker what W gives the target and leaves the other tokens nearly alone."""
    xa, xb = _normed_embedding(cfg, w, asker), _normed_embedding(cfg, w, target)
    return torch.eye(cfg["width"], dtype=torch.float64) + torch.outer(xb - xa, xa) / (xa @ xa)


def marked_attention(cfg, w, asker, target):
    """Layer 0 (an attention layer): every query head asks with its group's key projection, and the
    token `asker` asks as if it were `target`.  With a sharp scale, a row of `asker` hangs on the key
    of a `target` token when one is visible (on the part of the head that is not rotated; the rotated
    part adds or takes a little, by distance) and is spread over the other keys when none is."""
    w = dict(w)
    mx = cfg["layers"][0]["mixer"]
    H, G, d = mx["heads"], mx["kv_heads"], mx["dim"]
    k = w["l0.mix.k"].double().view(G, d, -1)
    q = torch.stack([k[h // (H // G)] for h in range(H)]).reshape(H * d, -1) @ _redirect(cfg, w, asker, target)
    w["l0.mix.q"] = q.to(w["l0.mix.q"].dtype)
    return w


def marked_latent(cfg, w, asker, target):
    """Layer 0 (a latent attention layer with q_rank == kv_rank): the queries' latent is the keys'
    latent and their plain parts go through the keys' up-projection, `asker` asking as `target`; the
    rotated parts are silenced.  A row of `asker` then hangs on the key of a visible `target`."""
    w = dict(w)
    mx = cfg["layers"][0]["mixer"]
    H, dq, r, rank = mx["heads"], mx["dim"], mx["rot_dim"], mx["kv_rank"]
    assert mx["q_rank"] == rank
    w["l0.mix.dq"] = (w["l0.mix.dkv"].double()[:rank] @ _redirect(cfg, w, asker, target)).to(w["l0.mix.dq"].dtype)
    w["l0.mix.dq.norm"] = w["l0.mix.dkv.norm"].clone()
    uq = torch.zeros((H, dq + r, rank), dtype=torch.float64)
    uq[:, :dq] = w["l0.mix.uk"].double().view(H, dq, rank)
    w["l0.mix.uq"] = uq.reshape(H * (dq + r), rank).to(w["l0.mix.uq"].dtype)
    return w


def build_engine(cfg, weights, dtype, max_tokens, block_size=8, max_requests=4, use_graphs=True, device="cuda:0"):
    from rllm_b200.config import config_from_dict
    from rllm_b200.engine import Engine
    from rllm_b200.models.model import DecoderModel, parse_dtype
    from rllm_b200.parts import Runtime
    model = DecoderModel(config_from_dict(cfg).model_spec(), Runtime(torch.device(device), parse_dtype(dtype)))
    model.load_tensors(dict(weights))
    return Engine(model, block_size=block_size, max_tokens=max_tokens, max_requests=max_requests,
                  use_graphs=use_graphs)


def tokens_for(cfg, n, seed, avoid=()):
    g = torch.Generator().manual_seed(2000 + seed)
    free = [t for t in range(cfg["vocab"]) if t not in avoid]
    return [free[int(i)] for i in torch.randint(0, len(free), (n,), generator=g)]


def row_error(row, ref):
    """max |row - ref| / max |ref| with the rows' means taken off (logits are defined up to a shift)."""
    row, ref = row.double() - row.double().mean(), ref.double() - ref.double().mean()
    return float((row - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
