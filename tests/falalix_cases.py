"""Small Falalix configurations and random weights for the tests, made here (not by the package's
random-weights mode), and the glue that runs a schedule through the engine and the plain
implementation.  Every configuration differs from the others in every size; between them they
cover one query head per key/value head and several, value heads smaller and larger than key
heads, no kept first keys and kept keys that span pages, state sizes that are no multiple of the
kernels' lane counts, one tap and several, no loop, a loop from layer 0, one pass and three, a
residual multiplier of 1 and others, layers without a feed-forward.
"""
from __future__ import annotations

import copy
import math

import torch

import plain_falalix


def att(heads, kv, dim, vdim, size, keep, scale=None):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "mask": {"size": size, "keep_first": keep},
            "scale": scale if scale is not None else dim ** -0.5}


def parallel(left, rheads, rdim, rank, ls=0.8, rs=1.1, ff=None):
    return {"type": "parallel", "mixer": {"left": left, "right": {"heads": rheads, "dim": rdim, "decay_rank": rank},
                                          "left_scale": ls, "right_scale": rs},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def mamba(inner, state, rank, conv, ff=None):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": rank, "conv": conv},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(layers, width, vocab, loop=None, mult=1.0, eps=1e-5):
    c = {"architecture": "Falalix", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
         "residual_mult": mult}
    if loop is not None:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    return c


CASES = {
    # one mechanism at a time
    "mamba": config([mamba(80, 5, 3, 4)], width=48, vocab=97),
    "mamba_wide_state": config([mamba(40, 33, 1, 1, ff=56)], width=24, vocab=61, mult=0.5),
    "attention": config([parallel(att(3, 3, 16, 8, 7, 0), 1, 8, 2, ls=1.0, rs=0.0, ff=64)], width=40, vocab=83),
    "attention_kept": config([parallel(att(4, 1, 24, 40, 9, 6), 1, 8, 2, ls=1.0, rs=0.0)], width=56, vocab=71,
                             mult=0.6),
    "time_mix": config([parallel(att(1, 1, 8, 8, 4, 0), 2, 24, 5, ls=0.0, rs=1.0)], width=36, vocab=59, mult=1.3),
    "time_mix_one_head": config([parallel(att(1, 1, 8, 8, 4, 0), 1, 72, 3, ls=0.0, rs=1.0, ff=48)], width=32,
                                vocab=53),
    # key and value heads of one size, 64 or 128: in bfloat16 the tensor-core attention kernels take these
    "heads64": config([parallel(att(4, 2, 64, 64, 19, 3), 2, 32, 4, ff=72)], width=64, vocab=113, mult=0.8),
    "heads128": config([parallel(att(2, 1, 128, 128, 23, 0), 1, 64, 4), mamba(48, 16, 3, 4, ff=64)], width=48,
                       vocab=103, loop=(0, 1, 2), mult=0.5),
    # everything together, loops of several shapes
    "loop3_from_0": config([parallel(att(6, 2, 32, 48, 20, 5), 3, 40, 7, ff=96), mamba(72, 17, 2, 2, ff=80),
                            parallel(att(2, 2, 16, 16, 11, 2), 2, 16, 4), mamba(64, 4, 5, 3)],
                           width=64, vocab=131, loop=(0, 2, 3), mult=0.7),
    "loop1_tail": config([mamba(48, 8, 4, 3, ff=72), parallel(att(4, 2, 16, 24, 13, 3), 2, 32, 6, ff=64),
                          parallel(att(4, 2, 16, 24, 13, 3), 2, 32, 6, ff=64)],
                         width=48, vocab=101, loop=(1, 3, 1), mult=0.4),
    "no_loop": config([parallel(att(2, 1, 64, 64, 16, 1), 4, 8, 8, ff=40), mamba(56, 16, 6, 4)], width=40, vocab=89,
                      mult=0.9),
}


def sharpened(cfg, scale):
    """The same model with every attention's score scale multiplied: rows then hang on a few keys."""
    cfg = copy.deepcopy(cfg)
    for layer in cfg["layers"]:
        if layer["type"] == "parallel":
            layer["mixer"]["left"]["scale"] *= scale
    return cfg


def with_mask(cfg, d_size=0, d_keep=0):
    """The same model with every window `d_size` larger and `d_keep` more kept first keys."""
    cfg = copy.deepcopy(cfg)
    for layer in cfg["layers"]:
        if layer["type"] == "parallel":
            layer["mixer"]["left"]["mask"]["size"] += d_size
            layer["mixer"]["left"]["mask"]["keep_first"] += d_keep
    return cfg


def marked(cfg, w, token, beta=6.0):
    """Layer 0's query bias pointed at the key that `token` makes there, with a large score scale: a
    query that sees such a key puts nearly all its weight on it, one that does not spreads it over
    the others, so whether ONE key is visible decides the row."""
    w = dict(w)
    f = lambda n: w[n].double()
    c = cfg["layers"][0]["mixer"]["left"]
    h = plain_falalix.rms_norm(f("embed")[token], f("l0.norm1"), cfg["norm"]["eps"])
    k = plain_falalix.rms_norm(plain_falalix.lin(f("l0.mix.left.k"), h, f("l0.mix.left.k.b")), f("l0.mix.left.k.norm"), cfg["norm"]["eps"])
    k = k.reshape(c["kv_heads"], c["dim"])
    k = k / k.norm(dim=-1, keepdim=True)
    per = c["heads"] // c["kv_heads"]
    bias = torch.cat([k[hd // per] for hd in range(c["heads"])]) * beta / f("l0.mix.left.q.norm")
    w["l0.mix.left.q.b"] = bias.to(w["l0.mix.left.q.b"].dtype)
    return w


def tensor_shapes(cfg):
    """name -> (shape, kind) from the configuration alone, written out from the model's description."""
    d, out = cfg["width"], {"embed": ((cfg["vocab"], cfg["width"]), "embed"), "final.norm": ((cfg["width"],), "norm"),
                            "head": ((cfg["vocab"], cfg["width"]), "matrix")}
    if cfg.get("loop"):
        out["loop.in"] = ((d, 2 * d), "matrix")
        out["loop.step"] = ((cfg["loop"]["times"], d), "vector")
    for i, layer in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = ((d,), "norm")
        if layer["type"] == "mamba1":
            I, N, R, K = mx["inner"], mx["state"], mx["dt_rank"], mx["conv"]
            out.update({p + "mix.in": ((2 * I, d), "matrix"), p + "mix.conv": ((I, K), "conv"),
                        p + "mix.conv.b": ((I,), "vector"), p + "mix.x": ((R + 2 * N, I), "matrix"),
                        p + "mix.dt": ((I, R), "matrix"), p + "mix.dt.b": ((I,), "dt_bias"),
                        p + "mix.A_log": ((I, N), "a_log"), p + "mix.D": ((I,), "norm"), p + "mix.o": ((d, I), "matrix")})
        else:
            lf, rt = mx["left"], mx["right"]
            wq, wk, wv = lf["heads"] * lf["dim"], lf["kv_heads"] * lf["dim"], lf["kv_heads"] * lf["vdim"]
            q = p + "mix.left."
            out.update({q + "q": ((wq, d), "matrix"), q + "q.b": ((wq,), "vector"), q + "k": ((wk, d), "matrix"),
                        q + "k.b": ((wk,), "vector"), q + "v": ((wv, d), "matrix"), q + "v.b": ((wv,), "vector"),
                        q + "q.norm": ((wq,), "norm"), q + "k.norm": ((wk,), "norm"),
                        q + "g": ((lf["heads"] * lf["vdim"], d), "matrix"), q + "o": ((d, lf["heads"] * lf["vdim"]), "matrix")})
            r, HD, low = p + "mix.right.", rt["heads"] * rt["dim"], rt["decay_rank"]
            out.update({r + "mu." + s: ((d,), "mix") for s in "rkvgw"})
            out.update({r + s: ((HD, d), "matrix") for s in "rkvg"})
            out.update({r + "w1": ((low, d), "matrix"), r + "w2": ((HD, low), "matrix"), r + "w0": ((HD,), "decay"),
                        r + "u": ((rt["heads"], rt["dim"]), "vector"), r + "norm": ((HD,), "norm"),
                        r + "o": ((d, HD), "matrix")})
        if layer.get("mlp"):
            F = layer["mlp"]["ff"]
            out.update({p + "norm2": ((d,), "norm"), p + "mlp.up": ((F, d), "matrix"), p + "mlp.down": ((d, F), "matrix")})
    return out


def make_weights(cfg, seed, dtype=torch.float32):
    """Random tensors of a size at which every mechanism moves the output: activations of order 1,
    decays and step sizes spread over their useful range.  Stored in `dtype`."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    out = {}
    for name, (shape, kind) in tensor_shapes(cfg).items():
        if kind == "matrix":
            t = rnd(*shape) / math.sqrt(shape[1])
        elif kind == "embed":
            t = rnd(*shape)
        elif kind == "norm":
            t = 1.0 + 0.2 * rnd(*shape)
        elif kind == "mix":
            t = torch.rand(*shape, generator=g, dtype=torch.float64)
        elif kind == "conv":
            t = rnd(*shape) * 0.6
        elif kind == "dt_bias":
            t = rnd(*shape) - 1.5
        elif kind == "a_log":
            t = torch.log(0.3 + 3.0 * torch.rand(*shape, generator=g, dtype=torch.float64))
        elif kind == "decay":
            t = rnd(*shape) - 1.0
        else:
            t = 0.4 * rnd(*shape)
        out[name] = t.to(dtype)
    return out


def oracle(cfg, weights, tokens):
    """float64 logits [T, vocab] of the plain implementation from the weights as stored."""
    return plain_falalix.forward(cfg, weights, tokens, dtype=torch.float64)


def build_engine(cfg, weights, dtype, max_tokens, block_size=8, max_requests=4, use_graphs=True, device="cuda:0"):
    from rllm_b200.config import config_from_dict
    from rllm_b200.engine import Engine
    from rllm_b200.models.model import DecoderModel, parse_dtype
    from rllm_b200.parts import Runtime
    model = DecoderModel(config_from_dict(cfg).model_spec(), Runtime(torch.device(device), parse_dtype(dtype)))
    model.load_tensors(dict(weights))
    return Engine(model, block_size=block_size, max_tokens=max_tokens, max_requests=max_requests,
                  use_graphs=use_graphs)


def tokens_for(cfg, n, seed):
    g = torch.Generator().manual_seed(1000 + seed)
    return [int(t) for t in torch.randint(0, cfg["vocab"], (n,), generator=g)]


def row_error(row, ref):
    """max |row - ref| / max |ref| with the rows' means taken off (logits are defined up to a shift)."""
    row, ref = row.double() - row.double().mean(), ref.double() - ref.double().mean()
    return float((row - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
