"""Govopel: typed configuration from config.json and the model it describes.

A decoder whose layers are listed one by one in config.json (`layers`: each entry names its mixer
`type`, the mixer's sizes and its feed-forward, or none).  The norms stand on the sublayers'
OUTPUTS: x <- x + norm1(mixer(x)), x <- x + norm2(ff(x)); the sublayers read the stream itself.
The embedding is followed by an RMSNorm of its own, the LM head is the embedding table, and the
logits are capped by `logit_softcap`.

Mixers: ``attention`` (grouped heads; the values are the keys as projected; rotary encoding on the
first rot.dims entries of a head with optional YaRN-style scaling; queries and keys divided by
their root mean square after the rotation; capped scores; a chunked mask of mask.size positions)
and ``latent_attention`` (queries and keys/values through low-rank latents, one rotated key part
shared by the heads, causal).  Feed-forwards: ``dense``, a gated unit with clamped branches,
g = min(gate, limit), u = clamp(up, +-limit), y = g sigmoid(1.702 g) (u + 1).

config.json keys: architecture, vocab, width, layers[].{type, mixer, mlp}, norm.eps,
logit_softcap.  Tensors: embed, embed.norm, final.norm and l<i>.{norm1, norm2, mix.*, mlp.*}.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping

from .base import ConfigError, LayerSpec, ModelConfig, ModelSpec, PartSpec, RunEntry, optional, require

GLU_ALPHA = 1.702          # the design fixes these two
GLU_SHIFT = 1.0


def _section(d, key, where):
    v = d.get(key)
    if not isinstance(v, Mapping):
        raise ConfigError(f"{where}: required section '{key}' is missing")
    return v


def _positive(d, keys, where):
    for k in keys:
        if require(d, k, int, where) <= 0:
            raise ConfigError(f"{where}: '{k}' must be positive")


def _check_rot(rot, where):
    if require(rot, "dims", int, where) <= 0 or rot["dims"] % 2:
        raise ConfigError(f"{where}: 'dims' must be positive and even")
    if not require(rot, "base", float, where) > 1.0:
        raise ConfigError(f"{where}: 'base' must be larger than 1")
    sc = rot.get("scaling")
    if sc is not None:
        if not isinstance(sc, Mapping):
            raise ConfigError(f"{where}.scaling must be an object or null")
        for k in ("factor", "original", "fast", "slow"):
            if not require(sc, k, float, where + ".scaling") > 0:
                raise ConfigError(f"{where}.scaling: '{k}' must be positive")


@dataclass(frozen=True)
class GovopelConfig(ModelConfig):
    vocab: int
    width: int
    layers: tuple                  # of plain dicts as config.json gives them (validated)
    norm_eps: float
    logit_softcap: float = 0.0
    architecture: str = "Govopel"

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "GovopelConfig":
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: required key 'layers' must be a non-empty list")
        checked = []
        for i, layer in enumerate(layers):
            where = f"config.json: layers[{i}]"
            if not isinstance(layer, Mapping):
                raise ConfigError(f"{where} must be an object")
            typ = require(layer, "type", str, where)
            mx = _section(layer, "mixer", where)
            mw = where + ".mixer"
            require(mx, "scale", float, mw)
            rot = _section(mx, "rot", mw)
            _check_rot(rot, mw + ".rot")
            if optional(mx, "softcap", float, 0.0, mw) < 0:
                raise ConfigError(f"{mw}: 'softcap' must not be negative")
            if typ == "attention":
                _positive(mx, ("heads", "kv_heads", "dim"), mw)
                if mx["heads"] % mx["kv_heads"]:
                    raise ConfigError(f"{mw}: heads {mx['heads']} is not a multiple of kv_heads {mx['kv_heads']}")
                if optional(mx, "vdim", int, mx["dim"], mw) != mx["dim"]:
                    raise ConfigError(f"{mw}: 'vdim' must equal 'dim' (the values are the keys)")
                if rot["dims"] > mx["dim"]:
                    raise ConfigError(f"{mw}.rot: 'dims' {rot['dims']} exceeds the head size {mx['dim']}")
                mask = mx.get("mask")
                if mask is not None:
                    if not isinstance(mask, Mapping):
                        raise ConfigError(f"{mw}.mask must be an object or null")
                    if require(mask, "size", int, mw + ".mask") <= 0:
                        raise ConfigError(f"{mw}.mask: 'size' must be positive")
            elif typ == "latent_attention":
                _positive(mx, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"), mw)
                if rot["dims"] != mx["rot_dim"]:
                    raise ConfigError(f"{mw}.rot: 'dims' {rot['dims']} must equal rot_dim {mx['rot_dim']}")
            else:
                raise ConfigError(f"{where}: mixer type {typ!r} is not supported (attention, latent_attention)")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping):
                    raise ConfigError(f"{where}.mlp must be an object or null")
                kind = require(mlp, "kind", str, where + ".mlp")
                if kind != "dense":
                    raise ConfigError(f"{where}.mlp: kind {kind!r} is not supported (dense)")
                if require(mlp, "ff", int, where + ".mlp") <= 0:
                    raise ConfigError(f"{where}.mlp: 'ff' must be positive")
                if not require(mlp, "limit", float, where + ".mlp") > 0:
                    raise ConfigError(f"{where}.mlp: 'limit' must be positive")
            checked.append(copy.deepcopy(dict(layer)))
        norm = _section(d, "norm", "config.json")
        cfg = cls(vocab=require(d, "vocab", int), width=require(d, "width", int), layers=tuple(checked),
                  norm_eps=require(norm, "eps", float, "config.json: norm"),
                  logit_softcap=optional(d, "logit_softcap", float, 0.0))
        if cfg.vocab <= 0 or cfg.width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        if not cfg.norm_eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        if cfg.logit_softcap < 0:
            raise ConfigError("config.json: 'logit_softcap' must not be negative")
        return cfg

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps}}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        return d

    # ------------------------------------------------------------------ the model as data
    def _mixer(self, i: int, layer) -> PartSpec:
        p, mx, d = f"l{i}.mix.", layer["mixer"], self.width
        softcap = float(mx.get("softcap") or 0.0)
        if layer["type"] == "attention":
            return PartSpec("chunked_attention", {
                "hidden_size": d, "num_heads": mx["heads"], "num_kv_heads": mx["kv_heads"], "head_dim": mx["dim"],
                "scale": float(mx["scale"]), "softcap": softcap, "chunk": int((mx.get("mask") or {}).get("size", 0)),
                "eps": self.norm_eps, "qk_norm": "unit", "tie_values": True}, p)
        return PartSpec("latent_attention", {
            "hidden_size": d, "num_heads": mx["heads"], "head_dim": mx["dim"], "rot_dim": mx["rot_dim"],
            "v_head_dim": mx["vdim"], "kv_rank": mx["kv_rank"], "q_rank": mx["q_rank"], "eps": self.norm_eps,
            "scale": float(mx["scale"]), "softcap": softcap}, p)

    @staticmethod
    def _position(layer) -> PartSpec:
        rot = layer["mixer"]["rot"]
        sc = rot.get("scaling")
        return PartSpec("rotary_scaled", {"dims": rot["dims"], "base": float(rot["base"]),
                                          "scaling": None if sc is None else {k: float(v) for k, v in sc.items()}})

    def model_spec(self) -> ModelSpec:
        d = self.width
        norm = lambda name: PartSpec("rms_norm", {"size": d, "eps": self.norm_eps, "tensor": name})
        layers = []
        for i, layer in enumerate(self.layers):
            mlp = layer.get("mlp")
            ffn = None if mlp is None else PartSpec(
                "clamped_glu", {"hidden_size": d, "intermediate_size": mlp["ff"], "limit": float(mlp["limit"]),
                                "alpha": GLU_ALPHA, "shift": GLU_SHIFT}, f"l{i}.mlp.")
            norms = {"mixer": norm(f"l{i}.norm1")}
            if ffn is not None:
                norms["ffn"] = norm(f"l{i}.norm2")
            layers.append(LayerSpec(block="post_norm", mixer=self._mixer(i, layer), ffn=ffn, norms=norms,
                                    position=self._position(layer)))
        return ModelSpec(
            vocab_size=self.vocab, hidden_size=d,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": d, "tensor": "embed",
                                             "norm": "embed.norm", "norm_eps": self.norm_eps}),
            layers=tuple(layers), run_order=tuple(RunEntry(i) for i in range(len(layers))),
            final_norm=norm("final.norm"),
            lm_head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": d, "tied_to": "embed",
                                         "tensor": "head", "softcap": self.logit_softcap}),
            max_position=0)
