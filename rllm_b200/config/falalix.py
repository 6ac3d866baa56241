"""Falalix: typed configuration from config.json and the model it describes.

A pre-norm decoder whose layers are listed one by one in config.json (`layers`: each entry names
its mixer `type`, the mixer's sizes and its feed-forward or none).  Two mixers: ``mamba1`` (a
selective scan behind a short causal convolution) and ``parallel`` (a gated sliding-window
attention that keeps the first tokens, beside RWKV-style time mixing, their outputs added with
two constant scales).  Every sublayer's output joins the residual stream multiplied by
`residual_mult`.  `loop` lets the layers start .. stop-1 run `times` times in a row with the same
weights and a cache or state of their own per pass; each pass begins with a junction that mixes
the stream with the embedding output and adds a vector of the pass.  Feed-forwards are dense with
a squared-relu activation.  The model has no position encoding and sets no limit on positions.

config.json keys: architecture, vocab, width, layers[].{type, mixer, mlp}, loop.{start, stop,
times}, norm.eps, residual_mult.  The width of the decay's bottleneck in the time mixing is the
shape of its tensors; `mixer.right.decay_rank` may state it (the random-weights mode needs it).  Tensors: embed, head, final.norm, loop.in, loop.step and
l<i>.{norm1, norm2, mix.*, mlp.*}.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping, Optional

from .base import (ConfigError, LayerSpec, ModelConfig, ModelSpec, PartSpec, RunEntry, coerce, optional, require)


def _section(d, key, where):
    v = d.get(key)
    if not isinstance(v, Mapping):
        raise ConfigError(f"{where}: required section '{key}' is missing")
    return v


@dataclass(frozen=True)
class FalalixConfig(ModelConfig):
    vocab: int
    width: int
    layers: tuple                  # of plain dicts as config.json gives them (validated)
    norm_eps: float
    residual_mult: float
    loop: Optional[Mapping[str, int]] = None     # {start, stop, times} or None
    architecture: str = "Falalix"

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "FalalixConfig":
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
            if typ == "mamba1":
                for k in ("inner", "state", "dt_rank", "conv"):
                    if require(mx, k, int, where + ".mixer") <= 0:
                        raise ConfigError(f"{where}.mixer: '{k}' must be positive")
            elif typ == "parallel":
                left, right = _section(mx, "left", where + ".mixer"), _section(mx, "right", where + ".mixer")
                for k in ("heads", "kv_heads", "dim", "vdim"):
                    if require(left, k, int, where + ".mixer.left") <= 0:
                        raise ConfigError(f"{where}.mixer.left: '{k}' must be positive")
                if left["heads"] % left["kv_heads"]:
                    raise ConfigError(f"{where}.mixer.left: heads {left['heads']} is not a multiple of kv_heads "
                                      f"{left['kv_heads']}")
                require(left, "scale", float, where + ".mixer.left")
                mask = _section(left, "mask", where + ".mixer.left")
                if require(mask, "size", int, where + ".mixer.left.mask") <= 0:
                    raise ConfigError(f"{where}.mixer.left.mask: 'size' must be positive")
                if require(mask, "keep_first", int, where + ".mixer.left.mask") < 0:
                    raise ConfigError(f"{where}.mixer.left.mask: 'keep_first' must not be negative")
                for k in ("heads", "dim"):
                    if require(right, k, int, where + ".mixer.right") <= 0:
                        raise ConfigError(f"{where}.mixer.right: '{k}' must be positive")
                if optional(right, "decay_rank", int, 1, where + ".mixer.right") <= 0:
                    raise ConfigError(f"{where}.mixer.right: 'decay_rank' must be positive")
                require(mx, "left_scale", float, where + ".mixer")
                require(mx, "right_scale", float, where + ".mixer")
            else:
                raise ConfigError(f"{where}: mixer type {typ!r} is not supported (mamba1, parallel)")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping):
                    raise ConfigError(f"{where}.mlp must be an object or null")
                kind = require(mlp, "kind", str, where + ".mlp")
                if kind != "dense":
                    raise ConfigError(f"{where}.mlp: kind {kind!r} is not supported (dense)")
                if require(mlp, "ff", int, where + ".mlp") <= 0:
                    raise ConfigError(f"{where}.mlp: 'ff' must be positive")
            checked.append(copy.deepcopy(dict(layer)))
        loop = d.get("loop")
        if loop is not None:
            if not isinstance(loop, Mapping):
                raise ConfigError("config.json: 'loop' must be an object or null")
            loop = {k: require(loop, k, int, "config.json: loop") for k in ("start", "stop", "times")}
            if not 0 <= loop["start"] <= loop["stop"] <= len(checked) or loop["times"] < 1:
                raise ConfigError(f"config.json: loop {loop} does not fit {len(checked)} layers "
                                  f"(0 <= start <= stop <= layers, times >= 1)")
        norm = _section(d, "norm", "config.json")
        cfg = cls(vocab=require(d, "vocab", int), width=require(d, "width", int), layers=tuple(checked),
                  norm_eps=require(norm, "eps", float, "config.json: norm"),
                  residual_mult=optional(d, "residual_mult", float, 1.0), loop=loop)
        if cfg.vocab <= 0 or cfg.width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        if not cfg.norm_eps > 0:
            raise ConfigError("config.json: norm.eps must be positive")
        return cfg

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps},
             "residual_mult": self.residual_mult}
        if self.loop is not None:
            d["loop"] = dict(self.loop)
        return d

    # ------------------------------------------------------------------ the model as data
    def _mixer(self, i: int, layer) -> PartSpec:
        p, mx, d = f"l{i}.mix.", layer["mixer"], self.width
        if layer["type"] == "mamba1":
            return PartSpec("mamba1", {"hidden_size": d, "inner": mx["inner"], "state": mx["state"],
                                       "dt_rank": mx["dt_rank"], "conv": mx["conv"]}, p)
        left, right = mx["left"], mx["right"]
        attention = PartSpec("gated_attention", {
            "hidden_size": d, "num_heads": left["heads"], "num_kv_heads": left["kv_heads"], "head_dim": left["dim"],
            "v_head_dim": left["vdim"], "bias": True, "qk_norm": "row", "eps": self.norm_eps,
            "window": left["mask"]["size"], "keep_first": left["mask"]["keep_first"], "scale": float(left["scale"]),
            "gate": "sigmoid"}, p + "left.")
        time_mix = PartSpec("rwkv_time_mix", {
            "hidden_size": d, "num_heads": right["heads"], "head_dim": right["dim"], "eps": self.norm_eps,
            "decay_rank": right.get("decay_rank")}, p + "right.")
        return PartSpec("parallel", {"left": attention, "right": time_mix, "left_scale": float(mx["left_scale"]),
                                     "right_scale": float(mx["right_scale"])}, p)

    def model_spec(self) -> ModelSpec:
        d = self.width
        norm = lambda name: PartSpec("rms_norm", {"size": d, "eps": self.norm_eps, "tensor": name})
        layers = []
        for i, layer in enumerate(self.layers):
            mlp = layer.get("mlp")
            ffn = None if mlp is None else PartSpec(
                "dense_act", {"hidden_size": d, "intermediate_size": mlp["ff"], "activation": "relu2"}, f"l{i}.mlp.")
            norms = {"mixer": norm(f"l{i}.norm1")}
            if ffn is not None:
                norms["ffn"] = norm(f"l{i}.norm2")
            layers.append(LayerSpec(block="pre_norm", mixer=self._mixer(i, layer), ffn=ffn, norms=norms,
                                    block_params={"residual_mult": self.residual_mult}))
        n = len(layers)
        junctions = ()
        if self.loop is None:
            order = [RunEntry(i) for i in range(n)]
        else:
            start, stop, times = self.loop["start"], self.loop["stop"], self.loop["times"]
            junctions = (PartSpec("loop_input", {"hidden_size": d, "passes": times, "in": "loop.in",
                                                 "step": "loop.step"}),)
            order = [RunEntry(i) for i in range(start)]
            for t in range(times):          # every pass owns its caches and states: no entry reads another's
                order += [RunEntry(i, junction=0 if i == start else None, junction_arg=t) for i in range(start, stop)]
            order += [RunEntry(i) for i in range(stop, n)]
        return ModelSpec(
            vocab_size=self.vocab, hidden_size=d,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": d, "tensor": "embed"}),
            layers=tuple(layers), run_order=tuple(order), final_norm=norm("final.norm"),
            lm_head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": d, "tied_to": None,
                                         "tensor": "head"}),
            max_position=0, junctions=junctions, residual_scale=self.residual_mult)
