"""Typed configuration of Dunelix, a small decoder whose layers mix tokens either with a minGRU recurrence or with
chunked differential attention, every layer normed by Dynamic Tanh, and a span of whose layers may run several
times in a row with the same weights.

config.json keys (all sizes and all constants that differ between models of the design come from here):

  architecture     "Dunelix"
  vocab, width     vocabulary and width of the residual stream
  residual_mult    what every branch is multiplied by before it joins the stream
  norm.eps         the eps of the unit norms inside the mixers (Dynamic Tanh itself uses none)
  layers[i]        {"type": "mingru" | "attention", "mixer": {...}, "mlp": {"kind": "dense", "ff": n} | null}
    mingru mixer     {"width": n}
    attention mixer  {"heads", "kv_heads", "dim", "vdim", "scale", "diff", "mask": {"size": n} | absent,
                      "rot": {"dims", "base", "scaling": {"factor", "low", "high", "original"} | absent} | absent}
  loop             {"start", "stop", "times"} | absent: layers start .. stop-1 run `times` times in a row, each pass
                   with caches and states of its own; the embedding output is added to the stream before every
                   pass but the first

Tensor names: `embed`, `head`, `final.norm`(`.b`, `.alpha`), and per layer `l<i>.norm1`, `l<i>.norm2`,
`l<i>.mix.*`, `l<i>.mlp.gate|up|down`."""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from .errors import ConfigError
from .registry import register_architecture
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec

# The design sets no limit on positions; this is what the engine's tables are sized for unless a caller asks for less.
DEFAULT_MAX_POSITIONS = 1 << 20


def _need(d: dict, key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f'config.json: {where}: required key "{key}" is missing')
    return d[key]


def _pos_int(d: dict, key: str, where: str) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f'config.json: {where}: "{key}" must be a positive integer, found {v!r}')
    return v


def _number(d: dict, key: str, where: str) -> float:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f'config.json: {where}: "{key}" must be a number, found {v!r}')
    return float(v)


@dataclass(frozen=True)
class DunelixConfig:
    vocab: int
    width: int
    residual_mult: float
    norm_eps: float
    layers: Tuple[Dict[str, Any], ...]
    loop: Optional[Tuple[int, int, int]] = None   # (start, stop, times)
    eos_token_ids: Tuple[int, ...] = ()
    initializer_range: float = 0.06

    architecture = "Dunelix"

    @classmethod
    def from_dict(cls, d: dict) -> "DunelixConfig":
        vocab, width = _pos_int(d, "vocab", "top level"), _pos_int(d, "width", "top level")
        layers_in = _need(d, "layers", "top level")
        if not isinstance(layers_in, list) or not layers_in:
            raise ConfigError('config.json: "layers" must be a non-empty list')
        layers = []
        for i, l in enumerate(layers_in):
            where = f"layers[{i}]"
            kind = _need(l, "type", where)
            mixer = _need(l, "mixer", where)
            if kind == "mingru":
                _pos_int(mixer, "width", where + ".mixer")
            elif kind == "attention":
                mw = where + ".mixer"
                heads, kv = _pos_int(mixer, "heads", mw), _pos_int(mixer, "kv_heads", mw)
                if heads % kv:
                    raise ConfigError(f'config.json: {mw}: "heads" ({heads}) must be a multiple of "kv_heads" ({kv})')
                dim = _pos_int(mixer, "dim", mw)
                _pos_int(mixer, "vdim", mw)
                _number(mixer, "scale", mw)
                _number(mixer, "diff", mw)
                if mixer.get("mask") is not None:
                    _pos_int(mixer["mask"], "size", mw + ".mask")
                rot = mixer.get("rot")
                if rot is not None:
                    dims = _pos_int(rot, "dims", mw + ".rot")
                    if dims % 2 or dims > dim:
                        raise ConfigError(f'config.json: {mw}.rot: "dims" ({dims}) must be even and at most "dim" ({dim})')
                    _number(rot, "base", mw + ".rot")
                    if rot.get("scaling") is not None:
                        for k in ("factor", "low", "high", "original"):
                            _number(rot["scaling"], k, mw + ".rot.scaling")
            else:
                raise ConfigError(f'config.json: {where}: unknown mixer type {kind!r} (known: mingru, attention)')
            mlp = l.get("mlp")
            if mlp is not None:
                if _need(mlp, "kind", where + ".mlp") != "dense":
                    raise ConfigError(f'config.json: {where}.mlp: unknown kind {mlp["kind"]!r} (known: dense)')
                _pos_int(mlp, "ff", where + ".mlp")
            layers.append(copy.deepcopy({"type": kind, "mixer": mixer, "mlp": mlp}))
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            start, stop, times = _need(lp, "start", "loop"), _need(lp, "stop", "loop"), _pos_int(lp, "times", "loop")
            if not (isinstance(start, int) and isinstance(stop, int) and 0 <= start < stop <= len(layers)):
                raise ConfigError(f'config.json: loop: layers {start!r} .. {stop!r} are not a span of the {len(layers)} layers')
            loop = (start, stop, times)
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(vocab=vocab, width=width, residual_mult=_number(d, "residual_mult", "top level"),
                   norm_eps=_number(_need(d, "norm", "top level"), "eps", "norm"), layers=tuple(layers), loop=loop,
                   eos_token_ids=eos_ids, initializer_range=float(d.get("initializer_range", 0.06)))

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "residual_mult": self.residual_mult, "norm": {"eps": self.norm_eps},
             "layers": copy.deepcopy(list(self.layers)), "initializer_range": self.initializer_range}
        if self.loop is not None:
            d["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    def run_order(self) -> List[LayerCall]:
        n = len(self.layers)
        if self.loop is None:
            return [LayerCall(i) for i in range(n)]
        start, stop, times = self.loop
        order = [LayerCall(i) for i in range(start)]
        for rep in range(times):
            order += [LayerCall(i, add_embedding=(rep > 0 and i == start)) for i in range(start, stop)]
        return order + [LayerCall(i) for i in range(stop, n)]

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("dynamic_tanh", {"size": self.width})
        layers = []
        for i, l in enumerate(self.layers):
            m = l["mixer"]
            if l["type"] == "mingru":
                mixer = PartSpec("min_gru", {"hidden_size": self.width, "width": m["width"]})
            else:
                rot = m.get("rot") or {}
                mixer = PartSpec("diff_attention", {
                    "hidden_size": self.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"],
                    "key_dim": m["dim"], "value_dim": m["vdim"], "scale": float(m["scale"]), "diff": float(m["diff"]),
                    "eps": self.norm_eps, "rot_dims": rot.get("dims", 0), "rot_base": float(rot.get("base", 10000.0)),
                    "rot_scaling": rot.get("scaling"), "chunk": (m.get("mask") or {}).get("size")})
            ffn = None
            if l["mlp"] is not None:
                ffn = PartSpec("swiglu", {"hidden_size": self.width, "intermediate_size": l["mlp"]["ff"],
                                          "names": ("gate", "up", "down")})
            layers.append(LayerSpec(prefix=f"l{i}.", norm1=norm, mixer=mixer, norm2=norm if ffn else None, ffn=ffn,
                                    mixer_prefix="mix.", ffn_prefix="mlp.", norm1_name="norm1", norm2_name="norm2",
                                    residual_scale=self.residual_mult))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width,
            max_positions=DEFAULT_MAX_POSITIONS, layers=layers, order=self.run_order(), final_norm=norm,
            embed_name="embed", final_norm_name="final.norm", lm_head_name="head", tie_word_embeddings=False,
            eos_token_ids=self.eos_token_ids, initializer_range=self.initializer_range)


register_architecture(DunelixConfig.architecture, DunelixConfig)
