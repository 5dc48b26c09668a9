"""Typed configuration of Zozenex, a small decoder with a learned position table, RMS norms, and layers whose
mixer is either a retention (linear attention with a fixed decay per head) or two mixers side by side on the same
input: attention without softmax over a sliding window plus pooled blocks of older keys, and gated linear attention
with a decay per key channel.  Feed-forwards are mixtures of small experts with a sigmoid router and a gated shared
expert.

config.json keys (every size and every constant that differs between models of the design comes from here):

  architecture     "Zozenex"
  vocab, width     vocabulary and width of the residual stream
  max_positions    rows of the learned position table
  norm.eps         eps of every RMS norm
  layers[i]        {"type": "retention" | "parallel", "mixer": {...}, "mlp": {...} | null}
    retention mixer  {"heads", "dim", "vdim", "decay": [one number per head]}
    parallel mixer   {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap" | absent,
                               "mask": {"size", "pool" | absent} | absent, "rot": {"dims", "base"} | absent},
                      "right": {"heads", "dim", "vdim", "tau", "rank" | absent}}   (the rank of the decay's projection
                               is the stored tensors' when it is absent; random-weights mode then takes 16)
    mlp              {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "scale"}, "shared": {"ff"} | absent}

Tensor names: `embed`, `pos`, `head`, `final.norm`, and per layer `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`
(`left.*`, `right.*` in a parallel mixer), `l<i>.mlp.router|correction|e<j>.up|e<j>.down|shared.up|shared.down|shared.sg`."""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Tuple

from .dunelix import _need, _number, _pos_int
from .errors import ConfigError
from .registry import register_architecture
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec


def _check_retention(m: dict, where: str) -> None:
    heads = _pos_int(m, "heads", where)
    _pos_int(m, "dim", where)
    _pos_int(m, "vdim", where)
    decay = _need(m, "decay", where)
    if not isinstance(decay, list) or len(decay) != heads or \
            any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
        raise ConfigError(f'config.json: {where}: "decay" must list one number per head ({heads})')


def _check_left(m: dict, where: str) -> None:
    heads, kv = _pos_int(m, "heads", where), _pos_int(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f'config.json: {where}: "heads" ({heads}) must be a multiple of "kv_heads" ({kv})')
    dim, vdim = _pos_int(m, "dim", where), _pos_int(m, "vdim", where)
    _number(m, "scale", where)
    if m.get("softcap") is not None and _number(m, "softcap", where) <= 0:
        raise ConfigError(f'config.json: {where}: "softcap" must be positive')
    mask = m.get("mask")
    if mask is not None:
        _pos_int(mask, "size", where + ".mask")
        if mask.get("pool") is not None:
            _pos_int(mask, "pool", where + ".mask")
    rot = m.get("rot")
    if rot is not None:
        dims = _pos_int(rot, "dims", where + ".rot")
        if dims % 2 or dims > dim:
            raise ConfigError(f'config.json: {where}.rot: "dims" ({dims}) must be even and at most "dim" ({dim})')
        if _number(rot, "base", where + ".rot") <= 0:
            raise ConfigError(f'config.json: {where}.rot: "base" must be positive')
        if vdim % 2:
            raise ConfigError(f'config.json: {where}: "vdim" ({vdim}) must be even, since values are rotated in pairs')


def _check_right(m: dict, where: str) -> None:
    for k in ("heads", "dim", "vdim"):
        _pos_int(m, k, where)
    if _number(m, "tau", where) <= 0:
        raise ConfigError(f'config.json: {where}: "tau" must be positive')
    if m.get("rank") is not None:
        _pos_int(m, "rank", where)


def _check_mlp(mlp: dict, where: str) -> None:
    if _need(mlp, "kind", where) != "moe":
        raise ConfigError(f'config.json: {where}: unknown kind {mlp["kind"]!r} (known: moe)')
    _pos_int(_need(mlp, "expert", where), "ff", where + ".expert")
    r = _need(mlp, "router", where)
    n, top = _pos_int(r, "experts", where + ".router"), _pos_int(r, "top", where + ".router")
    if top > n:
        raise ConfigError(f'config.json: {where}.router: "top" ({top}) exceeds "experts" ({n})')
    _number(r, "scale", where + ".router")
    if mlp.get("shared") is not None:
        _pos_int(mlp["shared"], "ff", where + ".shared")


@dataclass(frozen=True)
class ZozenexConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    layers: Tuple[Dict[str, Any], ...]
    eos_token_ids: Tuple[int, ...] = ()
    initializer_range: float = 0.06

    architecture = "Zozenex"

    @classmethod
    def from_dict(cls, d: dict) -> "ZozenexConfig":
        vocab, width = _pos_int(d, "vocab", "top level"), _pos_int(d, "width", "top level")
        layers_in = _need(d, "layers", "top level")
        if not isinstance(layers_in, list) or not layers_in:
            raise ConfigError('config.json: "layers" must be a non-empty list')
        layers = []
        for i, l in enumerate(layers_in):
            where = f"layers[{i}]"
            kind, mixer = _need(l, "type", where), _need(l, "mixer", where)
            if kind == "retention":
                _check_retention(mixer, where + ".mixer")
            elif kind == "parallel":
                _check_left(_need(mixer, "left", where + ".mixer"), where + ".mixer.left")
                _check_right(_need(mixer, "right", where + ".mixer"), where + ".mixer.right")
            else:
                raise ConfigError(f'config.json: {where}: unknown mixer type {kind!r} (known: retention, parallel)')
            mlp = l.get("mlp")
            if mlp is not None:
                _check_mlp(mlp, where + ".mlp")
            layers.append(copy.deepcopy({"type": kind, "mixer": mixer, "mlp": mlp}))
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(vocab=vocab, width=width, max_positions=_pos_int(d, "max_positions", "top level"),
                   norm_eps=_number(_need(d, "norm", "top level"), "eps", "norm"), layers=tuple(layers),
                   eos_token_ids=eos_ids, initializer_range=float(d.get("initializer_range", 0.06)))

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "max_positions": self.max_positions, "norm": {"eps": self.norm_eps},
             "layers": copy.deepcopy(list(self.layers)), "initializer_range": self.initializer_range}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    def _mixer(self, l: dict) -> PartSpec:
        m, w, eps = l["mixer"], self.width, self.norm_eps
        if l["type"] == "retention":
            return PartSpec("retention", {"hidden_size": w, "num_heads": m["heads"], "key_dim": m["dim"],
                                          "value_dim": m["vdim"], "decay": tuple(float(x) for x in m["decay"]), "eps": eps})
        le, ri = m["left"], m["right"]
        rot, mask = le.get("rot") or {}, le.get("mask") or {}
        left = PartSpec("pooled_window_attention", {
            "hidden_size": w, "num_heads": le["heads"], "num_kv_heads": le["kv_heads"], "key_dim": le["dim"],
            "value_dim": le["vdim"], "scale": float(le["scale"]),
            "softcap": None if le.get("softcap") is None else float(le["softcap"]),
            "window": mask.get("size"), "pool": mask.get("pool"), "rot_dims": rot.get("dims", 0),
            "rot_base": float(rot.get("base", 10000.0)), "rotate_values": bool(rot)})
        right = PartSpec("gated_linear_attention", {
            "hidden_size": w, "num_heads": ri["heads"], "key_dim": ri["dim"], "value_dim": ri["vdim"],
            "tau": float(ri["tau"]), "eps": eps, "rank": ri.get("rank") or 0})
        return PartSpec("side_by_side", {"hidden_size": w, "eps": eps, "weight": 0.5,
                                         "branches": (("left.", left, "left.out"), ("right.", right, "right.out"))})

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("rms_norm", {"size": self.width, "eps": self.norm_eps, "weight_suffix": ""})
        layers: List[LayerSpec] = []
        for i, l in enumerate(self.layers):
            ffn = None
            if l["mlp"] is not None:
                mlp = l["mlp"]
                ffn = PartSpec("routed_experts", {
                    "hidden_size": self.width, "num_experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
                    "expert_size": mlp["expert"]["ff"], "route_scale": float(mlp["router"]["scale"]),
                    "shared_size": None if mlp.get("shared") is None else mlp["shared"]["ff"]})
            layers.append(LayerSpec(prefix=f"l{i}.", norm1=norm, mixer=self._mixer(l), norm2=norm if ffn else None,
                                    ffn=ffn, mixer_prefix="mix.", ffn_prefix="mlp.", norm1_name="norm1",
                                    norm2_name="norm2"))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width,
            max_positions=self.max_positions, layers=layers, order=[LayerCall(i) for i in range(len(layers))],
            final_norm=norm, embed_name="embed", final_norm_name="final.norm", lm_head_name="head",
            tie_word_embeddings=False, eos_token_ids=self.eos_token_ids, initializer_range=self.initializer_range,
            after_embedding=PartSpec("learned_positions", {"size": self.width, "max_positions": self.max_positions}),
            after_embedding_name="pos")


register_architecture(ZozenexConfig.architecture, ZozenexConfig)
