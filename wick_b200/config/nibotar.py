"""Configuration of the Nibotar decoder, from its ``config.json``.

``config.json`` lists the layers one by one; every layer has a mixer (of type
``attention``) with its own sizes and constants and a feed-forward (``mlp``: dense, a
mixture of experts, or none).  Model-wide: ``vocab``, ``width``, ``norm.eps``,
``postln_alpha`` (the factor of the stream in every residual sum) and ``logit_softcap``.
Nothing here has a default that stands for a size: what the file does not give is an error,
except the options a layer may leave out (``mask``, ``rot``, ``v_mix``, ``shared``, the cap).
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any, Dict, Mapping, Optional, Tuple

from .base import ConfigError, ModelConfig


def _num(j: Mapping[str, Any], key: str, where: str, kind=float, positive: bool = True):
    v = j.get(key) if isinstance(j, Mapping) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (kind is int and int(v) != v) or not math.isfinite(v):
        raise ConfigError(f"config.json: {where}{key} is missing or no number")
    if positive and v <= 0:
        raise ConfigError(f"config.json: {where}{key} must be positive")
    return kind(v)


@dataclasses.dataclass(frozen=True)
class NibotarAttention:
    heads: int
    kv_heads: int
    dim: int                               # size of a query / key head
    vdim: int                              # size of a value head
    scale: float
    mask_size: Optional[int] = None        # positions per block of the mask; None: every earlier key
    rot_dims: int = 0                      # rotated elements per head; 0: no rotation
    rot_base: float = 10000.0
    v_mix: bool = False

    @classmethod
    def from_json(cls, j: Mapping[str, Any], where: str) -> "NibotarAttention":
        if not isinstance(j, Mapping):
            raise ConfigError(f"config.json: {where}mixer is missing")
        mask, rot = j.get("mask"), j.get("rot")
        a = cls(heads=_num(j, "heads", where, int), kv_heads=_num(j, "kv_heads", where, int), dim=_num(j, "dim", where, int),
                vdim=_num(j, "vdim", where, int), scale=_num(j, "scale", where),
                mask_size=_num(mask, "size", where + "mask.", int) if mask is not None else None,
                rot_dims=_num(rot, "dims", where + "rot.", int) if rot is not None else 0,
                rot_base=_num(rot, "base", where + "rot.") if rot is not None else 10000.0,
                v_mix=bool(j.get("v_mix", False)))
        if a.heads % a.kv_heads != 0:
            raise ConfigError(f"config.json: {where}heads must be a multiple of kv_heads")
        if a.rot_dims % 2 != 0 or a.rot_dims > a.dim:
            raise ConfigError(f"config.json: {where}rot.dims must be even and at most dim")
        return a

    def to_json(self) -> Dict[str, Any]:
        j: Dict[str, Any] = dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim, scale=self.scale,
                                 v_mix=self.v_mix)
        if self.mask_size is not None:
            j["mask"] = {"size": self.mask_size}
        if self.rot_dims:
            j["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        return j


@dataclasses.dataclass(frozen=True)
class NibotarMLP:
    kind: str                              # "dense" or "moe"
    ff: int                                # inner size (of every expert, for "moe")
    experts: int = 0
    top: int = 0
    shared_ff: Optional[int] = None        # inner size of the expert every token uses; None: there is none

    @classmethod
    def from_json(cls, j: Mapping[str, Any], where: str) -> "NibotarMLP":
        kind = j.get("kind")
        if kind == "dense":
            return cls("dense", _num(j, "ff", where, int))
        if kind == "moe":
            shared = j.get("shared")
            m = cls("moe", _num(j.get("expert"), "ff", where + "expert.", int),
                    experts=_num(j.get("router"), "experts", where + "router.", int),
                    top=_num(j.get("router"), "top", where + "router.", int),
                    shared_ff=_num(shared, "ff", where + "shared.", int) if shared is not None else None)
            if m.top > m.experts:
                raise ConfigError(f"config.json: {where}router.top is larger than router.experts")
            return m
        raise ConfigError(f"config.json: {where}kind {kind!r} is not known (dense, moe)")

    def to_json(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        j: Dict[str, Any] = {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff is not None:
            j["shared"] = {"ff": self.shared_ff}
        return j


@dataclasses.dataclass(frozen=True)
class NibotarLayer:
    mixer: NibotarAttention
    mlp: Optional[NibotarMLP]
    type: str = "attention"


@dataclasses.dataclass(frozen=True)
class NibotarConfig(ModelConfig):
    vocab_size: int = 0
    width: int = 0
    layers: Tuple[NibotarLayer, ...] = ()
    norm_eps: float = 1e-6
    postln_alpha: float = 1.0
    logit_softcap: Optional[float] = None

    @property
    def vocab(self) -> int:
        return self.vocab_size

    @property
    def max_position(self) -> int:
        return 1 << 30                     # (the design names no limit; positions are 32-bit integers)

    def param_count(self, tied: Optional[bool] = None) -> int:
        """Number of parameters (every expert counted)."""
        n = 2 * self.vocab_size * self.width + self.width
        for L in self.layers:
            m = L.mixer
            q, k, v = m.heads * m.dim, m.kv_heads * m.dim, m.kv_heads * m.vdim
            n += (q + k + v) * (self.width + 1) + q + k + m.heads + 1 + self.width * m.heads * m.vdim + self.width
            if L.mlp is None:
                continue
            n += self.width
            if L.mlp.kind == "dense":
                n += 2 * self.width * L.mlp.ff
            else:
                n += 3 * self.width * (L.mlp.experts * L.mlp.ff + (L.mlp.shared_ff or 0)) + self.vocab_size * L.mlp.top
        return n

    @classmethod
    def from_json(cls, j: Mapping[str, Any], architecture: str) -> "NibotarConfig":
        raw = j.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: layers is missing or empty")
        layers = []
        for i, L in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(L, Mapping) or L.get("type") != "attention":
                raise ConfigError(f"config.json: {where}type {L.get('type') if isinstance(L, Mapping) else L!r} is not "
                                  f"known (attention)")
            mlp = L.get("mlp")
            layers.append(NibotarLayer(NibotarAttention.from_json(L.get("mixer"), where + "mixer."),
                                       NibotarMLP.from_json(mlp, where + "mlp.") if mlp is not None else None))
        cap = j.get("logit_softcap")
        cfg = cls(architecture=architecture, vocab_size=_num(j, "vocab", "", int), width=_num(j, "width", "", int),
                  layers=tuple(layers), norm_eps=_num(j.get("norm"), "eps", "norm."),
                  postln_alpha=_num(j, "postln_alpha", ""),
                  logit_softcap=_num(j, "logit_softcap", "") if cap is not None else None)
        mixing = [L.mixer for L in cfg.layers if L.mixer.v_mix]
        if any((m.kv_heads, m.vdim) != (mixing[0].kv_heads, mixing[0].vdim) for m in mixing):
            raise ConfigError("config.json: layers that mix values must agree in kv_heads and vdim")
        return cfg

    def to_json(self) -> Dict[str, Any]:
        j: Dict[str, Any] = {
            "architecture": self.architecture,
            "layers": [{"type": L.type, "mixer": L.mixer.to_json(), "mlp": L.mlp.to_json() if L.mlp is not None else None}
                       for L in self.layers],
            "norm": {"eps": self.norm_eps}, "postln_alpha": self.postln_alpha, "vocab": self.vocab_size, "width": self.width}
        if self.logit_softcap is not None:
            j["logit_softcap"] = self.logit_softcap
        return j
