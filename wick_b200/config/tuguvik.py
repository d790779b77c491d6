"""Configuration of the Tuguvik decoder, from its ``config.json``.

``config.json`` lists the layers one by one.  Every layer names its mixer by ``type``
(``attention``: differential attention over grouped key/value heads; ``latent_attention``:
attention whose keys and values are made from a cached latent), gives the mixer's sizes
and constants under ``mixer`` and its feed-forward under ``mlp`` (``dense``, or null).
Model-wide: ``vocab``, ``width``, ``norm.eps`` and ``token_side.dim`` (the size of the
per-layer token input; absent: the layers have none).  Nothing here has a default that
stands for a size: what the file does not give is an error, except the options a layer
may leave out (``mask``, ``mask.keep_first``, ``rot``, ``rot.scaling``, ``kv_from``).
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any, Dict, Mapping, Optional, Tuple

from .base import ConfigError, ModelConfig


def _num(j: Any, key: str, where: str, kind=float, positive: bool = True):
    v = j.get(key) if isinstance(j, Mapping) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (kind is int and int(v) != v) or not math.isfinite(v):
        raise ConfigError(f"config.json: {where}{key} is missing or no number")
    if positive and v <= 0:
        raise ConfigError(f"config.json: {where}{key} must be positive")
    return kind(v)


@dataclasses.dataclass(frozen=True)
class Rotation:
    """Rotated elements per vector, the base of the frequencies, and the frequency scaling:
    a tuple of (key, number) pairs as ``config.json`` gives them, or () for none."""
    dims: int
    base: float
    scaling: Tuple[Tuple[str, float], ...] = ()

    @classmethod
    def from_json(cls, j: Any, where: str, keys: Tuple[str, ...]) -> Optional["Rotation"]:
        if j is None:
            return None
        sc = j.get("scaling") if isinstance(j, Mapping) else None
        r = cls(_num(j, "dims", where, int), _num(j, "base", where),
                tuple((k, _num(sc, k, where + "scaling.")) for k in keys) if sc is not None else ())
        if r.dims % 2 != 0:
            raise ConfigError(f"config.json: {where}dims must be even")
        return r

    def to_json(self) -> Dict[str, Any]:
        j: Dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling:
            j["scaling"] = dict(self.scaling)
        return j


def _mask(j: Any, where: str) -> Tuple[Optional[int], int]:
    if j is None:
        return None, 0
    keep = j.get("keep_first") if isinstance(j, Mapping) else None
    return _num(j, "size", where, int), (_num(j, "keep_first", where, int, positive=False) if keep is not None else 0)


@dataclasses.dataclass(frozen=True)
class DifferentialAttention:
    heads: int
    kv_heads: int
    dim: int                               # size of one map's query / key vector (a head holds two)
    vdim: int
    scale: float
    diff: float                            # the constant in lambda and in the result's factor 1 - diff
    mask_size: Optional[int] = None        # None: every earlier key
    keep_first: int = 0
    rot: Optional[Rotation] = None

    SCALING_KEYS = ("factor", "low", "high", "original")

    @classmethod
    def from_json(cls, j: Any, where: str) -> "DifferentialAttention":
        if not isinstance(j, Mapping):
            raise ConfigError(f"config.json: {where[:-1]} is missing")
        size, keep = _mask(j.get("mask"), where + "mask.")
        a = cls(heads=_num(j, "heads", where, int), kv_heads=_num(j, "kv_heads", where, int), dim=_num(j, "dim", where, int),
                vdim=_num(j, "vdim", where, int), scale=_num(j, "scale", where), diff=_num(j, "diff", where, positive=False),
                mask_size=size, keep_first=keep, rot=Rotation.from_json(j.get("rot"), where + "rot.", cls.SCALING_KEYS))
        if a.heads % a.kv_heads != 0:
            raise ConfigError(f"config.json: {where}heads must be a multiple of kv_heads")
        if a.rot is not None and a.rot.dims > a.dim:
            raise ConfigError(f"config.json: {where}rot.dims must be at most dim")
        return a

    def to_json(self) -> Dict[str, Any]:
        j: Dict[str, Any] = dict(heads=self.heads, kv_heads=self.kv_heads, dim=self.dim, vdim=self.vdim, scale=self.scale,
                                 diff=self.diff)
        if self.mask_size is not None:
            j["mask"] = {"size": self.mask_size, "keep_first": self.keep_first}
        if self.rot is not None:
            j["rot"] = self.rot.to_json()
        return j


@dataclasses.dataclass(frozen=True)
class LatentAttention:
    heads: int
    dim: int                               # unrotated query / key elements per head
    rot_dim: int                           # rotated ones (the key's are shared by the heads)
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    mask_size: Optional[int] = None
    rot: Optional[Rotation] = None
    kv_from: Optional[int] = None          # the layer whose cached latent this one reads; None: its own

    SCALING_KEYS = ("factor", "original", "fast", "slow")

    @classmethod
    def from_json(cls, j: Any, where: str) -> "LatentAttention":
        if not isinstance(j, Mapping):
            raise ConfigError(f"config.json: {where[:-1]} is missing")
        size, _ = _mask(j.get("mask"), where + "mask.")
        src = j.get("kv_from")
        a = cls(heads=_num(j, "heads", where, int), dim=_num(j, "dim", where, int), rot_dim=_num(j, "rot_dim", where, int),
                vdim=_num(j, "vdim", where, int), q_rank=_num(j, "q_rank", where, int), kv_rank=_num(j, "kv_rank", where, int),
                scale=_num(j, "scale", where), mask_size=size,
                rot=Rotation.from_json(j.get("rot"), where + "rot.", cls.SCALING_KEYS),
                kv_from=_num(j, "kv_from", where, int, positive=False) if src is not None else None)
        if a.rot is not None and a.rot.dims != a.rot_dim:
            raise ConfigError(f"config.json: {where}rot.dims must equal rot_dim")
        return a

    def to_json(self) -> Dict[str, Any]:
        j: Dict[str, Any] = dict(heads=self.heads, dim=self.dim, rot_dim=self.rot_dim, vdim=self.vdim, q_rank=self.q_rank,
                                 kv_rank=self.kv_rank, scale=self.scale)
        if self.mask_size is not None:
            j["mask"] = {"size": self.mask_size}
        if self.rot is not None:
            j["rot"] = self.rot.to_json()
        if self.kv_from is not None:
            j["kv_from"] = self.kv_from
        return j


MIXERS = {"attention": DifferentialAttention, "latent_attention": LatentAttention}


@dataclasses.dataclass(frozen=True)
class TuguvikLayer:
    type: str
    mixer: Any
    ff: Optional[int]                      # inner size of the gated feed-forward; None: the layer has none


@dataclasses.dataclass(frozen=True)
class TuguvikConfig(ModelConfig):
    vocab_size: int = 0
    width: int = 0
    layers: Tuple[TuguvikLayer, ...] = ()
    norm_eps: float = 1e-6
    side_dim: Optional[int] = None

    @property
    def vocab(self) -> int:
        return self.vocab_size

    @property
    def max_position(self) -> int:
        return 1 << 30                     # (the design names no limit; positions are 32-bit integers)

    def param_count(self, tied: Optional[bool] = None) -> int:
        D, n = self.width, 2 * self.vocab_size * self.width + 2 * self.width + 1
        for L in self.layers:
            m = L.mixer
            n += (2 * D + 1) + D
            if L.type == "attention":
                n += D * (2 * m.dim * (m.heads + m.kv_heads) + m.kv_heads * m.vdim + m.heads * m.vdim) + 4 * m.dim
            else:
                n += D * m.q_rank + m.q_rank + m.q_rank * m.heads * (m.dim + m.rot_dim) + m.kv_rank * m.heads * (m.dim + m.vdim)
                n += m.heads + m.heads * D + D * m.heads * m.vdim
                if m.kv_from is None:
                    n += D * (m.kv_rank + m.rot_dim) + m.kv_rank
            if L.ff is not None:
                n += 3 * D * L.ff + D + (2 * D + 1)
            if self.side_dim:
                n += self.vocab_size * self.side_dim + 2 * D * self.side_dim + D
        return n

    @classmethod
    def from_json(cls, j: Mapping[str, Any], architecture: str) -> "TuguvikConfig":
        raw = j.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: layers is missing or empty")
        layers = []
        for i, L in enumerate(raw):
            where = f"layers[{i}]."
            kind = L.get("type") if isinstance(L, Mapping) else None
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}type {kind!r} is not known ({', '.join(sorted(MIXERS))})")
            mlp = L.get("mlp")
            if mlp is not None and (not isinstance(mlp, Mapping) or mlp.get("kind") != "dense"):
                raise ConfigError(f"config.json: {where}mlp.kind {mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r} "
                                  f"is not known (dense)")
            layers.append(TuguvikLayer(kind, MIXERS[kind].from_json(L.get("mixer"), where + "mixer."),
                                       _num(mlp, "ff", where + "mlp.", int) if mlp is not None else None))
        for i, L in enumerate(layers):
            src = L.mixer.kv_from if L.type == "latent_attention" else None
            if src is None:
                continue
            S = layers[src] if 0 <= src < i else None
            if S is None or S.type != "latent_attention" or S.mixer.kv_from is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from names layer {src}, which is no earlier layer "
                                  f"with a latent of its own")
            if (S.mixer.kv_rank, S.mixer.rot_dim, S.mixer.rot) != (L.mixer.kv_rank, L.mixer.rot_dim, L.mixer.rot):
                raise ConfigError(f"config.json: layers[{i}] and layers[{src}] must agree in kv_rank, rot_dim and rot")
        side = j.get("token_side")
        return cls(architecture=architecture, vocab_size=_num(j, "vocab", "", int), width=_num(j, "width", "", int),
                   layers=tuple(layers), norm_eps=_num(j.get("norm"), "eps", "norm."),
                   side_dim=_num(side, "dim", "token_side.", int) if side is not None else None)

    def to_json(self) -> Dict[str, Any]:
        j: Dict[str, Any] = {
            "architecture": self.architecture,
            "layers": [{"type": L.type, "mixer": L.mixer.to_json(),
                        "mlp": {"kind": "dense", "ff": L.ff} if L.ff is not None else None} for L in self.layers],
            "norm": {"eps": self.norm_eps}, "vocab": self.vocab_size, "width": self.width}
        if self.side_dim is not None:
            j["token_side"] = {"dim": self.side_dim}
        return j
