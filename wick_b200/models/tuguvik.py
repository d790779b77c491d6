"""The Tuguvik decoder as a model spec.

Every layer is a pre-norm residual block whose sublayers' results are multiplied by
learned vectors before the sum: x <- x + s1 * mixer(norm1(x)), then x <- x + s2 *
ff(norm2(x)), the norms of the ``tanh`` kind (tanh(alpha x) * w + b).  The mixer is
differential attention (two softmax maps per head over grouped key/value heads, a window
that also keeps the first positions, frequencies scaled by wavelength) or attention through
a cached latent (a window, a sink per head, a gate per head, frequencies scaled by a ramp);
a latent layer may read the cached rows of an earlier one.  The feed-forward is the gated
one, or absent.  After it every layer adds a normed projection of a gated slice of the
token's row in a table that the layers share.  Tensor names: ``embed``, ``side.embed``,
``l<i>.norm1|norm2`` (+ ``.b``, ``.alpha``), ``l<i>.ls1|ls2``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``l<i>.side.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.base import Architecture, register_architecture
from ..config.tuguvik import TuguvikConfig
from ..parts import diff_attention as _diff, latent_attention as _latent, side_input as _side   # register the kinds  # noqa: F401
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, SharedPart

_DIFF_NAMES = dict(q="q", k="k", v="v", o="o", lq1="lq1", lk1="lk1", lq2="lq2", lk2="lk2")
_LATENT_NAMES = dict(dq="dq", dq_norm="dq.norm", uq="uq", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv", sink="sink",
                     gate="g", o="o")
_SIDE_TABLE = "token_side"


def _rotation(rot, head_dim: int, pairing: str, scaling_kind: str):
    if rot is None:
        return None
    scaling = dict(rot.scaling, kind=scaling_kind) if rot.scaling else None
    return PartSpec("rotary_pairs", {"head_dim": head_dim, "dims": rot.dims, "theta": rot.base, "pairing": pairing,
                                     "scaling": scaling})


def build_spec(cfg: TuguvikConfig) -> ModelSpec:
    def norm(optional=False):
        return PartSpec("tanh", {"width": cfg.width, "tensor": "", "names": {"bias": ".b", "alpha": ".alpha"},
                                 "optional": optional})

    layers = []
    for i, L in enumerate(cfg.layers):
        m = L.mixer
        if L.type == "attention":
            mixer = PartSpec("differential_attention", {
                "width": cfg.width, "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim, "v_dim": m.vdim,
                "scale": m.scale, "diff": m.diff, "eps": cfg.norm_eps,
                "position": _rotation(m.rot, m.dim, "halves", "wavelength"),
                "mask": {"size": m.mask_size, "keep_first": m.keep_first} if m.mask_size is not None else None,
                "names": _DIFF_NAMES})
        else:
            mixer = PartSpec("latent_attention", {
                "width": cfg.width, "heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "v_dim": m.vdim,
                "q_rank": m.q_rank, "kv_rank": m.kv_rank, "scale": m.scale, "eps": cfg.norm_eps,
                "position": _rotation(m.rot, m.rot_dim, "neighbours", "ramp"), "window": m.mask_size, "sink": True,
                "gate": True, "own_kv": m.kv_from is None, "names": _LATENT_NAMES})
        ffn = PartSpec("gated_mlp", {"width": cfg.width, "intermediate": L.ff, "activation": "silu",
                                     "names": {"gate": "gate", "up": "up", "down": "down"}}) if L.ff is not None else PartSpec("none")
        side = None
        if cfg.side_dim is not None:
            side = PartSpec("gated_token_rows", {"width": cfg.width, "dim": cfg.side_dim, "offset": i * cfg.side_dim,
                                                 "eps": cfg.norm_eps, "table": _SIDE_TABLE,
                                                 "names": {"gate": "gate", "proj": "proj", "norm": "norm"}})
        layers.append(LayerSpec(
            block=PartSpec("prenorm_residual", {"width": cfg.width, "layer_scale": {"mixer": "ls1", "ffn": "ls2"}}),
            mixer=mixer, mixer_norm=norm(), ffn=ffn, ffn_norm=norm(optional=L.ff is None), prefix=f"l{i}.", side=side,
            names={"mixer": "mix.", "mixer_norm": "norm1", "ffn": "mlp.", "ffn_norm": "norm2", "block": "", "side": "side."}))
    shared = ()
    if cfg.side_dim is not None:
        shared = (SharedPart(_SIDE_TABLE, "embedding", PartSpec("table", {"vocab": cfg.vocab_size,
                             "width": len(cfg.layers) * cfg.side_dim, "tensor": "embed"}), "side."),)
    spec = ModelSpec(
        architecture=cfg.architecture, vocab=cfg.vocab_size, width=cfg.width, max_position=cfg.max_position,
        embedding=PartSpec("table", {"vocab": cfg.vocab_size, "width": cfg.width, "tensor": ""}), embedding_prefix="embed",
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i, L.mixer.kv_from if L.type == "latent_attention" else None)
                       for i, L in enumerate(cfg.layers)),
        final_norm=norm(), final_norm_prefix="final.norm",
        head=PartSpec("linear", {"vocab": cfg.vocab_size, "width": cfg.width, "tied": False, "tensor": ""}), head_prefix="head",
        shared=shared)
    spec.validate()
    return spec


TUGUVIK = register_architecture(Architecture(names=("Tuguvik", "tuguvik"), config_cls=TuguvikConfig, build_spec=build_spec))
