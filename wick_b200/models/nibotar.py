"""The Nibotar decoder as a model spec.

Every layer is a post-norm residual block: x <- norm1(alpha x + mixer(x)), then
x <- norm2(alpha x + ff(x)), the norms RMS norms whose weights are stored around zero.  The
mixer is attention with projection biases, an RMS norm of q and k over the whole projection,
a rotation of neighbouring pairs over the first ``rot.dims`` elements of each head, a mask of
blocks of positions, a sink per head, and (in the layers that say so) values blended with
those of the first such layer.  The feed-forward is a plain one with a squared ReLU, or
gated experts chosen by a table of token ids plus an expert shared by all tokens, or absent.
The logits go through a soft cap.  Tensor names: ``embed``, ``l<i>.norm1|norm2``,
``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.base import Architecture, register_architecture
from ..config.nibotar import NibotarConfig
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

_MIX_NAMES = dict(q="q", k="k", v="v", o="o", q_bias="q.b", k_bias="k.b", v_bias="v.b", q_norm="q.norm", k_norm="k.norm",
                  sink="sink", blend="vmix")
_EXPERT_NAMES = dict(gate="gate", up="up", down="down")


def build_spec(cfg: NibotarConfig) -> ModelSpec:
    def norm(optional=False):
        return PartSpec("rms", {"width": cfg.width, "eps": cfg.norm_eps, "offset": 1.0, "tensor": "", "optional": optional})

    layers = []
    seen_mixing = False
    for i, L in enumerate(cfg.layers):
        m = L.mixer
        blend = None
        if m.v_mix:
            blend = {"role": "blend" if seen_mixing else "source", "group": "first"}
            seen_mixing = True
        position = PartSpec("rotary_pairs", {"head_dim": m.dim, "dims": m.rot_dims, "theta": m.rot_base,
                                             "pairing": "neighbours"}) if m.rot_dims else None
        mixer = PartSpec("attention", {
            "width": cfg.width, "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim, "v_dim": m.vdim, "bias": True,
            "scale": m.scale, "qk_norm": "projection", "eps": cfg.norm_eps, "position": position,
            "mask": {"kind": "block", "size": m.mask_size} if m.mask_size is not None else None, "sink": True,
            "value_blend": blend, "names": _MIX_NAMES})
        if L.mlp is None:
            ffn = PartSpec("none")
        elif L.mlp.kind == "dense":
            ffn = PartSpec("mlp", {"width": cfg.width, "intermediate": L.mlp.ff, "activation": "relu2",
                                   "names": {"up": "up", "down": "down"}})
        else:
            shared = PartSpec("gated_mlp", {"width": cfg.width, "intermediate": L.mlp.shared_ff, "activation": "silu",
                                            "names": _EXPERT_NAMES}) if L.mlp.shared_ff is not None else None
            ffn = PartSpec("table_moe", {"width": cfg.width, "vocab": cfg.vocab_size, "experts": L.mlp.experts,
                                         "top": L.mlp.top, "intermediate": L.mlp.ff, "shared": shared,
                                         "names": dict(_EXPERT_NAMES, expert="e{i}.", table="table", shared="shared.")})
        layers.append(LayerSpec(block=PartSpec("postnorm_residual", {"alpha": cfg.postln_alpha}), mixer=mixer,
                                mixer_norm=norm(), ffn=ffn, ffn_norm=norm(optional=L.mlp is None), prefix=f"l{i}.",
                                names={"mixer": "mix.", "mixer_norm": "norm1", "ffn": "mlp.", "ffn_norm": "norm2"}))
    spec = ModelSpec(
        architecture=cfg.architecture, vocab=cfg.vocab_size, width=cfg.width, max_position=cfg.max_position,
        embedding=PartSpec("table", {"vocab": cfg.vocab_size, "width": cfg.width, "tensor": ""}), embedding_prefix="embed",
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=norm(), final_norm_prefix="final.norm",
        head=PartSpec("linear", {"vocab": cfg.vocab_size, "width": cfg.width, "tied": False, "tensor": "",
                                 "soft_cap": cfg.logit_softcap}),
        head_prefix="head",
        # (a checkpoint may carry a blend factor for a layer that blends nothing)
        ignore_tensors=("l*.mix.vmix",))
    spec.validate()
    return spec


NIBOTAR = register_architecture(Architecture(names=("Nibotar", "nibotar"), config_cls=NibotarConfig, build_spec=build_spec))
