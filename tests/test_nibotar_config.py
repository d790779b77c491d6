"""Nibotar's configuration, its spec and the plain implementation's own invariants (no GPU)."""
import copy

import pytest
import torch

import wick_b200 as wick
from wick_b200.config.base import ConfigError
from wick_b200.weights.safetensors_io import SafeTensorsDir
from helpers import tmp_root
from plain import nibotar_plain as P

CONFIG = dict(architecture="Nibotar", vocab=97, width=32, norm={"eps": 1e-5}, postln_alpha=1.5, logit_softcap=7.0, layers=[
    dict(type="attention", mixer=dict(heads=2, kv_heads=1, dim=8, vdim=12, scale=0.3, v_mix=False, mask={"size": 6},
                                      rot={"dims": 4, "base": 50.0}), mlp={"kind": "dense", "ff": 40}),
    dict(type="attention", mixer=dict(heads=4, kv_heads=2, dim=8, vdim=6, scale=0.35, v_mix=True, mask={"size": 11},
                                      rot={"dims": 8, "base": 1e4}),
         mlp={"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 4, "top": 2}, "shared": {"ff": 24}}),
    dict(type="attention", mixer=dict(heads=2, kv_heads=2, dim=16, vdim=6, scale=0.25, v_mix=True), mlp=None),
])


def test_config_round_trip_and_registry():
    cfg = wick.config_from_json(CONFIG)
    assert isinstance(cfg, wick.NibotarConfig) and cfg.vocab == 97 and len(cfg.layers) == 3
    assert cfg.layers[0].mixer.mask_size == 6 and cfg.layers[2].mixer.mask_size is None and cfg.layers[2].mixer.rot_dims == 0
    assert cfg.layers[1].mlp.shared_ff == 24 and cfg.layers[2].mlp is None
    assert wick.config_from_json(cfg.to_json()) == cfg
    assert "Nibotar" in wick.architecture_names()


@pytest.mark.parametrize("breakage", [
    lambda c: c.pop("vocab"), lambda c: c["layers"][0]["mixer"].pop("scale"), lambda c: c["layers"][0].update(type="recurrent"),
    lambda c: c["layers"][1]["mlp"].update(kind="sparse"), lambda c: c["layers"][0]["mixer"].update(heads=3, kv_heads=2),
    lambda c: c["layers"][1]["mlp"]["router"].update(top=5), lambda c: c["layers"][2]["mixer"].update(vdim=7),
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), lambda c: c.update(layers=[])])
def test_broken_configs_are_refused(breakage):
    c = copy.deepcopy(CONFIG)
    breakage(c)
    with pytest.raises(ConfigError):
        wick.config_from_json(c)


def test_spec_names_every_tensor_and_marks_the_first_blending_layer():
    cfg = wick.config_from_json(CONFIG)
    spec = wick.get_architecture("Nibotar").build_spec(cfg)
    roles = [L.mixer.params["value_blend"] for L in spec.layers]
    assert roles[0] is None and roles[1]["role"] == "source" and roles[2]["role"] == "blend"
    assert spec.layers[2].ffn.kind == "none" and spec.layers[0].block.params["alpha"] == 1.5
    names = set(wick.Model(spec, torch.float32, "cpu").tensor_table())
    for n in ("embed", "head", "final.norm", "l0.norm1", "l0.norm2", "l0.mix.q", "l0.mix.q.b", "l0.mix.k.norm", "l0.mix.sink",
              "l0.mix.o", "l0.mlp.up", "l0.mlp.down", "l1.mix.vmix", "l1.mlp.e3.gate", "l1.mlp.e0.down", "l1.mlp.table",
              "l1.mlp.shared.up", "l2.mix.vmix", "l2.norm2"):
        assert n in names, n
    assert "l0.mix.vmix" not in names and "l2.mlp.up" not in names


def test_random_model_folder_loads_into_the_plain_model():
    d = wick.write_random_model(wick.config_from_json(CONFIG), 3, tmp_root() + "/nib-cpu", std=0.3)
    st = SafeTensorsDir(d)
    w = {n: st.get(n).tensor() for n in st.names()}
    table = w["l1.mlp.table"]
    assert table.dtype == torch.int32 and int(table.min()) >= 0 and int(table.max()) < 4 and (table[:, 0] != table[:, 1]).all()
    assert "l2.norm2" not in w                              # an optional tensor of a layer without a feed-forward
    toks = list(range(40))
    z, layers = P.forward(CONFIG, w, toks, return_layers=True)
    assert z.shape == (40, 97) and layers.shape == (3, 40, 32) and z.abs().max() <= 7.0
    # causal and cut into blocks: a later token changes nothing before it, and nothing beyond the blocks it shares
    other = list(toks)
    other[25] = 96
    z2 = P.forward(CONFIG, w, other)
    assert torch.equal(z[:25], z2[:25]) and not torch.equal(z[25], z2[25])


def test_plain_mechanisms_on_small_cases():
    vis = P.chunk_visible(7, 3)
    assert vis.int().tolist() == [[1, 0, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0, 0], [0, 0, 0, 1, 0, 0, 0],
                                  [0, 0, 0, 1, 1, 0, 0], [0, 0, 0, 1, 1, 1, 0], [0, 0, 0, 0, 0, 0, 1]]
    assert P.chunk_visible(3, 2, offset=1).int().tolist() == [[1, 0, 0], [0, 1, 0], [0, 1, 1]]
    x = torch.tensor([[[1.0, 0.0, 5.0, 7.0]]]).double()
    r = P.rotate_pairs(x, torch.tensor([1]), 2, 10.0)      # one pair, angle 1; the rest pass
    assert torch.allclose(r[0, 0], torch.tensor([0.5403023, 0.8414710, 5.0, 7.0]).double(), atol=1e-6)
    o = P.sink_softmax_mix(torch.zeros(1, 1, 1).double(), torch.ones(1, 1, dtype=torch.bool), torch.tensor([0.0]).double(),
                           torch.ones(1, 1, 2).double())
    assert torch.allclose(o, torch.full((1, 1, 2), 0.5).double())
