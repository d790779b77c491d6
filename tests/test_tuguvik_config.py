"""Tuguvik's configuration, its spec, the frequency scalings and the plain implementation's own invariants (no GPU)."""
import copy
import math

import pytest
import torch

import wick_b200 as wick
from wick_b200.config.base import ConfigError
from wick_b200.parts.attention import scaled_frequencies
from wick_b200.weights.safetensors_io import SafeTensorsDir
from helpers import tmp_root
from plain import tuguvik_plain as P

RAMP = {"factor": 5.0, "fast": 4.0, "slow": 0.5, "original": 100}
CONFIG = dict(architecture="Tuguvik", vocab=97, width=32, norm={"eps": 1e-5}, token_side={"dim": 6}, layers=[
    dict(type="latent_attention", mixer=dict(heads=2, dim=8, rot_dim=4, vdim=6, q_rank=12, kv_rank=10, scale=0.3, mask={"size": 7},
                                             rot={"dims": 4, "base": 50.0, "scaling": RAMP}), mlp={"kind": "dense", "ff": 40}),
    dict(type="attention", mixer=dict(heads=4, kv_heads=2, dim=6, vdim=10, scale=0.35, diff=0.3, mask={"size": 11, "keep_first": 2},
                                      rot={"dims": 4, "base": 1e4, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 32}}),
         mlp={"kind": "dense", "ff": 24}),
    dict(type="latent_attention", mixer=dict(heads=3, dim=4, rot_dim=4, vdim=8, q_rank=8, kv_rank=10, scale=0.25, mask={"size": 5},
                                             rot={"dims": 4, "base": 50.0, "scaling": RAMP}, kv_from=0), mlp=None),
])


def test_config_round_trip_and_registry():
    cfg = wick.config_from_json(CONFIG)
    assert isinstance(cfg, wick.TuguvikConfig) and cfg.vocab == 97 and len(cfg.layers) == 3 and cfg.side_dim == 6
    assert cfg.layers[0].mixer.mask_size == 7 and cfg.layers[1].mixer.keep_first == 2 and cfg.layers[2].mixer.kv_from == 0
    assert cfg.layers[2].ff is None and cfg.layers[1].ff == 24
    assert wick.config_from_json(cfg.to_json()) == cfg
    assert "Tuguvik" in wick.architecture_names()
    bare = copy.deepcopy(CONFIG)
    bare.pop("token_side")
    bare["layers"][1]["mixer"].pop("mask")
    bare["layers"][1]["mixer"]["rot"].pop("scaling")
    c2 = wick.config_from_json(bare)
    assert c2.side_dim is None and c2.layers[1].mixer.mask_size is None and c2.layers[1].mixer.rot.scaling == ()
    assert wick.config_from_json(c2.to_json()) == c2


@pytest.mark.parametrize("breakage", [
    lambda c: c.pop("vocab"), lambda c: c["layers"][0]["mixer"].pop("scale"), lambda c: c["layers"][0].update(type="recurrent"),
    lambda c: c["layers"][1]["mlp"].update(kind="moe"), lambda c: c["layers"][1]["mixer"].update(heads=3, kv_heads=2),
    lambda c: c["layers"][1]["mixer"].pop("diff"), lambda c: c["layers"][2]["mixer"].update(kv_from=1),
    lambda c: c["layers"][2]["mixer"].update(kv_from=2), lambda c: c["layers"][2]["mixer"].update(kv_rank=12),
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=2), lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("fast"),
    lambda c: c["layers"][1]["mixer"]["rot"].update(dims=8), lambda c: c.update(layers=[])])
def test_broken_configs_are_refused(breakage):
    c = copy.deepcopy(CONFIG)
    breakage(c)
    with pytest.raises(ConfigError):
        wick.config_from_json(c)


def test_spec_names_every_tensor_and_schedules_the_shared_cache():
    cfg = wick.config_from_json(CONFIG)
    spec = wick.get_architecture("Tuguvik").build_spec(cfg)
    assert [e.read_cache_of for e in spec.schedule] == [None, None, 0]
    assert spec.layers[2].ffn.kind == "none" and spec.layers[2].mixer.params["own_kv"] is False
    assert spec.layers[1].side.params["offset"] == 6 and spec.shared[0].spec.params["width"] == 18
    m = wick.Model(spec, torch.float32, "cpu")
    names = set(m.tensor_table())
    for n in ("embed", "side.embed", "head", "final.norm", "final.norm.b", "final.norm.alpha", "l0.norm1", "l0.norm1.alpha", "l0.ls1",
              "l0.ls2", "l0.mix.dq", "l0.mix.dq.norm", "l0.mix.uq", "l0.mix.dkv", "l0.mix.dkv.norm", "l0.mix.uk", "l0.mix.uv",
              "l0.mix.sink", "l0.mix.g", "l0.mix.o", "l0.mlp.gate", "l0.side.gate", "l0.side.proj", "l0.side.norm", "l1.mix.q",
              "l1.mix.lq1", "l1.mix.lk2", "l2.mix.uk", "l2.ls1", "l2.norm2", "l2.ls2"):
        assert n in names, n
    assert "l2.mix.dkv" not in names and "l2.mix.dkv.norm" not in names and "l2.mlp.up" not in names
    needs = m.cache_needs()
    assert needs[0].kind == "paged_rows" and needs[0].shape == (14,) and needs[2] is None
    assert needs[1].kind == "paged_kv" and (needs[1].kv_heads, needs[1].head_dim, needs[1].v_head_dim) == (2, 12, 10)
    n_params = sum(math.prod(ts.shape) for name, ts in m.tensor_table().items()
                   if not (ts.optional and name.startswith("l2.")))
    assert cfg.param_count() == n_params


def test_frequency_scalings_agree_with_the_plain_ones():
    for dims, base, sc in ((8, 1e4, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}), (16, 5e5, {"factor": 8.0, "low": 1.0,
                           "high": 4.0, "original": 8192}), (6, 100.0, None)):
        got, amp = scaled_frequencies(dims, base, dict(sc, kind="wavelength") if sc else None)
        assert amp == 1.0 and got == pytest.approx(P.frequencies_by_wavelength(dims, base, sc), rel=1e-12)
    got, _ = scaled_frequencies(8, 1e4, {"kind": "wavelength", "factor": 4.0, "low": 1.0, "high": 4.0, "original": 64})
    f = [1e4 ** (-i / 4) for i in range(4)]
    assert got[0] == f[0] and got[2] == f[2] / 4 and got[3] == f[3] / 4 and f[1] / 4 < got[1] < f[1]      # kept, blended, divided
    for dims, base, sc in ((8, 5e4, {"factor": 3.0, "fast": 8.0, "slow": 1.0, "original": 40}), (32, 1e4, {"factor": 40.0, "fast": 32.0,
                           "slow": 1.0, "original": 4096}), (4, 50.0, RAMP), (4, 50.0, None)):
        got, amp = scaled_frequencies(dims, base, dict(sc, kind="ramp") if sc else None)
        ref, ref_amp = P.frequencies_by_ramp(dims, base, sc)
        assert got == pytest.approx(ref, rel=1e-12) and amp == pytest.approx(ref_amp, rel=1e-12)
    got, amp = scaled_frequencies(32, 1e4, {"kind": "ramp", "factor": 40.0, "fast": 32.0, "slow": 1.0, "original": 4096})
    f = [1e4 ** (-i / 16) for i in range(16)]
    assert got[0] == f[0] and got[15] == pytest.approx(f[15] / 40) and amp == pytest.approx(0.1 * math.log(40.0) + 1)


def test_random_model_folder_loads_into_the_plain_model():
    d = wick.write_random_model(wick.config_from_json(CONFIG), 3, tmp_root() + "/tug-cpu", std=0.3)
    st = SafeTensorsDir(d)
    w = {n: st.get(n).tensor() for n in st.names()}
    assert "l2.norm2" not in w and "l2.ls2" not in w and w["side.embed"].shape == (97, 18) and w["l0.norm1.alpha"].shape == ()
    toks = list(range(40))
    z, layers = P.forward(CONFIG, w, toks, return_layers=True)
    assert z.shape == (40, 97) and layers.shape == (3, 40, 32) and torch.isfinite(z).all()
    # causal, and the windows' reach is bounded: windows of 7 and 11 (+ 2 kept) reach 6 + 10 positions back; the third layer's
    # keys are the FIRST layer's cached rows, which depend on their own token alone, so it adds nothing to the reach
    other = list(toks)
    other[10] = 96
    z2 = P.forward(CONFIG, w, other)
    assert torch.equal(z[:10], z2[:10]) and not torch.equal(z[10], z2[10])
    assert not torch.equal(z[26], z2[26]) and torch.equal(z[27:], z2[27:])
    kept = list(toks)
    kept[1] = 96                                            # a kept first token is seen from everywhere
    assert not torch.equal(z[39], P.forward(CONFIG, w, kept)[39])


def test_plain_mechanisms_on_small_cases():
    vis = P.window_visible(6, 2, 1)
    assert vis.int().tolist() == [[1, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0], [1, 0, 1, 1, 0, 0], [1, 0, 0, 1, 1, 0],
                                  [1, 0, 0, 0, 1, 1]]
    assert P.window_visible(3, None).int().tolist() == [[1, 0, 0], [1, 1, 0], [1, 1, 1]]
    x = torch.tensor([[[1.0, 0.0, 5.0, 7.0]]]).double()
    r = P.turn_neighbours(x[..., :2], torch.tensor([1]), [1.0], 2.0)
    assert torch.allclose(r[0, 0], 2 * torch.tensor([0.5403023, 0.8414710]).double(), atol=1e-6)
    r = P.turn_halves(x, torch.tensor([1]), [1.0, 0.0])      # pairs (0, 2) and (1, 3); the second does not turn
    assert torch.allclose(r[0, 0], torch.tensor([0.5403023 - 5 * 0.8414710, 0.0, 5 * 0.5403023 + 0.8414710, 7.0]).double(), atol=1e-6)
    w = P.softmax_visible(torch.zeros(1, 1, 1).double(), torch.ones(1, 1, dtype=torch.bool), torch.tensor([0.0]).double())
    assert torch.allclose(w, torch.full((1, 1, 1), 0.5).double())
    assert torch.allclose(P.tanh_norm(torch.tensor([0.5]), torch.tensor([2.0]), torch.tensor([1.0]), torch.tensor(2.0)),
                          torch.tensor([2 * math.tanh(1.0) + 1.0]))
    assert abs(P.gelu_tanh(torch.tensor(1.0)).item() - 0.841192) < 1e-5
