"""The Nibotar decoder and its mechanisms against the plain implementation in
``tests/plain/nibotar_plain.py``: every mechanism alone through its kernel, then whole
models through the engine (prompts, decoding, portions, batches, reused pages, mask edges,
generation).  The configurations differ from each other in every size and option,
and include the values that make mechanisms vanish (alpha 1, no mask, no rotation, one kv
head, as many kv heads as heads, top = 1, top = experts, no shared expert, no feed-forward)."""
import copy
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

import wick_b200 as wick  # noqa: E402
from wick_b200 import ops  # noqa: E402
from wick_b200.engine.batch import BatchLayout, StepBatch, fill_host  # noqa: E402
from wick_b200.weights.safetensors_io import SafeTensorsDir  # noqa: E402
from helpers import poison_free_pages, random_tokens, tmp_root  # noqa: E402
from plain import nibotar_plain as P  # noqa: E402

PAGE = 64
DEV = "cuda"


def attn(heads, kv, dim, vdim, scale, mask=None, rot=None, v_mix=False):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale, v_mix=v_mix)
    if mask is not None:
        m["mask"] = {"size": mask}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return m


def moe(experts, top, ff, shared=None):
    j = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        j["shared"] = {"ff": shared}
    return j


CONFIG_NA = dict(architecture="Nibotar", vocab=211, width=64, norm={"eps": 1e-5}, postln_alpha=1.7, logit_softcap=9.0, layers=[
    dict(type="attention", mixer=attn(4, 4, 16, 24, 0.31, mask=20, rot=(8, 100.0)), mlp={"kind": "dense", "ff": 96}),
    dict(type="attention", mixer=attn(4, 2, 16, 24, 0.25, mask=33, rot=(16, 1e4), v_mix=True), mlp=moe(5, 3, 40)),
    dict(type="attention", mixer=attn(2, 2, 24, 24, 0.2, v_mix=True), mlp=None),
    dict(type="attention", mixer=attn(6, 2, 8, 24, 0.4, mask=5, rot=(8, 3e5), v_mix=True), mlp=moe(3, 1, 24, shared=56)),
])
CONFIG_NB = dict(architecture="Nibotar", vocab=130, width=72, norm={"eps": 1e-6}, postln_alpha=1.0, layers=[
    dict(type="attention", mixer=attn(6, 1, 20, 12, 0.22, mask=64, rot=(10, 5e5), v_mix=True), mlp=moe(2, 2, 52, shared=20)),
    dict(type="attention", mixer=attn(3, 3, 12, 24, 0.3, mask=100, rot=(12, 1e3)), mlp={"kind": "dense", "ff": 44}),
    dict(type="attention", mixer=attn(6, 1, 20, 12, 0.22, mask=9, v_mix=True), mlp={"kind": "dense", "ff": 120}),
])
# sizes at which the bfloat16 path takes its tensor-core kernels
CONFIG_NC = dict(architecture="Nibotar", vocab=300, width=128, norm={"eps": 1e-5}, postln_alpha=2.0, logit_softcap=20.0, layers=[
    dict(type="attention", mixer=attn(4, 2, 64, 64, 0.125, mask=96, rot=(64, 1e4), v_mix=True), mlp={"kind": "dense", "ff": 256}),
    dict(type="attention", mixer=attn(4, 2, 64, 64, 0.125, mask=130, rot=(32, 1e4), v_mix=True), mlp=moe(4, 2, 64, shared=128)),
])
CONFIGS = {"NA": CONFIG_NA, "NB": CONFIG_NB, "NC": CONFIG_NC}
_models = {}


def model(name, seed=5, std=0.3):
    key = (name, seed, std)
    if key not in _models:
        d = os.path.join(tmp_root(), f"nib-{name}-{seed}-{std}")
        wick.write_random_model(wick.config_from_json(CONFIGS[name]), seed, d, std=std)
        st = SafeTensorsDir(d)
        _models[key] = (d, {n: st.get(n).tensor() for n in st.names()})
    return _models[key]


def engine(name, dtype, max_tokens=1024, **kw):
    return wick.Engine.from_dir(model(name)[0], dtype=dtype, max_tokens=max_tokens, **kw)


def plain(name, tokens):
    return P.forward(CONFIGS[name], model(name)[1], list(tokens)).float()


def close(got, ref, dtype, what=""):
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    assert got.shape == ref.shape, f"{what}: {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite"
    scale = max(1.0, ref.abs().max().item())
    worst = (got - ref).abs().max().item()
    tol = 2e-4 if dtype == "float32" else 6e-2
    if worst > tol * scale:
        row = int((got - ref).abs().reshape(got.shape[0], -1).max(-1).values.argmax())
        raise AssertionError(f"{what}: differs by {worst:.3e} (scale {scale:.3g}), worst row {row}")


DTYPES = ["float32", "bfloat16"]


# ---------------------------------------------------------------------------
# mechanisms alone
def one_seq_batch(n_new, start=0, pages=None):
    """A step of one sequence: ``n_new`` tokens after ``start`` cached ones."""
    n_pages = (start + n_new + PAGE - 1) // PAGE
    pages = pages if pages is not None else list(range(1, n_pages + 1))
    lay = BatchLayout(1, n_new, len(pages), 0)
    host = np.zeros(lay.size, dtype=np.int32)
    fill_host(lay, host, tokens=[[0] * n_new], starts=[start], slots=[1], pages=[pages], want=[[]])
    return StepBatch(lay, torch.from_numpy(host).to(DEV), q_lens=[n_new], starts=[start])


def test_norm_after_the_sum():
    g = torch.Generator().manual_seed(1)
    for width, rows in ((48, 9), (100, 9), (257, 9), (100, 600), (2052, 515)):
        x = torch.randn(rows, width, generator=g)
        d = torch.randn(3, rows, width, generator=g)
        w = 0.1 * torch.randn(width, generator=g)
        ref = P.norm_one_plus(1.3 * x.double() + d.double().sum(0), w.double(), 1e-5)
        xd = x.to(DEV)
        out = ops.scaled_add_rmsnorm(xd, d.to(DEV), 1.3, (1.0 + w).to(DEV), 1e-5, torch.bfloat16)
        close(xd, ref, "float32", f"stream, width {width}")
        assert torch.equal(out.float(), xd.to(torch.bfloat16).float())
        xd = x.to(DEV)
        assert ops.scaled_add_rmsnorm(xd, None, 1.0, (1.0 + w).to(DEV), 1e-5, torch.float32) is xd
        close(xd, P.norm_one_plus(x.double(), w.double(), 1e-5), "float32", "no partial sums")


def test_squared_relu_and_soft_cap():
    g = torch.Generator().manual_seed(2)
    a = torch.randn(1000, generator=g)
    for dt in (torch.float32, torch.bfloat16):
        ad = a.to(dt)
        close(ops.relu_squared_(ad.to(DEV)), torch.relu(ad.double()) ** 2, "float32" if dt == torch.float32 else "bfloat16")
    z = 40 * torch.randn(3, 77, generator=g)
    close(ops.soft_cap_(z.to(DEV), 12.0), P.softcap(z.double(), 12.0), "float32")


@pytest.mark.parametrize("H,G,d,e,span,rot,pairing", [(4, 2, 16, 24, "projection", 8, "neighbours"), (3, 3, 20, 12, "head", 20, "halves"),
                                                      (6, 1, 8, 8, None, 0, "neighbours")])
def test_projection_finish(H, G, d, e, span, rot, pairing):
    """Bias, norm over the whole projection or per head, rotation of pairs over part of a head, value
    blend, and the places of keys and values in the pages."""
    g = torch.Generator().manual_seed(3)
    n, start = 70, 30                                      # crosses a page border
    W = (H + G) * d + G * e
    parts = torch.randn(2, n, W, generator=g)
    bias = torch.randn(W, generator=g)
    qw = 1 + 0.1 * torch.randn(H * d if span == "projection" else d, generator=g)
    kw = 1 + 0.1 * torch.randn(G * d if span == "projection" else d, generator=g)
    inv = torch.tensor([100.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64).float() if rot else None
    v_first = torch.randn(n, G * e, generator=g)
    lam = torch.tensor([0.3])
    batch = one_seq_batch(n, start, pages=[3, 1])
    kv = torch.full((5, G * PAGE * (d + e)), float("nan"), device=DEV)
    cs = ops.rope_table(batch.positions, inv.to(DEV)) if rot else None
    q = ops.qkv_finish(parts.to(DEV), H, G, d, e, dtype=torch.float32, bias=bias.to(DEV),
                       q_weight=qw.to(DEV) if span else None, k_weight=kw.to(DEV) if span else None, eps=1e-5,
                       cos=cs[0] if rot else None, sin=cs[1] if rot else None, rot_dims=rot, pairing=pairing, v_keep=v_first.to(DEV), v_mode=2,
                       blend=lam.to(DEV), kv=kv, page_table=batch.page_table, seq_of_token=batch.seq_of_token,
                       positions=batch.positions)
    row = parts.double().sum(0) + bias.double()
    qr, kr, vr = row[:, :H * d], row[:, H * d:(H + G) * d], row[:, (H + G) * d:]
    if span == "projection":
        qr, kr = P.norm_plain_weight(qr, qw.double(), 1e-5), P.norm_plain_weight(kr, kw.double(), 1e-5)
    elif span == "head":
        qr = P.norm_plain_weight(qr.view(n, H, d), qw.double(), 1e-5).reshape(n, -1)
        kr = P.norm_plain_weight(kr.view(n, G, d), kw.double(), 1e-5).reshape(n, -1)
    qr, kr = qr.view(n, H, d), kr.view(n, G, d)
    pos = torch.arange(start, start + n)
    if rot:
        if pairing == "neighbours":
            qr, kr = P.rotate_pairs(qr, pos, rot, 100.0), P.rotate_pairs(kr, pos, rot, 100.0)
        else:                                                # the half-split pairing, written out here
            def halves(x):
                out, half = x.clone(), rot // 2
                for i in range(half):
                    a = pos.double() * 100.0 ** (-2.0 * i / rot)
                    c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
                    out[..., i] = x[..., i] * c - x[..., i + half] * s
                    out[..., i + half] = x[..., i + half] * c + x[..., i] * s
                return out
            qr, kr = halves(qr), halves(kr)
    vr = P.mix_values(vr, v_first.double(), 0.3).view(n, G, e)
    close(q, qr, "float32", "q")
    kvc = kv.cpu()
    for t in (0, 33, 34, n - 1):                           # positions 30, 63 | 64, 99: both pages
        p = start + t
        page = kvc[[3, 1][p // PAGE]]
        keys, vals = page[:G * PAGE * d].view(G, PAGE, d), page[G * PAGE * d:].view(G, PAGE, e)
        close(keys[:, p % PAGE], kr[t], "float32", f"key at {p}")
        close(vals[:, p % PAGE], vr[t], "float32", f"value at {p}")
    assert torch.isnan(kvc[0]).all() and torch.isnan(kvc[2]).all() and torch.isnan(kvc[4]).all()
    assert torch.isnan(kvc[3][:G * PAGE * d].view(G, PAGE, d)[:, :start]).all()      # nothing before the first new token


def fill_cache(k, v, pages, n_pages):
    """k [n, G, d], v [n, G, e] at positions 0.. into the named pages."""
    n, G, d = k.shape
    e = v.shape[2]
    kv = torch.full((n_pages, G * PAGE * (d + e)), float("nan"))
    for p in range(n):
        page = kv[pages[p // PAGE]]
        page[:G * PAGE * d].view(G, PAGE, d)[:, p % PAGE] = k[p]
        page[G * PAGE * d:].view(G, PAGE, e)[:, p % PAGE] = v[p]
    return kv


@pytest.mark.parametrize("mask,size", [("block", 50), ("block", 64), ("window", 37), ("causal", 0)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_masked_attention_with_a_sink(mask, size, dtype):
    """A prompt's portion after a cached prefix and single tokens, over pages in no order."""
    g = torch.Generator().manual_seed(4)
    H, G, d, e, n = 6, 2, 20, 12, 200
    q = torch.randn(n, H, d, generator=g).to(dtype)
    k = torch.randn(n, G, d, generator=g).to(dtype)
    v = torch.randn(n, G, e, generator=g).to(dtype)
    sink = torch.randn(H, generator=g)
    pages = [4, 2, 7, 1]
    kv = fill_cache(k.float(), v.float(), pages, 9).to(dtype).to(DEV)
    rep = H // G
    scores = (q.double().permute(1, 0, 2) @ k.double().permute(1, 0, 2).repeat_interleave(rep, 0).transpose(1, 2)) * 0.3
    p = torch.arange(n)
    vis = p[None, :] <= p[:, None]
    if mask == "block":
        vis &= (p[None, :] // size) == (p[:, None] // size)
    elif mask == "window":
        vis &= p[None, :] > p[:, None] - size
    else:
        assert torch.equal(vis, P.chunk_visible(n, None))
    if mask == "block":
        assert torch.equal(vis, P.chunk_visible(n, size))
    ref = P.sink_softmax_mix(scores, vis, sink.double(), v.double().permute(1, 0, 2).repeat_interleave(rep, 0)).permute(1, 0, 2)
    kind = "float32" if dtype == torch.float32 else "bfloat16"
    for start, n_new in ((0, n), (77, n - 77), (n - 1, 1), (size, 1) if size else (5, 1), (max(size - 1, 0), 1), (128, 1)):
        batch = one_seq_batch(n_new, start, pages=pages[:(start + n_new + PAGE - 1) // PAGE])
        out = ops.attention_masked(q[start:start + n_new].contiguous().to(DEV), kv, batch, 0.3, n_kv=G, v_dim=e, mask=mask,
                                   mask_size=size, sink=sink.to(DEV))
        close(out, ref[start:start + n_new], kind, f"{mask} {size}: {n_new} tokens after {start}")


@pytest.mark.parametrize("mask,size", [("block", 50), ("block", 64), ("block", 200), ("window", 37), ("causal", 0)])
@pytest.mark.parametrize("d,H,G", [(16, 4, 4), (48, 6, 2), (64, 4, 2), (128, 2, 1)])
def test_tensor_core_prompt_attention_equals_the_warp_kernel(mask, size, d, H, G):
    """Three sequences in one step: from position 0, after a prefix that ends inside a block and a page, and a
    single row; the tensor-core kernel against the warp kernel on the same cache."""
    g = torch.Generator().manual_seed(8)
    lens, starts = [150, 90, 1], [0, 77, 130]
    pages = [[5, 2, 8], [1, 9, 3], [4, 7, 6]]
    kv = torch.full((10, 2 * G * PAGE * d), float("nan"))
    for b in range(3):
        n = starts[b] + lens[b]
        k, v = torch.randn(n, G, d, generator=g), torch.randn(n, G, d, generator=g)
        one = fill_cache(k, v, pages[b], 10)
        for pg in pages[b][:(n + PAGE - 1) // PAGE]:
            kv[pg] = one[pg]
    kv = kv.to(torch.bfloat16).to(DEV)
    q = torch.randn(sum(lens), H, d, generator=g).to(torch.bfloat16).to(DEV)
    sink = torch.randn(H, generator=g).to(DEV)
    lay = BatchLayout(3, sum(lens), 3, 0)
    host = np.zeros(lay.size, dtype=np.int32)
    fill_host(lay, host, tokens=[[0] * n for n in lens], starts=starts, slots=[1, 2, 3], pages=pages, want=[[], [], []])
    batch = StepBatch(lay, torch.from_numpy(host).to(DEV), q_lens=lens, starts=starts)
    for sk in (sink, None):
        kw = dict(n_kv=G, v_dim=d, mask=mask, mask_size=size, sink=sk)
        ref = ops.attention_masked(q, kv, batch, 0.2, kind="warp", **kw)
        assert ops.attention_masked_kind(d, d, torch.bfloat16, False) == ("tc" if d in (64, 128) else "mma")
        for kind in ("mma", "tc") if d in (64, 128) else ("mma",):
            out = ops.attention_masked(q, kv, batch, 0.2, kind=kind, **kw)
            assert torch.isfinite(out.float()).all()
            # (both results are bfloat16: an ulp is 2^-8 of the value)
            assert ((out.float() - ref.float()).abs() <= 0.02 + 0.01 * ref.float().abs()).all(), (kind, mask, size, d, sk is None)
        ops.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mask,size", [("block", 50), ("block", 300), ("window", 37), ("causal", 0)])
@pytest.mark.parametrize("d,H,G", [(16, 4, 4), (48, 6, 1), (128, 8, 2)])
def test_bulk_copy_decode_attention_equals_the_warp_kernel(mask, size, d, H, G, dtype):
    """One token for each of four sequences of different lengths (one of them a single position, one that ends
    on a page's and a block's first position), pages in no order."""
    g = torch.Generator().manual_seed(9)
    lens = [1, 301, 129, 600]
    pages = [[3], [5, 2, 8, 11, 4], [1, 9, 12], [6, 7, 10, 13, 14, 15, 16, 17, 18, 19]]
    kv = torch.full((20, 2 * G * PAGE * d), float("nan"))
    for b, n in enumerate(lens):
        one = fill_cache(torch.randn(n, G, d, generator=g), torch.randn(n, G, d, generator=g), pages[b], 20)
        for pg in pages[b][:(n + PAGE - 1) // PAGE]:
            kv[pg] = one[pg]
    kv = kv.to(dtype).to(DEV)
    q = torch.randn(4, H, d, generator=g).to(dtype).to(DEV)
    sink = torch.randn(H, generator=g).to(DEV)
    lay = BatchLayout(4, 4, 10, 0)
    host = np.zeros(lay.size, dtype=np.int32)
    fill_host(lay, host, tokens=[[0]] * 4, starts=[n - 1 for n in lens], slots=[1, 2, 3, 4], pages=pages, want=[[]] * 4)
    batch = StepBatch(lay, torch.from_numpy(host).to(DEV), q_lens=[1] * 4, starts=[n - 1 for n in lens])
    assert batch.is_decode and ops.attention_masked_kind(d, d, dtype, True) == "bulk"
    for sk in (sink, None):
        kw = dict(n_kv=G, v_dim=d, mask=mask, mask_size=size, sink=sk)
        ref = ops.attention_masked(q, kv, batch, 0.2, kind="warp", **kw)
        out = ops.attention_masked(q, kv, batch, 0.2, kind="bulk", **kw)
        assert torch.isfinite(out.float()).all()
        assert (out.float() - ref.float()).abs().max().item() < (2e-5 if dtype == torch.float32 else 0.02), (mask, size, d)


@pytest.mark.parametrize("size", [50, 64])
def test_one_key_that_stands_out_shows_on_which_side_of_an_edge_it_lies(size):
    """Key j is made to dominate every query that sees it (its score is far above all others) and its value is
    a marker: the result of query i is the marker exactly when j is in i's block and not after i."""
    H, G, d, e, n = 2, 1, 16, 8, 3 * size + 5
    for j in (0, size - 1, size, 2 * size - 1, 2 * size, 63, 64):
        q = torch.zeros(n, H, d)
        q[:, :, 0] = 1.0
        k = torch.zeros(n, G, d)
        k[j, 0, 0] = 60.0
        v = torch.zeros(n, G, e)
        v[j] = 1.0
        pages = [2, 1, 3, 4][:(n + PAGE - 1) // PAGE]
        kv = fill_cache(k, v, pages, 5).to(DEV)
        sink = torch.full((H,), -3.0)
        sees = lambda i: j <= i and i // size == j // size
        batch = one_seq_batch(n, 0, pages=pages)
        out = ops.attention_masked(q.to(DEV), kv, batch, 1.0, n_kv=G, v_dim=e, mask="block", mask_size=size, sink=sink.to(DEV)).cpu()
        for i in range(n):
            want = 1.0 if sees(i) else 0.0
            assert abs(out[i, 0, 0].item() - want) < 1e-6, (size, j, i, out[i, 0, 0].item())
        for i in (j, j + 1, (j // size + 1) * size - 1, (j // size + 1) * size):        # the same, one token at a time
            if i >= n:
                continue
            batch = one_seq_batch(1, i, pages=pages[:i // PAGE + 1])
            o = ops.attention_masked(q[i:i + 1].to(DEV), kv, batch, 1.0, n_kv=G, v_dim=e, mask="block", mask_size=size,
                                     sink=sink.to(DEV)).cpu()
            assert abs(o[0, 0, 0].item() - (1.0 if sees(i) else 0.0)) < 1e-6, (size, j, i)


def test_the_sink_takes_its_share_and_has_no_value():
    """One visible key with score 0 and a sink s: the weight of the key is 1 / (1 + exp(s))."""
    H, d, e = 3, 8, 8
    kv = fill_cache(torch.zeros(1, 1, d), torch.ones(1, 1, e), [1], 2).to(DEV)
    sink = torch.tensor([-2.0, 0.0, 1.5])
    out = ops.attention_masked(torch.zeros(1, H, d, device=DEV), kv, one_seq_batch(1, 0), 1.0, n_kv=1, v_dim=e, sink=sink.to(DEV))
    close(out[0, :, 0], 1.0 / (1.0 + torch.exp(sink.double())), "float32")
    out = ops.attention_masked(torch.zeros(1, H, d, device=DEV), kv, one_seq_batch(1, 0), 1.0, n_kv=1, v_dim=e)
    close(out[0, :, 0], torch.ones(H), "float32", "no sink")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,width,ff", [(5, 3, 64, 40), (2, 2, 72, 52), (3, 1, 40, 24)])
def test_experts_chosen_by_a_table(dtype, experts, top, width, ff):
    g = torch.Generator().manual_seed(6)
    vocab, n = 31, 45
    x = torch.randn(n, width, generator=g).to(dtype)
    tokens = torch.randint(0, vocab, (n,), generator=g)
    table = torch.rand(vocab, experts, generator=g).argsort(1)[:, :top].int()
    t = {"m.table": table}
    for i in range(experts):
        t[f"m.e{i}.gate"] = (0.2 * torch.randn(ff, width, generator=g)).to(dtype)
        t[f"m.e{i}.up"] = (0.2 * torch.randn(ff, width, generator=g)).to(dtype)
        t[f"m.e{i}.down"] = (0.2 * torch.randn(width, ff, generator=g)).to(dtype)
    base = torch.randn(2, n, width, generator=g)
    ref = P.table_moe(x.double(), tokens, {k: (v.double() if v.is_floating_point() else v) for k, v in t.items()}, "m.",
                      {"router": {"top": top}}) + base.double().sum(0)
    gate_up = torch.stack([torch.stack([t[f"m.e{i}.gate"], t[f"m.e{i}.up"]]) for i in range(experts)]).to(DEV)
    down = torch.stack([t[f"m.e{i}.down"] for i in range(experts)]).to(DEV)
    tok = tokens.int().to(DEV)
    hidden = ops.moe_table_up(x.to(DEV), tok, table.to(DEV), gate_up)
    out = ops.moe_table_down(hidden, tok, table.to(DEV), down, 1.0 / top, base.to(DEV))
    close(out, ref, "float32" if dtype == torch.float32 else "bfloat16")


# ---------------------------------------------------------------------------
# whole models through the engine
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["NA", "NB", "NC"])
def test_prompt_decoding_and_portions_agree_with_the_plain_model(name, dtype):
    cfg = CONFIGS[name]
    toks = random_tokens(cfg["vocab"], 230, seed=11)
    ref = plain(name, toks)
    eng = engine(name, dtype)
    s = eng.open_seq()
    close(eng.step([s], [toks], [list(range(len(toks)))]), ref, dtype, "whole prompt")
    eng.close_seq(s)
    # the first tokens one by one, then portions of 2, 3, 61, 64 and 70 tokens, then one by one again
    s = eng.open_seq()
    at, rows = 0, []
    for n in [1] * 7 + [2, 3, 61, 2, 64, 70] + [1] * 13:
        rows.append(eng.step([s], [toks[at:at + n]], [list(range(n))]).clone())
        at += n
    close(torch.cat(rows), ref[:at], dtype, "portions")
    eng.close_seq(s)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_passes_block_edges_and_page_borders(dtype):
    name = "NA"                                            # blocks of 20, 33 and 5 positions, one layer without a mask
    toks = random_tokens(CONFIGS[name]["vocab"], 200, seed=12)
    ref = plain(name, toks)
    eng = engine(name, dtype)
    s = eng.open_seq()
    rows = [eng.step([s], [toks[:17]], [[16]]).clone()]
    for p in range(17, len(toks)):
        rows.append(eng.step([s], [[toks[p]]]).clone())
    close(torch.cat(rows), ref[16:], dtype, "decoded")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["NA", "NB"])
def test_a_batch_of_unequal_requests_equals_each_alone(name, dtype):
    cfg = CONFIGS[name]
    lens = [1, 65, 130, 9, 64]
    prompts = [random_tokens(cfg["vocab"], n + 12, seed=20 + i) for i, n in enumerate(lens)]
    eng = engine(name, dtype, max_tokens=2048)
    alone = []
    for p, n in zip(prompts, lens):
        s = eng.open_seq()
        rows = [eng.step([s], [p[:n]], [list(range(n))]).clone()]
        for t in p[n:]:
            rows.append(eng.step([s], [[t]]).clone())
        alone.append(torch.cat(rows))
        eng.close_seq(s)
        close(alone[-1], plain(name, p), dtype, f"alone, {n} tokens")
    slots = [eng.open_seq() for _ in prompts]
    got = [[] for _ in prompts]
    first = eng.step(slots, [p[:n] for p, n in zip(prompts, lens)], [list(range(n)) for n in lens])
    at = 0
    for i, n in enumerate(lens):
        got[i].append(first[at:at + n].clone())
        at += n
    live = list(range(len(prompts)))
    for step in range(12):
        if step == 5:                                      # two requests end early; the others go on
            for i in (1, 3):
                eng.close_seq(slots[i])
                live.remove(i)
        out = eng.step([slots[i] for i in live], [[prompts[i][lens[i] + step]] for i in live])
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1].clone())
    for i in range(len(prompts)):
        g = torch.cat(got[i])
        close(g, plain(name, prompts[i])[:g.shape[0]], dtype, f"request {i} in a batch")
        if dtype == "float32":
            # the 32-bit kernels cut a request's work the same way whatever else the step holds
            assert (g - alone[i][:g.shape[0]]).abs().max().item() <= 1e-5, f"request {i} differs in a batch"


@pytest.mark.parametrize("dtype", DTYPES)
def test_pages_and_slots_that_were_given_back_are_used_again(dtype):
    name = "NB"
    cfg = CONFIGS[name]
    eng = engine(name, dtype, max_tokens=320)
    a, b = random_tokens(cfg["vocab"], 150, seed=31), random_tokens(cfg["vocab"], 140, seed=32)
    s1 = eng.open_seq()
    eng.step([s1], [a])
    s2 = eng.open_seq()
    eng.step([s2], [b[:70]])
    eng.close_seq(s1)                                      # its three pages and its slot come back
    poison_free_pages(eng)
    s3 = eng.open_seq()
    assert s3 == s1
    out = eng.step([s3], [a[:100]], [list(range(100))])
    assert set(eng.cache.pages_of(s3)) & {1, 2, 3}
    close(out, plain(name, a[:100]), dtype, "in reused pages")
    rows = [eng.step([s2, s3], [[b[70 + i]], [a[100 + i]]]).clone() for i in range(30)]
    close(torch.stack([r[0] for r in rows]), plain(name, b[:100])[70:], dtype, "the request that stayed")
    close(torch.stack([r[1] for r in rows]), plain(name, a[:130])[100:], dtype, "the request in reused pages")
    eng.cache.check()


def test_rows_sorted_by_expert_equal_the_walk_over_tokens():
    """A step that is launched kernel by kernel sorts its rows by expert and uses the tensor-core products;
    a captured step walks the tokens.  Same model, same prompt."""
    from wick_b200.parts.feedforward import TableMoE
    name = "NC"
    toks = random_tokens(CONFIGS[name]["vocab"], 300, seed=71)
    ref = plain(name, toks)
    calls = []
    orig = TableMoE._forward_sorted
    TableMoE._forward_sorted = lambda self, *a: calls.append(1) or orig(self, *a)
    try:
        eng = engine(name, "bfloat16", use_graphs=False)
        s = eng.open_seq()
        close(eng.step([s], [toks], [list(range(300))]), ref, "bfloat16", "sorted by expert")
        assert calls, "the step did not sort its rows"
        n = len(calls)
        eng2 = engine(name, "float32", use_graphs=False)
        s = eng2.open_seq()
        close(eng2.step([s], [toks], [list(range(300))]), ref, "float32", "32-bit walks the tokens")
        assert len(calls) == n
    finally:
        TableMoE._forward_sorted = orig


def test_a_far_key_among_hundreds_is_found():
    """Layer weights are arranged so that attention is the only path from a marked early token to the logits:
    with blocks of 400 positions the marked token at position 3 decides position 390's logits; with blocks of
    100 it cannot."""
    base = copy.deepcopy(CONFIG_NB)
    outs = {}
    for size in (400, 100):
        cfg = copy.deepcopy(base)
        for L in cfg["layers"]:
            L["mixer"]["mask"] = {"size": size}
        d = os.path.join(tmp_root(), f"nib-far-{size}")
        wick.write_random_model(wick.config_from_json(cfg), 9, d, std=0.3)
        st = SafeTensorsDir(d)
        w = {n: st.get(n).tensor() for n in st.names()}
        toks = random_tokens(cfg["vocab"], 391, seed=40)
        other = list(toks)
        other[3] = (toks[3] + 1) % cfg["vocab"]
        eng = wick.Engine.from_dir(d, dtype="float32", max_tokens=1024)
        res = []
        for t in (toks, other):
            s = eng.open_seq()
            eng.step([s], [t[:380]], [[]])
            for p in range(380, 390):
                eng.step([s], [[t[p]]])
            res.append(eng.step([s], [[t[390]]]).clone())
            eng.close_seq(s)
            close(res[-1], P.forward(cfg, w, t).float()[390:], "float32", f"blocks of {size}")
        outs[size] = (res[0] - res[1]).abs().max().item()
    assert outs[400] > 1e-3, "a change 387 tokens back, inside the block, must show"
    assert outs[100] == 0.0, "a change in an earlier block must not show"


@pytest.mark.parametrize("name", ["NA", "NC"])
def test_greedy_generation_through_the_library_entry(name):
    cfg = CONFIGS[name]
    prompts = [random_tokens(cfg["vocab"], n, seed=50 + n) for n in (3, 40, 71)]
    eng = engine(name, "float32")
    out = wick.generate(eng, prompts, wick.GenOptions(max_tokens=24, sampler=wick.SamplerConfig.greedy()))
    for p, r in zip(prompts, out):
        assert len(r.tokens) == 24
        ref = plain(name, list(p) + r.tokens)               # (causal: row i is the prefix's last row)
        for i, t in enumerate(r.tokens):                    # every token is the plain model's best (or ties with it)
            row = ref[len(p) - 1 + i]
            assert row[t] >= row.max() - 1e-3, (name, len(p), i)
    eng_b = engine(name, "bfloat16")
    out_b = wick.generate(eng_b, prompts, wick.GenOptions(max_tokens=8, sampler=wick.SamplerConfig.greedy()))
    for p, r in zip(prompts, out_b):
        ref = plain(name, list(p) + r.tokens)
        for i, t in enumerate(r.tokens):
            row = ref[len(p) - 1 + i]
            assert row[t] >= row.max() - 0.06 * max(1.0, row.abs().max().item())


def test_the_trace_runner_serves_the_design():
    name = "NA"
    d = model(name)[0]
    cfg = CONFIGS[name]
    a, b = random_tokens(cfg["vocab"], 70, seed=61), random_tokens(cfg["vocab"], 9, seed=62)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": a[:66], "want": [0, 65]}, {"id": "y", "tokens": b[:5], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": a[66:67], "want": [0]}, {"id": "y", "tokens": b[5:6], "want": [0]}], "end": ["y"]},
             {"step": 2, "entries": [{"id": "x", "tokens": a[67:68], "want": []}], "end": []},
             {"step": 3, "entries": [{"id": "x", "tokens": a[68:69], "want": [0]}], "end": ["x"]}]
    out = os.path.join(tmp_root(), "nib-trace-out")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", out,
                        "--max-tokens", "256"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    V = cfg["vocab"]
    ra, rb = plain(name, a), plain(name, b)
    read = lambda i: torch.from_numpy(np.fromfile(os.path.join(out, f"{i}.f32"), dtype="<f4").reshape(-1, V))
    close(read(0), ra[[0, 65]], "float32", "step 0")
    close(read(1), torch.stack([ra[66], rb[5]]), "float32", "step 1")
    assert not os.path.exists(os.path.join(out, "2.f32"))
    close(read(3), ra[68:69], "float32", "step 3")
