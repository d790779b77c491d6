"""The Tuguvik decoder and its mechanisms against the plain implementation in
``tests/plain/tuguvik_plain.py``: every mechanism alone through its kernel, then whole
models through the engine (prompts, decoding, portions, batches, reused pages, window
edges, generation).  The configurations differ from each other in every size and option
and include the values that make mechanisms vanish or coincide (no mask, no kept first
tokens, no frequency scaling, one kv head, as many kv heads as heads, values as large as
two maps, no feed-forward, no token input)."""
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
from helpers import random_tokens, tmp_root  # noqa: E402
from plain import tuguvik_plain as P  # noqa: E402

PAGE = 64
DEV = "cuda"

WAVE = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}          # dims 8, base 1e4: one frequency of each kind
RAMP = {"factor": 3.0, "fast": 8.0, "slow": 1.0, "original": 40}


def diff(heads, kv, dim, vdim, scale, d, mask=None, rot=None):
    m = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale, diff=d)
    if mask is not None:
        m["mask"] = {"size": mask[0], "keep_first": mask[1]}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
        if len(rot) > 2:
            m["rot"]["scaling"] = rot[2]
    return dict(type="attention", mixer=m)


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, mask=None, rot=None, kv_from=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank, scale=scale)
    if mask is not None:
        m["mask"] = {"size": mask}
    if rot is not None:
        m["rot"] = {"dims": rot_dim, "base": rot[0]}
        if len(rot) > 1:
            m["rot"]["scaling"] = rot[1]
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="latent_attention", mixer=m)


def layer(mix, ff):
    return dict(mix, mlp={"kind": "dense", "ff": ff} if ff else None)


CONFIG_TA = dict(architecture="Tuguvik", vocab=211, width=64, norm={"eps": 1e-5}, token_side={"dim": 12}, layers=[
    layer(diff(4, 2, 12, 20, 0.3, 0.35, mask=(21, 5), rot=(8, 1e4, WAVE)), 96),
    layer(latent(3, 16, 8, 20, 24, 40, 0.2, mask=17, rot=(5e4, RAMP)), 80),
    layer(latent(2, 8, 8, 12, 16, 40, 0.25, mask=30, rot=(5e4, RAMP), kv_from=1), None),
    layer(diff(2, 2, 16, 16, 0.25, 0.8), 40),
])
CONFIG_TB = dict(architecture="Tuguvik", vocab=130, width=72, norm={"eps": 1e-6}, layers=[
    layer(latent(5, 12, 4, 8, 20, 136, 0.3, rot=(1e3,)), 52),
    layer(diff(6, 1, 10, 20, 0.33, 0.2, mask=(64, 0), rot=(10, 5e5)), 44),
    layer(latent(1, 24, 16, 24, 32, 24, 0.2, mask=100, rot=(1e4, {"factor": 2.0, "fast": 16.0, "slow": 2.0, "original": 300})), 120),
])
# sizes of 64 and 128 numbers a head
CONFIG_TC = dict(architecture="Tuguvik", vocab=300, width=128, norm={"eps": 1e-5}, token_side={"dim": 16}, layers=[
    layer(latent(2, 64, 64, 64, 96, 128, 0.09, mask=70, rot=(1e4, RAMP)), 256),
    layer(diff(2, 1, 64, 128, 0.125, 0.5, mask=(96, 3), rot=(32, 1e4)), 192),
    layer(latent(4, 32, 64, 32, 64, 128, 0.1, mask=130, rot=(1e4, RAMP), kv_from=0), 256),
])
CONFIGS = {"TA": CONFIG_TA, "TB": CONFIG_TB, "TC": CONFIG_TC}
_models = {}


# Whole models are drawn with weights of standard deviation 0.1: these attentions norm neither q nor k, and with larger
# weights their scores grow until the plain model itself differs between float32 and float64 by 1e-3 of its logits.
STD = 0.1


def write_model(cfg, d, seed=5, std=STD):
    wick.write_random_model(wick.config_from_json(cfg), seed, d, std=std)
    st = SafeTensorsDir(d)
    return {n: st.get(n).tensor() for n in st.names()}


def model(name, seed=5, std=STD):
    key = (name, seed, std)
    if key not in _models:
        d = os.path.join(tmp_root(), f"tug-{name}-{seed}-{std}")
        _models[key] = (d, write_model(CONFIGS[name], d, seed, std))
    return _models[key]


def engine(name, dtype, max_tokens=1024, **kw):
    return wick.Engine.from_dir(model(name)[0], dtype=dtype, max_tokens=max_tokens, **kw)


def plain(name, tokens):
    return P.forward(CONFIGS[name], model(name)[1], list(tokens)).float()


def close(got, ref, dtype, what="", tol=None):
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    assert got.shape == ref.shape, f"{what}: {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite"
    scale = max(1.0, ref.abs().max().item())
    worst = (got - ref).abs().max().item()
    tol = tol or (2e-4 if dtype == "float32" else 6e-2)
    if worst > tol * scale:
        row = int((got - ref).abs().reshape(got.shape[0], -1).max(-1).values.argmax())
        raise AssertionError(f"{what}: differs by {worst:.3e} (scale {scale:.3g}), worst row {row}")


DTYPES = ["float32", "bfloat16"]


def seq_batch(n_new, start=0, pages=None):
    """A step of one sequence: ``n_new`` tokens after ``start`` cached ones."""
    n_pages = (start + n_new + PAGE - 1) // PAGE
    pages = pages if pages is not None else list(range(1, n_pages + 1))
    lay = BatchLayout(1, n_new, len(pages), 0)
    host = np.zeros(lay.size, dtype=np.int32)
    fill_host(lay, host, tokens=[[0] * n_new], starts=[start], slots=[1], pages=[pages], want=[[]])
    return StepBatch(lay, torch.from_numpy(host).to(DEV), q_lens=[n_new], starts=[start])


# ---------------------------------------------------------------------------
# mechanisms alone
def test_the_stream_kernel_adds_scales_norms_and_selects_rows():
    g = torch.Generator().manual_seed(1)
    for width, rows in ((48, 9), (100, 9), (257, 5), (2052, 70)):
        x, d = torch.randn(rows, width, generator=g), torch.randn(3, rows, width, generator=g)
        s, rw = torch.randn(width, generator=g), 1 + 0.1 * torch.randn(width, generator=g)
        w, b, a = torch.randn(width, generator=g), torch.randn(width, generator=g), torch.tensor([0.37])
        X, D = x.double(), d.double().sum(0)
        norm = ("tanh", a.to(DEV), w.to(DEV), b.to(DEV))
        # the norm alone
        xd = x.to(DEV)
        out = ops.stream_update(xd, None, norm=norm, out_dtype=torch.float32)
        close(out, P.tanh_norm(X, w.double(), b.double(), 0.37), "float32", f"norm, width {width}", 2e-6)
        assert torch.equal(xd.cpu(), x)
        # a scaled sum, then the norm; the stream is brought up to date
        out = ops.stream_update(xd, d.to(DEV), scale=s.to(DEV), norm=norm, out_dtype=torch.bfloat16)
        close(xd, X + s.double() * D, "float32", "scaled sum", 2e-6)
        close(out, P.tanh_norm(X + s.double() * D, w.double(), b.double(), 0.37), "bfloat16", "norm of it", 1e-2)
        # a sum that is divided by its root mean square, no norm, a copy in the activation type
        xd = x.to(DEV)
        out = ops.stream_update(xd, d.to(DEV), rms=(rw.to(DEV), 1e-5), out_dtype=torch.bfloat16)
        ref = X + P.unit_rms(D, 1e-5) * rw.double()
        close(xd, ref, "float32", "normed sum", 2e-6)
        assert torch.equal(out.float(), xd.to(torch.bfloat16).float())
        xd2 = x.to(DEV)
        assert ops.stream_update(xd2, d.to(DEV), rms=(rw.to(DEV), 1e-5), out_dtype=torch.float32) is xd2
        assert torch.equal(xd2, xd)
        # selected rows (one named twice): only they go out, the stream stays
        xd = x.to(DEV)
        idx = torch.tensor([rows - 1, 0, rows - 1], dtype=torch.int32)
        out = ops.stream_update(xd, d.to(DEV), rms=(rw.to(DEV), 1e-5), norm=norm, out_dtype=torch.float32, rows=idx.to(DEV))
        close(out, P.tanh_norm(ref, w.double(), b.double(), 0.37)[idx.long()], "float32", "rows", 2e-6)
        assert torch.equal(xd.cpu(), x)


def test_gated_token_rows():
    g = torch.Generator().manual_seed(2)
    n, dim, vocab, cols = 37, 12, 50, 40
    z = 3 * torch.randn(n, dim, generator=g)
    tokens = torch.randint(0, vocab, (n,), generator=g)
    for dt in (torch.float32, torch.bfloat16):
        table = torch.randn(vocab, cols, generator=g).to(dt)
        out = ops.gelu_gate_rows(z.to(DEV), table.to(DEV), tokens.int().to(DEV), 17, dt)
        ref = P.gelu_tanh(z.double()) * table.double()[tokens][:, 17:17 + dim]
        close(out, ref, "float32" if dt == torch.float32 else "bfloat16", "gate", 2e-6 if dt == torch.float32 else 1e-2)
    # the whole side input: x + rms(Wproj (gelu(Wgate x) * e)) * w
    t = {"s.gate": torch.randn(dim, 64, generator=g), "s.proj": torch.randn(64, dim, generator=g), "s.norm": torch.randn(64, generator=g)}
    x = torch.randn(n, 64, generator=g)
    e = torch.randn(n, dim, generator=g)
    zz = x @ t["s.gate"].T
    gg = ops.gelu_gate_rows(zz.to(DEV), e.to(DEV), torch.arange(n, dtype=torch.int32, device=DEV), 0, torch.float32)
    y = (gg.cpu() @ t["s.proj"].T)[None]
    xd = x.to(DEV)
    ops.stream_update(xd, y.to(DEV), rms=(t["s.norm"].to(DEV), 1e-5))
    close(xd, x.double() + P.token_input(x.double(), e.double(), {k: v.double() for k, v in t.items()}, "s.", 1e-5), "float32",
          "side input", 2e-5)


def fill_pages(k, v, pages, n_pages, dtype=torch.float32):
    """Keys [n, G, d] and values [n, G, e] into pages of [G][64][d] keys then [G][64][e] values."""
    n, G, d = k.shape
    e = v.shape[2]
    kv = torch.full((n_pages, G * PAGE * (d + e)), float("nan"), dtype=dtype)
    for j in range(n):
        pg, r = pages[j // PAGE], j % PAGE
        for g_ in range(G):
            kv[pg, (g_ * PAGE + r) * d:(g_ * PAGE + r) * d + d] = k[j, g_].to(dtype)
            o = G * PAGE * d + (g_ * PAGE + r) * e
            kv[pg, o:o + e] = v[j, g_].to(dtype)
    return kv


def plain_two_maps(q, k, v, scale, window, keep, lam, eps, factor, offset=0):
    """q [n, H, 2, dm] (rows are positions offset ..), k [m, G, 2, dm], v [m, G, e] -> [n, H, e], from the oracle's pieces."""
    n, H = q.shape[:2]
    m, G = k.shape[:2]
    vis = P.window_visible(m, window or None, keep)[offset:offset + n]
    kk, vv = k.repeat_interleave(H // G, 1), v.repeat_interleave(H // G, 1)
    ys = []
    for a in range(2):
        s = torch.einsum("ihd,jhd->hij", q[:, :, a], kk[:, :, a]) * scale
        ys.append(torch.einsum("hij,jhe->ihe", P.softmax_visible(s, vis), vv))
    return P.unit_rms(ys[0] - lam * ys[1], eps) * factor


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dm,e,window,keep", [(4, 2, 12, 20, 21, 5), (6, 1, 10, 20, 64, 0), (2, 2, 16, 16, 0, 0), (2, 1, 64, 128, 70, 70),
                                                  (3, 3, 8, 132, 130, 2)])
def test_two_maps_over_a_window_with_kept_first_keys(dtype, H, G, dm, e, window, keep):
    g = torch.Generator().manual_seed(3)
    m = 200
    q = torch.randn(m, H, 2, dm, generator=g).to(dtype)
    k = torch.randn(m, G, 2, dm, generator=g).to(dtype)
    v = torch.randn(m, G, e, generator=g).to(dtype)
    pages = [3, 1, 4, 2]
    kv = fill_pages(k.reshape(m, G, 2 * dm), v, pages, 6, dtype).to(DEV)
    lam, eps, factor = 0.45, 1e-5, 0.65
    ref = plain_two_maps(q.double(), k.double(), v.double(), 0.3, window, keep, lam, eps, factor)
    kw = dict(maps=2, kv_heads=G, v_dim=e, window=window, keep_first=keep, combine=(lam, eps, factor), out_dtype=dtype)
    name = "float32" if dtype == torch.float32 else "bfloat16"
    out = ops.attention_multi(q.reshape(m, H, 2 * dm).to(DEV), kv, seq_batch(m, 0, pages), 0.3, **kw)
    close(out, ref, name, "a prompt", 3e-5 if dtype == torch.float32 else 3e-2)
    for start, n in ((0, 1), (1, 1), (keep, 2), (window + keep, 1), (63, 3), (128, 1), (150, 50), (199, 1)):   # portions and single tokens
        if start + n > m:
            continue
        b = seq_batch(n, start, pages[:(start + n + PAGE - 1) // PAGE])
        out = ops.attention_multi(q[start:start + n].reshape(n, H, 2 * dm).to(DEV), kv, b, 0.3, **kw)
        close(out, ref[start:start + n], name, f"{n} tokens after {start}", 3e-5 if dtype == torch.float32 else 3e-2)


@pytest.mark.parametrize("window,keep", [(50, 0), (64, 7), (10, 64)])
def test_a_key_that_stands_out_shows_on_which_side_of_the_window_it_lies(window, keep):
    """Key j dominates map 1 of every query that sees it, and its value is a marker; with lambda = 0 the result is the
    marker's unit vector exactly when j is visible: j <= i and (i - j < window or j < keep)."""
    H, G, dm, e, n = 1, 1, 8, 8, 3 * 64 + 9
    hit = 1.0 / math.sqrt(1.0 / e + 1e-6)
    for j in (0, keep - 1, keep, 63, 64, 100, 128):
        if j < 0:
            continue
        q = torch.zeros(n, H, 2 * dm)
        q[:, :, 0] = 1.0
        k = torch.zeros(n, G, 2 * dm)
        k[j, 0, 0] = 60.0
        v = torch.zeros(n, G, e)
        v[j, 0, 0] = 1.0
        pages = [2, 1, 3, 4]
        kv = fill_pages(k, v, pages, 5).to(DEV)
        sees = lambda i: j <= i and (i - j < window or j < keep)
        kw = dict(maps=2, kv_heads=G, v_dim=e, window=window, keep_first=keep, combine=(0.0, 1e-6, 1.0), out_dtype=torch.float32)
        out = ops.attention_multi(q.to(DEV), kv, seq_batch(n, 0, pages), 1.0, **kw).cpu()
        for i in range(n):
            assert abs(out[i, 0, 0].item() - (hit if sees(i) else 0.0)) < 1e-3, (window, keep, j, i, out[i, 0, 0].item())
        for i in (j, j + 1, j + window - 1, j + window, j + window + 1, n - 1):          # the same, one token at a time
            if not 0 <= i < n:
                continue
            o = ops.attention_multi(q[i:i + 1].to(DEV), kv, seq_batch(1, i, pages[:i // PAGE + 1]), 1.0, **kw).cpu()
            assert abs(o[0, 0, 0].item() - (hit if sees(i) else 0.0)) < 1e-3, (window, keep, j, i)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,r,dr,window", [(3, 40, 8, 17), (5, 136, 4, 0), (1, 24, 16, 100), (4, 128, 64, 64), (2, 300, 2, 65)])
def test_one_map_over_cached_rows_with_a_sink(dtype, H, r, dr, window):
    g = torch.Generator().manual_seed(4)
    m, R = 200, r + dr
    q = torch.randn(m, H, R, generator=g)
    rows = torch.randn(m, R, generator=g).to(dtype)
    sink = torch.randn(H, generator=g)
    pages = [2, 4, 1, 3]
    store = torch.full((6, PAGE, R), float("nan"), dtype=dtype)
    for j in range(m):
        store[pages[j // PAGE], j % PAGE] = rows[j]
    s = torch.einsum("ihd,jd->hij", q.double(), rows.double()) * 0.2
    w = P.softmax_visible(s, P.window_visible(m, window or None), sink.double())
    ref = torch.einsum("hij,je->ihe", w, rows.double()[:, :r])
    name = "float32" if dtype == torch.float32 else "bfloat16"
    kw = dict(maps=1, kv_heads=1, v_dim=r, window=window, sink=sink.to(DEV), rows_of=R, out_dtype=torch.float32)
    out = ops.attention_multi(q.to(DEV), store.to(DEV), seq_batch(m, 0, pages), 0.2, **kw)
    close(out, ref, name, "a prompt", 3e-5)
    for start, n in ((0, 1), (1, 2), (window, 1), (window + 1, 1), (64, 1), (127, 2), (199, 1)):
        b = seq_batch(n, start, pages[:(start + n + PAGE - 1) // PAGE])
        out = ops.attention_multi(q[start:start + n].to(DEV), store.to(DEV), b, 0.2, **kw)
        close(out, ref[start:start + n], name, f"{n} tokens after {start}", 3e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_rows_of_keys_are_cut_into_runs_and_merged(dtype):
    """A step of few tokens over many keys: the keys go through several blocks whose records are merged (with the sink,
    with the two maps' combination), and heads that read the same rows share a block (groups of 4, 2 and 1 heads)."""
    g = torch.Generator().manual_seed(8)
    m = 1300
    name = "float32" if dtype == torch.float32 else "bfloat16"
    pages = list(range(21, 0, -1))
    for H, r, dr, window in ((8, 40, 8, 0), (6, 136, 8, 1100), (3, 24, 16, 0)):
        R = r + dr
        q = torch.randn(m, H, R, generator=g)
        rows = torch.randn(m, R, generator=g).to(dtype)
        sink = torch.randn(H, generator=g)
        store = torch.full((23, PAGE, R), float("nan"), dtype=dtype)
        for j in range(m):
            store[pages[j // PAGE], j % PAGE] = rows[j]
        s = torch.einsum("ihd,jd->hij", q.double(), rows.double()) * 0.1
        ref = torch.einsum("hij,je->ihe", P.softmax_visible(s, P.window_visible(m, window or None), sink.double()), rows.double()[:, :r])
        for start, n in ((1299, 1), (1024, 2), (600, 1), (5, 1)):
            b = seq_batch(n, start, pages[:(start + n + PAGE - 1) // PAGE])
            out = ops.attention_multi(q[start:start + n].to(DEV), store.to(DEV), b, 0.1, maps=1, kv_heads=1, v_dim=r, window=window,
                                      sink=sink.to(DEV), rows_of=R, out_dtype=torch.float32)
            close(out, ref[start:start + n], name, f"rows: {n} tokens after {start}, {H} heads", 3e-5)
    H, G, dm, e, window, keep = 4, 2, 16, 24, 900, 40
    q = torch.randn(m, H, 2, dm, generator=g).to(dtype)
    k = torch.randn(m, G, 2, dm, generator=g).to(dtype)
    v = torch.randn(m, G, e, generator=g).to(dtype)
    kv = fill_pages(k.reshape(m, G, 2 * dm), v, pages, 23, dtype).to(DEV)
    ref = plain_two_maps(q.double(), k.double(), v.double(), 0.2, window, keep, 0.45, 1e-5, 0.65)
    for start, n in ((1299, 1), (939, 2), (600, 1)):
        b = seq_batch(n, start, pages[:(start + n + PAGE - 1) // PAGE])
        out = ops.attention_multi(q[start:start + n].reshape(n, H, 2 * dm).to(DEV), kv, b, 0.2, maps=2, kv_heads=G, v_dim=e, window=window,
                                  keep_first=keep, combine=(0.45, 1e-5, 0.65), out_dtype=dtype)
        close(out, ref[start:start + n], name, f"two maps: {n} tokens after {start}", 3e-5 if dtype == torch.float32 else 3e-2)


def test_the_sink_takes_its_share_and_a_row_outside_the_window_none():
    """One visible row with score 0 and a sink s: the row's weight is 1 / (1 + exp(s)).  A row that dominates is seen
    from positions j .. j + window - 1 and from no other."""
    H, R = 3, 8
    store = torch.zeros(2, PAGE, R)
    store[1, 0] = 1.0
    sink = torch.tensor([-2.0, 0.0, 1.5])
    kw = dict(maps=1, kv_heads=1, v_dim=6, rows_of=R, out_dtype=torch.float32)
    out = ops.attention_multi(torch.zeros(1, H, R, device=DEV), store.to(DEV), seq_batch(1, 0), 1.0, sink=sink.to(DEV), **kw)
    close(out[0, :, 0], 1.0 / (1.0 + torch.exp(sink.double())), "float32", tol=1e-6)
    out = ops.attention_multi(torch.zeros(1, H, R, device=DEV), store.to(DEV), seq_batch(1, 0), 1.0, **kw)
    close(out[0, :, 0], torch.ones(H), "float32", "no sink", 1e-6)
    n, window = 150, 37
    for j in (0, 27, 63, 64, 100):
        store = torch.zeros(4, PAGE, R)
        store[1 + j // PAGE, j % PAGE, 0] = 50.0
        q = torch.zeros(n, 1, R)
        q[:, :, 0] = 1.0
        out = ops.attention_multi(q.to(DEV), store.to(DEV), seq_batch(n, 0), 1.0, sink=torch.tensor([-3.0], device=DEV),
                                  maps=1, kv_heads=1, v_dim=4, window=window, rows_of=R, out_dtype=torch.float32).cpu()
        for i in range(n):
            want = 50.0 if 0 <= i - j < window else 0.0
            assert abs(out[i, 0, 0].item() - want) < 1e-3, (j, i, out[i, 0, 0].item())
        for i in (j + window - 1, j + window):
            if i < n:
                o = ops.attention_multi(q[i:i + 1].to(DEV), store.to(DEV), seq_batch(1, i), 1.0, sink=torch.tensor([-3.0], device=DEV),
                                        maps=1, kv_heads=1, v_dim=4, window=window, rows_of=R, out_dtype=torch.float32).cpu()
                assert abs(o[0, 0, 0].item() - (50.0 if i - j < window else 0.0)) < 1e-3, (j, i)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dm,e,rot", [(4, 2, 12, 20, (8, 1e4, WAVE)), (6, 1, 10, 20, (10, 5e5)), (2, 2, 16, 16, None)])
def test_projection_finish_turns_every_map_on_its_own(dtype, H, G, dm, e, rot):
    g = torch.Generator().manual_seed(5)
    n, start = 70, 30
    W = 2 * dm * (H + G) + G * e
    parts = torch.randn(3, n, W, generator=g)
    batch = seq_batch(n, start)
    pos = torch.arange(start, start + n)
    row = parts.double().sum(0)
    q = row[:, :2 * dm * H].reshape(n, 2 * H, dm)
    k = row[:, 2 * dm * H:2 * dm * (H + G)].reshape(n, 2 * G, dm)
    cos = sin = None
    if rot:
        freqs = P.frequencies_by_wavelength(rot[0], rot[1], rot[2] if len(rot) > 2 else None)
        inv = torch.tensor(freqs, dtype=torch.float64).float()
        cos, sin = ops.rope_table(batch.positions, inv.to(DEV))
        q = torch.cat([P.turn_halves(q[..., :rot[0]], pos, freqs), q[..., rot[0]:]], -1)
        k = torch.cat([P.turn_halves(k[..., :rot[0]], pos, freqs), k[..., rot[0]:]], -1)
    kv = torch.zeros(4, G * PAGE * (2 * dm + e), dtype=dtype, device=DEV)
    out = ops.qkv_finish(parts.to(DEV), H, G, 2 * dm, e, dtype=dtype, cos=cos, sin=sin, rot_dims=rot[0] if rot else 0,
                         pairing="halves", maps=2, kv=kv, page_table=batch.page_table, seq_of_token=batch.seq_of_token,
                         positions=batch.positions)
    name = "float32" if dtype == torch.float32 else "bfloat16"
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    close(out.reshape(n, 2 * H, dm), q, name, "q", tol)
    kvc = kv.float().cpu()
    for t in (0, 33, 34, n - 1):                              # (position 63 -> 64: a page border)
        pg, r = 1 + (start + t) // PAGE, (start + t) % PAGE
        for h in range(G):
            got = kvc[pg, (h * PAGE + r) * 2 * dm:(h * PAGE + r + 1) * 2 * dm]
            close(got[None], k[t, 2 * h:2 * h + 2].reshape(1, -1), name, f"key of token {t}", tol)
            o = G * PAGE * 2 * dm + (h * PAGE + r) * e
            close(kvc[pg, o:o + e][None], row[t, 2 * dm * (H + G) + h * e:2 * dm * (H + G) + (h + 1) * e][None], name, "value", tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,d,dr,e,qr,r,own", [(3, 16, 8, 20, 24, 40, True), (2, 8, 8, 12, 16, 40, False), (5, 12, 4, 8, 20, 136, True),
                                               (2, 64, 64, 64, 96, 300, True)])
def test_the_kernels_around_the_latent(dtype, H, d, dr, e, qr, r, own):
    g = torch.Generator().manual_seed(6)
    n, start = 41, 50
    name = "float32" if dtype == torch.float32 else "bfloat16"
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    batch = seq_batch(n, start)
    pos = torch.arange(start, start + n)
    freqs, amp = P.frequencies_by_ramp(dr, 5e4, RAMP)
    cos, sin = ops.rope_table(batch.positions, torch.tensor(freqs, dtype=torch.float64).float().to(DEV), amp)
    W = qr + (r + dr if own else 0) + H
    parts = torch.randn(2, n, W, generator=g)
    wq, wkv = torch.randn(qr, generator=g), torch.randn(r, generator=g)
    rows = torch.zeros(4, PAGE, r + dr, dtype=dtype, device=DEV)
    cq, gate = ops.latent_finish(parts.to(DEV), qr, r if own else 0, dr if own else 0, H, dtype=dtype, q_weight=wq.to(DEV),
                                 kv_weight=wkv.to(DEV) if own else None, eps=1e-5, cos=cos, sin=sin, rows=rows if own else None,
                                 page_table=batch.page_table, seq_of_token=batch.seq_of_token, positions=batch.positions)
    row = parts.double().sum(0)
    close(cq, P.unit_rms(row[:, :qr], 1e-5) * wq.double(), name, "query latent", tol)
    close(gate, torch.sigmoid(row[:, W - H:]), "float32", "gates", 1e-5)
    if own:
        c = P.unit_rms(row[:, qr:qr + r], 1e-5) * wkv.double()
        kr = P.turn_neighbours(row[:, None, qr + r:qr + r + dr], pos, freqs, amp)[:, 0]
        got = torch.stack([rows[1 + (start + t) // PAGE, (start + t) % PAGE] for t in range(n)]).float().cpu()
        close(got, torch.cat([c, kr], -1), name, "cached rows", tol)
    # the query in the rows' space and the way back to a head's values
    uk = (0.3 * torch.randn(H * d, r, generator=g)).to(dtype)
    uv = (0.3 * torch.randn(H * e, r, generator=g)).to(dtype)
    qp = torch.randn(3, n, H * (d + dr), generator=g)
    ql = ops.latent_absorb(qp.to(DEV), uk.to(DEV), H, d, dr, r, cos=cos, sin=sin)
    qq = qp.double().sum(0).reshape(n, H, d + dr)
    ref = torch.cat([torch.einsum("nhd,hdr->nhr", qq[..., :d], uk.double().reshape(H, d, r)),
                     P.turn_neighbours(qq[..., d:], pos, freqs, amp)], -1)
    close(ql, ref, "float32", "query in the rows' space", 1e-4)
    y = torch.randn(n, H, r, generator=g)
    gt = torch.rand(n, H, generator=g)
    out = ops.latent_expand(y.to(DEV), uv.to(DEV), gt.to(DEV), H, e, r, dtype=dtype)
    ref = torch.einsum("nhr,her->nhe", y.double(), uv.double().reshape(H, e, r)) * gt.double()[:, :, None]
    close(out.reshape(n, H, e), ref, name, "values of the heads", tol)


def flex_two_maps(q, kv, batch, scale, H, G, dm, e, window, keep, combine):
    """The tensor-core form of two maps over the paged keys and values: every map of every head a head of its own."""
    n, d = q.shape[0], 2 * dm
    page, per = G * PAGE * (d + e), 2 * (H // G)
    k0 = ops.flex_source(kv, tile_elems=page, hdiv=per, hmul=PAGE * d, hmod=2, hmul2=dm, row_stride=d, length=dm, paged=True)
    v = ops.flex_source(kv, tile_elems=page, const_off=G * PAGE * d, hdiv=per, hmul=PAGE * e, row_stride=e, length=e, paged=True)
    maps = ops.attention_flex(q.view(n, 2 * H, dm), k0, ops.flex_source(), v, batch, scale, dv=e, window=window, keep_first=keep,
                              out_dtype=torch.float32)
    return ops.combine_maps(maps.view(n, H, 2, e), *combine, lib=(dm, e))


def ragged_batch(lens, starts, pages):
    lay = BatchLayout(len(lens), sum(lens), max(len(p) for p in pages), 0)
    host = np.zeros(lay.size, dtype=np.int32)
    fill_host(lay, host, tokens=[[0] * n for n in lens], starts=starts, slots=list(range(1, len(lens) + 1)), pages=pages,
              want=[[] for _ in lens])
    return StepBatch(lay, torch.from_numpy(host).to(DEV), q_lens=lens, starts=starts)


@pytest.mark.parametrize("H,G,dm,e,window,keep", [(4, 2, 16, 32, 21, 5), (2, 1, 32, 64, 64, 0), (2, 2, 64, 128, 0, 0), (3, 1, 16, 16, 100, 70)])
def test_two_maps_on_the_tensor_cores(H, G, dm, e, window, keep):
    """Prompts (whole, ragged batches, later portions over cached keys) through the tensor-core kernel against the plain form."""
    g = torch.Generator().manual_seed(9)
    m = 300
    q = torch.randn(m, H, 2, dm, generator=g).to(torch.bfloat16)
    k = torch.randn(m, G, 2, dm, generator=g).to(torch.bfloat16)
    v = torch.randn(m, G, e, generator=g).to(torch.bfloat16)
    pages = [3, 1, 4, 2, 5]
    kv = fill_pages(k.reshape(m, G, 2 * dm), v, pages, 12, torch.bfloat16).to(DEV)
    comb = (0.45, 1e-5, 0.65)
    ref = plain_two_maps(q.double(), k.double(), v.double(), 0.2, window, keep, *comb)
    for start, n in ((0, 300), (0, 64), (0, 65), (37, 100), (128, 172), (299, 1)):
        b = seq_batch(n, start, pages[:(start + n + PAGE - 1) // PAGE])
        out = flex_two_maps(q[start:start + n].reshape(n, H, 2 * dm).to(DEV), kv, b, 0.2, H, G, dm, e, window, keep, comb)
        close(out, ref[start:start + n], "bfloat16", f"{n} tokens after {start}", 3e-2)
    # three requests in one step: the same rows at other places of the cache, one of them a later portion
    kv2 = torch.full_like(kv, float("nan"))
    lens, starts, pgs = [70, 130, 100], [0, 0, 200], [[6, 7], [8, 9, 10], [3, 1, 4, 2, 5]]
    for src, dst in ((3, 6), (1, 7), (3, 8), (1, 9), (4, 10), (3, 3), (1, 1), (4, 4), (2, 2), (5, 5)):
        kv2[dst] = kv[src]
    b = ragged_batch(lens, starts, pgs)
    qq = torch.cat([q[:70], q[:130], q[200:300]]).reshape(300, H, 2 * dm).to(DEV)
    out = flex_two_maps(qq, kv2, b, 0.2, H, G, dm, e, window, keep, comb)
    close(out, torch.cat([ref[:70], ref[:130], ref[200:300]]), "bfloat16", "a ragged step", 3e-2)


@pytest.mark.parametrize("window,keep", [(50, 0), (64, 7), (10, 64), (130, 66)])
def test_a_key_that_stands_out_on_the_tensor_cores(window, keep):
    """As above, through the tensor-core kernel: key j's marker is the result exactly when j is visible."""
    H, G, dm, e, n = 1, 1, 16, 16, 5 * 64 + 9
    hit = 1.0 / math.sqrt(1.0 / e + 1e-6)
    pages = [2, 1, 3, 4, 6, 5]
    for j in (0, keep - 1, keep, 63, 64, 100, 128, 200):
        if j < 0:
            continue
        q = torch.zeros(n, H, 2 * dm)
        q[:, :, 0] = 1.0
        k = torch.zeros(n, G, 2 * dm)
        k[j, 0, 0] = 60.0
        v = torch.zeros(n, G, e)
        v[j, 0, 0] = 1.0
        kv = fill_pages(k, v, pages, 7, torch.bfloat16).to(DEV)
        sees = lambda i: j <= i and (i - j < window or j < keep)
        for start in (0, 70):                                # a prompt from position 0, and a portion after 70 cached tokens
            b = seq_batch(n - start, start, pages)
            out = flex_two_maps(q[start:].to(torch.bfloat16).to(DEV), kv, b, 1.0, H, G, dm, e, window, keep, (0.0, 1e-6, 1.0)).float().cpu()
            for i in range(start, n):
                assert abs(out[i - start, 0, 0].item() - (hit if sees(i) else 0.0)) < 3e-2, (window, keep, j, start, i, out[i - start, 0, 0].item())


@pytest.mark.parametrize("H,d,dr,e,window", [(2, 16, 16, 16, 50), (3, 64, 32, 64, 0), (2, 128, 64, 128, 130)])
def test_keys_of_two_parts_from_the_steps_own_rows(H, d, dr, e, window):
    """The tensor-core kernel over flat arrays: a head's key is its own part followed by a part all heads share; a sink; a
    gate on the result; two requests in a step."""
    g = torch.Generator().manual_seed(10)
    lens = [150, 201]
    n = sum(lens)
    q = torch.randn(n, H, d + dr, generator=g).to(torch.bfloat16)
    kvx = torch.randn(n, H * d + H * e, generator=g).to(torch.bfloat16)
    kr = torch.randn(n, dr, generator=g).to(torch.bfloat16)
    sink, gate = torch.randn(H, generator=g), torch.rand(n, H, generator=g)
    b = ragged_batch(lens, [0, 0], [[1, 2, 3], [4, 5, 6, 7]])
    kvd, krd = kvx.to(DEV), kr.to(DEV)
    k0 = ops.flex_source(kvd, hmul=d, row_stride=H * (d + e), length=d)
    out = ops.attention_flex(q.to(DEV), k0, ops.flex_source(krd, row_stride=dr, length=dr),
                             ops.flex_source(kvd, const_off=H * d, hmul=e, row_stride=H * (d + e), length=e), b, 0.1, dv=e,
                             window=window, sink=sink.to(DEV), gate=gate.to(DEV))
    at = 0
    for L in lens:
        qq, kk = q[at:at + L].double(), kvx[at:at + L].double()
        keys = torch.cat([kk[:, :H * d].reshape(L, H, d), kr[at:at + L].double()[:, None, :].expand(L, H, dr)], -1)
        vals = kk[:, H * d:].reshape(L, H, e)
        s = torch.einsum("ihd,jhd->hij", qq, keys) * 0.1
        w = P.softmax_visible(s, P.window_visible(L, window or None), sink.double())
        ref = torch.einsum("hij,jhe->ihe", w, vals) * gate[at:at + L].double()[:, :, None]
        close(out[at:at + L], ref, "bfloat16", f"request of {L} tokens", 3e-2)
        at += L
    # a key that stands out is seen from its window's positions only
    if window:
        j = 77
        q2 = torch.zeros(n, H, d + dr)
        q2[:, :, 0] = 1.0
        kv2 = torch.zeros(n, H * d + H * e)
        kv2[j, 0] = 60.0                                        # head 0's own key part
        kv2[j, H * d] = 1.0                                     # head 0's value
        kv2d, kr2d = kv2.to(torch.bfloat16).to(DEV), torch.zeros(n, dr, dtype=torch.bfloat16, device=DEV)
        out = ops.attention_flex(q2.to(torch.bfloat16).to(DEV), ops.flex_source(kv2d, hmul=d, row_stride=H * (d + e), length=d),
                                 ops.flex_source(kr2d, row_stride=dr, length=dr),
                                 ops.flex_source(kv2d, const_off=H * d, hmul=e, row_stride=H * (d + e), length=e), b, 1.0, dv=e,
                                 window=window, sink=torch.full((H,), -3.0, device=DEV)).float().cpu()
        for i in range(lens[0]):
            assert abs(out[i, 0, 0].item() - (1.0 if 0 <= i - j < window else 0.0)) < 2e-2, (i, out[i, 0, 0].item())
        assert out[lens[0]:, 0, 0].abs().max().item() == 0.0     # the other request sees none of it


@pytest.mark.parametrize("graphs", [False, True])
def test_long_prompts_take_the_tensor_core_kernels(graphs):
    """Sizes the tensor-core prompt kernels take: prompts from position 0 alone and in a ragged step, then later portions and
    single tokens over what they cached, launched and replayed from captured steps."""
    name = "TC"
    calls = []
    orig = ops.attention_flex
    ops.attention_flex = lambda *a, **k: calls.append(1) or orig(*a, **k)
    try:
        eng = engine(name, "bfloat16", max_tokens=4096, use_graphs=graphs)
        toks = [random_tokens(CONFIGS[name]["vocab"], n, seed=80 + n) for n in (700, 90, 333)]
        refs = [plain(name, t) for t in toks]
        s = eng.open_seq()
        close(eng.step([s], [toks[0][:600]], [list(range(600))]), refs[0][:600], "bfloat16", "a prompt of 600 tokens")
        assert len(calls) == 3, "every layer's attention of a long prompt runs on the tensor cores"
        close(eng.step([s], [toks[0][600:690]], [list(range(90))]), refs[0][600:690], "bfloat16", "a later portion")
        rows = [eng.step([s], [[t]]).clone() for t in toks[0][690:]]
        close(torch.cat(rows), refs[0][690:], "bfloat16", "decoded")
        eng.close_seq(s)
        slots = [eng.open_seq() for _ in toks]
        cut = [650, 80, 300]
        out = eng.step(slots, [t[:c] for t, c in zip(toks, cut)], [list(range(c)) for c in cut])
        close(out, torch.cat([r[:c] for r, c in zip(refs, cut)]), "bfloat16", "a ragged step")
        for i in range(10):
            out = eng.step(slots, [[t[c + i]] for t, c in zip(toks, cut)])
            close(out, torch.stack([r[c + i] for r, c in zip(refs, cut)]), "bfloat16", f"decode step {i}")
    finally:
        ops.attention_flex = orig


# ---------------------------------------------------------------------------
# whole models through the engine
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["TA", "TB", "TC"])
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
def test_the_stream_after_every_layer(dtype):
    """The residual stream after each layer (with everything of the layer added) against the plain model's."""
    from wick_b200.parts.standard import PreNormResidual
    name = "TA"
    toks = random_tokens(CONFIGS[name]["vocab"], 90, seed=13)
    _, layers = P.forward(CONFIGS[name], model(name)[1], toks, return_layers=True)
    seen, orig = [], PreNormResidual.forward

    def forward(self, h, batch, cache, write):
        h = orig(self, h, batch, cache, write)
        x = h.x.clone()
        if h.pending is not None:
            ops.stream_update(x, h.pending, scale=h.scale, rms=h.rms)
        seen.append(x.cpu())
        return h

    PreNormResidual.forward = forward
    try:
        eng = engine(name, dtype, use_graphs=False)
        s = eng.open_seq()
        eng.step([s], [toks])
    finally:
        PreNormResidual.forward = orig
    assert len(seen) == len(layers)
    for i, (got, ref) in enumerate(zip(seen, layers)):
        close(got, ref, dtype, f"after layer {i}", 1e-4 if dtype == "float32" else 4e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_passes_windows_kept_tokens_and_page_borders(dtype):
    name = "TA"                                            # windows of 21 (+ 5 kept), 17 and 30 positions, one layer without a mask
    toks = random_tokens(CONFIGS[name]["vocab"], 200, seed=12)
    ref = plain(name, toks)
    eng = engine(name, dtype)
    s = eng.open_seq()
    rows = [eng.step([s], [toks[:3]], [[2]]).clone()]
    for p in range(3, len(toks)):
        rows.append(eng.step([s], [[toks[p]]]).clone())
    close(torch.cat(rows), ref[2:], dtype, "decoded")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["TA", "TB"])
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
            assert (g - alone[i][:g.shape[0]]).abs().max().item() <= 2e-5, f"request {i} differs in a batch"


def poison_free(eng):
    """NaN in every page that no sequence holds, in every paged group."""
    held = eng.cache.pages.held()
    free = [p for p in range(1, eng.cache.n_pages) if p not in held]
    for g in eng.cache.groups:
        if g.need.kind in ("paged_kv", "paged_rows") and free:
            g.storage[:, torch.tensor(free, device=g.storage.device)] = float("nan")


@pytest.mark.parametrize("dtype", DTYPES)
def test_pages_and_slots_that_were_given_back_are_used_again(dtype):
    name = "TB"
    cfg = CONFIGS[name]
    eng = engine(name, dtype, max_tokens=320)
    a, b = random_tokens(cfg["vocab"], 150, seed=31), random_tokens(cfg["vocab"], 140, seed=32)
    s1 = eng.open_seq()
    eng.step([s1], [a])
    s2 = eng.open_seq()
    eng.step([s2], [b[:70]])
    eng.close_seq(s1)                                      # its three pages and its slot come back
    poison_free(eng)
    s3 = eng.open_seq()
    assert s3 == s1
    out = eng.step([s3], [a[:100]], [list(range(100))])
    assert set(eng.cache.pages_of(s3)) & {1, 2, 3}
    close(out, plain(name, a[:100]), dtype, "in reused pages")
    rows = [eng.step([s2, s3], [[b[70 + i]], [a[100 + i]]]).clone() for i in range(30)]
    close(torch.stack([r[0] for r in rows]), plain(name, b[:100])[70:], dtype, "the request that stayed")
    close(torch.stack([r[1] for r in rows]), plain(name, a[:130])[100:], dtype, "the request in reused pages")
    eng.cache.check()


def _uniform_windows(cfg, size, keep):
    cfg = copy.deepcopy(cfg)
    for L in cfg["layers"]:
        L["mixer"]["mask"] = {"size": size, "keep_first": keep} if L["type"] == "attention" else {"size": size}
    return cfg


def test_a_far_token_shows_only_through_windows_or_as_a_kept_one():
    """Attention is the only path between positions.  With windows of 400 a change at position 7 shows at position 390;
    with windows of 90 in all four layers (reach 4 x 89) it cannot, unless the first 8 positions are kept."""
    outs = {}
    for tag, size, keep in (("wide", 400, 0), ("narrow", 90, 0), ("kept", 90, 8)):
        cfg = _uniform_windows(CONFIG_TA, size, keep)
        d = os.path.join(tmp_root(), f"tug-far-{tag}")
        w = write_model(cfg, d, seed=9, std=0.3)
        toks = random_tokens(cfg["vocab"], 391, seed=40)
        other = list(toks)
        other[7] = (toks[7] + 1) % cfg["vocab"]
        eng = wick.Engine.from_dir(d, dtype="float32", max_tokens=1024)
        res = []
        for t in (toks, other):
            s = eng.open_seq()
            eng.step([s], [t[:380]], [[]])
            for p in range(380, 390):
                eng.step([s], [[t[p]]])
            res.append(eng.step([s], [[t[390]]]).clone())
            eng.close_seq(s)
            close(res[-1], P.forward(cfg, w, t).float()[390:], "float32", tag)
        outs[tag] = (res[0] - res[1]).abs().max().item()
    assert outs["wide"] > 1e-4, "a change 383 tokens back, inside the windows, must show"
    assert outs["narrow"] == 0.0, "a change beyond the windows' reach must not show"
    assert outs["kept"] > 1e-4, "a change in a kept first token must show"


@pytest.mark.parametrize("name", ["TA", "TC"])
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


def test_the_command_line_writes_runs_and_times_the_design(tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root)
    cmd = [sys.executable, os.path.join(root, "bin", "wick")]
    cfg_path, d = str(tmp_path / "cfg.json"), str(tmp_path / "m")
    with open(cfg_path, "w") as f:
        json.dump(CONFIG_TA, f)
    r = subprocess.run(cmd + ["random", d, "--config", cfg_path, "--seed", "4"], capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr
    st = SafeTensorsDir(d)
    w = {n: st.get(n).tensor() for n in st.names()}
    prompts = [[5, 17, 3], [9, 9, 200, 1, 77, 3, 3, 14]]
    r = subprocess.run(cmd + ["run", d, "--ids", "5,17,3", "--ids", "9,9,200,1,77,3,3,14", "-n", "6", "-t", "0", "-q", "f32"],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr
    assert "Tuguvik" in r.stderr and "4 layers" in r.stderr
    lines = [json.loads(l) for l in r.stdout.strip().splitlines()]
    for p, toks in zip(prompts, lines):
        assert len(toks) == 6
        ref = P.forward(CONFIG_TA, w, p + toks).float()
        for i, t in enumerate(toks):
            row = ref[len(p) - 1 + i]
            assert row[t] >= row.max() - 1e-3, (p, i)
    # sampling with a temperature and a cut: the same seed gives the same tokens, all inside the vocabulary
    args = ["run", d, "--ids", "5,17,3", "-n", "12", "-t", "0.9", "--top-k", "20", "--seed", "7", "-q", "bf16"]
    a = subprocess.run(cmd + args, capture_output=True, text=True, env=env, timeout=600)
    b = subprocess.run(cmd + args, capture_output=True, text=True, env=env, timeout=600)
    assert a.returncode == 0 and a.stdout == b.stdout, a.stderr
    assert all(0 <= t < CONFIG_TA["vocab"] for t in json.loads(a.stdout.strip().splitlines()[0]))
    r = subprocess.run(cmd + ["bench", d, "--prompt-len", "16", "-n", "4", "--batch", "2", "-q", "bf16"],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0 and "tok/s" in r.stdout, r.stderr


def test_the_trace_runner_serves_the_design():
    name = "TA"
    d = model(name)[0]
    cfg = CONFIGS[name]
    a, b = random_tokens(cfg["vocab"], 70, seed=61), random_tokens(cfg["vocab"], 9, seed=62)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": a[:66], "want": [0, 65]}, {"id": "y", "tokens": b[:5], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": a[66:67], "want": [0]}, {"id": "y", "tokens": b[5:6], "want": [0]}], "end": ["y"]},
             {"step": 2, "entries": [{"id": "x", "tokens": a[67:68], "want": []}], "end": []},
             {"step": 3, "entries": [{"id": "x", "tokens": a[68:69], "want": [0]}], "end": ["x"]}]
    out = os.path.join(tmp_root(), "tug-trace-out")
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
