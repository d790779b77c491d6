"""Differential attention: two softmax maps per head over the same values, subtracted.

=============  ==========================  ======================================
category       kind                        params
=============  ==========================  ======================================
mixer          ``differential_attention``  width, heads, kv_heads, head_dim (of
                                           ONE map), v_dim, scale, diff, eps,
                                           position (PartSpec ``rotary_pairs``
                                           over a map, or None), mask (None or
                                           {"size": n, "keep_first": m}),
                                           names (q, k, v, o, lq1, lk1, lq2, lk2
                                           -> local names)
=============  ==========================  ======================================

For a token at position p with input h (H query heads, G key/value heads, query head i uses
key/value head floor(i / (H / G)), maps of size d, values of size e):

* q = Wq h has H heads of [map 1 | map 2] (2 d numbers), k = Wk h has G such heads,
  v = Wv h has G heads of e numbers; the position encoding turns every map on its own;
* map a of head i: scores (q_a . k_a) * scale over the keys j <= p with p - j < size or
  j < keep_first (no mask: every j <= p), an ordinary softmax, and the weighted sum y_a
  of the values: both maps weigh the same values;
* y = y_1 - lambda y_2 with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff, one number of
  the layer; then y / sqrt(mean(y^2) + eps) over the head's e numbers, times (1 - diff);
* the heads' results, side by side, go through Wo.

The cache holds a key head as the 2 d numbers of both maps and a value head beside it (the
paged key/value storage).  Scores, weights, sums, lambda and the head norm are float32.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..layout import PAGE
from ..models.spec import PartSpec
from .attention import RotaryPairs
from .base import CacheNeed, Mixer, TensorSpec, build_part, register_part
from .linear import Linear
from .standard import NoPosition


class DifferentialAttention(Mixer):
    PROMPT_CAPTURABLE = True
    MAPS = 2
    TENSOR_CORES_FROM = 16      # tokens of a prompt step from which its attention takes the tensor-core kernel

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        p = params
        self.width, self.heads, self.kv_heads = int(p["width"]), int(p["heads"]), int(p["kv_heads"])
        self.map_dim, self.v_dim = int(p["head_dim"]), int(p["v_dim"])
        self.head_dim = self.MAPS * self.map_dim
        if self.heads <= 0 or self.kv_heads <= 0 or self.heads % self.kv_heads != 0:
            raise ValueError("heads must be a positive multiple of kv_heads")
        if self.v_dim > ops.ATTN_MULTI_MAX_V:
            raise ValueError(f"the attention kernel takes values of up to {ops.ATTN_MULTI_MAX_V} elements, not {self.v_dim}")
        self.scale = float(p["scale"]) if p.get("scale") is not None else self.map_dim ** -0.5
        self.diff, self.eps = float(p["diff"]), float(p.get("eps", 0.0))
        mask = p.get("mask")
        self.window = int(mask["size"]) if mask else 0
        self.keep_first = int(mask.get("keep_first", 0)) if mask else 0
        if mask and self.window <= 0:
            raise ValueError(f"a window holds a positive number of positions, not {mask}")
        self.position = build_part("position", p.get("position") or PartSpec("none"), ctx)
        if not isinstance(self.position, (RotaryPairs, NoPosition)):
            raise ValueError("this mixer's kernel turns pairs (rotary_pairs) or nothing")
        if isinstance(self.position, RotaryPairs) and self.position.head_dim != self.map_dim:
            raise ValueError("the position encoding works on one map")
        names = dict(q="q_proj.weight", k="k_proj.weight", v="v_proj.weight", o="o_proj.weight", lq1="lambda_q1",
                     lk1="lambda_k1", lq2="lambda_q2", lk2="lambda_k2")
        names.update(p.get("names") or {})
        self.names = names
        self.q_dim, self.k_dim, self.v_all = self.heads * self.head_dim, self.kv_heads * self.head_dim, self.kv_heads * self.v_dim
        self.qkv = Linear(self.q_dim + self.k_dim + self.v_all, self.width, ctx)
        self.o = Linear(self.width, self.heads * self.v_dim, ctx)
        self.lambdas = {}
        self.lam = 0.0

    def tensor_specs(self):
        nm = self.names
        return [TensorSpec(nm["q"], (self.q_dim, self.width)), TensorSpec(nm["k"], (self.k_dim, self.width)),
                TensorSpec(nm["v"], (self.v_all, self.width)), TensorSpec(nm["o"], (self.width, self.heads * self.v_dim))] + \
               [TensorSpec(nm[k], (self.map_dim,), "vector", init="around_zero") for k in ("lq1", "lk1", "lq2", "lk2")]

    def load(self, fetch):
        nm = self.names
        self.qkv.load_rows([fetch(nm["q"]), fetch(nm["k"]), fetch(nm["v"])])
        self.o.load_rows([fetch(nm["o"])])
        self.lambdas = {k: self.ctx.hold(fetch(nm[k]), "vector") for k in ("lq1", "lk1", "lq2", "lk2")}
        # (one number of the layer, from its float32 vectors, made once)
        L = {k: v.to("cpu", torch.float32) for k, v in self.lambdas.items()}
        lam = torch.exp((L["lq1"] * L["lk1"]).sum()) - torch.exp((L["lq2"] * L["lk2"]).sum()) + torch.tensor(self.diff, dtype=torch.float32)
        self.lam = float(lam)

    def tensor(self, name):
        nm, q, k = self.names, self.q_dim, self.k_dim
        if name == nm["q"]:
            return self.qkv.rows(0, q)
        if name == nm["k"]:
            return self.qkv.rows(q, q + k)
        if name == nm["v"]:
            return self.qkv.rows(q + k, q + k + self.v_all)
        if name == nm["o"]:
            return self.o.rows(0, self.width)
        for key, t in self.lambdas.items():
            if name == nm[key]:
                return t
        return None

    def cache_need(self):
        return CacheNeed("paged_kv", kv_heads=self.kv_heads, head_dim=self.head_dim,
                         v_head_dim=None if self.v_dim == self.head_dim else self.v_dim)

    def weight_bytes(self):
        return self.qkv.weight_bytes() + self.o.weight_bytes()

    def forward(self, x, batch, cache, write_cache):
        n = x.shape[0]
        parts = self.qkv.forward_delta(x)                 # float32 [splits, n, 2 H d + 2 G d + G e]
        rot = self.position if isinstance(self.position, RotaryPairs) else None
        cos, sin = rot.tables(batch) if rot else (None, None)
        q = ops.qkv_finish(parts, self.heads, self.kv_heads, self.head_dim, self.v_dim, dtype=self.ctx.dtype,
                           cos=cos, sin=sin, rot_dims=rot.dims if rot else 0, pairing=rot.pairing if rot else "neighbours",
                           maps=self.MAPS, kv=cache.kv, page_table=batch.page_table, seq_of_token=batch.seq_of_token,
                           positions=batch.positions, write_kv=write_cache)
        combine = (self.lam, self.eps, 1.0 - self.diff)
        if n >= self.TENSOR_CORES_FROM and not batch.is_decode and ops.attention_flex_supported(self.map_dim, self.v_dim, self.ctx.dtype):
            # a prompt's tokens: every map of every head is a head of its own for the tensor-core kernel (its keys one
            # half of a cached key row, its values the head's), and a second kernel combines the two results of a head
            G, d, e = self.kv_heads, self.head_dim, self.v_dim
            page, per = G * PAGE * (d + e), self.MAPS * (self.heads // G)
            k0 = ops.flex_source(cache.kv, tile_elems=page, hdiv=per, hmul=PAGE * d, hmod=self.MAPS, hmul2=self.map_dim,
                                 row_stride=d, length=self.map_dim, paged=True)
            v = ops.flex_source(cache.kv, tile_elems=page, const_off=G * PAGE * d, hdiv=per, hmul=PAGE * e, row_stride=e, length=e,
                                paged=True)
            maps = ops.attention_flex(q.view(n, self.MAPS * self.heads, self.map_dim), k0, ops.flex_source(), v, batch, self.scale,
                                      dv=e, window=self.window, keep_first=self.keep_first, out_dtype=torch.float32)
            att = ops.combine_maps(maps.view(n, self.heads, self.MAPS, e), *combine, lib=(self.map_dim, e))
        else:
            att = ops.attention_multi(q, cache.kv, batch, self.scale, maps=self.MAPS, kv_heads=self.kv_heads, v_dim=self.v_dim,
                                      window=self.window, keep_first=self.keep_first, combine=combine, out_dtype=self.ctx.dtype)
        return self.o.forward_delta(att.view(n, self.heads * self.v_dim))


register_part("mixer", "differential_attention", DifferentialAttention)
