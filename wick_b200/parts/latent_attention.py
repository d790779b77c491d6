"""Attention whose keys and values are made from a cached latent.

=============  ======================  ==========================================
category       kind                    params
=============  ======================  ==========================================
mixer          ``latent_attention``    width, heads, head_dim (unrotated query /
                                       key elements of a head), rot_dim (rotated
                                       ones), v_dim, q_rank, kv_rank, scale, eps,
                                       position (PartSpec ``rotary_pairs`` over
                                       rot_dim elements, or None), window (None
                                       or positions), sink, gate, own_kv,
                                       names (dq, dq_norm, uq, dkv, dkv_norm, uk,
                                       uv, sink, gate, o -> local names)
=============  ======================  ==========================================

For a token at position p with input h (H heads, d unrotated and dr rotated query / key
elements, values of size e, latent of r numbers):

* cq = rms(Wdq h) * wq, then q = Wuq cq: per head [d unrotated | dr rotated] numbers;
* Wdkv h has r + dr numbers: c = rms(first r) * wkv is the latent, the last dr, turned by
  the position encoding, are the rotated key part that all heads share; c and that part
  are all the cache holds for the position (one row of r + dr numbers);
* head i's key at position j is [Wuk_i c_j | rotated part_j], its value Wuv_i c_j; the
  score is (q . key) * scale over the keys with 0 <= p - j < window; the weights are
  exp(s_j) / (sum exp(s_j) + exp(sink_i));
* the head's result is multiplied by sigmoid(Wg h)_i; Wo follows.

A layer with ``own_kv`` False has no Wdkv: it is scheduled to read the cache of an earlier
layer, and applies its own Wuk and Wuv to that layer's rows.

Two forms compute this.  A step over cached rows (decoding, a prompt's later portion, the
32-bit path) never expands a row into keys and values: since q_i . (Wuk_i c) =
(Wuk_i^T q_i) . c, a head's query is carried into the latent's space once per token
([Wuk_i^T q_i | rotated q_i], r + dr numbers), the attention runs over the cached rows
themselves as one shared key head whose first r numbers are also the value, and Wuv_i is
applied to the weighted sum of rows; query in latent space, scores, weights and the sum
are float32.  A bfloat16 prompt from position 0 (launched, not replayed from a captured
step) makes the step's own keys and values once, [Wuk; Wuv] c as one matrix product, and
runs the tensor-core attention over them and the shared key part, with the gate in its
epilogue; the layer that owns the rows leaves the step's latents in the step's memo for a
layer that reads its cache.
"""
from __future__ import annotations

import torch

from .. import ops
from ..models.spec import PartSpec
from .attention import RotaryPairs
from .base import CacheNeed, Mixer, TensorSpec, build_part, register_part
from .linear import Linear
from .standard import NoPosition


class LatentAttention(Mixer):
    PROMPT_CAPTURABLE = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        p = params
        self.width, self.heads = int(p["width"]), int(p["heads"])
        self.head_dim, self.rot_dim, self.v_dim = int(p["head_dim"]), int(p["rot_dim"]), int(p["v_dim"])
        self.q_rank, self.kv_rank = int(p["q_rank"]), int(p["kv_rank"])
        if self.kv_rank > ops.ATTN_MULTI_MAX_V:
            raise ValueError(f"the attention kernel takes a latent of up to {ops.ATTN_MULTI_MAX_V} numbers, not {self.kv_rank}")
        self.row = self.kv_rank + self.rot_dim
        self.scale = float(p["scale"]) if p.get("scale") is not None else (self.head_dim + self.rot_dim) ** -0.5
        self.eps = float(p.get("eps", 0.0))
        self.window = int(p.get("window") or 0)
        self.has_sink, self.has_gate, self.own_kv = bool(p.get("sink", False)), bool(p.get("gate", False)), bool(p.get("own_kv", True))
        self.position = build_part("position", p.get("position") or PartSpec("none"), ctx)
        if not isinstance(self.position, (RotaryPairs, NoPosition)):
            raise ValueError("this mixer's kernel turns pairs (rotary_pairs) or nothing")
        if isinstance(self.position, RotaryPairs) and (self.position.head_dim != self.rot_dim or self.position.dims != self.rot_dim):
            raise ValueError("the position encoding turns the whole rotated part")
        names = dict(dq="q_a_proj.weight", dq_norm="q_a_norm.weight", uq="q_b_proj.weight", dkv="kv_a_proj.weight",
                     dkv_norm="kv_a_norm.weight", uk="k_b_proj.weight", uv="v_b_proj.weight", sink="sinks", gate="gate.weight",
                     o="o_proj.weight")
        names.update(p.get("names") or {})
        self.names = names
        # one product for everything that reads h: [dq | dkv (own_kv) | gate (gate)]
        self.kv_rows = self.row if self.own_kv else 0
        self.down = Linear(self.q_rank + self.kv_rows + (self.heads if self.has_gate else 0), self.width, ctx)
        self.uq = Linear(self.heads * (self.head_dim + self.rot_dim), self.q_rank, ctx)
        self.o = Linear(self.width, self.heads * self.v_dim, ctx)
        self.uk = self.uv = self.q_weight = self.kv_weight = self.sink = None
        self.ukv = Linear(self.heads * (self.head_dim + self.v_dim), self.kv_rank, ctx)     # [Wuk; Wuv] for prompts

    def tensor_specs(self):
        nm, H = self.names, self.heads
        specs = [TensorSpec(nm["dq"], (self.q_rank, self.width)), TensorSpec(nm["dq_norm"], (self.q_rank,), "vector"),
                 TensorSpec(nm["uq"], (H * (self.head_dim + self.rot_dim), self.q_rank))]
        if self.own_kv:
            specs += [TensorSpec(nm["dkv"], (self.row, self.width)), TensorSpec(nm["dkv_norm"], (self.kv_rank,), "vector")]
        specs += [TensorSpec(nm["uk"], (H * self.head_dim, self.kv_rank)), TensorSpec(nm["uv"], (H * self.v_dim, self.kv_rank))]
        if self.has_sink:
            specs.append(TensorSpec(nm["sink"], (H,), "vector", init="around_zero"))
        if self.has_gate:
            specs.append(TensorSpec(nm["gate"], (H, self.width)))
        specs.append(TensorSpec(nm["o"], (self.width, H * self.v_dim)))
        return specs

    def load(self, fetch):
        nm, hold = self.names, self.ctx.hold
        rows = [fetch(nm["dq"])] + ([fetch(nm["dkv"])] if self.own_kv else []) + ([fetch(nm["gate"])] if self.has_gate else [])
        self.down.load_rows(rows)
        self.uq.load_rows([fetch(nm["uq"])])
        self.o.load_rows([fetch(nm["o"])])
        self.uk, self.uv = hold(fetch(nm["uk"]), "matrix"), hold(fetch(nm["uv"]), "matrix")
        self.expands = ops.attention_flex_supported(self.head_dim + self.rot_dim, self.v_dim, self.ctx.dtype) and self.uk.is_cuda \
            and self.head_dim % 8 == 0 and self.rot_dim % 8 == 0 and self.kv_rank % 8 == 0
        if self.expands:                                   # (held a second time, in the matrix product's own layout)
            self.ukv.use(torch.cat([self.uk, self.uv], 0))
        self.q_weight = hold(fetch(nm["dq_norm"]), "vector")
        self.kv_weight = hold(fetch(nm["dkv_norm"]), "vector") if self.own_kv else None
        self.sink = hold(fetch(nm["sink"]), "vector") if self.has_sink else None

    def tensor(self, name):
        nm, a, b = self.names, self.q_rank, self.q_rank + self.kv_rows
        held = {nm["uk"]: self.uk, nm["uv"]: self.uv, nm["dq_norm"]: self.q_weight}
        if self.own_kv:
            held[nm["dkv_norm"]] = self.kv_weight
        if self.has_sink:
            held[nm["sink"]] = self.sink
        if name in held:
            return held[name]
        if name == nm["dq"]:
            return self.down.rows(0, a)
        if self.own_kv and name == nm["dkv"]:
            return self.down.rows(a, b)
        if self.has_gate and name == nm["gate"]:
            return self.down.rows(b, b + self.heads)
        if name == nm["uq"]:
            return self.uq.rows(0, self.uq.out_features)
        return self.o.rows(0, self.width) if name == nm["o"] else None

    def cache_need(self):
        return CacheNeed("paged_rows", shape=(self.row,)) if self.own_kv else None

    def weight_bytes(self):
        el = 2 if self.ctx.dtype == torch.bfloat16 else 4
        return self.down.weight_bytes() + self.uq.weight_bytes() + self.o.weight_bytes() + \
            self.heads * (self.head_dim + self.v_dim) * self.kv_rank * el

    TENSOR_CORES_FROM = 16      # tokens of a prompt step from which its attention takes the tensor-core kernel

    def _from_position_zero(self, batch) -> bool:
        """Whether the step is a launched prompt step whose sequences all start at position 0 (a captured step's host
        lists describe no real prompt: it takes the other form)."""
        return (not batch.is_decode and batch.q_tiles is None and batch.n_tokens >= self.TENSOR_CORES_FROM
                and all(s == 0 for s in batch.starts))

    def forward(self, x, batch, cache, write_cache):
        n, H = x.shape[0], self.heads
        if cache is None or getattr(cache, "rows", None) is None:
            raise RuntimeError("this layer has no cached rows to read: its schedule entry must name the entry whose cache it reads")
        parts = self.down.forward_delta(x)                # float32 [splits, n, q_rank (+ r + dr) (+ H)]
        rot = self.position if isinstance(self.position, RotaryPairs) else None
        cos, sin = rot.tables(batch) if rot else (None, None)
        expand = self.expands and self._from_position_zero(batch)
        memo_key = ("latent_rows", cache.rows.data_ptr())
        writes = write_cache and self.own_kv
        res = ops.latent_finish(parts, self.q_rank, self.kv_rank if self.own_kv else 0, self.rot_dim if self.own_kv else 0,
                                H if self.has_gate else 0, dtype=self.ctx.dtype, q_weight=self.q_weight,
                                kv_weight=self.kv_weight, eps=self.eps, cos=cos, sin=sin,
                                rows=cache.rows if writes else None, page_table=batch.page_table,
                                seq_of_token=batch.seq_of_token, positions=batch.positions, flat=writes and self._from_position_zero(batch))
        cq, gate = res[0], res[1]
        if len(res) == 4:
            batch.memo[memo_key] = (res[2], res[3])       # the step's own latents and key parts, for this layer and its readers
        q = self.uq.forward_delta(cq)                     # float32 [splits, n, H (d + dr)]
        if expand and memo_key in batch.memo:
            c, kr = batch.memo[memo_key]
            d, e, dr = self.head_dim, self.v_dim, self.rot_dim
            qb = ops.latent_query(q, H, d, dr, cos=cos, sin=sin, dtype=self.ctx.dtype)
            kv = self.ukv.forward(c, self.ctx.dtype)      # [n, H d + H e]: every head's unrotated keys, then every head's values
            k0 = ops.flex_source(kv, hmul=d, row_stride=H * (d + e), length=d)
            k1 = ops.flex_source(kr, row_stride=dr, length=dr) if dr else ops.flex_source()
            v = ops.flex_source(kv, const_off=H * d, hmul=e, row_stride=H * (d + e), length=e)
            out = ops.attention_flex(qb, k0, k1, v, batch, self.scale, dv=e, window=self.window, sink=self.sink, gate=gate)
            return self.o.forward_delta(out.view(n, H * e))
        q_lat = ops.latent_absorb(q, self.uk, H, self.head_dim, self.rot_dim, self.kv_rank, cos=cos, sin=sin)
        att = ops.attention_multi(q_lat, cache.rows, batch, self.scale, maps=1, kv_heads=1, v_dim=self.kv_rank,
                                  window=self.window, sink=self.sink, rows_of=self.row, out_dtype=torch.float32)
        out = ops.latent_expand(att, self.uv, gate, H, self.v_dim, self.kv_rank, dtype=self.ctx.dtype)
        return self.o.forward_delta(out)


register_part("mixer", "latent_attention", LatentAttention)
