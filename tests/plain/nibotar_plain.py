"""A plain, slow implementation of the Nibotar decoder, one function per mechanism.

Written from the design's equations in torch on the CPU (float64 by default), it
shares no code with the package: it takes the ``config.json`` dictionary and a
dictionary of tensors by checkpoint name, and runs whole sequences at once.

Notation: n tokens, width D, H query heads, G key/value heads, head size d (keys
and queries) and e (values), positions p counted from 0.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """RMS norm whose stored weight lies around zero: rms(x) * (1 + w)."""
    return rms(x, eps) * (1.0 + w)


def norm_plain_weight(x, w, eps):
    """RMS norm over the whole vector with an ordinary weight."""
    return rms(x, eps) * w


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [n, heads, d]: the first ``dims`` elements of every head are rotated as
    neighbouring pairs (2i, 2i+1) by the angle p * base^(-2i/dims); the rest pass."""
    out = x.clone()
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        a = positions.to(x.dtype) * f
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def chunk_visible(n: int, size: Optional[int], offset: int = 0) -> torch.Tensor:
    """[n, n] bool: query i sees key j iff j <= i and both lie in the same block of
    ``size`` positions counted from position 0 (size None: every earlier key)."""
    p = torch.arange(offset, offset + n)
    vis = p[None, :] <= p[:, None]
    if size is not None:
        vis &= (p[None, :] // size) == (p[:, None] // size)
    return vis


def sink_softmax_mix(scores: torch.Tensor, visible: torch.Tensor, sink: Optional[torch.Tensor],
                     v: torch.Tensor) -> torch.Tensor:
    """scores [H, n, n] (already scaled), visible [n, n], sink [H] or None, v [H, n, e].
    The weights are exp(s_j) / (sum over visible j of exp(s_j) + exp(sink)): the sink
    adds to the denominator only."""
    s = scores.masked_fill(~visible[None], -math.inf)
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink[:, None, None] - m)
    return (e / den) @ v


def mix_values(v: torch.Tensor, v_first: torch.Tensor, lam: torch.Tensor) -> torch.Tensor:
    return (1.0 - lam) * v + lam * v_first


def attention_mixer(h, t: Dict[str, torch.Tensor], pre: str, m: dict, eps: float, positions,
                    v_first: Optional[torch.Tensor]):
    """Returns (output [n, D], the values this layer caches [n, G*e])."""
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    q = h @ t[pre + "q"].T + t[pre + "q.b"]
    k = h @ t[pre + "k"].T + t[pre + "k.b"]
    v = h @ t[pre + "v"].T + t[pre + "v.b"]
    q = norm_plain_weight(q, t[pre + "q.norm"], eps)
    k = norm_plain_weight(k, t[pre + "k.norm"], eps)
    rot = m.get("rot")
    q, k = q.view(n, H, d), k.view(n, G, d)
    if rot:
        q = rotate_pairs(q, positions, rot["dims"], rot["base"])
        k = rotate_pairs(k, positions, rot["dims"], rot["base"])
    if m.get("v_mix") and v_first is not None:
        v = mix_values(v, v_first, t[pre + "vmix"])
    vh = v.view(n, G, e)
    rep = H // G
    kh = k.permute(1, 0, 2).repeat_interleave(rep, 0)            # [H, n, d]
    vv = vh.permute(1, 0, 2).repeat_interleave(rep, 0)           # [H, n, e]
    scores = (q.permute(1, 0, 2) @ kh.transpose(1, 2)) * m["scale"]
    size = (m.get("mask") or {}).get("size")
    vis = chunk_visible(n, size, int(positions[0]))
    o = sink_softmax_mix(scores, vis, t.get(pre + "sink"), vv)   # [H, n, e]
    o = o.permute(1, 0, 2).reshape(n, H * e)
    return o @ t[pre + "o"].T, v


def relu2_ffn(h, up, down):
    z = torch.relu(h @ up.T)
    return (z * z) @ down.T


def gated_expert(h, gate, up, down):
    g = h @ gate.T
    return ((g * torch.sigmoid(g)) * (h @ up.T)) @ down.T


def table_moe(h, tokens, t, pre, mlp):
    """Every token id owns ``top`` experts by a table; each weighs 1/top; a shared expert is added."""
    top = mlp["router"]["top"]
    table = t[pre + "table"].long()
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        for e in table[int(tokens[i])].tolist():
            p = f"{pre}e{e}."
            out[i] += gated_expert(h[i:i + 1], t[p + "gate"], t[p + "up"], t[p + "down"])[0] / top
    if mlp.get("shared"):
        p = pre + "shared."
        out = out + gated_expert(h, t[p + "gate"], t[p + "up"], t[p + "down"])
    return out


def feed_forward(h, tokens, t, pre, mlp):
    if mlp["kind"] == "dense":
        return relu2_ffn(h, t[pre + "up"], t[pre + "down"])
    if mlp["kind"] == "moe":
        return table_moe(h, tokens, t, pre, mlp)
    raise ValueError(mlp["kind"])


def softcap(z, cap):
    return cap * torch.tanh(z / cap)


def forward(config: dict, tensors: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            return_layers: bool = False):
    """Logits [n, vocab] of one sequence from position 0 (and the stream after every layer)."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps, alpha = config["norm"]["eps"], config["postln_alpha"]
    tok = torch.tensor(tokens, dtype=torch.long)
    pos = torch.arange(len(tokens))
    x = t["embed"][tok]
    v_first = None
    layers = []
    for i, L in enumerate(config["layers"]):
        if L["type"] != "attention":
            raise ValueError(L["type"])
        pre = f"l{i}."
        mixes = bool(L["mixer"].get("v_mix"))
        a, v = attention_mixer(x, t, pre + "mix.", L["mixer"], eps, pos, v_first if mixes else None)
        if mixes and v_first is None:
            v_first = v
        x = norm_one_plus(alpha * x + a, t[pre + "norm1"], eps)
        if L.get("mlp") is not None:
            x = norm_one_plus(alpha * x + feed_forward(x, tok, t, pre + "mlp.", L["mlp"]), t[pre + "norm2"], eps)
        layers.append(x)
    z = norm_one_plus(x, t["final.norm"], eps) @ t["head"].T
    cap = config.get("logit_softcap")
    if cap:
        z = softcap(z, cap)
    return (z, torch.stack(layers)) if return_layers else z
