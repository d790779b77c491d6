"""A plain, slow implementation of the Tuguvik decoder, one function per mechanism.

Written from the design's equations in torch on the CPU (float64 by default), it
shares no code with the package: it takes the ``config.json`` dictionary and a
dictionary of tensors by checkpoint name, and runs one whole sequence at once
(every score matrix is [n, n]).

Notation: n tokens, width D, H query heads, positions p counted from 0, query i,
key j.  A layer:

    x <- x + s1 * M(N1(x));   x <- x + s2 * F(N2(x));   x <- x + T(x, token)

with N(v) = tanh(a v) * w + b (a one number), s1 and s2 vectors of D numbers, M one
of two mixers, F a gated feed-forward, and T the layer's token input.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


# ---- norms -------------------------------------------------------------------
def tanh_norm(x, w, b, a):
    """tanh(a x) * w + b: no mean, no variance."""
    return torch.tanh(a * x) * w + b


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ---- rotation frequencies ----------------------------------------------------
def base_frequencies(dims: int, base: float) -> List[float]:
    return [base ** (-2.0 * i / dims) for i in range(dims // 2)]


def frequencies_by_wavelength(dims: int, base: float, sc: Optional[dict]) -> List[float]:
    """Scaling by wavelength l = 2 pi / f: short waves (l < original / high) stay, long ones
    (l > original / low) are divided by ``factor``, those between are blended."""
    out = []
    for f in base_frequencies(dims, base):
        if sc:
            l = 2.0 * math.pi / f
            if l < sc["original"] / sc["high"]:
                pass
            elif l > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            else:
                s = (sc["original"] / l - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        out.append(f)
    return out


def frequencies_by_ramp(dims: int, base: float, sc: Optional[dict]):
    """Scaling by a ramp over the pair index; returns (frequencies, amplitude of cos and sin)."""
    fs = base_frequencies(dims, base)
    if not sc:
        return fs, 1.0

    def index_of(turns):
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(sc["fast"])), 0)
    hi = min(math.ceil(index_of(sc["slow"])), dims - 1)
    out = []
    for i, f in enumerate(fs):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / sc["factor"] * r + f * (1.0 - r))
    return out, 0.1 * math.log(sc["factor"]) + 1.0


def turn_neighbours(x, positions, freqs, amplitude=1.0):
    """x [n, heads, dims]: the pair (2i, 2i+1) turns by p * f_i."""
    out = x.clone()
    for i, f in enumerate(freqs):
        a = positions.to(x.dtype) * f
        c, s = (torch.cos(a) * amplitude)[:, None], (torch.sin(a) * amplitude)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def turn_halves(x, positions, freqs):
    """x [n, heads, dims]: the pair (i, i + dims/2) turns by p * f_i."""
    half = len(freqs)
    out = x.clone()
    for i, f in enumerate(freqs):
        a = positions.to(x.dtype) * f
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


# ---- visibility --------------------------------------------------------------
def window_visible(n: int, size: Optional[int], keep_first: int = 0) -> torch.Tensor:
    """[n, n] bool: i sees j iff j <= i and (i - j < size or j < keep_first)."""
    p = torch.arange(n)
    i, j = p[:, None], p[None, :]
    vis = j <= i
    if size is not None:
        vis &= ((i - j) < size) | (j < keep_first)
    return vis


def softmax_visible(scores, visible, sink=None):
    """scores [H, n, n]; a sink [H] is one more term exp(sink) in the denominator."""
    s = scores.masked_fill(~visible[None], -math.inf)
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink[:, None, None])
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink[:, None, None] - m)
    return e / den


# ---- mixer: attention through a latent --------------------------------------
def latent_kv(h, t, pre, m, eps, positions):
    """What a layer with a down-projection of its own caches: the normed latent [n, r] and
    the turned key part [n, dr] that all heads share."""
    r, dr = m["kv_rank"], m["rot_dim"]
    z = h @ t[pre + "dkv"].T
    c = unit_rms(z[:, :r], eps) * t[pre + "dkv.norm"]
    freqs, amp = frequencies_by_ramp(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    k_rot = turn_neighbours(z[:, None, r:r + dr], positions, freqs, amp)[:, 0]
    return c, k_rot


def latent_attention(h, t, pre, m, eps, positions, shared_kv):
    H, d, dr, e = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    n = h.shape[0]
    c, k_rot = shared_kv
    cq = unit_rms(h @ t[pre + "dq"].T, eps) * t[pre + "dq.norm"]
    q = (cq @ t[pre + "uq"].T).view(n, H, d + dr)
    freqs, amp = frequencies_by_ramp(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    q_flat, q_rot = q[..., :d], turn_neighbours(q[..., d:], positions, freqs, amp)
    k_flat = (c @ t[pre + "uk"].T).view(n, H, d)
    v = (c @ t[pre + "uv"].T).view(n, H, e)
    scores = (torch.einsum("ihd,jhd->hij", q_flat, k_flat) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    vis = window_visible(n, (m.get("mask") or {}).get("size"))
    w = softmax_visible(scores, vis, t[pre + "sink"])
    o = torch.einsum("hij,jhe->ihe", w, v)
    gate = torch.sigmoid(h @ t[pre + "g"].T)                    # [n, H]
    o = o * gate[:, :, None]
    return o.reshape(n, H * e) @ t[pre + "o"].T


# ---- mixer: differential attention --------------------------------------------
def differential_attention(h, t, pre, m, eps, positions):
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    q = (h @ t[pre + "q"].T).view(n, H, 2, d)
    k = (h @ t[pre + "k"].T).view(n, G, 2, d)
    v = (h @ t[pre + "v"].T).view(n, G, e)
    rot = m.get("rot")
    if rot:
        freqs = frequencies_by_wavelength(rot["dims"], rot["base"], rot.get("scaling"))
        dims = rot["dims"]
        q = torch.cat([turn_halves(q[..., :dims].reshape(n, 2 * H, dims), positions, freqs).view(n, H, 2, dims),
                       q[..., dims:]], -1)
        k = torch.cat([turn_halves(k[..., :dims].reshape(n, 2 * G, dims), positions, freqs).view(n, G, 2, dims),
                       k[..., dims:]], -1)
    rep = H // G
    kk = k.repeat_interleave(rep, 1)                            # [n, H, 2, d]
    vv = v.repeat_interleave(rep, 1)                            # [n, H, e]
    mask = m.get("mask") or {}
    vis = window_visible(n, mask.get("size"), mask.get("keep_first", 0))
    maps = []
    for a in range(2):
        s = torch.einsum("ihd,jhd->hij", q[:, :, a], kk[:, :, a]) * m["scale"]
        maps.append(torch.einsum("hij,jhe->ihe", softmax_visible(s, vis), vv))
    lam = torch.exp((t[pre + "lq1"] * t[pre + "lk1"]).sum()) - torch.exp((t[pre + "lq2"] * t[pre + "lk2"]).sum()) + m["diff"]
    o = maps[0] - lam * maps[1]
    o = unit_rms(o, eps) * (1.0 - m["diff"])
    return o.reshape(n, H * e) @ t[pre + "o"].T


# ---- feed-forward and token input ----------------------------------------------
def gated_ffn(h, gate, up, down):
    g = h @ gate.T
    return ((g * torch.sigmoid(g)) * (h @ up.T)) @ down.T


def token_input(x, rows, t, pre, eps):
    """rows [n, ds]: this layer's part of the tokens' rows of the side table."""
    g = gelu_tanh(x @ t[pre + "gate"].T) * rows
    y = g @ t[pre + "proj"].T
    return unit_rms(y, eps) * t[pre + "norm"]


# ---- the model -------------------------------------------------------------------
def forward(config: dict, tensors: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            return_layers: bool = False):
    """Logits [n, vocab] of one sequence from position 0 (and the stream after every layer)."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    side = config.get("token_side")
    tok = torch.tensor(tokens, dtype=torch.long)
    pos = torch.arange(len(tokens))
    x = t["embed"][tok]

    def norm(v, name):
        return tanh_norm(v, t[name], t[name + ".b"], t[name + ".alpha"])

    kv_of = {}
    layers = []
    for i, L in enumerate(config["layers"]):
        pre, m = f"l{i}.", L["mixer"]
        h = norm(x, pre + "norm1")
        if L["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                kv_of[i] = latent_kv(h, t, pre + "mix.", m, eps, pos)
                src = i
            a = latent_attention(h, t, pre + "mix.", m, eps, pos, kv_of[src])
        elif L["type"] == "attention":
            a = differential_attention(h, t, pre + "mix.", m, eps, pos)
        else:
            raise ValueError(L["type"])
        x = x + t[pre + "ls1"] * a
        if L.get("mlp") is not None:
            if L["mlp"]["kind"] != "dense":
                raise ValueError(L["mlp"]["kind"])
            p = pre + "mlp."
            x = x + t[pre + "ls2"] * gated_ffn(norm(x, pre + "norm2"), t[p + "gate"], t[p + "up"], t[p + "down"])
        if side:
            ds = side["dim"]
            x = x + token_input(x, t["side.embed"][tok][:, i * ds:(i + 1) * ds], t, pre + "side.", eps)
        layers.append(x)
    z = norm(x, "final.norm") @ t["head"].T
    return (z, torch.stack(layers)) if return_layers else z
