"""Plain restatement of the Zudarax decoder (test infrastructure; nothing under vllm_neuron_b200/ imports it).

Zudarax is a decoder with PARALLEL residual branches: one grouped RMS norm per layer, h = N(x), feeds both the mixer and
the feed-forward, and x += mixer(h) + ff(h).  The mixers are three kinds of attention:
  * 'attention'   -- biased q / k / v projections, a short causal convolution on each, an RMS norm over the WHOLE q (and k)
                     projection, partial rotate-half rotary positions, soft-capped scores, a chunked causal mask, softmax;
  * 'attention_2' -- differential attention: two softmax maps per head over the same values, a1 - lambda a2, a weightless
                     per-head RMS norm times (1 - diff), a per-head sigmoid output gate;
  * 'attention_3' -- short convolutions, YaRN-blended rotary angles, causal, and sigmoid(score + per-head bias) weights that
                     are NOT normalised over the keys.
Feed-forward: W_down PolyNorm(W_up h).  One function per mechanism, whole sequences, no cache: a token's output depends
on earlier tokens only, so every way of cutting a sequence into engine steps must reproduce `forward` on the full list.
`dtype` float64 gives the reference values.  `cfg` is the configuration in its file form (a dict).
"""
from __future__ import annotations

import math

import torch


def rms_unit(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def group_rms_norm(x, w, groups, eps):
    """x [T, W] cut into `groups` equal consecutive parts, each scaled to unit RMS on its own; then the whole times w."""
    T, W = x.shape
    return rms_unit(x.view(T, groups, W // groups), eps).reshape(T, W) * w


def short_conv(u, w):
    """u [T, C]; w [C, taps], the last column multiplies the current token; zeros before the start; no bias, no activation."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([u.new_zeros(taps - 1, C), u])
    out = u.new_zeros(T, C)
    for j in range(taps):
        out = out + pad[j : j + T] * w[:, j]
    return out


def rotary_frequencies(rot, dtype):
    """f_i = base^(-2i/dims) for the dims/2 pairs; with `scaling` each is blended with f_i / factor by a linear ramp over the
    pair index between the pairs that make `fast` and `slow` full turns within `original` positions.  Returns (f, magnitude)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    mag = 1.0
    if sc:
        def pair_of(turns):
            return dims * math.log(sc["original"] / (2 * math.pi * turns)) / (2 * math.log(base))

        lo = max(math.floor(pair_of(sc["fast"])), 0)
        hi = min(math.ceil(pair_of(sc["slow"])), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
        f = f / sc["factor"] * ramp + f * (1 - ramp)
        mag = 0.1 * math.log(sc["factor"]) + 1.0
    return f, mag


def rotate_half(x, rot):
    """x [T, heads, D]: column i < dims/2 is paired with column i + dims/2; (u, v) -> (u cos - v sin, v cos + u sin) at angle
    position * f_i; columns from `dims` on pass unchanged."""
    T, _, D = x.shape
    dims = int(rot["dims"])
    half = dims // 2
    f, mag = rotary_frequencies(rot, x.dtype)
    a = torch.arange(T, dtype=x.dtype)[:, None] * f
    c, s = (torch.cos(a) * mag)[:, None, :], (torch.sin(a) * mag)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def visible(T, chunk=None):
    """[T, T] bool: key j <= query i, and in the same chunk of `chunk` positions counted from 0 when chunked."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if chunk:
        m = m & (i // chunk == j // chunk)
    return m


def softmax_attention(q, k, v, scale, mask, softcap=None):
    """q [T, H, D], k [T, G, D], v [T, Gv, P] with H a multiple of G and of Gv -> [T, H, P]."""
    T, H, D = q.shape
    out = q.new_zeros(T, H, v.shape[2])
    for h in range(H):
        s = (q[:, h] @ k[:, h // (H // k.shape[1])].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~mask, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, h // (H // v.shape[1])]
    return out


def sigmoid_attention(q, k, v, scale, mask, bias):
    """Weights sigmoid(score + bias[h]) on the visible keys, zero elsewhere; no normalisation over keys."""
    T, H, D = q.shape
    out = q.new_zeros(T, H, v.shape[2])
    for h in range(H):
        g = h // (H // k.shape[1])
        s = (q[:, h] @ k[:, g].T) * scale + bias[h]
        out[:, h] = (torch.sigmoid(s) * mask) @ v[:, g]
    return out


def chunked_attention_mixer(h, W, p, m, eps):
    """The 'attention' mixer."""
    T = h.shape[0]
    H, G, D, P = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = (h @ W[p + n].T + W[p + n + ".b"] for n in "qkv")
    if m.get("conv"):
        q, k, v = (short_conv(u, W[p + n + ".conv"]) for u, n in ((q, "q"), (k, "k"), (v, "v")))
    q = rms_unit(q, eps) * W[p + "q.norm"]   # over all heads' rows at once
    k = rms_unit(k, eps) * W[p + "k.norm"]
    q, k = rotate_half(q.view(T, H, D), m["rot"]), rotate_half(k.view(T, G, D), m["rot"])
    mask = visible(T, (m.get("mask") or {}).get("size"))
    a = softmax_attention(q, k, v.view(T, G, P), m["scale"], mask, m.get("softcap"))
    return a.reshape(T, H * P) @ W[p + "o"].T


def differential_attention_mixer(h, W, p, m, eps):
    """The 'attention_2' mixer: per head  o = a1 - lambda a2,  lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff."""
    T = h.shape[0]
    H, G, D, P, diff = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["diff"]
    q = (h @ W[p + "q"].T).view(T, H, 2, D)
    k = (h @ W[p + "k"].T).view(T, G, 2, D)
    v = (h @ W[p + "v"].T).view(T, G, P)
    mask = visible(T)
    a = []
    for part in range(2):
        qm, km = rotate_half(q[:, :, part], m["rot"]), rotate_half(k[:, :, part], m["rot"])
        a.append(softmax_attention(qm, km, v, m["scale"], mask))
    lam = torch.exp((W[p + "lq1"] * W[p + "lk1"]).sum()) - torch.exp((W[p + "lq2"] * W[p + "lk2"]).sum()) + diff
    o = rms_unit(a[0] - lam * a[1], eps) * (1 - diff)
    o = o * torch.sigmoid(h @ W[p + "g"].T)[:, :, None]
    return o.reshape(T, H * P) @ W[p + "o"].T


def sigmoid_attention_mixer(h, W, p, m, eps):
    """The 'attention_3' mixer."""
    T = h.shape[0]
    H, G, D, P = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = (h @ W[p + n].T for n in "qkv")
    if m.get("conv"):
        q, k, v = (short_conv(u, W[p + n + ".conv"]) for u, n in ((q, "q"), (k, "k"), (v, "v")))
    q, k = rotate_half(q.view(T, H, D), m["rot"]), rotate_half(k.view(T, G, D), m["rot"])
    a = sigmoid_attention(q, k, v.view(T, G, P), m["scale"], visible(T), W[p + "pb"])
    return a.reshape(T, H * P) @ W[p + "o"].T


def poly_norm(z, coef, eps):
    """a N(z) + b N(z^2) + c N(z^3) + e with elementwise powers, N = division by the row's RMS."""
    a, b, c, e = coef
    return a * rms_unit(z, eps) + b * rms_unit(z * z, eps) + c * rms_unit(z * z * z, eps) + e


def feed_forward(h, W, p, eps):
    return poly_norm(h @ W[p + "up"].T, W[p + "act"], eps) @ W[p + "down"].T


MIXERS = {"attention": chunked_attention_mixer, "attention_2": differential_attention_mixer,
          "attention_3": sigmoid_attention_mixer}


def forward(cfg: dict, weights: dict, tokens, dtype=torch.float64, capture: list | None = None):
    """Logits [T, vocab] of one whole sequence.  capture: given the residual stream after every layer."""
    W = {k: v.to(dtype) for k, v in weights.items()}
    eps, groups = cfg["norm"]["eps"], cfg["norm"].get("groups", 1)
    x = W["embed"][torch.tensor(tokens, dtype=torch.int64)]
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = group_rms_norm(x, W[p + "norm1"], groups, eps)
        y = MIXERS[L["type"]](h, W, p + "mix.", L["mixer"], eps)
        if L.get("mlp"):
            y = y + feed_forward(h, W, p + "mlp.", eps)
        x = x + y
        if capture is not None:
            capture.append(x.clone())
    return group_rms_norm(x, W["final.norm"], groups, eps) @ W["head"].T
