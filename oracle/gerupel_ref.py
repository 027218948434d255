"""Plain restatement of the Gerupel decoder (test infrastructure; nothing under vllm_neuron_b200/ imports it).

Gerupel is a decoder whose layers add two branches that read two norms of the same residual stream,
    x <- x + m (mixer(N1(x)) + ff(N2(x))),
behind a normed token embedding, with a run of layers that is repeated with shared weights (every repetition keeping a
cache of its own), and logits from the embedding table.  A mixer is two mixers side by side over the same input:
  * left  -- grouped-query attention with partial rotate-half rotary positions (frequencies rescaled by wavelength bands),
             a per-head temperature on the scores, a sliding window BESIDE which every block of `pool` positions that lies
             wholly before the window is seen as ONE key / value (the block's mean), and a softmax whose denominator
             carries an extra 1;
  * right -- a gated linear recurrence per head, S <- diag(f) S + (1 - f) v^T, o = S^T q, whose forget gate f is bounded
             from below per channel and also decides what is written; each head's o is RMS-normed.
Feed-forward: SiLU experts chosen by the largest softmax scores, weighed by their renormalised scores times a constant.
One function per mechanism, whole sequences, no cache: a token's output depends on earlier tokens only, so every way of
cutting a sequence into engine steps must reproduce `forward` on the full list.  `dtype` float64 gives the reference
values.  `cfg` is the configuration in its file form (a dict).
"""
from __future__ import annotations

import math

import torch


def rms_norm(x, w, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def banded_frequencies(rot, dtype):
    """f_i = base^(-2i/dims) for the dims/2 pairs.  With `scaling` (factor, low, high, original) a pair whose wavelength
    2 pi / f is shorter than original / high keeps f, one longer than original / low turns `factor` times slower, and in
    between the two are blended linearly in original / wavelength."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = (float(sc[k]) for k in ("factor", "low", "high", "original"))
        wave = 2 * math.pi / f
        s = (orig / wave - low) / (high - low)
        mid = (1 - s) * f / factor + s * f
        f = torch.where(wave < orig / high, f, torch.where(wave > orig / low, f / factor, mid))
    return f.to(dtype)


def rotate_half(x, rot):
    """x [T, heads, D]: column i < dims/2 pairs with column i + dims/2; (u, v) -> (u cos a - v sin a, v cos a + u sin a) at
    a = position * f_i; columns from `dims` on pass unchanged."""
    T = x.shape[0]
    dims = int(rot["dims"])
    half = dims // 2
    a = torch.arange(T, dtype=x.dtype)[:, None] * banded_frequencies(rot, x.dtype)
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def window_pool_attention(q, k, v, scale, temp, size, pool, pool_dtype=None):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] (k already rotated).  Query i sees keys i - size < j <= i and, for every block
    b of `pool` positions with b pool + pool - 1 <= i - size, the mean key and mean value of the block.  Weights
    exp(s) / (1 + sum exp(s)) over tokens and blocks together; scores q . k * scale * temp[head].  size None: every earlier
    key, no blocks.  pool_dtype: the block means pass through this type (a cache of that type holds them)."""
    T, H, D = q.shape
    G, Dv = k.shape[1], v.shape[2]
    rep = H // G
    out = q.new_zeros(T, H, Dv)
    nblk = T // pool if (pool and size) else 0
    if nblk:
        kb = k[: nblk * pool].view(nblk, pool, G, D).mean(1)
        vb = v[: nblk * pool].view(nblk, pool, G, Dv).mean(1)
        if pool_dtype is not None:
            kb, vb = kb.to(pool_dtype).to(q.dtype), vb.to(pool_dtype).to(q.dtype)
    for i in range(T):
        lo = 0 if size is None else max(0, i - size + 1)
        nb = 0 if not nblk else max(0, (i - size + 1) // pool)
        for h in range(H):
            g = h // rep
            keys, vals = k[lo : i + 1, g], v[lo : i + 1, g]
            if nb:
                keys, vals = torch.cat([kb[:nb, g], keys]), torch.cat([vb[:nb, g], vals])
            s = (keys @ q[i, h]) * scale * temp[h]
            m = torch.clamp(s.max(), min=0.0)
            e = torch.exp(s - m)
            out[i, h] = (e @ vals) / (torch.exp(-m) + e.sum())
    return out


def left_mixer(h, W, p, m, cache_dtype=None):
    """Attention branch.  cache_dtype: the keys and values pass through this type before they are pooled and read (what a
    cache of that type holds)."""
    T = h.shape[0]
    H, G, D, Dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ W[p + "q"].T).view(T, H, D)
    k = (h @ W[p + "k"].T).view(T, G, D)
    v = (h @ W[p + "v"].T).view(T, G, Dv)
    if m.get("rot"):
        q, k = rotate_half(q, m["rot"]), rotate_half(k, m["rot"])
    if cache_dtype is not None:
        k, v = k.to(cache_dtype).to(h.dtype), v.to(cache_dtype).to(h.dtype)
    mask = m.get("mask") or {}
    o = window_pool_attention(q, k, v, float(m["scale"]), W[p + "temp"], mask.get("size"), int(mask.get("pool") or 0), cache_dtype)
    return o.reshape(T, H * Dv) @ W[p + "o"].T


def gated_recurrence(q, f, v):
    """q, f [T, H, D], v [T, H, P]: S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T (S [D, P], zero at the start), o_t = S_t^T q_t."""
    T, H, D = q.shape
    P = v.shape[2]
    S = q.new_zeros(H, D, P)
    o = q.new_zeros(T, H, P)
    for t in range(T):
        S = f[t][:, :, None] * S + (1 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdp,hd->hp", S, q[t])
    return o


def right_mixer(h, W, p, m, eps):
    T = h.shape[0]
    H, D, P = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = torch.nn.functional.silu(h @ W[p + "q"].T).view(T, H, D)
    lower = W[p + "lower"]
    f = (lower + (1 - lower) * torch.sigmoid(h @ W[p + "f"].T + W[p + "f.b"])).view(T, H, D)
    v = (h @ W[p + "v"].T).view(T, H, P)
    o = rms_norm(gated_recurrence(q, f, v), W[p + "norm"], eps)
    return o.reshape(T, H * P) @ W[p + "o"].T


def expert_mixture(h, W, p, f):
    """Scores = softmax of the router logits over all experts; the `top` largest are kept, divided by their sum (+ 1e-20)
    and multiplied by router.scale; the output is the weighted sum of the kept experts' down(silu(gate h) * up h)."""
    E, top, scale = int(f["router"]["experts"]), int(f["router"]["top"]), float(f["router"].get("scale", 1.0))
    s = torch.softmax(h @ W[p + "router"].T, dim=-1)
    val, idx = torch.topk(s, top, dim=-1)
    wt = val / (val.sum(-1, keepdim=True) + 1e-20) * scale
    out = torch.zeros_like(h)
    for e in range(E):
        for j in range(top):
            rows = (idx[:, j] == e).nonzero().flatten()
            if rows.numel():
                x = h[rows]
                y = (torch.nn.functional.silu(x @ W[f"{p}e{e}.gate"].T) * (x @ W[f"{p}e{e}.up"].T)) @ W[f"{p}e{e}.down"].T
                out[rows] += wt[rows, j][:, None] * y
    return out


def layer_runs(cfg):
    """[(layer index, pass number or None)] in the order the layers run: layers loop.start .. loop.stop - 1 run loop.times
    times in a row."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, None) for i in range(a)]
    for t in range(times):
        runs += [(i, t) for i in range(a, b)]
    return runs + [(i, None) for i in range(b, n)]


def forward(cfg, weights, tokens, dtype=torch.float64, cache_dtype=None, streams=None):
    """tokens: list of ids -> logits [T, vocab].  streams: a list that receives x after every layer run."""
    W = {k: v.to(dtype) for k, v in weights.items()}
    eps, mult = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    x = rms_norm(W["embed"][torch.tensor(tokens, dtype=torch.long)], W["embed.norm"], eps)
    x0 = x
    loop = cfg.get("loop")
    for i, t in layer_runs(cfg):
        L = cfg["layers"][i]
        p = f"l{i}."
        if t is not None and i == int(loop["start"]):
            if t > 0:
                x = x + x0
            x = x + W["loop.step"][t]
        m = L["mixer"]
        h1 = rms_norm(x, W[p + "norm1"], eps)
        y = float(m["left_scale"]) * left_mixer(h1, W, p + "mix.left.", m["left"], cache_dtype) + \
            float(m["right_scale"]) * right_mixer(h1, W, p + "mix.right.", m["right"], eps)
        if L.get("mlp"):
            y = y + expert_mixture(rms_norm(x, W[p + "norm2"], eps), W, p + "mlp.", L["mlp"])
        x = x + mult * y
        if streams is not None:
            streams.append(x.clone())
    return rms_norm(x, W["final.norm"], eps) @ W["embed"].T
