"""Prefill / decode throughput of the hybrid decoders (bench.py --hybrid): the Pumopel design next to the dense Llama decoder
at equal size (`small`, `1b`), the Kenetar design next to Pumopel at equal size (`kenetar-small`, `kenetar-1b`), the
Zudarax design next to the dense Llama decoder at equal size (`zudarax-small`, `zudarax-1b`), and the Gerupel design next to
Pumopel (its closest relative: windowed sink attention, a recurrence, experts) at equal size (`gerupel-small`, `gerupel-1b`).

For each size: random weights, both models in bf16 on one GPU, same width / layer count / vocabulary; the dense model's
intermediate size equals the hybrid's ACTIVE feed-forward width (top * ff + shared ff) so a token costs about the same FLOPs.
  prefill : one prompt of S tokens in one step                       -> tokens/s
  decode  : B sequences holding `ctx` tokens each, one token apiece  -> tokens/s
Timed with CUDA events around each step (eager launches, L2 flushed between steps, >= 3 warm-ups).  A second, untimed pass
records every kernel with CUDA events (ops.kernel_timer) and sets it against its own floor: max(FLOPs / measured bf16 GEMM
peak, algorithmic bytes / measured copy bandwidth), both from MEASURED_PEAKS.json.  One JSON line per size.
"""
from __future__ import annotations

import json
import os
import re

import torch

from . import ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# width, layers, then the mixers / feed-forward of the hybrid; layer pattern 'm m a m' repeated
SIZES = {
    "1b": dict(width=2048, layers=8, vocab=32000, ssm=dict(heads=32, vdim=128, state=128, groups=8, conv=4, norm_groups=8),
               attn=dict(heads=16, kv_heads=4, dim=128, vdim=128, window=1024),
               moe=dict(experts=16, top=2, ff=1024, shared=2048), prefill=4096, batch=64, ctx=2048),
    "small": dict(width=1024, layers=8, vocab=32000, ssm=dict(heads=32, vdim=64, state=64, groups=4, conv=4, norm_groups=4),
                  attn=dict(heads=16, kv_heads=4, dim=64, vdim=64, window=512),
                  moe=dict(experts=8, top=2, ff=512, shared=1024), prefill=2048, batch=32, ctx=1024),
}


# the post-norm design at the same width / layers / vocabulary / expert sizes: layer pattern 'd d l d' repeated, the first
# layer with a dense feed-forward of the experts' active width
KENETAR_MIXERS = {
    "1b": dict(delta=dict(heads=16, kv_heads=8, dim=128, vdim=128, conv=4),
               latent=dict(heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=256, q_rank=768)),
    "small": dict(delta=dict(heads=16, kv_heads=8, dim=64, vdim=64, conv=4),
                  latent=dict(heads=16, dim=64, rot_dim=32, vdim=64, kv_rank=128, q_rank=384)),
}


# the parallel-branch design at the same width / layers / vocabulary: layer pattern 'differential, sigmoid, chunked, differential'
# repeated, feed-forward width = the dense decoder's intermediate size; the differential layers carry two maps of half a head
ZUDARAX_MIXERS = {
    "1b": dict(heads=16, kv_heads=4, dim=128, vdim=128, conv=4, chunk=1024, softcap=30.0),
    "small": dict(heads=16, kv_heads=4, dim=64, vdim=64, conv=4, chunk=512, softcap=30.0),
}


# the dual-norm parallel design at the same width / vocabulary / attention sizes and as many layer RUNS: six layers of which the
# third and fourth run twice; window as the hybrid's, blocks of `pool` positions behind it; the recurrence as wide as the
# attention; top * ff = the hybrid's active feed-forward width (it has no shared expert)
GERUPEL_MIXERS = {
    "1b": dict(pool=16, right=dict(heads=16, dim=128, vdim=128), experts=16, top=4, ff=1024),
    "small": dict(pool=8, right=dict(heads=16, dim=64, vdim=64), experts=8, top=4, ff=512),
}


def gerupel_config(name: str):
    from .hybrid import HybridConfig

    sz, gm = SIZES[name], GERUPEL_MIXERS[name]
    a = sz["attn"]
    band = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}
    left = {"heads": a["heads"], "kv_heads": a["kv_heads"], "dim": a["dim"], "vdim": a["vdim"], "scale": a["dim"] ** -0.5,
            "rot": {"dims": a["dim"] // 2, "base": 500000.0, "scaling": band}, "mask": {"size": a["window"], "pool": gm["pool"]}}
    layer = {"type": "parallel", "mixer": {"left": left, "right": dict(gm["right"]), "left_scale": 0.9, "right_scale": 1.2},
             "mlp": {"kind": "moe", "router": {"experts": gm["experts"], "top": gm["top"], "scale": 2.0}, "expert": {"ff": gm["ff"]}}}
    assert sz["layers"] == 8
    return HybridConfig.from_dict({"architecture": "Gerupel", "vocab": sz["vocab"], "width": sz["width"], "norm": {"eps": 1e-6},
                                   "residual_mult": 0.6, "loop": {"start": 2, "stop": 4, "times": 2}, "layers": [layer] * 6})


def _gerupel_floors(name, t, s_pre, ctx, b, prefill):
    """Algorithmic (flops, bytes) per launch of the dual-norm parallel design's own kernels at `t` tokens."""
    sz, gm = SIZES[name], GERUPEL_MIXERS[name]
    a, r, w = sz["attn"], gm["right"], sz["width"]
    h, g, d, dv, win, pool = a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["window"], gm["pool"]
    seen = lambda i: min(i + 1, win) + max(0, (i - win + 1) // pool)  # noqa: E731  keys and blocks that position i sees
    if prefill:
        pairs_qk = float(sum(seen(i) for i in range(s_pre)))
        kv_rows = s_pre + s_pre // pool
        nseq = 1
    else:
        pairs_qk = float(b * seen(ctx))
        kv_rows = b * seen(ctx)
        nseq = b
    att = (2.0 * h * pairs_qk * (d + dv), 2.0 * kv_rows * g * (d + dv) + t * h * (4 * d + 2 * dv))
    hd, hp = r["heads"] * r["dim"], r["heads"] * r["vdim"]
    c = (h + g) * d + g * dv
    npairs = t * gm["top"]
    used = min(gm["experts"], npairs)
    out = {k + "[pool]": att for k in ("swa_sink_attn_prefill", "swa_sink_attn", "swa_sink_attn_decode_tc")}
    out.update({
        "gated_scan": (6.0 * t * hd * r["vdim"], t * 4.0 * (2 * hd + 2 * hp) + 8.0 * nseq * hd * r["vdim"]),
        "gated_scan_prep": (0.0, t * 16.0 * hd),
        "head_rmsnorm_gate": (0.0, t * hp * 6.0),
        "qk_norm_rope_kv_write": (0.0, t * (4.0 * c + 4.0 * h * d + 2.0 * g * (d + dv))),
        "kv_pool_mean": (0.0, (t // pool + (0 if prefill else t)) * 2.0 * g * (d + dv) * (pool + 1)),
        "scaled_add_rmsnorm2": (0.0, t * w * (4 + 4 + 4 + 4 + 4 * gm["top"] + 2 + 2.0)),
        "embed_rmsnorm": (0.0, t * w * 6.0),
        "moe_gate_up_glu": (4.0 * npairs * gm["ff"] * w, used * 4.0 * gm["ff"] * w + t * 2 * w + npairs * 2 * gm["ff"]),
        "moe_down": (2.0 * npairs * gm["ff"] * w, used * 2.0 * gm["ff"] * w + npairs * (2 * gm["ff"] + 4 * w)),
        "moe_gather_scale": (0.0, npairs * w * 4.0),
    })
    return out


def zudarax_config(name: str):
    from .hybrid import HybridConfig

    sz, a = SIZES[name], ZUDARAX_MIXERS[name]
    ff = {"kind": "dense", "ff": dense_shape(sz).intermediate}
    base = {"heads": a["heads"], "kv_heads": a["kv_heads"], "vdim": a["vdim"], "scale": a["dim"] ** -0.5}
    yarn = {"factor": 4.0, "original": 2048, "fast": 32.0, "slow": 1.0}
    chunked = {"type": "attention", "mlp": ff, "mixer": dict(base, dim=a["dim"], conv=a["conv"], softcap=a["softcap"],
                                                            mask={"size": a["chunk"]}, rot={"dims": a["dim"] // 2, "base": 10000.0})}
    diff = {"type": "attention_2", "mlp": ff, "mixer": dict(base, dim=a["dim"] // 2, diff=0.5, rot={"dims": a["dim"] // 2, "base": 10000.0})}
    sig = {"type": "attention_3", "mlp": ff, "mixer": dict(base, dim=a["dim"], conv=a["conv"],
                                                          rot={"dims": a["dim"], "base": 10000.0, "scaling": yarn})}
    layers = [(diff, sig, chunked, diff)[i % 4] for i in range(sz["layers"])]
    return HybridConfig.from_dict({"architecture": "Zudarax", "vocab": sz["vocab"], "width": sz["width"],
                                   "norm": {"eps": 1e-6, "groups": 4}, "layers": layers})


def _zudarax_floors(name, t, s_pre, ctx, b, prefill):
    """Algorithmic (flops, bytes) per launch of the parallel-branch design's own kernels at `t` tokens."""
    sz, a = SIZES[name], ZUDARAX_MIXERS[name]
    w, h, g, d, dv, ff = sz["width"], a["heads"], a["kv_heads"], a["dim"], a["vdim"], dense_shape(sz).intermediate
    c = (h + g) * d + g * dv

    def att(keys_per_query, kv_tokens, maps=1):
        dm = d // maps  # two maps of half a head: the scores cost the same, the value product is done per map
        return (2.0 * t * h * maps * keys_per_query * (dm + dv),
                2.0 * kv_tokens * g * (d + dv) + t * h * maps * (4 * dm + (4 if maps > 1 else 2) * dv))

    ck = a["chunk"]
    if prefill:
        full, chk, kv_full, kv_chk = s_pre / 2, min(ck, s_pre) / 2, s_pre, s_pre
    else:
        full, chk, kv_full, kv_chk = ctx + 1, ctx % ck + 1, b * (ctx + 1), b * (ctx % ck + 1)
    out = {}
    for kern in ("swa_sink_attn_prefill", "swa_sink_attn_prefill_tc", "swa_sink_attn", "swa_sink_attn_decode_tc"):
        out[kern + "[chunk+cap]"] = att(chk, kv_chk)
        out[kern + "[sigmoid]"] = att(full, kv_full)
        out[kern + "[maps]"] = att(full, kv_full, 2)
    out.update({
        "causal_conv": (0.0, t * 8.0 * c),
        "qk_norm_rope_kv_write": (0.0, t * (4.0 * c + 4.0 * h * d + 2.0 * g * (d + dv))),
        "diff_head_norm_gate": (0.0, t * h * dv * (8 + 2.0)),
        "poly_norm": (0.0, t * ff * 6.0),
        "add_group_rmsnorm": (0.0, t * w * (4 + 4 + 4 + 4 + 2.0)),
        "embed_scale": (0.0, t * w * 6.0),
    })
    return out


def kenetar_config(name: str):
    from .hybrid import HybridConfig

    sz, mx = SIZES[name], KENETAR_MIXERS[name]
    m, la = sz["moe"], mx["latent"]
    moe = {"kind": "moe", "router": {"experts": m["experts"], "top": m["top"]}, "expert": {"ff": m["ff"]}}
    dense = {"kind": "dense", "ff": m["top"] * m["ff"]}
    rot = {"dims": la["rot_dim"], "base": 10000.0, "scaling": {"factor": 4.0, "original": 2048, "fast": 32.0, "slow": 1.0}}
    lat = {"type": "latent_attention", "mlp": moe, "mixer": dict(la, scale=(la["dim"] + la["rot_dim"]) ** -0.5, rot=rot)}
    layers = [lat if i % 4 == 2 else {"type": "delta", "mlp": dense if i == 0 else moe, "mixer": dict(mx["delta"])}
              for i in range(sz["layers"])]
    return HybridConfig.from_dict({"architecture": "Kenetar", "vocab": sz["vocab"], "width": sz["width"], "norm": {"eps": 1e-6},
                                   "logit_scale": 1.0, "embedding": {"scale": 1.0, "bigram": {"buckets": 8191, "mul_prev": 31,
                                                                                             "mul_cur": 7}}, "layers": layers})


def _kenetar_floors(name, t, keys_per_query, kv_tokens, nseq):
    """Algorithmic (flops, bytes) per launch of the post-norm design's own kernels at `t` tokens."""
    sz, mx = SIZES[name], KENETAR_MIXERS[name]
    d, la, m, w = mx["delta"], mx["latent"], sz["moe"], sz["width"]
    c = 2 * d["kv_heads"] * d["dim"] + d["heads"] * d["vdim"]
    hp = d["heads"] * d["vdim"]
    row = la["kv_rank"] + la["rot_dim"]
    pairs = t * m["top"]
    used = min(m["experts"], pairs)
    att = (2.0 * t * la["heads"] * keys_per_query * (row + la["kv_rank"]),
           2.0 * kv_tokens * row + t * la["heads"] * (4 * row + 2 * la["kv_rank"]))
    return {
        "swa_sink_attn_prefill": att, "swa_sink_attn": att, "latent_attn_decode": att,
        "delta_scan": (8.0 * t * d["heads"] * d["dim"] * d["vdim"],
                       t * (4 * c + 4 * hp) + 8.0 * nseq * d["heads"] * d["dim"] * d["vdim"]),
        "delta_prep": (0.0, t * 16.0 * d["kv_heads"] * d["dim"]),
        "moe_gate_up_glu": (4.0 * pairs * m["ff"] * w, used * 4.0 * m["ff"] * w + t * 2 * w + pairs * 2 * m["ff"]),
        "moe_down": (2.0 * pairs * m["ff"] * w, used * 2.0 * m["ff"] * w + pairs * (2 * m["ff"] + 4 * w)),
        "moe_gather_scale": (0.0, pairs * w * 4.0),
        "causal_conv_silu": (0.0, t * 8.0 * c),
        "head_rmsnorm_gate": (0.0, t * hp * 10.0),
        "rms_residual": (0.0, t * w * (4 + 4 + 4 + 2.0)),
        "latent_kv_write": (0.0, t * row * 6.0),
        "latent_q_prep": (0.0, t * la["heads"] * ((la["dim"] + la["rot_dim"]) * 4 + la["dim"] * 2 + la["rot_dim"] * 4.0)),
        "rmsnorm_cols": (0.0, t * la["q_rank"] * 6.0),
        "glu": (0.0, t * m["top"] * m["ff"] * 10.0),
    }


def _batched_floor(name):
    g = re.match(r"batched_linear\[(\d+)x(\d+)x(\d+)x(\d+)\]", name)
    if not g:
        return None
    b, mm, n, k = (int(g.group(i)) for i in range(1, 5))
    return 2.0 * b * mm * n * k, 2.0 * b * (mm * k + n * k) + 3.0 * b * mm * n


def hybrid_config(sz: dict):
    from .hybrid import HybridConfig

    a, s, m = sz["attn"], sz["ssm"], sz["moe"]
    mlp = {"kind": "moe", "router": {"experts": m["experts"], "top": m["top"]}, "expert": {"ff": m["ff"], "limit": 7.0},
           "shared": {"ff": m["shared"], "limit": 7.0}}
    att = {"type": "attention", "mlp": mlp, "mixer": {"heads": a["heads"], "kv_heads": a["kv_heads"], "dim": a["dim"],
                                                     "vdim": a["vdim"], "scale": a["dim"] ** -0.5, "mask": {"size": a["window"]},
                                                     "v_mix": True}}
    ssm = {"type": "mamba2", "mlp": mlp, "mixer": dict(s)}
    layers = [att if i % 4 == 2 else ssm for i in range(sz["layers"])]
    return HybridConfig.from_dict({"architecture": "Pumopel", "vocab": sz["vocab"], "width": sz["width"], "norm": {"eps": 1e-6},
                                   "embedding": {"scale": 1.0}, "layers": layers})


def dense_shape(sz: dict):
    from .config import ModelShape

    m = sz["moe"]
    return ModelShape(f"dense-{sz['width']}", sz["width"], sz["layers"], sz["width"] // 128, max(1, sz["width"] // 512), 128,
                      m["top"] * m["ff"] + m["shared"], sz["vocab"])


def _peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return p["hbm_gbs"] * 1e9, p["bf16_tflops"] * 1e12, "measured"
    except Exception:
        return 6.65e12, 1.59e15, "fallback"


def _timed(fn, steps, warmup, flush):
    for _ in range(max(3, warmup)):
        fn()
    ms = []
    for _ in range(steps):
        flush.fill_(1.0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ms.append(e0.elapsed_time(e1))
    ms.sort()
    return ms[len(ms) // 2]


def _floors(cfg, sz, t, keys_per_query, kv_tokens, nseq):
    """Algorithmic (flops, bytes) per launch of the hybrid decoder's own kernels at `t` tokens."""
    a, s, m, w = sz["attn"], sz["ssm"], sz["moe"], sz["width"]
    inner, c = s["heads"] * s["vdim"], s["heads"] * s["vdim"] + 2 * s["groups"] * s["state"]
    pairs = t * m["top"]
    used = min(m["experts"], pairs)
    att = (2.0 * t * a["heads"] * keys_per_query * (a["dim"] + a["vdim"]),
           2.0 * kv_tokens * a["kv_heads"] * (a["dim"] + a["vdim"]) + t * a["heads"] * (4 * a["dim"] + 2 * a["vdim"]))
    return {
        "swa_sink_attn_prefill": att, "swa_sink_attn_decode_tc": att,
        "swa_sink_attn": (2.0 * t * a["heads"] * keys_per_query * (a["dim"] + a["vdim"]),
                          2.0 * kv_tokens * a["kv_heads"] * (a["dim"] + a["vdim"]) + t * a["heads"] * (4 * a["dim"] + 2 * a["vdim"])),
        "ssd_scan": (6.0 * t * s["heads"] * s["state"] * s["vdim"],
                     t * (2 * c + 4 * s["heads"] + 4 * inner) + 8.0 * nseq * s["heads"] * s["state"] * s["vdim"]),
        "moe_gate_up_glu": (4.0 * pairs * m["ff"] * w, used * 4.0 * m["ff"] * w + t * 2 * w + pairs * 2 * m["ff"]),
        "moe_down": (2.0 * pairs * m["ff"] * w, used * 2.0 * m["ff"] * w + pairs * (2 * m["ff"] + 4 * w)),
        "moe_gather_scale": (0.0, pairs * w * 4.0),
        "causal_conv_silu": (0.0, t * (4 * c + 2 * c)),
        "gated_group_rmsnorm": (0.0, t * inner * 10.0),
        "dyt_residual": (0.0, t * w * (4 + 4 + 4 + 2.0)),
        "kv_write_vmix": (0.0, t * a["kv_heads"] * (a["dim"] + a["vdim"]) * 6.0),
        "clamped_glu": (0.0, t * m["shared"] * 10.0),
    }


def _gemm_floor(name):
    g = re.match(r"(gemm\w*|linear_simt)\[(\d+)x(\d+)x(\d+)\]", name)
    if not g:
        return None
    mm, n, k = int(g.group(2)), int(g.group(3)), int(g.group(4))
    return 2.0 * mm * n * k, 2.0 * (mm * k + n * k) + 4.0 * mm * n


def _breakdown(fn, floors, hbm, peak):
    with ops.kernel_timer() as kt:
        fn()
    out = {}
    for name, (cnt, ms) in sorted(kt.summary().items(), key=lambda kv: -kv[1][0] * kv[1][1]):
        fb = _gemm_floor(name) or _batched_floor(name) or floors.get(name)
        row = {"launches": cnt, "ms": round(ms, 4)}
        if fb:
            floor_ms = max(fb[0] / peak, fb[1] / hbm) * 1e3
            row.update(floor_ms=round(floor_ms, 5), frac_of_floor=round(floor_ms / ms, 4) if ms > 0 else None)
        out[name] = row
    return out


def _time_hybrid(cfg, sz, args, floors_fn, flush, hbm, peak):
    """Prefill and decode of one hybrid model: step times and the per-kernel table."""
    from .hybrid import HybridCausalLM, StepMeta

    dev = torch.device("cuda:0")
    s_pre, b, ctx, bs = sz["prefill"], sz["batch"], sz["ctx"], 32
    mml = max(s_pre, ctx + 64)
    per = -(-mml // bs)
    nblocks = b * per + 1
    hm = HybridCausalLM(cfg, None, num_blocks=nblocks, max_num_seqs=b, max_model_len=mml, block_size=bs, device=dev)
    rows = {r: list(range(1 + r * per, 1 + (r + 1) * per)) for r in range(b)}
    for r, blk in rows.items():
        hm.block_table[r, :per] = torch.tensor(blk, dtype=torch.int32, device=dev)
    g = torch.Generator(device="cpu").manual_seed(0)
    ptoks = torch.randint(0, sz["vocab"], (s_pre,), generator=g, dtype=torch.int32).to(dev)
    pmeta = StepMeta.build([(0, 0, s_pre)], rows, bs, dev)
    last = torch.tensor([s_pre - 1], device=dev)
    dtoks = torch.randint(0, sz["vocab"], (b,), generator=g, dtype=torch.int32).to(dev)
    dmeta = StepMeta.build([(r, ctx, 1) for r in range(b)], rows, bs, dev)
    drows = torch.arange(b, device=dev)
    h_pre = lambda: hm.forward(ptoks, pmeta, last)  # noqa: E731
    h_dec = lambda: hm.forward(dtoks, dmeta, drows)  # noqa: E731
    ms_p = _timed(h_pre, args.steps, args.warmup, flush)
    ms_d = _timed(h_dec, args.steps, args.warmup, flush)
    out = {"prefill_tok_s": round(s_pre / ms_p * 1e3), "prefill_ms": round(ms_p, 3),
           "decode_tok_s": round(b / ms_d * 1e3), "decode_ms": round(ms_d, 3),
           "kv_bytes_per_block": hm.kv_bytes_per_block(), "state_bytes_per_slot": hm.state_bytes_per_slot(),
           "prefill_kernels": _breakdown(h_pre, floors_fn(s_pre, True), hbm, peak),
           "decode_kernels": _breakdown(h_dec, floors_fn(b, False), hbm, peak)}
    del hm
    torch.cuda.empty_cache()
    return out, rows, nblocks, mml, ptoks, dtoks


def run(args):
    from .model import B200CausalLM

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    hbm, peak, src = _peaks()
    flush = torch.empty(192 << 20, dtype=torch.float32, device=dev)  # 768 MB > L2
    names = list(SIZES) if args.hybrid == "all" else [args.hybrid]
    for name in names:
        kenetar, zudarax, gerupel = name.startswith("kenetar-"), name.startswith("zudarax-"), name.startswith("gerupel-")
        short = name.split("-", 1)[1] if kenetar or zudarax or gerupel else name
        sz = SIZES[short]
        cfg = hybrid_config(sz)
        s_pre, b, ctx = sz["prefill"], sz["batch"], sz["ctx"]
        bs = 32
        res = {"metric": "gerupel_vs_pumopel_tokens_per_s" if gerupel else "kenetar_vs_pumopel_tokens_per_s" if kenetar else "zudarax_vs_dense_tokens_per_s" if zudarax else
               "hybrid_vs_dense_tokens_per_s", "size": name,
               "dtype": "bf16", "data": "synthetic (random weights)",
               "roofline_peaks": {"hbm_gbs": hbm / 1e9, "bf16_tflops": peak / 1e12, "source": src},
               "config": {"width": sz["width"], "layers": sz["layers"], "prefill_tokens": s_pre, "decode_batch": b,
                          "decode_ctx": ctx, "l2": "flushed between timed steps"}}
        win = sz["attn"]["window"]
        pum_floors = lambda t, pre: _floors(cfg, sz, t, min(win, s_pre / 2) if pre else min(win, ctx + 1),  # noqa: E731
                                            s_pre if pre else b * min(win, ctx + 1), 1 if pre else b)
        if gerupel:
            ger_floors = lambda t, pre: _gerupel_floors(short, t, s_pre, ctx, b, pre)  # noqa: E731
            res["gerupel"] = _time_hybrid(gerupel_config(short), sz, args, ger_floors, flush, hbm, peak)[0]
            res["pumopel"] = _time_hybrid(cfg, sz, args, pum_floors, flush, hbm, peak)[0]
            res["gpu_launches"] = ops.launch_count()
            print(json.dumps(res), flush=True)
            continue
        if kenetar:
            ken_floors = lambda t, pre: _kenetar_floors(short, t, s_pre / 2 if pre else ctx + 1,  # noqa: E731
                                                        s_pre if pre else b * (ctx + 1), 1 if pre else b)
            res["kenetar"] = _time_hybrid(kenetar_config(short), sz, args, ken_floors, flush, hbm, peak)[0]
            res["pumopel"] = _time_hybrid(cfg, sz, args, pum_floors, flush, hbm, peak)[0]
            res["gpu_launches"] = ops.launch_count()
            print(json.dumps(res), flush=True)
            continue
        # ---------------- hybrid
        if zudarax:
            zud_floors = lambda t, pre: _zudarax_floors(short, t, s_pre, ctx, b, pre)  # noqa: E731
            res["zudarax"], rows, nblocks, mml, ptoks, dtoks = _time_hybrid(zudarax_config(short), sz, args, zud_floors, flush, hbm, peak)
        else:
            res["hybrid"], rows, nblocks, mml, ptoks, dtoks = _time_hybrid(cfg, sz, args, pum_floors, flush, hbm, peak)
        per = -(-mml // bs)
        # ---------------- dense decoder of equal size
        shape = dense_shape(sz)
        dm = B200CausalLM(shape, None, quant="bf16", num_blocks=nblocks, max_num_seqs=b, max_model_len=mml, block_size=bs, device=dev)
        for r, blk in rows.items():
            dm.block_table[r, :per] = torch.tensor(blk, dtype=torch.int32, device=dev)
        ptok64 = ptoks.long()
        d_pre = lambda: dm.prefill(0, ptok64, s_pre, 0)  # noqa: E731
        bufs = dm.decode_buffers(b)
        bufs.tokens.copy_(dtoks.long())

        def d_dec():
            dm.num_tokens[:b] = ctx + 1
            dm.decode_step(b, max_ctx_blocks=-(-(ctx + 1) // bs))

        ms_p2 = _timed(d_pre, args.steps, args.warmup, flush)
        ms_d2 = _timed(d_dec, args.steps, args.warmup, flush)
        hq, hkv, d = shape.num_q_heads, shape.num_kv_heads, shape.head_dim
        dfl_p = {"paged_attn_prefill": (4.0 * hq * d * s_pre * (s_pre + 1) / 2, 4.0 * s_pre * hkv * d + 4.0 * s_pre * hq * d)}
        dfl_d = {"paged_attn_decode": (4.0 * b * hq * d * (ctx + 1), 4.0 * b * (ctx + 1) * hkv * d)}
        res["dense"] = {
            "prefill_tok_s": round(s_pre / ms_p2 * 1e3), "prefill_ms": round(ms_p2, 3),
            "decode_tok_s": round(b / ms_d2 * 1e3), "decode_ms": round(ms_d2, 3), "intermediate": shape.intermediate,
            "prefill_kernels": _breakdown(d_pre, dfl_p, hbm, peak), "decode_kernels": _breakdown(d_dec, dfl_d, hbm, peak)}
        del dm
        torch.cuda.empty_cache()
        res["gpu_launches"] = ops.launch_count()
        print(json.dumps(res), flush=True)
