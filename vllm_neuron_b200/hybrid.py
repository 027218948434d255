"""Hybrid decoders: state-space and sliding-window-attention mixers with Dynamic-Tanh norms and a mixture-of-experts
feed-forward, served from a configuration that lists the layers one by one (the "Pumopel" design).

A layer is   x += N1b(mixer(N1(x)));  x += N2b(ff(N2(x)))   with N(x) = gain * tanh(a x) + shift (elementwise).  Mixers:
  * 'mamba2'    -- in-projection -> [z | x | B | C | dt]; causal depthwise convolution + SiLU over [x | B | C]; selective scan
                   S <- exp(-exp(A_log) d) S + d B x^T, y = S^T C + D x with step size d = softplus(raw + dt_bias), per head;
                   y * silu(z), RMS norm in `norm_groups` equal parts, out-projection.  State per sequence: S (fp32) and the last
                   taps - 1 convolution inputs.
  * 'attention' -- q / k / v projections without bias or rotation, GQA, key width `dim` != value width `vdim`, sliding window
                   (query i attends keys i - mask.size < j <= i), a per-head sink logit that only enlarges the softmax
                   denominator, and value mixing: every v_mix layer after the first caches v + lambda (v_first - v), v_first being
                   the first such layer's value of the same token.
Feed-forward: sigmoid router, `top` experts by score, weights = scores (not renormalised) applied to the expert's INPUT,
experts down((b + 1) a / (1 + exp(-1.702 a))) with a = min(gate(h), L), b = clip(up(h), -L, L), plus an always-on shared
expert.  Every size and constant above is read from the configuration.

A second block style, post-norm RMS (the "Kenetar" design), shares the step, the pools and the state slots:
  x += R1(mixer(x));  x += R2(ff(x))   with R(y) = y / sqrt(mean(y^2) + eps) * (1 + w); the sublayers read x itself.  The
embedding is table[token] * scale plus a hashed bigram row (the previous token is per-sequence state); the logits are
head . Rf(x) * logit_scale.  Mixers:
  * 'delta'            -- q / k / v projections, each through a short causal convolution + SiLU; q and k unit vectors per key
                          head (q also / sqrt(dim)); beta = sigmoid(b h), decay g = exp(-exp(A_log) softplus(a h + dt_bias));
                          gated delta rule  S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q  per head; per-head RMS
                          norm of o, times silu(g h), out-projection.  State per sequence: S (fp32) and the last taps - 1
                          convolution inputs.
  * 'latent_attention' -- queries through a normed latent (dq, uq), keys and values as up-projections (uk, uv) of ONE
                          normed latent c per token plus one rotated key part shared by the heads; interleaved-pair rotary
                          angles with YaRN frequency blending; causal softmax; a per-head sigmoid output gate.  Cached per
                          token: [c | rotated key part]; attention runs in the latent space (uk folded into the query, uv
                          applied to the attended latent).
Feed-forward: dense W_down(gelu_tanh(W_gate h) * W_up h), or SiLU experts chosen by the `top` largest router logits (+ bias)
and weighed, on their OUTPUTS, by the softmax over the chosen logits.

A third block style, parallel branches behind one grouped RMS norm (the "Zudarax" design):
  h = N(x);  x += mixer(h) + ff(h)   with N cutting a row into `norm.groups` equal parts, each divided by its own RMS, times w.
Mixers are rotating attentions over the paged pools, all one code path with per-layer variants (`RotAttnSpec`):
  * 'attention'   -- biased q / k / v projections, a short causal convolution on each (no activation), an RMS norm over the whole
                     q and k projection, rotary positions on the leading rot.dims columns of a head (pairs (i, i + dims/2)),
                     soft-capped scores, keys confined to the query's chunk of mask.size positions, softmax;
  * 'attention_2' -- differential attention: two score maps per head over the same values, a1 - lambda a2 with
                     lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff, a weightless per-head RMS norm times (1 - diff), and a
                     per-head sigmoid output gate read from the mixer's input;
  * 'attention_3' -- short convolutions, YaRN-blended rotary frequencies, causal, weights sigmoid(score + bias[head]) that are
                     not normalised over the keys.
Feed-forward: W_down P(W_up h) with the polynomial activation P(z) = a N(z) + b N(z^2) + c N(z^3) + e, N = division by the
row's RMS.  q / k / v (/ gate) and W_up are ONE GEMM, since both branches read the same h.  State per sequence: the K / V pages
and the last taps - 1 projected (biased) inputs of the convolutions.

A fourth block style, parallel branches behind TWO RMS norms of the same stream (the "Gerupel" design):
  x += m (mixer(N1(x)) + ff(N2(x)))   behind a normed token embedding, with logits from the embedding table.  A run of
layers [loop.start, loop.stop) is repeated loop.times times with the same weights, every repetition with pools and state of
its own; before a repetition the embedding output (all but the first) and a learned vector per repetition join the stream.
The mixer 'parallel' is two mixers side by side over the same input, left_scale * left + right_scale * right:
  * left  -- rotating attention (`RotAttnSpec`) with frequencies rescaled by wavelength bands, a per-head temperature on the
             scores, a sliding window beside which every block of mask.pool positions that lies wholly before the window is
             seen as ONE key / value (the mean of the block's cached rows), and a softmax with 1 added to its denominator;
  * right -- a gated linear recurrence per head (`GatedScanSpec`): S <- diag(f) S + (1 - f) v^T, o = S^T q with q = silu(.),
             f = lower + (1 - lower) sigmoid(. + bias), a per-head RMS norm of o.  State per sequence: S (fp32).
Feed-forward: SiLU experts chosen by the largest softmax scores over all experts, weighed on their outputs by the chosen
scores divided by their sum, times router.scale.

The step is ONE ragged batch (`StepMeta`): portions of prompts and single decoded tokens run through the same kernels, each
sequence continuing from its KV pages (block table row) and its state slot.  fp32 everywhere the design asks for it
(residual stream, norms, softmax, router, recurrence); GEMM operands, weights and KV pools are bf16, or fp32 when the model is
built with dtype=torch.float32 (then no tensor-core GEMM is used at all).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field

import torch

import math

from . import ops

ARCHITECTURE = "Pumopel"
# block style per architecture: how the norms sit around the sublayers (and which norm it is)
BLOCK_STYLES = {"Pumopel": "dyt_sandwich", "Kenetar": "rms_post", "Zudarax": "rms_parallel", "Gerupel": "rms_dual"}
ROT_ATTN_KINDS = ("attention", "attention_2", "attention_3")  # the parallel style's mixers
_NO_WINDOW = 1 << 30


# ------------------------------------------------------------------------------------------------ configuration
@dataclass
class SsmSpec:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @property
    def inner(self) -> int:
        return self.heads * self.vdim

    @property
    def channels(self) -> int:  # what the convolution sees: [x | B | C]
        return self.inner + 2 * self.groups * self.state

    @property
    def proj(self) -> int:  # rows of the in-projection: [z | x | B | C | dt]
        return self.inner + self.channels + self.heads


@dataclass
class AttnSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int = _NO_WINDOW
    v_mix: bool = False


@dataclass
class DeltaSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @property
    def channels(self) -> int:  # what the convolution sees: [q | k | v]
        return 2 * self.kv_heads * self.dim + self.heads * self.vdim

    @property
    def proj(self) -> int:  # rows of the in-projection: [q | k | v | b | a | g]
        return self.channels + 2 * self.heads + self.heads * self.vdim


@dataclass
class RotSpec:
    """Rotary angles over the first `dims` columns, pairs (2i, 2i + 1) or, with `half`, (i, i + dims / 2); `scaling` is either
    YaRN (factor, original, fast, slow) or wavelength bands (factor, low, high, original)."""
    dims: int
    base: float
    scaling: dict | None = None
    half: bool = False

    def tables(self, positions: int):
        """(cos, sin) fp32 [positions, dims / 2], computed in float64.  Pair i turns by p * f_i, f_i = base^(-2i/dims); with
        YaRN scaling, f_i is blended with f_i / factor by a linear ramp between the pair indices where `fast` and `slow` full turns
        fit into `original` positions, and cos / sin carry the factor 0.1 ln(factor) + 1.  With band scaling (keys low / high) a
        pair whose wavelength 2 pi / f is below original / high keeps f, one above original / low turns at f / factor, and in
        between f / factor and f are blended linearly in u = (original / wavelength - low) / (high - low)."""
        i = torch.arange(self.dims // 2, dtype=torch.float64)
        f = self.base ** (-2.0 * i / self.dims)
        mscale = 1.0
        sc = self.scaling
        if sc and "low" in sc:
            factor, low, high, orig = (float(sc[k]) for k in ("factor", "low", "high", "original"))
            wave = 2 * math.pi / f
            u = (orig / wave - low) / (high - low)
            f = torch.where(wave < orig / high, f, torch.where(wave > orig / low, f / factor, (1 - u) * f / factor + u * f))
        elif sc:
            turns_at = lambda turns: self.dims * math.log(sc["original"] / (2 * math.pi * turns)) / (2 * math.log(self.base))
            lo = max(math.floor(turns_at(sc["fast"])), 0)
            hi = min(math.ceil(turns_at(sc["slow"])), self.dims - 1)
            ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
            f = f / sc["factor"] * ramp + f * (1 - ramp)
            mscale = 0.1 * math.log(sc["factor"]) + 1.0
        a = torch.arange(positions, dtype=torch.float64)[:, None] * f
        return (torch.cos(a) * mscale).float().contiguous(), (torch.sin(a) * mscale).float().contiguous()


@dataclass
class LatentAttnSpec:
    heads: int
    dim: int       # unrotated query / key columns per head
    rot_dim: int   # rotated columns per head (the key's are shared by the heads)
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot: RotSpec = None


@dataclass
class RotAttnSpec:
    """Rotating attention over paged K / V with per-layer variants; a variant that is off costs nothing."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotSpec = None
    conv: int = 0            # taps of the short causal convolution on q, k and v (0: none)
    bias: bool = False       # q / k / v projection biases
    qk_norm: bool = False    # RMS norm over the whole q and k projection, weights per column
    chunk: int = 0           # > 0: keys visible only inside the query's chunk of this many positions
    softcap: float = 0.0     # > 0: cap * tanh(score / cap)
    sigmoid: bool = False    # weights sigmoid(score + bias[head]) instead of a softmax
    diff: float | None = None  # differential attention: two maps per head, this is the constant of lambda and of (1 - diff)
    gate: bool = False       # per-head sigmoid output gate from the mixer's input
    window: int = 0          # > 0: a query at position i sees keys i - window < j <= i
    pool: int = 0            # > 0 (with a window): blocks of this many positions wholly before the window are one key / value each
    unit_sink: bool = False  # softmax with 1 added to its denominator
    temp: bool = False       # a per-head factor on the scores

    @property
    def maps(self) -> int:
        return 1 if self.diff is None else 2

    @property
    def q_cols(self) -> int:
        return self.heads * self.maps * self.dim

    @property
    def k_cols(self) -> int:
        return self.kv_heads * self.maps * self.dim

    @property
    def v_cols(self) -> int:
        return self.kv_heads * self.vdim

    @property
    def channels(self) -> int:  # what the convolutions see: [q | k | v]
        return self.q_cols + self.k_cols + self.v_cols


@dataclass
class GatedScanSpec:
    """Gated linear recurrence per head: S <- diag(f) S + (1 - f) v^T, o = S^T q; q, f have `dim` channels, v has `vdim`."""
    heads: int
    dim: int
    vdim: int


@dataclass
class DualMixerSpec:
    """Two mixers side by side over the same input: left_scale * attention + right_scale * recurrence."""
    left: RotAttnSpec
    right: GatedScanSpec
    left_scale: float
    right_scale: float


@dataclass
class PolySpec:
    """Dense feed-forward with the polynomial unit-RMS activation."""
    ff: int


@dataclass
class MoeSpec:
    experts: int
    top: int
    ff: int
    limit: float = 0.0
    shared_ff: int = 0
    shared_limit: float = 0.0
    # 'sigmoid_in': weights = sigmoid scores applied to the expert's input, clamped-swish experts;
    # 'softmax_out': weights = softmax over the chosen logits (+ router bias) applied to the experts' outputs, SiLU experts
    # 'softmax_renorm': weights = softmax over ALL experts, the chosen ones divided by their sum, times `scale`; on the outputs
    route: str = "sigmoid_in"
    scale: float = 1.0


@dataclass
class DenseSpec:
    ff: int


@dataclass
class LayerSpec:
    kind: str  # 'mamba2' | 'attention'
    mixer: object
    mlp: MoeSpec | None


@dataclass
class HybridConfig:
    vocab: int
    width: int
    eps: float
    embed_scale: float
    layers: list = field(default_factory=list)
    name: str = ARCHITECTURE
    bigram: dict | None = None   # buckets, mul_prev, mul_cur
    logit_scale: float = 1.0
    norm_groups: int = 1         # parallel style: equal parts of a row that are normed on their own
    residual_mult: float = 1.0   # dual-norm style: factor on the sum of a layer's branches
    loop: dict | None = None     # dual-norm style: start, stop, times -- layers [start, stop) run `times` times in a row

    @property
    def style(self) -> str:
        return BLOCK_STYLES[self.name]

    def layer_runs(self) -> list:
        """[(layer index, repetition or None)] in execution order; a repeated layer appears once per repetition."""
        n = len(self.layers)
        if not self.loop:
            return [(i, None) for i in range(n)]
        a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        return [(i, None) for i in range(a)] + [(i, t) for t in range(times) for i in range(a, b)] + [(i, None) for i in range(b, n)]

    @staticmethod
    def from_dict(d: dict) -> "HybridConfig":
        layers = []
        name = d.get("architecture", ARCHITECTURE)
        if name not in BLOCK_STYLES:
            raise ValueError(f"unknown hybrid architecture {name!r}")
        post = BLOCK_STYLES[name] == "rms_post"
        par = BLOCK_STYLES[name] == "rms_parallel"
        dual = BLOCK_STYLES[name] == "rms_dual"
        for L in d["layers"]:
            m = L["mixer"]
            if dual:
                if L["type"] != "parallel":
                    raise ValueError(f"layer type {L['type']!r} is not part of the {name} design")
                r = m["right"]
                mixer = DualMixerSpec(_window_pool_attn_spec(m["left"]), GatedScanSpec(int(r["heads"]), int(r["dim"]), int(r["vdim"])),
                                      float(m.get("left_scale", 1.0)), float(m.get("right_scale", 1.0)))
            elif par:
                if L["type"] not in ROT_ATTN_KINDS:
                    raise ValueError(f"layer type {L['type']!r} is not part of the {name} design")
                mixer = _rot_attn_spec(L["type"], m)
            elif L["type"] == "mamba2":
                mixer = SsmSpec(int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"]), int(m["conv"]),
                                int(m.get("norm_groups", 1)))
                if mixer.heads % mixer.groups or mixer.inner % mixer.norm_groups:
                    raise ValueError(f"mamba2 layer: heads {mixer.heads} / groups {mixer.groups} / norm_groups {mixer.norm_groups}")
            elif L["type"] == "attention":
                mask = m.get("mask") or {}
                mixer = AttnSpec(int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), float(m["scale"]),
                                 int(mask.get("size", _NO_WINDOW)), bool(m.get("v_mix", False)))
                if mixer.heads % mixer.kv_heads:
                    raise ValueError(f"attention layer: {mixer.heads} query heads over {mixer.kv_heads} kv heads")
            elif L["type"] == "delta":
                mixer = DeltaSpec(int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), int(m["conv"]))
                if mixer.heads % mixer.kv_heads:
                    raise ValueError(f"delta layer: {mixer.heads} heads over {mixer.kv_heads} key heads")
            elif L["type"] == "latent_attention":
                r = m["rot"]
                mixer = LatentAttnSpec(int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"]),
                                       int(m["q_rank"]), float(m["scale"]),
                                       RotSpec(int(r["dims"]), float(r["base"]), dict(r["scaling"]) if r.get("scaling") else None))
                if mixer.rot.dims > mixer.rot_dim or mixer.rot.dims % 2:
                    raise ValueError(f"latent attention: {mixer.rot.dims} rotating columns in a rotated part of {mixer.rot_dim}")
            else:
                raise ValueError(f"unknown layer type {L['type']!r}")
            if not par and not dual and post != (L["type"] in ("delta", "latent_attention")):
                raise ValueError(f"layer type {L['type']!r} is not part of the {name} design")
            f = L.get("mlp")
            mlp = None
            if f:
                kind = f.get("kind", "moe")
                if dual:
                    if kind != "moe":
                        raise ValueError(f"unknown feed-forward kind {kind!r}")
                    mlp = MoeSpec(int(f["router"]["experts"]), int(f["router"]["top"]), int(f["expert"]["ff"]), route="softmax_renorm",
                                  scale=float(f["router"].get("scale", 1.0)))
                    if not 1 <= mlp.top <= mlp.experts:
                        raise ValueError(f"router: top {mlp.top} of {mlp.experts} experts")
                elif par:
                    if kind != "dense":
                        raise ValueError(f"unknown feed-forward kind {kind!r}")
                    mlp = PolySpec(int(f["ff"]))
                elif kind == "dense" and post:
                    mlp = DenseSpec(int(f["ff"]))
                elif kind == "moe" and post:
                    mlp = MoeSpec(int(f["router"]["experts"]), int(f["router"]["top"]), int(f["expert"]["ff"]), route="softmax_out")
                elif kind == "moe":
                    sh = f.get("shared") or {}
                    mlp = MoeSpec(int(f["router"]["experts"]), int(f["router"]["top"]), int(f["expert"]["ff"]),
                                  float(f["expert"]["limit"]), int(sh.get("ff", 0)), float(sh.get("limit", 0.0)))
                else:
                    raise ValueError(f"unknown feed-forward kind {kind!r}")
            layers.append(LayerSpec(L["type"], mixer, mlp))
        emb = d.get("embedding") or {}
        big = emb.get("bigram")
        groups = int(d["norm"].get("groups", 1))
        if int(d["width"]) % groups:
            raise ValueError(f"rows of {d['width']} do not split into {groups} equal norm groups")
        loop = None
        if dual and d.get("loop"):
            loop = {k: int(d["loop"][k]) for k in ("start", "stop", "times")}
            if not (0 <= loop["start"] < loop["stop"] <= len(layers) and loop["times"] >= 1):
                raise ValueError(f"loop {loop} over {len(layers)} layers")
        return HybridConfig(int(d["vocab"]), int(d["width"]), float(d["norm"]["eps"]), float(emb.get("scale", 1.0)), layers, name,
                            {k: int(big[k]) for k in ("buckets", "mul_prev", "mul_cur")} if big else None,
                            float(d.get("logit_scale", 1.0)), groups, float(d.get("residual_mult", 1.0)) if dual else 1.0, loop)

    @staticmethod
    def from_pretrained(path: str) -> "HybridConfig":
        with open(os.path.join(path, "config.json")) as f:
            return HybridConfig.from_dict(json.load(f))

    def to_dict(self) -> dict:
        """The configuration in its file form (what from_dict reads)."""
        out = {"architecture": self.name, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "embedding": {"scale": self.embed_scale}, "layers": []}
        if self.style == "rms_parallel":
            out["norm"]["groups"] = self.norm_groups
            del out["embedding"]
        if self.bigram:
            out["embedding"]["bigram"] = dict(self.bigram)
        if self.style == "rms_post":
            out["logit_scale"] = self.logit_scale
        if self.style == "rms_dual":
            del out["embedding"]
            out["residual_mult"] = self.residual_mult
            if self.loop:
                out["loop"] = dict(self.loop)
        for L in self.layers:
            m = L.mixer
            if isinstance(m, DualMixerSpec):
                a, r = m.left, m.right
                left = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale}
                if a.rot is not None:
                    left["rot"] = {"dims": a.rot.dims, "base": a.rot.base}
                    if a.rot.scaling:
                        left["rot"]["scaling"] = dict(a.rot.scaling)
                if a.window:
                    left["mask"] = {"size": a.window, **({"pool": a.pool} if a.pool else {})}
                mixer = {"left": left, "right": {"heads": r.heads, "dim": r.dim, "vdim": r.vdim}, "left_scale": m.left_scale,
                         "right_scale": m.right_scale}
            elif isinstance(m, RotAttnSpec):
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                         "rot": {"dims": m.rot.dims, "base": m.rot.base}}
                if m.rot.scaling:
                    mixer["rot"]["scaling"] = dict(m.rot.scaling)
                if m.conv:
                    mixer["conv"] = m.conv
                if m.chunk:
                    mixer["mask"] = {"size": m.chunk}
                if m.softcap:
                    mixer["softcap"] = m.softcap
                if m.diff is not None:
                    mixer["diff"] = m.diff
            elif L.kind == "delta":
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.conv}
            elif L.kind == "latent_attention":
                mixer = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank,
                         "q_rank": m.q_rank, "scale": m.scale,
                         "rot": {"dims": m.rot.dims, "base": m.rot.base, "scaling": dict(m.rot.scaling) if m.rot.scaling else None}}
            elif L.kind == "mamba2":
                mixer = {"heads": m.heads, "vdim": m.vdim, "state": m.state, "groups": m.groups, "conv": m.conv,
                         "norm_groups": m.norm_groups}
            else:
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                         "v_mix": m.v_mix}
                if m.window != _NO_WINDOW:
                    mixer["mask"] = {"size": m.window}
            f = None
            if isinstance(L.mlp, (DenseSpec, PolySpec)):
                f = {"kind": "dense", "ff": L.mlp.ff}
            elif L.mlp and L.mlp.route == "softmax_renorm":
                f = {"kind": "moe", "router": {"experts": L.mlp.experts, "top": L.mlp.top, "scale": L.mlp.scale}, "expert": {"ff": L.mlp.ff}}
            elif L.mlp and L.mlp.route == "softmax_out":
                f = {"kind": "moe", "router": {"experts": L.mlp.experts, "top": L.mlp.top}, "expert": {"ff": L.mlp.ff}}
            elif L.mlp:
                f = {"kind": "moe", "router": {"experts": L.mlp.experts, "top": L.mlp.top},
                     "expert": {"ff": L.mlp.ff, "limit": L.mlp.limit},
                     "shared": {"ff": L.mlp.shared_ff, "limit": L.mlp.shared_limit} if L.mlp.shared_ff else None}
            out["layers"].append({"type": L.kind, "mixer": mixer, "mlp": f})
        return out


def _rot_attn_spec(kind: str, m: dict) -> RotAttnSpec:
    """One of the parallel style's mixers from its configuration entry.  The kind fixes which mechanisms a layer has; every
    size and constant comes from the entry."""
    r = m["rot"]
    rot = RotSpec(int(r["dims"]), float(r["base"]), dict(r["scaling"]) if r.get("scaling") else None, half=True)
    spec = RotAttnSpec(int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), float(m["scale"]), rot)
    if spec.heads % spec.kv_heads:
        raise ValueError(f"{kind} layer: {spec.heads} query heads over {spec.kv_heads} kv heads")
    if rot.dims % 2 or rot.dims > spec.dim:
        raise ValueError(f"{kind} layer: {rot.dims} rotating columns in heads of {spec.dim}")
    if kind == "attention":
        spec.bias = spec.qk_norm = True
        spec.conv = int(m.get("conv") or 0)
        spec.chunk = int((m.get("mask") or {}).get("size") or 0)
        spec.softcap = float(m.get("softcap") or 0.0)
    elif kind == "attention_2":
        spec.diff, spec.gate = float(m["diff"]), True
    else:
        spec.sigmoid = True
        spec.conv = int(m.get("conv") or 0)
    return spec


def _window_pool_attn_spec(m: dict) -> RotAttnSpec:
    """The attention half of a 'parallel' mixer: rotary positions (optional band scaling), per-head temperature, unit sink, and a
    sliding window with pooled blocks before it (mask.size / mask.pool; no mask: every earlier key)."""
    r = m.get("rot")
    rot = RotSpec(int(r["dims"]), float(r["base"]), dict(r["scaling"]) if r.get("scaling") else None, half=True) if r else None
    spec = RotAttnSpec(int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), float(m["scale"]), rot, unit_sink=True,
                       temp=True)
    if spec.heads % spec.kv_heads:
        raise ValueError(f"parallel layer: {spec.heads} query heads over {spec.kv_heads} kv heads")
    if rot is not None and (rot.dims % 2 or rot.dims > spec.dim):
        raise ValueError(f"parallel layer: {rot.dims} rotating columns in heads of {spec.dim}")
    mask = m.get("mask") or {}
    spec.window = int(mask.get("size") or 0)
    spec.pool = int(mask.get("pool") or 0) if spec.window else 0
    if spec.window < 0 or spec.pool < 0:
        raise ValueError(f"parallel layer: window {spec.window}, blocks of {spec.pool}")
    return spec


def tensor_shapes(cfg: HybridConfig) -> dict[str, tuple]:
    """Checkpoint tensor name -> shape (a linear layer's matrix has one row per output)."""
    W = cfg.width
    s: dict[str, tuple] = {"embed": (cfg.vocab, W), "head": (cfg.vocab, W)}
    post = cfg.style == "rms_post"
    if cfg.bigram:
        s["bigram"] = (cfg.bigram["buckets"] + 1, W)

    par = cfg.style == "rms_parallel"
    dual = cfg.style == "rms_dual"
    if dual:  # the logits come from the embedding table; the embedding has a norm of its own
        del s["head"]
        s["embed.norm"] = (W,)
        if cfg.loop:
            s["loop.step"] = (cfg.loop["times"], W)

    def norm(n):
        if post or par or dual:
            s[n] = (W,)
        else:
            s[n], s[n + ".b"], s[n + ".alpha"] = (W,), (W,), ()

    norm("final.norm")
    for i, L in enumerate(cfg.layers):
        p = f"l{i}."
        for n in ("norm1",) if par else (("norm1",) + (("norm2",) if L.mlp else ())) if post or dual else \
                (("norm1", "norm1b") + (("norm2", "norm2b") if L.mlp else ())):
            norm(p + n)
        m = L.mixer
        if isinstance(m, DualMixerSpec):
            a, r = m.left, m.right
            s.update({p + "mix.left.q": (a.q_cols, W), p + "mix.left.k": (a.k_cols, W), p + "mix.left.v": (a.v_cols, W),
                      p + "mix.left.temp": (a.heads,), p + "mix.left.o": (W, a.heads * a.vdim),
                      p + "mix.right.q": (r.heads * r.dim, W), p + "mix.right.f": (r.heads * r.dim, W),
                      p + "mix.right.f.b": (r.heads * r.dim,), p + "mix.right.lower": (r.heads * r.dim,),
                      p + "mix.right.v": (r.heads * r.vdim, W), p + "mix.right.norm": (r.vdim,),
                      p + "mix.right.o": (W, r.heads * r.vdim)})
        elif isinstance(m, RotAttnSpec):
            s.update({p + "mix.q": (m.q_cols, W), p + "mix.k": (m.k_cols, W), p + "mix.v": (m.v_cols, W),
                      p + "mix.o": (W, m.heads * m.vdim)})
            for n, c in (("q", m.q_cols), ("k", m.k_cols), ("v", m.v_cols)):
                if m.bias:
                    s[f"{p}mix.{n}.b"] = (c,)
                if m.conv:
                    s[f"{p}mix.{n}.conv"] = (c, m.conv)
                if m.qk_norm and n != "v":
                    s[f"{p}mix.{n}.norm"] = (c,)
            if m.sigmoid:
                s[p + "mix.pb"] = (m.heads,)
            if m.diff is not None:
                s.update({p + "mix." + n: (m.dim,) for n in ("lq1", "lk1", "lq2", "lk2")})
            if m.gate:
                s[p + "mix.g"] = (m.heads, W)
        elif L.kind == "delta":
            gd, hp = m.kv_heads * m.dim, m.heads * m.vdim
            s.update({p + "mix.q": (gd, W), p + "mix.q.conv": (gd, m.conv), p + "mix.k": (gd, W), p + "mix.k.conv": (gd, m.conv),
                      p + "mix.v": (hp, W), p + "mix.v.conv": (hp, m.conv), p + "mix.b": (m.heads, W), p + "mix.a": (m.heads, W),
                      p + "mix.A_log": (m.heads,), p + "mix.dt_bias": (m.heads,), p + "mix.norm": (m.vdim,),
                      p + "mix.g": (hp, W), p + "mix.o": (W, hp)})
        elif L.kind == "latent_attention":
            s.update({p + "mix.dq": (m.q_rank, W), p + "mix.dq.norm": (m.q_rank,),
                      p + "mix.uq": (m.heads * (m.dim + m.rot_dim), m.q_rank), p + "mix.dkv": (m.kv_rank + m.rot_dim, W),
                      p + "mix.dkv.norm": (m.kv_rank,), p + "mix.uk": (m.heads * m.dim, m.kv_rank),
                      p + "mix.uv": (m.heads * m.vdim, m.kv_rank), p + "mix.g": (m.heads, W), p + "mix.o": (W, m.heads * m.vdim)})
        elif L.kind == "mamba2":
            s.update({p + "mix.in": (m.proj, W), p + "mix.conv": (m.channels, m.conv), p + "mix.conv.b": (m.channels,),
                      p + "mix.dt_bias": (m.heads,), p + "mix.A_log": (m.heads,), p + "mix.D": (m.heads,),
                      p + "mix.norm": (m.inner,), p + "mix.o": (W, m.inner)})
        else:
            s.update({p + "mix.q": (m.heads * m.dim, W), p + "mix.k": (m.kv_heads * m.dim, W), p + "mix.v": (m.kv_heads * m.vdim, W),
                      p + "mix.sink": (m.heads,), p + "mix.o": (W, m.heads * m.vdim)})
            if m.v_mix:
                s[p + "mix.vmix"] = ()
        f = L.mlp
        if isinstance(f, PolySpec):
            s.update({p + "mlp.up": (f.ff, W), p + "mlp.down": (W, f.ff), p + "mlp.act": (4,)})
        elif isinstance(f, DenseSpec):
            s.update({p + "mlp.gate": (f.ff, W), p + "mlp.up": (f.ff, W), p + "mlp.down": (W, f.ff)})
        elif f:
            s[p + "mlp.router"] = (f.experts, W)
            if f.route == "softmax_out":
                s[p + "mlp.router.b"] = (f.experts,)
            for e in range(f.experts):
                s.update({f"{p}mlp.e{e}.gate": (f.ff, W), f"{p}mlp.e{e}.up": (f.ff, W), f"{p}mlp.e{e}.down": (W, f.ff)})
            if f.shared_ff:
                s.update({p + "mlp.shared.gate": (f.shared_ff, W), p + "mlp.shared.up": (f.shared_ff, W),
                          p + "mlp.shared.down": (W, f.shared_ff)})
    return s


def random_weights(cfg: HybridConfig, seed: int = 0, std: float | None = None) -> dict[str, torch.Tensor]:
    """Seeded random weights under the checkpoint names (bf16), scaled so that activations stay O(1) through the layers."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    out = {}
    post = cfg.style == "rms_post"
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if post and leaf in ("norm1", "norm2") or (post and name == "final.norm"):
            t = 0.1 * torch.randn(shape, generator=g)  # stored around zero: the norm multiplies by 1 + w
        elif leaf == "alpha":
            t = 0.5 + 0.5 * torch.rand((), generator=g)
        elif leaf == "vmix":
            t = 0.2 + 0.5 * torch.rand((), generator=g)
        elif leaf == "temp":
            t = 0.6 + 0.8 * torch.rand(shape, generator=g)
        elif leaf == "lower":
            t = 0.9 * torch.rand(shape, generator=g)
        elif leaf == "step":
            t = 0.2 * torch.randn(shape, generator=g)
        elif leaf == "b" and len(shape) == 1:
            t = 0.05 * torch.randn(shape, generator=g)
        elif leaf == "act":
            t = torch.tensor([0.6, 0.3, 0.2, 0.05]) + 0.1 * torch.randn(shape, generator=g)
        elif leaf == "pb":
            t = -2.0 + torch.randn(shape, generator=g)
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif leaf in ("norm1", "norm2", "norm1b", "norm2b", "norm") and len(shape) == 1:
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif leaf == "A_log":
            t = torch.log(0.5 + 1.5 * torch.rand(shape, generator=g))
        elif leaf == "dt_bias":
            t = -2.0 + 1.5 * torch.rand(shape, generator=g)
        elif leaf in ("D", "sink"):
            t = torch.randn(shape, generator=g)
        elif leaf == "conv":
            t = torch.randn(shape, generator=g) / shape[1] ** 0.5
        elif len(shape) == 2:
            t = torch.randn(shape, generator=g) * (std if std is not None else shape[1] ** -0.5)
        else:
            t = 0.1 * torch.randn(shape, generator=g)
        out[name] = t.to(torch.bfloat16)
    return out


# ------------------------------------------------------------------------------------------------ the ragged step
@dataclass
class StepMeta:
    """Index tensors of one step (device int32 unless noted).  Sequence s of the step owns block-table row / state slot
    seq_slot[s], brings tokens [seq_start[s], seq_start[s+1]) and continues at position seq_pos0[s]."""
    num_seqs: int
    num_tokens: int
    seq_start: torch.Tensor
    seq_slot: torch.Tensor
    seq_pos0: torch.Tensor
    tok_seq: torch.Tensor
    tok_row: torch.Tensor
    tok_pos: torch.Tensor
    slot_mapping: torch.Tensor  # int64 [T]: KV slot = block id * block_size + offset
    max_new: int = 0            # longest portion of the step (host)
    max_end: int = 0            # most tokens any sequence of the step holds once the step is done (host)
    # long portions cut into segments the selective scan runs in parallel: int32 [num_segs, 4] = (first token, end token,
    # sequence, 1 = first of its sequence | 2 = last) and int32 [num_seqs + 1] first segment per sequence; None when no
    # portion of the step is long enough
    scan_segs: torch.Tensor | None = None
    scan_seq_seg0: torch.Tensor | None = None
    num_segs: int = 0

    @staticmethod
    def build(entries, block_rows, block_size: int, device) -> "StepMeta":
        """entries: [(row, pos0, n_new)]; block_rows: row -> list of block ids (host mirror of the block table).
        One pinned staging tensor, one asynchronous copy."""
        import numpy as np

        b = len(entries)
        n = np.array([e[2] for e in entries], dtype=np.int64)
        t = int(n.sum())
        start = np.zeros(b + 1, dtype=np.int64)
        np.cumsum(n, out=start[1:])
        rows = np.array([e[0] for e in entries], dtype=np.int64)
        pos0 = np.array([e[1] for e in entries], dtype=np.int64)
        tok_seq = np.repeat(np.arange(b, dtype=np.int64), n)
        tok_pos = np.arange(t, dtype=np.int64) - start[tok_seq] + pos0[tok_seq]
        slots = np.empty(t, dtype=np.int64)
        for s, (row, p0, k) in enumerate(entries):
            blocks = np.asarray(block_rows[row], dtype=np.int64)
            p = np.arange(p0, p0 + k)
            slots[start[s]:start[s + 1]] = blocks[p // block_size] * block_size + p % block_size
        parts = [start, rows, pos0, tok_seq, rows[tok_seq], tok_pos]
        i32 = np.concatenate(parts).astype(np.int32)
        if i32.size % 2:  # the int64 slots that follow must start on an 8-byte boundary
            i32 = np.concatenate([i32, np.zeros(1, np.int32)])
        host = torch.from_numpy(np.concatenate([i32, slots.view(np.int32)]))
        if torch.device(device).type == "cuda":
            host = host.pin_memory()
        dev = host.to(device, non_blocking=True)
        cut, o = [], 0
        for a in parts:
            cut.append(dev[o:o + a.size])
            o += a.size
        meta = StepMeta(b, t, *cut, dev[i32.size:i32.size + 2 * t].view(torch.int64), int(n.max()) if b else 0,
                        int((pos0 + n).max()) if b else 0)
        seg = ops.SCAN_SEGMENT
        if meta.max_new >= 2 * seg:
            per = np.maximum(1, -(-n // seg))
            seg0 = np.zeros(b + 1, dtype=np.int64)
            np.cumsum(per, out=seg0[1:])
            v = int(seg0[-1])
            sq = np.repeat(np.arange(b, dtype=np.int64), per)
            k = np.arange(v, dtype=np.int64) - seg0[sq]
            first = start[sq] + k * seg
            end = np.minimum(first + seg, start[sq + 1])
            flags = (k == 0) * 1 + (k == per[sq] - 1) * 2
            hs = torch.from_numpy(np.concatenate([np.stack([first, end, sq, flags], axis=1).reshape(-1), seg0]).astype(np.int32))
            if torch.device(device).type == "cuda":
                hs = hs.pin_memory()
            ds = hs.to(device, non_blocking=True)
            meta.scan_segs, meta.scan_seq_seg0, meta.num_segs = ds[:4 * v].view(v, 4), ds[4 * v:], v
        return meta


# ------------------------------------------------------------------------------------------------ the model
class HybridCausalLM:
    """Weights, KV pools, recurrent state and the step function of a hybrid decoder.  Rows of `block_table` and slots of the
    recurrent state are the model runner's persistent per-request rows."""

    mixed_batch = True  # prompt portions and decoded tokens of many requests run as one ragged batch

    def __init__(self, cfg: HybridConfig, weights, *, num_blocks: int, max_num_seqs: int, max_model_len: int,
                 block_size: int = 32, device="cuda", dtype=torch.bfloat16):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"hybrid decoders run in bfloat16 or float32, not {dtype}")
        self.cfg, self.device, self.et = cfg, torch.device(device), dtype
        ops.device_check(self.device.index or 0)
        self.block_size, self.num_blocks = block_size, num_blocks
        self.max_num_seqs, self.max_model_len = max_num_seqs, max_model_len
        self.max_blocks = -(-max_model_len // block_size)
        self.pad_row = max_num_seqs
        dev, et = self.device, dtype
        if weights is None:
            weights = random_weights(cfg)
        want = tensor_shapes(cfg)

        def get(name):
            t = weights[name]
            if tuple(t.shape) != want[name]:
                raise ValueError(f"tensor {name!r} has shape {tuple(t.shape)}, the configuration says {want[name]}")
            return t

        def lin(*names):  # GEMM operand: rows of several tensors stacked
            return torch.cat([get(n) for n in names], dim=0).to(dev, et).contiguous()

        def vec(name):
            return get(name).to(dev, torch.float32).contiguous()

        post = cfg.style == "rms_post"
        par = cfg.style == "rms_parallel"
        dual = cfg.style == "rms_dual"

        def norm(name):
            if post or par or dual:  # RMS norm: weight stored around zero (post-norm) or plain (in groups: parallel)
                return vec(name)
            return (vec(name), vec(name + ".b"), float(get(name + ".alpha").float()))

        self.embed = lin("embed")
        self.head = self.embed if dual else lin("head")  # dual-norm style: the logits come from the embedding table
        if dual:
            self.embed_norm = vec("embed.norm")
            self.loop_step = vec("loop.step") if cfg.loop else None
        self.final_norm = norm("final.norm")
        self.layers = []
        slots = max_num_seqs + 1
        self.bigram = self.prev_token = None
        if cfg.bigram:
            self.bigram = lin("bigram")
            self.prev_token = torch.zeros((slots,), dtype=torch.int32, device=dev)  # each sequence's last token
        if post:  # the logit scale rides on the final norm's factor: (1 + w) * logit_scale
            self.final_norm_scaled = (self.final_norm * cfg.logit_scale).contiguous()
        rot_tables: dict = {}
        first_vmix = True
        for i, L in enumerate(cfg.layers):
            p, m = f"l{i}.", L.mixer
            lw = {"spec": L, "norm1": norm(p + "norm1")}
            if not post and not par and not dual:
                lw["norm1b"] = norm(p + "norm1b")
            if isinstance(m, DualMixerSpec):
                a, r = m.left, m.right
                if a.rot is not None:
                    key = (a.rot.dims, a.rot.base, json.dumps(a.rot.scaling, sort_keys=True))
                    if key not in rot_tables:
                        rot_tables[key] = tuple(t.to(dev) for t in a.rot.tables(self.max_blocks * block_size))
                    lw["rot"] = rot_tables[key]
                # ONE GEMM for everything that reads norm1(x): [left q | k | v | right q | f | v]
                lw.update(w_in=lin(*(p + "mix." + n for n in ("left.q", "left.k", "left.v", "right.q", "right.f", "right.v"))),
                          w_o=lin(p + "mix.left.o"), w_o2=lin(p + "mix.right.o"), temp=vec(p + "mix.left.temp"),
                          sink=torch.zeros((a.heads,), dtype=torch.float32, device=dev),  # exp(0) = the 1 in the denominator
                          f_bias=vec(p + "mix.right.f.b"), lower=vec(p + "mix.right.lower"), onorm=vec(p + "mix.right.norm"))
            elif isinstance(m, RotAttnSpec):
                key = (m.rot.dims, m.rot.base, json.dumps(m.rot.scaling, sort_keys=True))
                if key not in rot_tables:
                    rot_tables[key] = tuple(t.to(dev) for t in m.rot.tables(self.max_blocks * block_size))
                wq = get(p + "mix.q")
                if m.diff is not None:
                    # two maps per head, stored head by head as [map 1 | map 2]: the query rows are re-laid per kv group as
                    # [the group's first maps | its second maps], so that query head i reads key head i // (heads / kv_heads)
                    # of the 2 * kv_heads key heads (kv head g's maps are key heads 2g and 2g + 1, both over value head g)
                    rep = m.heads // m.kv_heads
                    wq = wq.view(m.kv_heads, rep, 2, m.dim, -1).transpose(1, 2).reshape(m.q_cols, -1)
                    f64 = lambda n: get(p + "mix." + n).double()
                    lw["lam"] = float(torch.exp((f64("lq1") * f64("lk1")).sum()) - torch.exp((f64("lq2") * f64("lk2")).sum()) + m.diff)
                names = [p + "mix.k", p + "mix.v"] + ([p + "mix.g"] if m.gate else []) + ([p + "mlp.up"] if L.mlp else [])
                lw.update(w_in=torch.cat([wq] + [get(n) for n in names], dim=0).to(dev, et).contiguous(), w_o=lin(p + "mix.o"),
                          rot=rot_tables[key],
                          k_pool=torch.zeros((num_blocks, m.kv_heads * m.maps, block_size, m.dim), dtype=et, device=dev),
                          v_pool=torch.zeros((num_blocks, m.kv_heads, block_size, m.vdim), dtype=et, device=dev))
                if m.bias:
                    lw["in_bias"] = torch.cat([get(p + f"mix.{n}.b") for n in "qkv"]).to(dev, torch.float32).contiguous()
                if m.conv or m.bias:  # taps == 0 with a bias: one tap of weight 1 adds the bias
                    cw = torch.cat([get(p + f"mix.{n}.conv") for n in "qkv"]) if m.conv else torch.ones((m.channels, 1))
                    lw.update(conv_w=cw.to(dev, torch.float32).contiguous(),
                              conv_state=torch.zeros((slots, max(cw.shape[1] - 1, 1), m.channels), dtype=torch.float32, device=dev))
                if m.qk_norm:
                    lw.update(q_norm=vec(p + "mix.q.norm"), k_norm=vec(p + "mix.k.norm"))
                if m.sigmoid:
                    lw["pb"] = vec(p + "mix.pb")
            elif L.kind == "delta":
                lw.update(w_in=lin(p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.b", p + "mix.a", p + "mix.g"),
                          conv_w=torch.cat([get(p + "mix.q.conv"), get(p + "mix.k.conv"), get(p + "mix.v.conv")]
                                           ).to(dev, torch.float32).contiguous(),
                          a_log=vec(p + "mix.A_log"), dt_bias=vec(p + "mix.dt_bias"), onorm=vec(p + "mix.norm"),
                          w_o=lin(p + "mix.o"),
                          conv_state=torch.zeros((slots, max(m.conv - 1, 1), m.channels), dtype=torch.float32, device=dev),
                          delta_state=torch.zeros((slots, m.heads, m.vdim, m.dim), dtype=torch.float32, device=dev))
            elif L.kind == "latent_attention":
                key = (m.rot.dims, m.rot.base, json.dumps(m.rot.scaling, sort_keys=True))
                if key not in rot_tables:
                    rot_tables[key] = tuple(t.to(dev) for t in m.rot.tables(self.max_blocks * block_size))
                lw.update(w_in=lin(p + "mix.dq", p + "mix.dkv", p + "mix.g"), dq_norm=vec(p + "mix.dq.norm"),
                          dkv_norm=vec(p + "mix.dkv.norm"), w_uq=lin(p + "mix.uq"), w_o=lin(p + "mix.o"), rot=rot_tables[key],
                          # per head: the key up-projection transposed (it is folded into the query), the value up-projection
                          w_absorb=get(p + "mix.uk").view(m.heads, m.dim, m.kv_rank).transpose(1, 2).to(dev, et).contiguous(),
                          w_uv=get(p + "mix.uv").view(m.heads, m.vdim, m.kv_rank).to(dev, et).contiguous(),
                          k_pool=torch.zeros((num_blocks, 1, block_size, m.kv_rank + m.rot_dim), dtype=et, device=dev))
            elif L.kind == "mamba2":
                lw.update(w_in=lin(p + "mix.in"), conv_w=vec(p + "mix.conv"), conv_b=vec(p + "mix.conv.b"),
                          dt_bias=vec(p + "mix.dt_bias"), a_log=vec(p + "mix.A_log"), d=vec(p + "mix.D"),
                          gnorm=vec(p + "mix.norm"), w_o=lin(p + "mix.o"),
                          conv_state=torch.zeros((slots, max(m.conv - 1, 1), m.channels), dtype=torch.float32, device=dev),
                          ssm_state=torch.zeros((slots, m.heads, m.vdim, m.state), dtype=torch.float32, device=dev))
            else:
                lw.update(w_qkv=lin(p + "mix.q", p + "mix.k", p + "mix.v"), sink=vec(p + "mix.sink"), w_o=lin(p + "mix.o"),
                          k_pool=torch.zeros((num_blocks, m.kv_heads, block_size, m.dim), dtype=et, device=dev),
                          v_pool=torch.zeros((num_blocks, m.kv_heads, block_size, m.vdim), dtype=et, device=dev))
                lw["vmix_mode"] = 0
                if m.v_mix:
                    lw["vmix_mode"] = 1 if first_vmix else 2
                    if not first_vmix:  # the first value-mixing layer's coefficient has no use
                        lw["lam"] = float(get(p + "mix.vmix").float())
                    if first_vmix:
                        self._vfirst_cols = m.kv_heads * m.vdim
                    elif m.kv_heads * m.vdim != self._vfirst_cols:
                        raise ValueError("value mixing needs the same kv_heads * vdim in every v_mix layer")
                    first_vmix = False
            f = L.mlp
            if f and not par:
                lw["norm2"] = norm(p + "norm2")
                if not post and not dual:
                    lw["norm2b"] = norm(p + "norm2b")
            if isinstance(f, PolySpec):  # W_up rides in w_in
                lw.update(w_down=lin(p + "mlp.down"), act=vec(p + "mlp.act"))
            elif isinstance(f, DenseSpec):
                lw.update(w_gu=lin(p + "mlp.gate", p + "mlp.up"), w_down=lin(p + "mlp.down"))
            elif f:
                lw["w_router"] = lin(p + "mlp.router")
                if f.route == "softmax_out":
                    lw["router_b"] = vec(p + "mlp.router.b")
                lw["w_gu"] = torch.stack([torch.cat([get(f"{p}mlp.e{e}.gate"), get(f"{p}mlp.e{e}.up")]) for e in range(f.experts)]
                                         ).to(dev, et).contiguous()
                lw["w_down"] = torch.stack([get(f"{p}mlp.e{e}.down") for e in range(f.experts)]).to(dev, et).contiguous()
                if f.shared_ff:
                    lw["sh_gu"] = lin(p + "mlp.shared.gate", p + "mlp.shared.up")
                    lw["sh_down"] = lin(p + "mlp.shared.down")
            self.layers.append(lw)
        # dual-norm style: one entry per layer RUN (a repeated layer runs loop.times times with the same weights); every run has
        # K / V pools, pooled-block pools and recurrent state of its own
        self.runs = []
        if dual:
            for i, rep in cfg.layer_runs():
                a, r = cfg.layers[i].mixer.left, cfg.layers[i].mixer.right
                run = {"lw": self.layers[i], "layer": i, "rep": rep, "starts_pass": rep is not None and i == cfg.loop["start"],
                       "k_pool": torch.zeros((num_blocks, a.kv_heads, block_size, a.dim), dtype=et, device=dev),
                       "v_pool": torch.zeros((num_blocks, a.kv_heads, block_size, a.vdim), dtype=et, device=dev),
                       "scan_state": torch.zeros((slots, r.heads, r.vdim, r.dim), dtype=torch.float32, device=dev)}
                if a.pool:
                    ppb = -(-block_size // a.pool)
                    run.update(pk_pool=torch.zeros((num_blocks, a.kv_heads, ppb, a.dim), dtype=et, device=dev),
                               pv_pool=torch.zeros((num_blocks, a.kv_heads, ppb, a.vdim), dtype=et, device=dev))
                self.runs.append(run)
        self.block_table = torch.zeros((slots, self.max_blocks), dtype=torch.int32, device=dev)
        self.num_tokens = torch.zeros((slots,), dtype=torch.int32, device=dev)
        self.gemm_ws = None
        self.last_logits = None
        self.last_logprobs = None

    # ------------------------------------------------------------------ sizes
    def kv_bytes_per_block(self) -> int:
        es = 2 if self.et == torch.bfloat16 else 4
        if self.cfg.style == "rms_dual":  # per run: K / V rows of a page and its pooled-block rows
            return sum(sum(t.shape[1] * t.shape[2] * t.shape[3] * es for n, t in run.items() if n.endswith("_pool")) for run in self.runs)
        return sum(L.mixer.kv_heads * self.block_size * (L.mixer.dim * getattr(L.mixer, "maps", 1) + L.mixer.vdim) * es
                   for L in self.cfg.layers if isinstance(L.mixer, (AttnSpec, RotAttnSpec))) + \
            sum(self.block_size * (L.mixer.kv_rank + L.mixer.rot_dim) * es for L in self.cfg.layers if L.kind == "latent_attention")

    def state_bytes_per_slot(self) -> int:
        if self.cfg.style == "rms_dual":
            return sum(4 * run["scan_state"][0].numel() for run in self.runs)
        return sum(4 * (L.mixer.heads * L.mixer.state * L.mixer.vdim + (L.mixer.conv - 1) * L.mixer.channels)
                   for L in self.cfg.layers if L.kind == "mamba2") + \
            sum(4 * (L.mixer.heads * L.mixer.dim * L.mixer.vdim + (L.mixer.conv - 1) * L.mixer.channels)
                for L in self.cfg.layers if L.kind == "delta") + (4 if self.cfg.bigram else 0) + \
            sum(4 * max(L.mixer.conv - 1, 0) * L.mixer.channels for L in self.cfg.layers if isinstance(L.mixer, RotAttnSpec))

    # ------------------------------------------------------------------ building blocks
    def _linear(self, a, w):
        """fp32 [M, N] = a @ w^T.  bf16 serving: the tcgen05 GEMM (TMA needs K * 2 bytes to be a multiple of 16); anything
        else, and all of 32-bit serving, runs on the CUDA cores with true fp32 arithmetic.  A prompt-sized batch against a
        very narrow weight (the router) would leave the 128-row tcgen05 weight tile almost empty: it takes the mma.sync
        kernel behind linear_simt instead."""
        if self.et == torch.bfloat16 and w.shape[1] % 8 == 0 and not (w.shape[0] <= 32 and a.shape[0] > 128):
            m, (n, k) = a.shape[0], w.shape
            need = ops.gemm_workspace_bytes(m, n, k, ops.BF16, 0)
            if need and (self.gemm_ws is None or self.gemm_ws.numel() < need):
                self.gemm_ws = torch.zeros(need, dtype=torch.uint8, device=self.device)  # stream-K counters start at zero
            return ops.gemm(a, w, out_dtype=torch.float32, workspace=self.gemm_ws if need else None)
        return ops.linear_simt(a, w)

    def _ssm(self, lw, h, meta):
        m = lw["spec"].mixer
        proj = self._linear(h, lw["w_in"])  # fp32 [T, z | x | B | C | dt]
        xbc = ops.causal_conv_silu(proj, m.inner, m.channels, lw["conv_w"], lw["conv_b"], lw["conv_state"], meta, self.et)
        y = ops.ssd_scan(xbc, proj, m.inner + m.channels, lw["a_log"], lw["dt_bias"], lw["d"], lw["ssm_state"], meta, m.heads,
                         m.vdim, m.state, m.groups)
        g = ops.gated_group_rmsnorm(y, proj, lw["gnorm"], m.norm_groups, self.cfg.eps, self.et)
        return self._linear(g, lw["w_o"])

    def _attention(self, lw, h, meta, ctx):
        m = lw["spec"].mixer
        qkv = self._linear(h, lw["w_qkv"])  # fp32 [T, q | k | v]
        kc, vc = m.heads * m.dim, (m.heads + m.kv_heads) * m.dim
        mode = lw["vmix_mode"]
        if mode == 1:
            ctx["v_first"] = torch.empty((h.shape[0], self._vfirst_cols), dtype=torch.float32, device=self.device)
        ops.kv_write_vmix(qkv, kc, vc, lw["k_pool"], lw["v_pool"], meta.slot_mapping, v_first=ctx.get("v_first"),
                          lam=lw.get("lam", 0.0), mode=mode)
        a = ops.swa_sink_attn(qkv, m.heads, lw["k_pool"], lw["v_pool"], self.block_table, meta, lw["sink"], m.scale,
                              min(m.window, _NO_WINDOW))
        return self._linear(a, lw["w_o"])

    def _delta(self, lw, h, meta):
        m = lw["spec"].mixer
        c = m.channels
        proj = self._linear(h, lw["w_in"])  # fp32 [T, q | k | v | b | a | g]
        qkv = ops.causal_conv_silu(proj, 0, c, lw["conv_w"], None, lw["conv_state"], meta, torch.float32)
        o = ops.delta_rule(qkv, proj, c, c + m.heads, lw["a_log"], lw["dt_bias"], lw["delta_state"], meta, m.heads, m.kv_heads,
                           m.dim, m.vdim, m.dim ** -0.5)
        return self._linear(ops.head_rmsnorm_gate(o, proj, c + 2 * m.heads, lw["onorm"], self.cfg.eps, m.heads, self.et), lw["w_o"])

    def _latent_attention(self, lw, h, meta):
        m = lw["spec"].mixer
        cos, sin = lw["rot"]
        kr = m.kv_rank + m.rot_dim
        proj = self._linear(h, lw["w_in"])  # fp32 [T, query latent | kv latent | shared rotated key part | head gates]
        ops.latent_kv_write(proj, m.q_rank, m.kv_rank, m.rot_dim, m.rot.dims, lw["dkv_norm"], self.cfg.eps, cos, sin, meta,
                            lw["k_pool"])
        cq = ops.rmsnorm_cols(proj, 0, m.q_rank, lw["dq_norm"], self.cfg.eps, self.et)
        q = self._linear(cq, lw["w_uq"])  # fp32 [T, H * (dim + rot_dim)]
        nope, q_att = ops.latent_q_prep(q, m.heads, m.dim, m.rot_dim, m.rot.dims, m.kv_rank, cos, sin, meta, self.et)
        ops.batched_linear(nope, lw["w_absorb"], q_att, a_batch_stride=m.dim, out_batch_stride=kr)
        lat = ops.swa_sink_attn(q_att, m.heads, lw["k_pool"], None, self.block_table, meta, None, m.scale, _NO_WINDOW,
                                latent_values=m.kv_rank)  # [T, H * kv_rank]
        vals = torch.empty((h.shape[0], m.heads * m.vdim), dtype=self.et, device=self.device)
        ops.batched_linear(lat, lw["w_uv"], vals, a_batch_stride=m.kv_rank, out_batch_stride=m.vdim,
                           gate=proj[:, m.q_rank + kr:])
        return self._linear(vals, lw["w_o"])

    def _rot_attention(self, lw, proj, meta):
        """A rotating attention of the parallel style from the joint projection rows proj = fp32 [T, q | k | v | (gate) | (up)]."""
        m = lw["spec"].mixer
        src = proj
        if "conv_w" in lw:  # short convolutions over [q | k | v] (the projection's bias joins its inputs), no activation
            src = ops.causal_conv_silu(proj, 0, m.channels, lw["conv_w"], None, lw["conv_state"], meta, torch.float32,
                                       in_bias=lw.get("in_bias"), silu=False)
        cos, sin = lw["rot"]
        hq = m.heads * m.maps
        q = ops.qk_norm_rope_kv_write(src, 0, m.q_cols, m.q_cols + m.k_cols, hq, lw["k_pool"], lw["v_pool"], meta,
                                      q_norm=lw.get("q_norm"), k_norm=lw.get("k_norm"), eps=self.cfg.eps, rot_n=m.rot.dims,
                                      rot_half=m.rot.half, cos=cos, sin=sin)
        a = ops.swa_sink_attn(q, hq, lw["k_pool"], lw["v_pool"], self.block_table, meta, None, m.scale, _NO_WINDOW, chunk=m.chunk,
                              softcap=m.softcap, sigmoid_bias=lw.get("pb"), out_f32=m.diff is not None, split_p=True)
        if m.diff is not None:  # both maps' outputs stay fp32 until they are combined and normed
            a = ops.diff_head_norm_gate(a, lw["lam"], 1.0 - m.diff, proj if m.gate else None, m.channels, self.cfg.eps, m.heads,
                                        m.heads // m.kv_heads, self.et)
        return self._linear(a, lw["w_o"])

    def _forward_parallel(self, tokens, meta, logit_rows, capture):
        """h = N(x); x += mixer(h) + ff(h): one grouped norm per layer, one GEMM for everything that reads h, and one pass over
        the residual per layer that adds both branches and norms for the next layer (or for the logits)."""
        et, cfg, n = self.et, self.cfg, len(self.layers)
        x = ops.embed_scale(tokens, self.embed, cfg.embed_scale)
        h = ops.add_group_rmsnorm(x, None, None, self.layers[0]["norm1"] if n else self.final_norm, cfg.norm_groups, cfg.eps, et)
        for i, lw in enumerate(self.layers):
            m, f = lw["spec"].mixer, lw["spec"].mlp
            proj = self._linear(h, lw["w_in"])
            y = self._rot_attention(lw, proj, meta)
            y2 = None
            if f:
                y2 = self._linear(ops.poly_norm(proj, m.channels + (m.heads if m.gate else 0), f.ff, lw["act"], cfg.eps, et), lw["w_down"])
            h = ops.add_group_rmsnorm(x, y, y2, self.layers[i + 1]["norm1"] if i + 1 < n else self.final_norm, cfg.norm_groups,
                                      cfg.eps, et)
            if capture is not None:
                capture.append(x.clone())
        if logit_rows is None or logit_rows.numel() == 0:
            self.last_logits = None
            return None
        self.last_logits = self._linear(h.index_select(0, logit_rows).contiguous(), self.head)
        return self.last_logits

    def _dual_mixer(self, run, h, meta):
        """Both halves of a 'parallel' mixer from norm1(x) -> (attention branch, recurrence branch), fp32 [T, W] each, unscaled."""
        lw = run["lw"]
        m = lw["spec"].mixer
        a, r = m.left, m.right
        proj = self._linear(h, lw["w_in"])  # fp32 [T, left q | k | v | right q | f | v]
        k0 = a.q_cols
        v0 = k0 + a.k_cols
        rq0 = v0 + a.v_cols
        rf0 = rq0 + r.heads * r.dim
        rv0 = rf0 + r.heads * r.dim
        cos, sin = lw.get("rot", (None, None))
        q = ops.qk_norm_rope_kv_write(proj, 0, k0, v0, a.heads, run["k_pool"], run["v_pool"], meta, rot_n=a.rot.dims if a.rot else 0,
                                      rot_half=True, cos=cos, sin=sin, q_head_scale=lw["temp"])
        pooled = None
        if a.pool:  # means of the blocks this step completes, from what the cache now holds
            ops.kv_pool_mean(run["k_pool"], run["v_pool"], run["pk_pool"], run["pv_pool"], self.block_table, meta, a.pool)
            pooled = (run["pk_pool"], run["pv_pool"], a.pool)
        att = ops.swa_sink_attn(q, a.heads, run["k_pool"], run["v_pool"], self.block_table, meta, lw["sink"], a.scale,
                                a.window or _NO_WINDOW, split_p=True, pooled=pooled)
        o = ops.gated_scan(proj, rq0, rf0, rv0, lw["f_bias"], lw["lower"], run["scan_state"], meta, r.heads, r.dim, r.vdim)
        g = ops.head_rmsnorm_gate(o, None, 0, lw["onorm"], self.cfg.eps, r.heads, self.et)
        return self._linear(att, lw["w_o"]), self._linear(g, lw["w_o2"])

    def _forward_dual(self, tokens, meta, logit_rows, capture):
        """x += m (ls left(N1 x) + rs right(N1 x) + ff(N2 x)): one pass over the residual per layer run adds the three branches
        (the experts' rows weighed on the way), what joins the stream ahead of the next run (a repetition's embedding output and
        step vector), and writes both norms of the result for the next run."""
        et, cfg, runs = self.et, self.cfg, self.runs
        x = ops.embed_rmsnorm(tokens, self.embed, self.embed_norm, cfg.eps)
        x0 = x.clone() if cfg.loop and cfg.loop["times"] > 1 else None

        def entering(k):  # what joins the stream right before run k, and the norms that run reads
            if k == len(runs):
                return None, None, self.final_norm, None
            run = runs[k]
            rows = x0 if run["starts_pass"] and run["rep"] > 0 else None
            step = self.loop_step[run["rep"]] if run["starts_pass"] else None
            return rows, step, run["lw"]["norm1"], run["lw"].get("norm2")

        rows, step, w1, w2 = entering(0)
        h1, h2 = ops.scaled_add_rmsnorm2(x, cfg.eps, add_rows=rows, add_vec=step, w1=w1, w2=w2, out_dtype=et)
        for k, run in enumerate(runs):
            lw = run["lw"]
            m, f = lw["spec"].mixer, lw["spec"].mlp
            yl, yr = self._dual_mixer(run, h1, meta)
            pairs = wt = None
            if f:
                idx, wt = ops.moe_topk(self._linear(h2, lw["w_router"]), f.top, mode=ops.ROUTE_SOFTMAX_RENORM)
                align = ops.moe_align(idx, f.experts, ops.moe_wide_tiles(h2, lw["w_gu"], idx.numel()))
                pairs = ops.moe_experts(h2, wt, align, lw["w_gu"], lw["w_down"], f.top, act=ops.ACT_SILU, scale_input=False)
            mult = cfg.residual_mult
            branches = dict(y1=yl, c1=mult * m.left_scale, y2=yr, c2=mult * m.right_scale, y3=pairs, nsum=f.top if f else 1,
                            y3_weight=wt, c3=mult * (f.scale if f else 1.0))
            rows, step, w1, w2 = entering(k + 1)
            if capture is not None:  # the stream as the layer leaves it, before anything of the next run joins
                ops.scaled_add_rmsnorm2(x, cfg.eps, **branches)
                capture.append(x.clone())
                branches = {}
            h1, h2 = ops.scaled_add_rmsnorm2(x, cfg.eps, **branches, add_rows=rows, add_vec=step, w1=w1, w2=w2, out_dtype=et)
        if logit_rows is None or logit_rows.numel() == 0:
            self.last_logits = None
            return None
        self.last_logits = self._linear(h1.index_select(0, logit_rows).contiguous(), self.head)
        return self.last_logits

    def _post_ff(self, lw, h):
        """Feed-forward of the post-norm style -> (fp32 branch rows, rows per token, their weights or None)."""
        f = lw["spec"].mlp
        if isinstance(f, DenseSpec):
            return self._linear(ops.glu(self._linear(h, lw["w_gu"]), ops.ACT_GELU_TANH, self.et), lw["w_down"]), 1, None
        idx, wt = ops.moe_topk(self._linear(h, lw["w_router"]), f.top, bias=lw["router_b"], mode=ops.ROUTE_SOFTMAX_TOP)
        align = ops.moe_align(idx, f.experts, ops.moe_wide_tiles(h, lw["w_gu"], idx.numel()))
        pairs = ops.moe_experts(h, wt, align, lw["w_gu"], lw["w_down"], f.top, act=ops.ACT_SILU, scale_input=False)
        return pairs, f.top, wt

    def _forward_post(self, tokens, meta, logit_rows, capture):
        """x += R1(mixer(x)); x += R2(ff(x)): every sublayer reads the residual stream itself (rounded to the operand type)."""
        et, cfg = self.et, self.cfg
        b = cfg.bigram or {}
        x, h = ops.embed_bigram(tokens, self.embed, cfg.embed_scale, meta, bigram=self.bigram, buckets=b.get("buckets", 0),
                                mul_prev=b.get("mul_prev", 0), mul_cur=b.get("mul_cur", 0), prev_state=self.prev_token)
        for lw in self.layers:
            y = self._delta(lw, h, meta) if lw["spec"].kind == "delta" else self._latent_attention(lw, h, meta)
            h = ops.rms_residual(x, y, lw["norm1"], cfg.eps, out_dtype=et)
            if lw["spec"].mlp:
                y, nsum, wt = self._post_ff(lw, h)
                h = ops.rms_residual(x, y, lw["norm2"], cfg.eps, nsum=nsum, y_weight=wt, out_dtype=et)
            if capture is not None:
                capture.append(x.clone())
        if logit_rows is None or logit_rows.numel() == 0:
            self.last_logits = None
            return None
        hf = ops.rmsnorm_cols(x.index_select(0, logit_rows).contiguous(), 0, cfg.width, self.final_norm_scaled, cfg.eps, et,
                              offset=cfg.logit_scale)
        self.last_logits = self._linear(hf, self.head)
        return self.last_logits

    def _moe(self, lw, h):
        f = lw["spec"].mlp
        idx, wt = ops.moe_topk(self._linear(h, lw["w_router"]), f.top)  # fp32 logits, sigmoid scores
        align = ops.moe_align(idx, f.experts, ops.moe_wide_tiles(h, lw["w_gu"], idx.numel()))
        pairs = ops.moe_experts(h, wt, align, lw["w_gu"], lw["w_down"], f.top, f.limit)
        shared = None
        if f.shared_ff:
            shared = self._linear(ops.clamped_glu(self._linear(h, lw["sh_gu"]), f.shared_limit, self.et), lw["sh_down"])
        return pairs, shared

    # ------------------------------------------------------------------ the step
    def forward(self, tokens: torch.Tensor, meta: StepMeta, logit_rows: torch.Tensor | None, capture: list | None = None):
        """tokens int32 [T] (device) of the ragged batch `meta`; returns fp32 logits [len(logit_rows), vocab] (None when no
        row is asked for).  KV pools and recurrent state of the sequences advance by the step's tokens.
        capture: a list that is given, layer by layer, a copy of x as that layer leaves it."""
        if self.cfg.style == "rms_post":
            return self._forward_post(tokens, meta, logit_rows, capture)
        if self.cfg.style == "rms_parallel":
            return self._forward_parallel(tokens, meta, logit_rows, capture)
        if self.cfg.style == "rms_dual":
            return self._forward_dual(tokens, meta, logit_rows, capture)
        et, n = self.et, len(self.layers)
        x = ops.embed_scale(tokens, self.embed, self.cfg.embed_scale)
        h = ops.dyt_norm(x, *self.layers[0]["norm1"], et) if n else None
        ctx: dict = {}
        for i, lw in enumerate(self.layers):
            nxt = self.layers[i + 1]["norm1"] if i + 1 < n else self.final_norm
            y = self._ssm(lw, h, meta) if lw["spec"].kind == "mamba2" else self._attention(lw, h, meta, ctx)
            if lw["spec"].mlp:
                h2 = ops.dyt_residual(x, y, lw["norm1b"], lw["norm2"], et)
                pairs, shared = self._moe(lw, h2)
                h = ops.dyt_residual(x, pairs, lw["norm2b"], nxt, et, y2=shared, nsum=lw["spec"].mlp.top)
            else:
                h = ops.dyt_residual(x, y, lw["norm1b"], nxt, et)
            if capture is not None:
                capture.append(x.clone())
        if not n:
            h = ops.dyt_norm(x, *self.final_norm, et)
        if logit_rows is None or logit_rows.numel() == 0:
            self.last_logits = None
            return None
        self.last_logits = self._linear(h.index_select(0, logit_rows).contiguous(), self.head)
        return self.last_logits
