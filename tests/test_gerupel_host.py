"""CPU: host side of the dual-norm parallel decoder (Gerupel) -- configuration reader and its refusals, tensor names and
shapes, the order of layer runs, registry, band-scaled rotary tables -- and properties of the plain restatement that the GPU
tests lean on."""
import json
import math

import pytest
import torch

from vllm_neuron_b200.hybrid import DualMixerSpec, GatedScanSpec, HybridConfig, MoeSpec, RotAttnSpec, RotSpec, random_weights, tensor_shapes


def _layer(mask=None, mlp=True, scaling=None, **left):
    lm = {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 5, "scale": 0.3, "rot": {"dims": 4, "base": 100.0}}
    lm.update(left)
    if scaling:
        lm["rot"] = {**lm["rot"], "scaling": scaling}
    if mask:
        lm["mask"] = mask
    return {"type": "parallel", "mixer": {"left": lm, "right": {"heads": 3, "dim": 7, "vdim": 4}, "left_scale": 0.7, "right_scale": 1.25},
            "mlp": {"kind": "moe", "router": {"experts": 5, "top": 2, "scale": 1.5}, "expert": {"ff": 9}} if mlp else None}


def _cfg(layers=None, loop=None):
    band = {"factor": 5.0, "low": 1.0, "high": 3.0, "original": 16}
    d = {"architecture": "Gerupel", "vocab": 20, "width": 12, "norm": {"eps": 1e-5}, "residual_mult": 0.6,
         "layers": layers if layers is not None else [_layer({"size": 9, "pool": 4}, scaling=band), _layer({"size": 5}, mlp=False),
                                                      _layer(None)]}
    if loop:
        d["loop"] = loop
    return d


def test_config_reader_round_trip_and_shapes():
    d = _cfg(loop={"start": 1, "stop": 3, "times": 2})
    cfg = HybridConfig.from_dict(d)
    assert cfg.style == "rms_dual" and cfg.residual_mult == 0.6 and cfg.loop == {"start": 1, "stop": 3, "times": 2}
    assert cfg.to_dict() == d and HybridConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
    m0, m1, m2 = (L.mixer for L in cfg.layers)
    assert all(isinstance(m, DualMixerSpec) and isinstance(m.left, RotAttnSpec) and isinstance(m.right, GatedScanSpec) for m in (m0, m1, m2))
    assert (m0.left.window, m0.left.pool, m1.left.window, m1.left.pool, m2.left.window, m2.left.pool) == (9, 4, 5, 0, 0, 0)
    assert m0.left.unit_sink and m0.left.temp and m0.left.rot.half and m0.left.rot.scaling["low"] == 1.0 and m1.left.rot.scaling is None
    assert (m0.left_scale, m0.right_scale) == (0.7, 1.25) and (m0.right.heads, m0.right.dim, m0.right.vdim) == (3, 7, 4)
    f = cfg.layers[0].mlp
    assert isinstance(f, MoeSpec) and (f.experts, f.top, f.ff, f.route, f.scale) == (5, 2, 9, "softmax_renorm", 1.5)
    assert cfg.layers[1].mlp is None
    sh = tensor_shapes(cfg)
    assert "head" not in sh and sh["embed"] == (20, 12) and sh["embed.norm"] == sh["final.norm"] == (12,) and sh["loop.step"] == (2, 12)
    assert sh["l0.norm1"] == sh["l0.norm2"] == (12,) and "l1.norm2" not in sh and "l0.norm1b" not in sh
    assert sh["l0.mix.left.q"] == (24, 12) and sh["l0.mix.left.k"] == (12, 12) and sh["l0.mix.left.v"] == (10, 12)
    assert sh["l0.mix.left.temp"] == (4,) and sh["l0.mix.left.o"] == (12, 20)
    assert sh["l0.mix.right.q"] == sh["l0.mix.right.f"] == (21, 12) and sh["l0.mix.right.f.b"] == sh["l0.mix.right.lower"] == (21,)
    assert sh["l0.mix.right.v"] == (12, 12) and sh["l0.mix.right.norm"] == (4,) and sh["l0.mix.right.o"] == (12, 12)
    assert sh["l0.mlp.router"] == (5, 12) and sh["l0.mlp.e4.gate"] == (9, 12) and sh["l0.mlp.e0.down"] == (12, 9) and "l0.mlp.router.b" not in sh
    assert "l1.mlp.router" not in sh and set(random_weights(cfg)) == set(sh)
    assert "loop.step" not in tensor_shapes(HybridConfig.from_dict(_cfg()))


def test_order_of_layer_runs():
    runs = lambda loop: HybridConfig.from_dict(_cfg(loop=loop)).layer_runs()
    assert runs(None) == [(0, None), (1, None), (2, None)]
    assert runs({"start": 1, "stop": 3, "times": 2}) == [(0, None), (1, 0), (2, 0), (1, 1), (2, 1)]
    assert runs({"start": 0, "stop": 1, "times": 3}) == [(0, 0), (0, 1), (0, 2), (1, None), (2, None)]
    assert runs({"start": 0, "stop": 3, "times": 1}) == [(0, 0), (1, 0), (2, 0)]
    from oracle.gerupel_ref import layer_runs

    for loop in (None, {"start": 1, "stop": 2, "times": 4}, {"start": 0, "stop": 3, "times": 2}):
        assert layer_runs(_cfg(loop=loop)) == runs(loop)


def test_config_reader_refuses_what_the_design_does_not_have():
    for bad in ({"type": "attention", "mlp": None, "mixer": _layer()["mixer"]["left"]},
                {"type": "mamba2", "mlp": None, "mixer": {"heads": 2, "vdim": 3, "state": 5, "groups": 1, "conv": 3}},
                _layer(kv_heads=3), _layer(rot={"dims": 8, "base": 10.0}), _layer(rot={"dims": 3, "base": 10.0}),
                {**_layer(), "mlp": {"kind": "dense", "ff": 8}},
                {**_layer(), "mlp": {"kind": "moe", "router": {"experts": 2, "top": 3}, "expert": {"ff": 8}}}):
        with pytest.raises(ValueError):
            HybridConfig.from_dict(_cfg(layers=[bad]))
    for loop in ({"start": 2, "stop": 2, "times": 2}, {"start": 0, "stop": 4, "times": 1}, {"start": 0, "stop": 1, "times": 0}):
        with pytest.raises(ValueError):
            HybridConfig.from_dict(_cfg(loop=loop))
    with pytest.raises(ValueError):  # a layer of this design in another one
        HybridConfig.from_dict({**_cfg(), "architecture": "Zudarax", "norm": {"eps": 1e-5, "groups": 1}})


def test_registry_serves_it_in_both_modes():
    from vllm_neuron_b200.registry import resolve

    arch, entry = resolve(_cfg())
    assert arch == "Gerupel" and entry.family == "hybrid" and set(entry.dtypes) == {torch.bfloat16, torch.float32}
    assert entry.read_config(_cfg()) == HybridConfig.from_dict(_cfg())


def test_band_scaled_rotary_tables():
    """The three bands by hand: with base 10000 over 16 columns and original 64, pair 0 (wavelength 6.3) is kept, the last pairs
    (wavelengths in the thousands) turn `factor` times slower, and a pair in between is a blend."""
    from oracle.gerupel_ref import banded_frequencies

    sc = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    spec = RotSpec(16, 10000.0, sc, half=True)
    cos, sin = spec.tables(50)
    f = banded_frequencies({"dims": 16, "base": 10000.0, "scaling": sc}, torch.float64)
    plain = 10000.0 ** (-2.0 * torch.arange(8, dtype=torch.float64) / 16)
    wave = 2 * math.pi / plain
    assert wave[0] < 16 and f[0] == plain[0]
    assert wave[7] > 64 and abs(f[7] - plain[7] / 8) < 1e-15
    mid = [i for i in range(8) if 16 <= wave[i] <= 64]
    assert mid and all(plain[i] / 8 < f[i] < plain[i] for i in mid)
    i = mid[0]
    u = (64 / wave[i] - 1.0) / 3.0
    assert abs(f[i] - ((1 - u) * plain[i] / 8 + u * plain[i])) < 1e-15
    a = torch.arange(50, dtype=torch.float64)[:, None] * f
    assert (cos.double() - torch.cos(a)).abs().max() < 1e-7 and (sin.double() - torch.sin(a)).abs().max() < 1e-7
    c0, _ = RotSpec(16, 10000.0, None, half=True).tables(50)
    assert (c0.double() - torch.cos(torch.arange(50, dtype=torch.float64)[:, None] * plain)).abs().max() < 1e-7


def test_restatement_window_blocks_and_sink():
    from oracle.gerupel_ref import window_pool_attention

    g = torch.Generator().manual_seed(0)
    T, H, G, D, P = 40, 4, 2, 6, 5
    q, k, v = (torch.randn(T, n, d, generator=g, dtype=torch.float64) for n, d in ((H, D), (G, D), (G, P)))
    temp = 0.5 + torch.rand(H, generator=g, dtype=torch.float64)
    full = window_pool_attention(q, k, v, 0.4, temp, None, 0)
    # by hand for one query and head: softmax over [0 | scores] with the 0 carrying no value
    i, h = 17, 3
    s = torch.cat([torch.zeros(1, dtype=torch.float64), (k[:i + 1, 1] @ q[i, h]) * 0.4 * temp[h]])
    w = torch.softmax(s, 0)[1:]
    assert (full[i, h] - w @ v[:i + 1, 1]).abs().max() < 1e-12
    # a window as long as the sequence changes nothing; blocks of one position behind a window bring every key back
    assert (window_pool_attention(q, k, v, 0.4, temp, T, 8) - full).abs().max() < 1e-12
    assert (window_pool_attention(q, k, v, 0.4, temp, 7, 1) - full).abs().max() < 1e-12
    # query 20, window 6, blocks of 4: keys 15 .. 20 and blocks 0 .. 2 (positions 0 .. 11, since 11 <= 14 and 15 > 14); 12 .. 14 unseen
    got = window_pool_attention(q, k, v, 0.4, temp, 6, 4)[20, 0]
    keys = torch.cat([k[:12, 0].view(3, 4, D).mean(1), k[15:21, 0]])
    vals = torch.cat([v[:12, 0].view(3, 4, P).mean(1), v[15:21, 0]])
    s = torch.cat([torch.zeros(1, dtype=torch.float64), (keys @ q[20, 0]) * 0.4 * temp[0]])
    assert (got - torch.softmax(s, 0)[1:] @ vals).abs().max() < 1e-12


def test_restatement_recurrence_and_router():
    from oracle.gerupel_ref import expert_mixture, gated_recurrence

    g = torch.Generator().manual_seed(1)
    T, H, D, P = 12, 2, 3, 4
    q, v = torch.randn(T, H, D, generator=g, dtype=torch.float64), torch.randn(T, H, P, generator=g, dtype=torch.float64)
    f = torch.rand(T, H, D, generator=g, dtype=torch.float64)
    o = gated_recurrence(q, f, v)
    # unrolled: S_t[d] = sum_s (prod_{s < r <= t} f_r[d]) (1 - f_s[d]) v_s
    t, h = 9, 1
    S = torch.zeros(D, P, dtype=torch.float64)
    for s in range(t + 1):
        decay = f[s + 1:t + 1, h].prod(0)
        S += (decay * (1 - f[s, h]))[:, None] * v[s, h][None, :]
    assert (o[t, h] - S.T @ q[t, h]).abs().max() < 1e-12
    # a forget gate of 1 writes nothing; of 0 keeps only the current value
    assert gated_recurrence(q, torch.ones_like(f), v).abs().max() == 0
    assert (gated_recurrence(q, torch.zeros_like(f), v) - q.sum(-1, keepdim=True) * v).abs().max() < 1e-12
    # router: with top = experts the weights are the softmax itself times the scale
    W, E, ff = 6, 3, 5
    Wt = {"router": torch.randn(E, W, generator=g, dtype=torch.float64)}
    for e in range(E):
        Wt.update({f"e{e}.gate": torch.randn(ff, W, generator=g, dtype=torch.float64), f"e{e}.up": torch.randn(ff, W, generator=g, dtype=torch.float64),
                   f"e{e}.down": torch.randn(W, ff, generator=g, dtype=torch.float64)})
    hcol = torch.randn(7, W, generator=g, dtype=torch.float64)
    got = expert_mixture(hcol, Wt, "", {"router": {"experts": E, "top": E, "scale": 2.0}})
    s = torch.softmax(hcol @ Wt["router"].T, -1)
    want = sum(s[:, e:e + 1] * 2.0 * ((torch.nn.functional.silu(hcol @ Wt[f"e{e}.gate"].T) * (hcol @ Wt[f"e{e}.up"].T)) @ Wt[f"e{e}.down"].T)
               for e in range(E))
    assert (got - want).abs().max() < 1e-12
