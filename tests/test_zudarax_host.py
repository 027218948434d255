"""CPU: host side of the parallel-branch decoder (Zudarax) -- configuration reader and its refusals, tensor names and shapes,
registry, rotary tables -- and properties of the plain restatement that the GPU tests lean on."""
import json
import math

import pytest
import torch

from vllm_neuron_b200.hybrid import HybridConfig, PolySpec, RotAttnSpec, RotSpec, random_weights, tensor_shapes


def _cfg(layers=None, groups=2):
    yarn = {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}
    a1 = {"type": "attention", "mlp": {"kind": "dense", "ff": 14},
          "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 5, "conv": 3, "scale": 0.3, "softcap": 7.0, "mask": {"size": 9},
                    "rot": {"dims": 4, "base": 100.0}}}
    a2 = {"type": "attention_2", "mlp": None,
          "mixer": {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 6, "diff": 0.4, "scale": 0.5, "rot": {"dims": 2, "base": 50.0}}}
    a3 = {"type": "attention_3", "mlp": {"kind": "dense", "ff": 10},
          "mixer": {"heads": 3, "kv_heads": 3, "dim": 8, "vdim": 4, "conv": 2, "scale": 0.35,
                    "rot": {"dims": 8, "base": 1000.0, "scaling": yarn}}}
    return {"architecture": "Zudarax", "vocab": 20, "width": 12, "norm": {"eps": 1e-5, "groups": groups},
            "layers": layers if layers is not None else [a3, a1, a2]}


def test_config_reader_round_trip_and_shapes():
    d = _cfg()
    cfg = HybridConfig.from_dict(d)
    assert cfg.style == "rms_parallel" and cfg.norm_groups == 2 and cfg.embed_scale == 1.0 and cfg.bigram is None
    assert cfg.to_dict() == d and HybridConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
    s3, s1, s2 = (L.mixer for L in cfg.layers)
    assert all(isinstance(m, RotAttnSpec) and m.rot.half for m in (s1, s2, s3))
    assert s3.sigmoid and s3.conv == 2 and not (s3.bias or s3.qk_norm or s3.chunk or s3.softcap or s3.gate) and s3.diff is None
    assert s1.bias and s1.qk_norm and (s1.conv, s1.chunk, s1.softcap) == (3, 9, 7.0) and not s1.sigmoid and s1.maps == 1
    assert s2.diff == 0.4 and s2.gate and s2.maps == 2 and (s2.q_cols, s2.k_cols, s2.v_cols) == (16, 8, 6) and not s2.conv
    assert isinstance(cfg.layers[0].mlp, PolySpec) and cfg.layers[2].mlp is None
    sh = tensor_shapes(cfg)
    assert sh["embed"] == sh["head"] == (20, 12) and sh["final.norm"] == (12,) and "l0.norm2" not in sh and "l0.norm1b" not in sh
    assert sh["l0.mix.q"] == (24, 12) and sh["l0.mix.k.conv"] == (24, 2) and sh["l0.mix.v.conv"] == (12, 2) and sh["l0.mix.pb"] == (3,)
    assert "l0.mix.q.b" not in sh and "l0.mix.q.norm" not in sh and sh["l0.mlp.act"] == (4,) and sh["l0.mlp.up"] == (10, 12)
    assert sh["l1.mix.q.b"] == (24,) and sh["l1.mix.k.norm"] == (12,) and sh["l1.mix.v.b"] == (10,) and "l1.mix.v.norm" not in sh
    assert sh["l1.mix.q.conv"] == (24, 3) and sh["l1.mix.o"] == (12, 20) and sh["l1.mlp.down"] == (12, 14)
    assert sh["l2.mix.q"] == (16, 12) and sh["l2.mix.k"] == (8, 12) and sh["l2.mix.v"] == (6, 12) and sh["l2.mix.g"] == (2, 12)
    assert sh["l2.mix.lq1"] == sh["l2.mix.lk2"] == (4,) and sh["l2.mix.o"] == (12, 12) and "l2.mlp.up" not in sh
    assert set(random_weights(cfg)) == set(sh)


def test_config_reader_refuses_what_the_design_does_not_have():
    d = _cfg()
    bad_rot = json.loads(json.dumps(d["layers"][1]))
    bad_rot["mixer"]["rot"]["dims"] = 8                                       # more rotating columns than the head has
    odd_rot = json.loads(json.dumps(d["layers"][1]))
    odd_rot["mixer"]["rot"]["dims"] = 3
    bad_heads = json.loads(json.dumps(d["layers"][1]))
    bad_heads["mixer"]["kv_heads"] = 3
    for bad in ({"type": "delta", "mlp": None, "mixer": {"heads": 2, "kv_heads": 2, "dim": 4, "vdim": 4, "conv": 2}},
                {"type": "mamba2", "mlp": None, "mixer": {"heads": 2, "vdim": 3, "state": 5, "groups": 1, "conv": 3}},
                bad_rot, odd_rot, bad_heads, {**d["layers"][0], "mlp": {"kind": "moe"}}):
        with pytest.raises(ValueError):
            HybridConfig.from_dict(_cfg(layers=[bad]))
    with pytest.raises(ValueError):
        HybridConfig.from_dict(_cfg(groups=5))                                # 12 columns do not split into 5 equal parts
    with pytest.raises(ValueError):                                          # the other designs do not take these mixers
        HybridConfig.from_dict({**_cfg(layers=[d["layers"][2]]), "architecture": "Kenetar", "embedding": {"scale": 1.0}})


def test_registry_picks_the_model_class_by_config():
    from vllm_neuron_b200 import registry

    arch, entry = registry.resolve(_cfg())
    assert arch == "Zudarax" and entry.family == "hybrid" and torch.float32 in entry.dtypes and torch.bfloat16 in entry.dtypes
    assert isinstance(entry.read_config(_cfg()), HybridConfig)


def test_rotary_tables_follow_the_restatement():
    from oracle.zudarax_ref import rotary_frequencies

    for rot in ({"dims": 16, "base": 250.0}, {"dims": 8, "base": 10000.0, "scaling": {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 1.0}},
                {"dims": 32, "base": 5e5, "scaling": {"factor": 3.0, "original": 4096, "fast": 32.0, "slow": 2.0}}):
        cos, sin = RotSpec(rot["dims"], rot["base"], rot.get("scaling")).tables(50)
        f, mag = rotary_frequencies(rot, torch.float64)
        a = torch.arange(50, dtype=torch.float64)[:, None] * f
        assert (cos.double() - torch.cos(a) * mag).abs().max() < 1e-6 and (sin.double() - torch.sin(a) * mag).abs().max() < 1e-6
        if rot.get("scaling"):
            plain = rot["base"] ** (-2.0 * torch.arange(rot["dims"] // 2, dtype=torch.float64) / rot["dims"])
            assert abs(mag - (0.1 * math.log(rot["scaling"]["factor"]) + 1)) < 1e-12
            assert torch.all(f <= plain + 1e-15) and torch.all(f >= plain / rot["scaling"]["factor"] - 1e-15)
            assert f[0] == plain[0] or rot["dims"] == 32                      # the fastest pair keeps its frequency


def test_restatement_scores_depend_on_relative_position_and_only_rotating_columns_turn():
    from oracle.zudarax_ref import rotate_half

    g = torch.Generator().manual_seed(0)
    rot = {"dims": 6, "base": 30.0}
    q, k = torch.randn(1, 1, 10, generator=g).double(), torch.randn(1, 1, 10, generator=g).double()
    qs, ks = rotate_half(q.expand(12, 1, 10), rot), rotate_half(k.expand(12, 1, 10), rot)
    assert torch.equal(qs[:, :, 6:], q.expand(12, 1, 10)[:, :, 6:])
    s = qs[:, 0] @ ks[:, 0].T
    for d in range(5):
        assert (torch.diagonal(s, -d) - s[d, 0]).abs().max() < 1e-12
    assert (qs[0] - q[0]).abs().max() < 1e-15                                  # position 0 turns nothing


def test_restatement_chunks_first_tokens_and_causality():
    """A token of a new chunk sees nothing of the chunks before it through the chunked layer; no token sees a later one."""
    from oracle import zudarax_ref

    d = _cfg()
    only_chunked = _cfg(layers=[d["layers"][1]])
    only_chunked["layers"][0]["mixer"]["conv"] = 1                            # one tap: the convolution looks at no earlier token
    cfg = HybridConfig.from_dict(only_chunked)
    W = random_weights(cfg, seed=3)
    a = torch.randint(0, 20, (27,), generator=torch.Generator().manual_seed(1)).tolist()
    b = list(a)
    b[:9] = [(t + 1) % 20 for t in a[:9]]                                      # another first chunk
    la, lb = zudarax_ref.forward(only_chunked, W, a), zudarax_ref.forward(only_chunked, W, b)
    assert (la[9:] - lb[9:]).abs().max() < 1e-12 and (la[:9] - lb[:9]).abs().max() > 1e-3
    full = _cfg()
    Wf = random_weights(HybridConfig.from_dict(full), seed=4)
    whole = zudarax_ref.forward(full, Wf, a)
    assert (zudarax_ref.forward(full, Wf, a[:11]) - whole[:11]).abs().max() < 1e-10
    assert (zudarax_ref.forward(full, Wf, a[:1]) - whole[:1]).abs().max() < 1e-10


def test_restatement_differential_and_polynomial_parts():
    from oracle.zudarax_ref import group_rms_norm, poly_norm, rms_unit

    z = torch.randn(3, 40, generator=torch.Generator().manual_seed(2)).double()
    out = poly_norm(z, torch.tensor([0.0, 1.0, 0.0, 0.25]).double(), 1e-12)
    assert ((out - 0.25).pow(2).mean(-1).sqrt() - 1).abs().max() < 1e-9      # N(z^2) has unit RMS; e is added after
    assert (poly_norm(z, torch.tensor([1.0, 0, 0, 0]).double(), 1e-12) - rms_unit(z, 1e-12)).abs().max() < 1e-12
    x = torch.randn(2, 12).double()
    parts = group_rms_norm(x, torch.ones(12).double(), 3, 1e-12).view(2, 3, 4)
    assert (parts.pow(2).mean(-1) - 1).abs().max() < 1e-9
