"""GPU: the dual-norm parallel decoder (Gerupel) through the stand-alone engine (runner step, page pool, state slots) against
the plain restatement on whole sequences: whole prompts, token-by-token decoding from the first token, ragged portions down
to two tokens, mixed batches with rows and pages that are freed and reused, decoding far past every window, configurations
drawn at random, greedy generation through the scheduler and the trace command line.  The 32-bit mode is held to 1e-4 of
the logit spread; the bf16 mode to its rounding noise.  In bf16 every router keeps ALL its experts: with fewer, a near-tie
between two scores that bf16 rounding flips would swap an expert and move one token's logits by far more than rounding does
(which experts are chosen is tested in 32-bit, where nothing flips)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = scaling
    return r


def _layer(left, right, mlp, ls=1.0, rs=1.0):
    """left: (heads, kv_heads, dim, vdim, scale, rot, mask); right: (heads, dim, vdim); mlp: (experts, top, ff, scale) or None."""
    h, g, d, v, scale, rot, mask = left
    lm = {"heads": h, "kv_heads": g, "dim": d, "vdim": v, "scale": scale, "rot": rot}
    if mask:
        lm["mask"] = mask
    f = None
    if mlp:
        f = {"kind": "moe", "router": {"experts": mlp[0], "top": mlp[1], "scale": mlp[3]}, "expert": {"ff": mlp[2]}}
    return {"type": "parallel", "mixer": {"left": lm, "right": dict(zip(("heads", "dim", "vdim"), right)), "left_scale": ls,
                                          "right_scale": rs}, "mlp": f}


def cfg_a():
    """Sizes off every grid (the CUDA-core kernels in both modes, GEMMs off the tensor cores): three query heads on one kv head
    and two on two, rotation over half a head and over a whole one, a window that is no multiple of its blocks, blocks that do
    not divide the page, a window shorter than a block, a layer without window (no blocks either), a layer without
    feed-forward, one expert of one, top = experts; the first two layers run twice."""
    band = {"factor": 3.0, "low": 1.0, "high": 3.0, "original": 24}
    return {"architecture": "Gerupel", "vocab": 90, "width": 42, "norm": {"eps": 1e-5}, "residual_mult": 0.7,
            "loop": {"start": 0, "stop": 2, "times": 2}, "layers": [
        _layer((3, 1, 12, 20, 0.29, _rot(6, 300.0, band), {"size": 9, "pool": 4}), (2, 10, 7), (5, 2, 24, 1.5), 0.9, 1.2),
        _layer((2, 2, 10, 6, 0.32, _rot(10, 50.0), {"size": 3, "pool": 5}), (3, 5, 9), None, 1.1, 0.6),
        _layer((4, 2, 8, 14, 0.35, _rot(4, 1000.0), None), (1, 33, 6), (1, 1, 20, 0.8)),
        _layer((2, 1, 14, 10, 0.27, _rot(8, 10000.0, band), {"size": 13, "pool": 1}), (2, 6, 12), (3, 3, 16, 2.0), 0.5, 1.0),
    ]}


def cfg_b():
    """Tensor-core sizes throughout (prompt portions of 16 tokens and more on the tensor-core attention kernel, single tokens on
    the tensor-core decode kernel): windows of one page and a half and of 20 positions, blocks of 16, 4 and 48 positions (more
    than a page), key and value sizes that differ, the last two layers run three times (the repetition ends the model)."""
    band = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    return {"architecture": "Gerupel", "vocab": 200, "width": 64, "norm": {"eps": 1e-6}, "residual_mult": 0.6,
            "loop": {"start": 2, "stop": 4, "times": 3}, "layers": [
        _layer((4, 1, 32, 16, 0.18, _rot(32, 5000.0, band), {"size": 48, "pool": 16}), (2, 32, 16), (8, 2, 32, 2.0), 0.85, 1.15),
        _layer((4, 2, 16, 32, 0.25, _rot(8, 1000.0), {"size": 20, "pool": 4}), (4, 16, 16), (4, 1, 48, 1.0), 1.0, 0.7),
        _layer((2, 2, 48, 48, 0.14, _rot(16, 100000.0, band), {"size": 33, "pool": 48}), (1, 64, 32), None, 1.2, 1.0),
        _layer((8, 2, 16, 16, 0.25, _rot(16, 100.0), {"size": 64, "pool": 2}), (3, 48, 16), (6, 3, 32, 0.5)),
    ]}


def cfg_c():
    """No repeated layers at all, a residual factor of 1, a window with no blocks behind it, and head sizes of 64 / 128."""
    return {"architecture": "Gerupel", "vocab": 160, "width": 128, "norm": {"eps": 1e-6}, "layers": [
        _layer((2, 1, 64, 128, 0.125, _rot(16, 10000.0), {"size": 72, "pool": 8}), (2, 128, 64), (4, 2, 64, 1.0)),
        _layer((4, 4, 64, 64, 0.125, _rot(64, 30000.0), {"size": 50}), (4, 64, 32), (4, 4, 32, 3.0), 0.7, 1.3),
        _layer((2, 2, 128, 64, 0.09, _rot(32, 500.0), {"size": 7, "pool": 32}), (1, 256, 48), None),
    ]}


class Case:
    def __init__(self, cfgd, dtype, seed=0, max_num_seqs=3, pool_tokens=1024):
        from vllm_neuron_b200.engine import B200Engine
        from vllm_neuron_b200.hybrid import HybridConfig, random_weights

        if dtype == "bfloat16":
            for L in cfgd["layers"]:
                if L["mlp"]:
                    L["mlp"]["router"]["top"] = L["mlp"]["router"]["experts"]
        self.cfgd, self.dtype = cfgd, dtype
        self.cfg = HybridConfig.from_dict(cfgd)
        self.W = random_weights(self.cfg, seed=seed)
        self.engine = B200Engine(self.cfg, self.W, dtype=dtype, max_num_seqs=max_num_seqs, max_pool_tokens=pool_tokens,
                                 max_num_batched_tokens=1 << 20)
        self.tol = 1e-4 if dtype == "float32" else 0.06
        self._ref = {}

    def tokens(self, n, seed):
        return torch.randint(0, self.cfg.vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()

    def ref(self, toks):
        from oracle import gerupel_ref

        key = tuple(toks)
        if key not in self._ref:
            self._ref[key] = gerupel_ref.forward(self.cfgd, self.W, toks)
        return self._ref[key]

    def replay(self, reqs, schedule):
        """reqs: id -> tokens; schedule: list of steps, each [(id, n)].  Logits of every position, per request."""
        at = {i: 0 for i in reqs}
        got = {i: [] for i in reqs}
        for step in schedule:
            entries, end = [], []
            for i, n in step:
                entries.append((i, reqs[i][at[i]:at[i] + n], list(range(n))))
                at[i] += n
                if at[i] == len(reqs[i]):
                    end.append(i)
            taps = self.engine.replay_step(entries, end)
            for i, n in step:
                assert taps[i].shape == (n, self.cfg.vocab)
                got[i].append(taps[i])
        assert all(at[i] == len(reqs[i]) for i in reqs)
        return {i: torch.cat(v) for i, v in got.items()}

    def errs(self, got, toks):
        want = self.ref(toks)
        d = got.double() - want
        d = d - d.mean(-1, keepdim=True)
        spread = (want - want.mean(-1, keepdim=True)).pow(2).mean().sqrt()
        return d.pow(2).mean(-1).sqrt() / spread

    def check(self, got, reqs):
        e = torch.cat([self.errs(got[i], toks) for i, toks in reqs.items()])
        assert e.max().item() < self.tol, (e.max().item(), e.median().item())


def _portions(n, sizes):
    out, k = [], 0
    while n > 0:
        c = min(sizes[k % len(sizes)], n)
        out.append(c)
        n -= c
        k += 1
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cfg", [cfg_a, cfg_b, cfg_c])
def test_whole_prompt_decode_and_portions_agree_with_the_restatement(cfg, dtype):
    c = Case(cfg(), dtype)
    toks = c.tokens(150, 1)
    whole = c.replay({"w": toks}, [[("w", 150)]])
    c.check(whole, {"w": toks})
    short = c.tokens(90, 2)
    one_by_one = c.replay({"d": short}, [[("d", 1)] for _ in short])          # the first tokens, then decoding past windows and blocks
    c.check(one_by_one, {"d": short})
    sizes = _portions(150, [2, 3, 2, 27, 30, 2, 1, 33, 7, 31, 1, 1, 10])     # cuts inside pages, windows and blocks, and at their edges
    cut = c.replay({"p": toks}, [[("p", n)] for n in sizes])
    c.check(cut, {"p": toks})
    d = (cut["p"] - whole["w"]).abs().max().item() / whole["w"].abs().max().item()
    assert d < (1e-5 if dtype == "float32" else 0.05), d                      # how the prompt was cut does not matter


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompt_whole_in_portions_and_in_a_batch(dtype):
    """A 700-token prompt (hundreds of pooled blocks behind the window) whole, in portions, and beside two other requests (one
    decoding, one with a long portion of its own) through three rows."""
    c = Case(cfg_c(), dtype, max_num_seqs=3, pool_tokens=2048)
    toks, other, short = c.tokens(700, 5), c.tokens(300, 6), c.tokens(40, 7)
    whole = c.replay({"w": toks}, [[("w", 700)]])
    c.check(whole, {"w": toks})
    cut = c.replay({"p": toks}, [[("p", n)] for n in _portions(700, [130, 2, 127, 128, 1, 200, 31, 81])])
    c.check(cut, {"p": toks})
    d = (cut["p"] - whole["w"]).abs().max().item() / whole["w"].abs().max().item()
    assert d < (1e-5 if dtype == "float32" else 0.05), d
    reqs = {"a": toks, "b": other, "c": short}
    sched = [[("a", 300), ("c", 1)], [("a", 1), ("b", 129), ("c", 1)], [("a", 270), ("b", 171), ("c", 2)]] + \
            [[("a", 1), ("c", 1)] for _ in range(36)] + [[("a", 93)]]
    c.check(c.replay(reqs, sched), reqs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cfg", [cfg_a, cfg_b])
def test_mixed_batches_with_reused_rows_and_pages(cfg, dtype):
    """Seven requests of unequal length (1 .. 130 tokens) through THREE rows and a pool that cannot hold them all at once:
    portions beside single tokens, requests that sit out steps, rows, pages, pooled-block rows and recurrent state taken over by
    later requests."""
    c = Case(cfg(), dtype, max_num_seqs=3, pool_tokens=320)
    lens = {"a": 130, "b": 1, "c": 37, "d": 2, "e": 64, "f": 33, "g": 90}
    reqs = {i: c.tokens(n, 10 + k) for k, (i, n) in enumerate(lens.items())}
    sched = [
        [("a", 40), ("b", 1), ("c", 2)],            # b ends: its row and page go back
        [("a", 1), ("c", 30), ("d", 1)],
        [("c", 1), ("d", 1)],                        # a sits out; d ends
        [("a", 25), ("c", 1), ("e", 31)],
        [("a", 1), ("c", 1), ("e", 1)],
        [("a", 1), ("c", 2), ("e", 32)],            # c and e end
        [("a", 62), ("f", 33), ("g", 2)],           # f is whole in one step and ends
        [("g", 60)],
        [("g", 1)], [("g", 1)],
        [("g", 26)],
    ]
    got = c.replay(reqs, sched)
    c.check(got, reqs)
    assert c.engine.pool.num_free == c.engine.num_blocks - 1 and not c.engine.scheduler.running
    if dtype == "float32":                                                     # each alone gives the same numbers
        alone = Case(cfg(), dtype, max_num_seqs=1, pool_tokens=160)
        for i in ("a", "e", "g"):
            solo = alone.replay({i: reqs[i]}, [[(i, len(reqs[i]))]])
            d = (solo[i] - got[i]).abs().max().item() / solo[i].abs().max().item()
            assert d < 1e-5, (i, d)


def _random_cfg(rng):
    """A configuration drawn at random: 2-5 layers, head counts, sizes, windows, blocks and constants that need not be multiples of
    anything, with or without feed-forward, band scaling, window, blocks and repeated layers."""
    width = rng.choice([48, 96, 120, 192])
    layers = []
    for _ in range(rng.randint(2, 5)):
        h = rng.choice([1, 2, 3, 4, 6, 8])
        g = rng.choice([x for x in (1, 2, 3, 4, 6, 8) if h % x == 0])
        d, v = rng.choice([8, 12, 16, 32, 40, 64]), rng.choice([8, 16, 20, 48, 80])
        rot = _rot(rng.choice([x for x in (2, 4, 8, 12, 16, 32, 64) if x <= d]), rng.choice([100.0, 10000.0, 500000.0]))
        if rng.random() < 0.6:
            rot["scaling"] = {"factor": rng.choice([2.0, 4.0, 32.0]), "low": rng.choice([1.0, 2.0]), "high": rng.choice([4.0, 8.0]),
                              "original": rng.choice([16, 64, 4096])}
        mask = None
        if rng.random() < 0.85:
            mask = {"size": rng.choice([1, 5, 32, 44, 100, 300])}
            if rng.random() < 0.8:
                mask["pool"] = rng.choice([1, 2, 3, 8, 10, 32, 37, 64])
        e = rng.choice([1, 2, 5, 8, 16])
        mlp = None if rng.random() < 0.2 else (e, rng.randint(1, e), rng.choice([24, 64, 100]), rng.choice([0.5, 1.0, 3.0]))
        layers.append(_layer((h, g, d, v, rng.choice([d ** -0.5, 0.1, 0.3]), rot, mask),
                             (rng.choice([1, 2, 3, 6]), rng.choice([4, 9, 16, 48, 100, 130]), rng.choice([5, 16, 24, 64])), mlp,
                             rng.choice([0.5, 1.0, 1.3]), rng.choice([0.4, 1.0, 1.1])))
    out = {"architecture": "Gerupel", "vocab": rng.choice([100, 257, 512]), "width": width, "norm": {"eps": rng.choice([1e-6, 1e-5])},
           "residual_mult": rng.choice([0.3, 0.6, 1.0]), "layers": layers}
    if rng.random() < 0.8:
        a = rng.randint(0, len(layers) - 1)
        out["loop"] = {"start": a, "stop": rng.randint(a + 1, len(layers)), "times": rng.randint(1, 3)}
    return out


@pytest.mark.parametrize("seed", [1, 4, 7, 11, 13, 16])
def test_random_configurations_in_32_bit(seed):
    """Whole prompt, ragged portions and a mixed batch of a prompt beside a decoding request, for configurations nobody
    picked by hand."""
    import random

    c = Case(_random_cfg(random.Random(seed)), "float32", seed=seed, max_num_seqs=3, pool_tokens=1024)
    toks, short = c.tokens(420, 50 + seed), c.tokens(30, 60 + seed)
    c.check(c.replay({"w": toks}, [[("w", 420)]]), {"w": toks})
    c.check(c.replay({"p": toks}, [[("p", n)] for n in _portions(420, [2, 3, 130, 1, 33, 7, 64, 1, 1, 257])]), {"p": toks})
    mixed = c.replay({"a": toks, "b": short}, [[("a", 300), ("b", 1)]] + [[("a", 1), ("b", 1)] for _ in range(29)] + [[("a", 91)]])
    c.check(mixed, {"a": toks, "b": short})


@pytest.mark.parametrize("seed", [2, 9, 21])
def test_random_configurations_in_bf16(seed):
    import random

    c = Case(_random_cfg(random.Random(seed)), "bfloat16", seed=seed, max_num_seqs=2, pool_tokens=512)
    toks = c.tokens(200, 70 + seed)
    c.check(c.replay({"p": toks}, [[("p", n)] for n in _portions(200, [40, 2, 1, 1, 65, 17])]), {"p": toks})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    """280 single tokens after a short prompt: every window slides over decoded tokens, blocks close and become visible while
    decoding, and the recurrence runs 300 steps."""
    c = Case(cfg_b(), dtype, max_num_seqs=2, pool_tokens=512)
    toks = c.tokens(300, 3)
    got = c.replay({"x": toks}, [[("x", 20)]] + [[("x", 1)] for _ in range(280)])
    c.check(got, {"x": toks})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(dtype):
    """engine.generate: five prompts over three rows, prompts cut by a 48-token budget next to decodes.  Every generated
    token must be the restatement's argmax given the same history (or lie within rounding noise of it)."""
    from vllm_neuron_b200.engine import B200Engine

    c = Case(cfg_b(), dtype)
    eng = B200Engine(c.cfg, c.W, dtype=dtype, max_num_seqs=3, max_pool_tokens=512, max_num_batched_tokens=48)
    prompts = [c.tokens(n, 20 + n) for n in (70, 3, 33, 1, 100)]
    outs = eng.generate(prompts, max_new_tokens=12)
    assert eng.pool.num_free == eng.num_blocks - 1
    exact = far = 0
    for p, o in zip(prompts, outs):
        assert len(o) == 12
        ref = c.ref(p + o)
        for k, tok in enumerate(o):
            row = ref[len(p) + k - 1]
            best = int(row.argmax())
            exact += best == tok
            gap = (row[best] - row[tok]).item() / row.std().item()
            far += gap > (1e-4 if dtype == "float32" else 0.1)
    assert far <= (0 if dtype == "float32" else 3) and exact >= (60 if dtype == "float32" else 45), (far, exact)


def test_served_from_a_checkpoint_directory_and_layer_streams(tmp_path):
    """config.json + model.safetensors on disk -> registry -> engine; same logits as the in-memory weights, and the residual
    stream after every layer RUN (a repeated layer counts each time) equals the restatement's."""
    import json

    from oracle import gerupel_ref
    from safetensors.torch import save_file
    from vllm_neuron_b200.engine import B200Engine
    from vllm_neuron_b200.registry import load_config

    c = Case(cfg_a(), "float32")
    with open(tmp_path / "config.json", "w") as f:
        json.dump(c.cfgd, f)
    save_file({k: v.contiguous() for k, v in c.W.items()}, str(tmp_path / "model.safetensors"))
    arch, entry, cfg = load_config(str(tmp_path))
    assert arch == "Gerupel" and entry.family == "hybrid" and cfg == c.cfg
    eng = B200Engine.from_pretrained(str(tmp_path), dtype="float32", max_num_seqs=2, max_pool_tokens=128)
    toks = c.tokens(50, 5)
    cap, fwd = [], eng.model.forward
    eng.model.forward = lambda tokens, meta, rows: fwd(tokens, meta, rows, capture=cap)
    got = eng.replay_step([("r", toks, list(range(50)))], ["r"])["r"]
    assert c.errs(got, toks).max().item() < 1e-4
    streams = []
    gerupel_ref.forward(c.cfgd, c.W, toks, streams=streams)
    assert len(cap) == len(c.cfgd["layers"]) + 2 == len(streams)
    for got_x, want_x in zip(cap, streams):
        assert (got_x.double().cpu() - want_x).abs().max().item() < 1e-4 * want_x.abs().max().item()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_command_line(tmp_path, dtype):
    """bin/trace_run as a user runs it: a checkpoint folder, steps on standard input (two requests, portions beside single
    tokens, a step that reports nothing, a request that ends and frees its row), logits files per step."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np
    from safetensors.torch import save_file

    c = Case(cfg_b(), dtype)
    model_dir, out_dir = tmp_path / "model", tmp_path / "out"
    model_dir.mkdir()
    with open(model_dir / "config.json", "w") as f:
        json.dump(c.cfgd, f)
    save_file({k: v.contiguous() for k, v in c.W.items()}, str(model_dir / "model.safetensors"))
    a, b = c.tokens(70, 31), c.tokens(9, 32)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:33], "want": [0, 32]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[33:35], "want": []}, {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[8:], "want": [0]}, {"id": "a", "tokens": a[35:36], "want": [0]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": a[36:], "want": [0, 33]}], "end": ["a"]},
    ]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(model_dir), "--dtype", dtype,
                        "--out", str(out_dir), "--max-tokens", "192"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [ln for ln in p.stdout.splitlines() if ln.startswith("done")] == [f"done {i}" for i in range(4)]
    ra, rb = c.ref(a), c.ref(b)
    want = {0: [ra[0], ra[32]], 1: [rb[7]], 2: [rb[8], ra[35]], 3: [ra[36], ra[69]]}
    for n, rows in want.items():
        got = np.fromfile(out_dir / f"{n}.f32", dtype="<f4").reshape(len(rows), -1)
        for g, w in zip(got, rows):
            d = torch.from_numpy(g).double() - w
            assert (d - d.mean()).pow(2).mean().sqrt().item() < c.tol * (w - w.mean()).pow(2).mean().sqrt().item()
