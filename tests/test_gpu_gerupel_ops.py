"""GPU: every mechanism of the dual-norm parallel decoder (Gerupel) alone, against the plain restatement in
oracle/gerupel_ref.py (fp64).  Sizes are awkward on purpose (odd widths, head sizes that are no multiple of a warp, a vector
or a page; pages handed out in reverse), and where random numbers would hide a fault (a window's edge, a block that is just
seen or not yet, a far block, the 1 in the denominator) the inputs are made so that it shows."""
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _ops():
    from vllm_neuron_b200 import ops

    return ops


def _meta(entries, blocks, bs=8):
    from vllm_neuron_b200.hybrid import StepMeta

    return StepMeta.build(entries, blocks, bs, DEV)


def _err(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    return (got - want).abs().max().item() / max(want.abs().max().item(), 1e-30)


def _close(got, want, tol):
    e = _err(got, want)
    assert e < tol, e


def _bf16_values(*shape, g, scale=1.0):
    """Random numbers that bf16 holds exactly: fp32 and bf16 pools then cache the same values."""
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).float()


# ------------------------------------------------------------------------------------------------ embedding, residual step, norms
@pytest.mark.parametrize("width", [7, 60, 264, 2048])
@pytest.mark.parametrize("table_dtype", [torch.float32, torch.bfloat16])
def test_normed_embedding(width, table_dtype):
    from oracle.gerupel_ref import rms_norm

    ops = _ops()
    g = torch.Generator().manual_seed(width)
    table = (torch.randn(50, width, generator=g) * 3).to(table_dtype)
    w = 1 + 0.3 * torch.randn(width, generator=g)
    toks = torch.tensor([0, 49, 7, 7, 13], dtype=torch.int32)
    got = ops.embed_rmsnorm(toks.to(DEV), table.to(DEV), w.to(DEV), 1e-5)
    _close(got, rms_norm(table.double()[toks.long()], w.double(), 1e-5), 3e-6)


@pytest.mark.parametrize("width", [7, 60, 264, 2048])
def test_scaled_residual_step_with_two_norms(width):
    from oracle.gerupel_ref import rms_norm

    ops = _ops()
    g = torch.Generator().manual_seed(width + 1)
    T, top, eps = 9, 3, 1e-5
    x = torch.randn(T, width, generator=g) * 3
    wide = torch.randn(T, 2 * width + 5, generator=g)            # two branches are column ranges of wider rows
    y3, wt = torch.randn(T * top, width, generator=g), torch.rand(T, top, generator=g)
    rows, vec = torch.randn(T, width, generator=g), torch.randn(width, generator=g)
    w1, w2 = 1 + 0.2 * torch.randn(width, generator=g), 1 + 0.2 * torch.randn(width, generator=g)
    c1, c2, c3 = 0.4, 0.55, 1.25
    wd = wide.to(DEV)
    full = dict(y1=wd[:, 3:3 + width], c1=c1, y2=wd[:, width + 5:], c2=c2, y3=y3.to(DEV), nsum=top, y3_weight=wt.to(DEV), c3=c3,
                add_rows=rows.to(DEV), add_vec=vec.to(DEV))
    want_full = x.double() + c1 * wide[:, 3:3 + width].double() + c2 * wide[:, width + 5:].double() + \
        c3 * (y3.double().view(T, top, width) * wt.double()[:, :, None]).sum(1) + rows.double() + vec.double()
    cases = [(full, want_full), ({}, x.double()), (dict(add_vec=vec.to(DEV)), x.double() + vec.double()),
             (dict(y2=wd[:, width + 5:], c2=c2, y3=y3.to(DEV), nsum=top, c3=c3),           # experts without weights: the plain sum
              x.double() + c2 * wide[:, width + 5:].double() + c3 * y3.double().view(T, top, width).sum(1))]
    for terms, want_x in cases:
        for dt, tol in ((torch.float32, 3e-6), (torch.bfloat16, 6e-3)):
            xi = x.to(DEV)
            h1, h2 = ops.scaled_add_rmsnorm2(xi, eps, **terms, w1=w1.to(DEV), w2=w2.to(DEV), out_dtype=dt)
            _close(xi, want_x, 3e-7)
            _close(h1, rms_norm(want_x, w1.double(), eps), tol)
            _close(h2, rms_norm(want_x, w2.double(), eps), tol)
    xi = x.to(DEV)                                                # one norm, or none: the stream is updated all the same
    h1, h2 = ops.scaled_add_rmsnorm2(xi, eps, **full, w1=w1.to(DEV), out_dtype=torch.float32)
    assert h2 is None
    _close(h1, rms_norm(want_full, w1.double(), eps), 3e-6)
    xi = x.to(DEV)
    assert ops.scaled_add_rmsnorm2(xi, eps, **full) == (None, None)
    _close(xi, want_full, 3e-7)


def test_head_norm_without_a_gate():
    from oracle.gerupel_ref import rms_norm

    ops = _ops()
    g = torch.Generator().manual_seed(2)
    T, H, P = 6, 5, 36
    o = torch.randn(T, H, P, generator=g) * torch.tensor([0.01, 1.0, 30.0, 2.0, 0.5])[None, :, None]
    w = 1 + 0.3 * torch.randn(P, generator=g)
    got = ops.head_rmsnorm_gate(o.reshape(T, -1).to(DEV), None, 0, w.to(DEV), 1e-6, H, torch.float32)
    _close(got, rms_norm(o.double(), w.double(), 1e-6).reshape(T, -1), 3e-6)


# ------------------------------------------------------------------------------------------------ rotation, temperature, cache write
@pytest.mark.parametrize("kv_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("lead", [3, 4])   # columns before q: 3 puts the rows off the 16-byte grid (scalar kernel), 4 on it
def test_band_scaled_rotation_temperature_and_cache_write(kv_dtype, lead):
    """Rotation over 16 of 24 columns with frequencies in all three wavelength bands, q times a factor per head."""
    from oracle.gerupel_ref import banded_frequencies, rotate_half
    from vllm_neuron_b200.hybrid import RotSpec

    ops = _ops()
    g = torch.Generator().manual_seed(11)
    H, G, D, Dv, rot_n, bs = 5, 1, 24, 20, 16, 8
    pos0, n = 37, 13                                                          # positions that cross page borders
    sc = {"factor": 6.0, "low": 1.0, "high": 4.0, "original": 40}
    rot = {"dims": rot_n, "base": 300.0, "scaling": sc}
    f, plain = banded_frequencies(rot, torch.float64), banded_frequencies({"dims": rot_n, "base": 300.0}, torch.float64)
    ratio = f / plain                                                         # kept, blended and slowed pairs are all there
    assert (ratio == 1).any() and ((ratio - 1 / 6.0).abs() < 1e-12).any() and ((ratio > 0.2) & (ratio < 0.99)).any()
    rows = torch.randn(n, lead + H * D + G * D + G * Dv, generator=g)
    temp = torch.tensor([0.5, 1.0, 1.7, 0.9, 2.5])
    cos, sin = (t.to(DEV) for t in RotSpec(rot_n, 300.0, sc, half=True).tables(64))
    pages = [6, 5, 4, 3, 2, 1, 7]                                              # not in order
    meta = _meta([(0, pos0, n)], {0: pages}, bs)
    k_pool = torch.zeros(8, G, bs, D, dtype=kv_dtype, device=DEV)
    v_pool = torch.zeros(8, G, bs, Dv, dtype=kv_dtype, device=DEV)
    q = ops.qk_norm_rope_kv_write(rows.to(DEV), lead, lead + H * D, lead + H * D + G * D, H, k_pool, v_pool, meta, rot_n=rot_n,
                                  rot_half=True, cos=cos, sin=sin, q_head_scale=temp.to(DEV))
    r = rows.double()
    rq, rk, rv = r[:, lead:lead + H * D], r[:, lead + H * D:lead + H * D + G * D], r[:, lead + H * D + G * D:]

    def turn(u, heads):
        u = torch.cat([u.new_zeros(pos0, heads, D), u.view(n, heads, D)])     # the restatement counts positions from 0
        return rotate_half(u, rot)[pos0:]

    tol = 3e-6 if kv_dtype == torch.float32 else 5e-3
    _close(q, (turn(rq, H) * temp.double()[None, :, None]).reshape(n, -1), 3e-6)
    wk, wv = turn(rk, G), rv.view(n, G, Dv)
    for i in range(n):
        p = pos0 + i
        _close(k_pool[pages[p // bs], :, p % bs], wk[i], tol)
        _close(v_pool[pages[p // bs], :, p % bs], wv[i], tol)


# ------------------------------------------------------------------------------------------------ window + pooled blocks + unit sink
def _attend(q, k, v, scale, window, pool, *, kv_dtype, portions, bs=8, sink=True):
    """One sequence through the pools: q [T, H, D], k [T, G, D], v [T, G, P], cut into `portions`; pages in reverse order, in
    row 1 of the block table.  Each portion is cached, its closed blocks are averaged, and then it is attended, as a layer does
    it.  Returns (outputs [T, H, P], pooled key pool, pooled value pool, pages)."""
    ops = _ops()
    T, H, D = q.shape
    G, P = k.shape[1], v.shape[2]
    nb = -(-T // bs) + 1
    pages = list(range(nb - 1, 0, -1))
    k_pool = torch.zeros(nb, G, bs, D, dtype=kv_dtype, device=DEV)
    v_pool = torch.zeros(nb, G, bs, P, dtype=kv_dtype, device=DEV)
    ppb = -(-bs // pool) if pool else 1
    pk = torch.full((nb, G, ppb, D), 77.0, dtype=kv_dtype, device=DEV)          # stale rows are loud: reading one shows
    pv = torch.full((nb, G, ppb, P), 77.0, dtype=kv_dtype, device=DEV)
    table = torch.zeros(3, nb, dtype=torch.int32, device=DEV)
    table[1, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
    rows = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1).to(DEV)
    zero = torch.zeros(H, device=DEV) if sink else None
    out, at = [], 0
    for n in portions:
        meta = _meta([(1, at, n)], {1: pages}, bs)
        qd = ops.qk_norm_rope_kv_write(rows[at:at + n], 0, H * D, (H + G) * D, H, k_pool, v_pool, meta)
        if pool:
            ops.kv_pool_mean(k_pool, v_pool, pk, pv, table, meta, pool)
        out.append(ops.swa_sink_attn(qd, H, k_pool, v_pool, table, meta, zero, scale, window, split_p=True,
                                     pooled=(pk, pv, pool) if pool else None).float().view(n, H, P))
        at += n
    assert at == T
    return torch.cat(out), pk, pv, pages


def _cuts(T):
    """Whole (the tensor-core prompt kernel in bf16), token by token (the decode kernels), and ragged portions down to two tokens."""
    ragged, k = [], 0
    sizes = [2, 3, 17, 2, 40, 1, 1, 29, 64, 5]
    while sum(ragged) < T:
        ragged.append(min(sizes[k % len(sizes)], T - sum(ragged)))
        k += 1
    return {"whole": [T], "single": [1] * T, "ragged": ragged}


@pytest.mark.parametrize("kv_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,pool,bs", [(9, 4, 8), (16, 8, 8), (5, 8, 8), (44, 3, 8), (1, 1, 8), (33, 20, 8), (24, 16, 32)])
def test_block_means_are_the_means_of_the_cached_rows(kv_dtype, window, pool, bs):
    """Blocks that divide the page, straddle pages and exceed a page; closed inside a portion, by a portion's first token and by a
    single decoded token.  Every closed block's row is where the attention kernels look for it; no other row is touched."""
    g = torch.Generator().manual_seed(window + pool)
    T, H, G, D, P = 100, 2, 2, 12, 20
    q, k, v = _bf16_values(T, H, D, g=g), _bf16_values(T, G, D, g=g), _bf16_values(T, G, P, g=g)
    for name, portions in _cuts(T).items():
        _, pk, pv, pages = _attend(q, k, v, 0.3, window, pool, kv_dtype=kv_dtype, portions=portions, bs=bs)
        seen = torch.zeros(pk.shape[0], pk.shape[2], dtype=torch.bool)
        for b in range(T // pool):
            e = b * pool + pool - 1
            page, idx = pages[e // bs], (e % bs) // pool
            seen[page, idx] = True
            tol = 1e-6 if kv_dtype == torch.float32 else 5e-3
            _close(pk[page, :, idx], k[b * pool:(b + 1) * pool].double().mean(0), tol)
            _close(pv[page, :, idx], v[b * pool:(b + 1) * pool].double().mean(0), tol)
        assert (pk.float().cpu().permute(0, 2, 1, 3)[~seen] == 77.0).all(), name


@pytest.mark.parametrize("kv_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,pool", [(9, 4), (16, 8), (5, 8), (44, 3), (1, 1), (33, 20), (64, 32), (7, 0)])
def test_window_with_pooled_blocks_at_every_edge(kv_dtype, window, pool):
    """Loud keys (eight times the others) sit on both sides of the window's edge of late queries and fill whole blocks, so a
    window that is one position off, a block that is seen one position early or late, or a block that is lost moves the output
    by its whole size.  All positions are compared, whole, token by token and in ragged portions."""
    from oracle.gerupel_ref import window_pool_attention

    g = torch.Generator().manual_seed(window * 7 + pool)
    T, H, G, scale = 150, 4, 2, 0.4
    D, P = (20, 36) if kv_dtype == torch.float32 else (32, 48)
    q, k, v = _bf16_values(T, H, D, g=g), _bf16_values(T, G, D, g=g), _bf16_values(T, G, P, g=g)
    for j in (3, 31, 32, 64, 65, 100):                                        # single keys, also at page borders
        k[j] *= 4
    if pool:
        for b in {0, min(5, T // pool - 1), (T // pool) // 2}:                # whole blocks of one loud row: their mean is as loud
            k[b * pool:(b + 1) * pool] = k[b * pool] * 4
    k = k.to(torch.bfloat16).float()
    temp = torch.ones(H, dtype=torch.float64)
    pdt = None if kv_dtype == torch.float32 else kv_dtype                     # a bf16 cache holds bf16 block means
    want = window_pool_attention(q.double(), k.double(), v.double(), scale, temp, window, pool, pdt)
    off_by_one = window_pool_attention(q.double(), k.double(), v.double(), scale, temp, window + 1, pool, pdt)
    no_blocks = window_pool_attention(q.double(), k.double(), v.double(), scale, temp, window, 0)
    # edges and blocks matter for these inputs (blocks of one position bring every key back, wherever the window ends)
    assert (pool == 1 or _err(off_by_one, want) > 0.05) and (not pool or _err(no_blocks, want) > 0.05)
    for name, portions in _cuts(T).items():
        got, *_ = _attend(q, k, v, scale, window, pool, kv_dtype=kv_dtype, portions=portions)
        assert _err(got, want) < (2e-5 if kv_dtype == torch.float32 else 6e-3), (name, _err(got, want))


@pytest.mark.parametrize("kv_dtype", [torch.float32, torch.bfloat16])
def test_a_far_block_among_hundreds_the_first_tokens_and_the_sink(kv_dtype):
    """700 positions behind a window of 24 with blocks of 4: block 1 (positions 4 .. 7) is made to win for the late queries, so a
    kernel that loses the first page's blocks, or starts its walk late, shows.  Early queries, whose keys all score far below
    zero, are ruled by the 1 in the denominator: their outputs are nearly zero, not a mean of values."""
    from oracle.gerupel_ref import window_pool_attention

    g = torch.Generator().manual_seed(3)
    T, H, G, scale, window, pool = 700, 6, 3, 0.3, 24, 4
    D, P = (20, 36) if kv_dtype == torch.float32 else (48, 80)
    q, k, v = _bf16_values(T, H, D, g=g), _bf16_values(T, G, D, g=g), _bf16_values(T, G, P, g=g)
    k[4:8] = 0
    k[4:8, :, 0] = 8.0
    q[600:, :, 0] = 8.0
    q[:3] = 0
    q[:3, :, 1] = -8.0                                                        # queries 0 .. 2: every score is very negative
    k[:3, :, 1] = 8.0
    temp = torch.ones(H, dtype=torch.float64)
    want = window_pool_attention(q.double(), k.double(), v.double(), scale, temp, window, pool,
                                 None if kv_dtype == torch.float32 else kv_dtype)
    far = v[4:8, 0].double().mean(0)
    assert (want[650, 0] - far).abs().max() < 0.2 * far.abs().max()           # the far block carries the output
    assert want[:3].abs().max() < 1e-3                                        # the sink carries the denominator
    for name, portions in (("whole", [T]), ("prompt then single tokens", [640] + [1] * 60), ("ragged", [3, 2, 250, 1, 300, 144])):
        got, *_ = _attend(q, k, v, scale, window, pool, kv_dtype=kv_dtype, portions=portions)
        assert _err(got, want) < (2e-5 if kv_dtype == torch.float32 else 6e-3), (name, _err(got, want))
        assert got[:3].abs().max().item() < 1e-3


@pytest.mark.parametrize("kv_dtype", [torch.float32, torch.bfloat16])
def test_unequal_sequences_in_one_step_see_their_own_blocks(kv_dtype):
    """Three sequences in one ragged step (a long portion that continues, a short prompt, a single decoded token), each with its
    own block-table row; every output equals the sequence run alone."""
    from oracle.gerupel_ref import window_pool_attention

    ops = _ops()
    g = torch.Generator().manual_seed(8)
    H, G, D, P, scale, window, pool, bs = 4, 1, 32, 16, 0.35, 12, 4, 8
    lens, done = [90, 21, 57], [40, 0, 56]                                    # tokens in all, tokens cached by earlier steps
    seqs = [tuple(_bf16_values(n, h, d, g=g) for h, d in ((H, D), (G, D), (G, P))) for n in lens]
    nb = 40
    k_pool = torch.zeros(nb, G, bs, D, dtype=kv_dtype, device=DEV)
    v_pool = torch.zeros(nb, G, bs, P, dtype=kv_dtype, device=DEV)
    pk = torch.zeros(nb, G, bs // pool, D, dtype=kv_dtype, device=DEV)
    pv = torch.zeros(nb, G, bs // pool, P, dtype=kv_dtype, device=DEV)
    pages = {0: list(range(1, 13)), 1: list(range(39, 35, -1)), 2: list(range(20, 28))}
    table = torch.zeros(3, nb, dtype=torch.int32, device=DEV)
    for r, p in pages.items():
        table[r, :len(p)] = torch.tensor(p, dtype=torch.int32)
    zero = torch.zeros(H, device=DEV)

    def step(entries):
        rows = torch.cat([torch.cat([s[i][a:a + n].reshape(n, -1) for i in range(3)], dim=1) for r, a, n in entries for s in [seqs[r]]])
        meta = _meta(entries, pages, bs)
        qd = ops.qk_norm_rope_kv_write(rows.to(DEV), 0, H * D, (H + G) * D, H, k_pool, v_pool, meta)
        ops.kv_pool_mean(k_pool, v_pool, pk, pv, table, meta, pool)
        return ops.swa_sink_attn(qd, H, k_pool, v_pool, table, meta, zero, scale, window, split_p=True, pooled=(pk, pv, pool)).float()

    for r in (0, 2):
        step([(r, 0, done[r])])
    entries = [(r, done[r], lens[r] - done[r]) for r in range(3)]
    got = step(entries).view(-1, H, P)
    at = 0
    for r, a, n in entries:
        qq, kk, vv = seqs[r]
        want = window_pool_attention(qq.double(), kk.double(), vv.double(), scale, torch.ones(H, dtype=torch.float64), window, pool,
                                     None if kv_dtype == torch.float32 else kv_dtype)
        assert _err(got[at:at + n], want[a:a + n]) < (2e-5 if kv_dtype == torch.float32 else 6e-3), r
        at += n


# ------------------------------------------------------------------------------------------------ gated linear recurrence
@pytest.mark.parametrize("H,D,P,lead", [(2, 10, 7, 3), (3, 40, 72, 0), (1, 33, 20, 1), (2, 128, 32, 4), (1, 256, 16, 8), (4, 4, 5, 0), (1, 500, 3, 0)])
def test_gated_recurrence_over_portions_slots_and_reuse(H, D, P, lead):
    """Raw projections -> silu / bounded forget gate -> recurrence, for a sequence cut into portions beside another sequence in the
    same steps; then the first sequence's slot is taken over by a new one, which must not see the old state."""
    from oracle.gerupel_ref import gated_recurrence

    ops = _ops()
    g = torch.Generator().manual_seed(H * D + P)
    n = H * D
    lens = {0: 75, 2: 40}
    lower, fb = 0.95 * torch.rand(n, generator=g), 0.5 * torch.randn(n, generator=g)
    state = torch.full((4, H, P, D), 55.0, device=DEV)                         # stale state is loud
    width = lead + 2 * n + H * P + (2 if lead % 4 else 0)                   # rows on the 16-byte grid (vector copies) and off it
    pages = {0: list(range(1, 12)), 2: list(range(12, 20))}

    def want(raw):
        r = raw.double()
        q = torch.nn.functional.silu(r[:, lead:lead + n]).view(-1, H, D)
        f = (lower.double() + (1 - lower.double()) * torch.sigmoid(r[:, lead + n:lead + 2 * n] + fb.double())).view(-1, H, D)
        return gated_recurrence(q, f, r[:, lead + 2 * n:lead + 2 * n + H * P].view(-1, H, P)).reshape(-1, H * P)

    raws = {s: torch.randn(L, width, generator=g) * 1.5 for s, L in lens.items()}
    steps = [{0: 2, 2: 1}, {0: 33, 2: 1}, {0: 1}, {0: 17, 2: 38}, {0: 22}]
    at, got = {s: 0 for s in lens}, {s: [] for s in lens}
    for st in steps:
        entries = [(s, at[s], c) for s, c in st.items()]
        rows = torch.cat([raws[s][at[s]:at[s] + c] for s, c in st.items()]).to(DEV)
        o = ops.gated_scan(rows, lead, lead + n, lead + 2 * n, fb.to(DEV), lower.to(DEV), state, _meta(entries, pages), H, D, P)
        k = 0
        for s, c in st.items():
            got[s].append(o[k:k + c])
            at[s] += c
            k += c
    for s in lens:
        assert at[s] == lens[s]
        _close(torch.cat(got[s]), want(raws[s]), 2e-5)
    assert (state[1] == 55.0).all() and (state[3] == 55.0).all()               # other slots are not touched
    fresh = torch.randn(9, width, generator=g)
    o = ops.gated_scan(fresh.to(DEV), lead, lead + n, lead + 2 * n, fb.to(DEV), lower.to(DEV), state, _meta([(0, 0, 9)], pages), H, D, P)
    _close(o, want(fresh), 2e-5)


@pytest.mark.parametrize("H,D,P,lead", [(2, 10, 7, 3), (2, 64, 48, 0), (1, 200, 20, 4)])
def test_gated_recurrence_with_long_portions_cut_into_parallel_segments(H, D, P, lead):
    """Portions of 256 tokens and more run as segments of 128 that are chained afterwards: a long portion from position 0, one
    that continues a sequence (its first segment starts from the slot's state), a length that is no multiple of the segment, and
    short portions of other sequences in the same step."""
    from oracle.gerupel_ref import gated_recurrence

    ops = _ops()
    g = torch.Generator().manual_seed(D + P)
    n = H * D
    lens = {0: 1000, 1: 40, 3: 300}
    lower, fb = 0.97 * torch.rand(n, generator=g), 0.5 * torch.randn(n, generator=g)
    state = torch.full((5, H, P, D), 55.0, device=DEV)
    width = lead + 2 * n + H * P + (2 if lead % 4 else 0)
    pages = {0: list(range(1, 130)), 1: list(range(130, 140)), 3: list(range(140, 180))}
    raws = {s: torch.randn(L, width, generator=g) * 1.5 for s, L in lens.items()}
    steps = [{0: 333, 1: 2}, {0: 1, 1: 1, 3: 300}, {0: 410, 1: 37}, {0: 256}]
    at, got = {s: 0 for s in lens}, {s: [] for s in lens}
    for st in steps:
        entries = [(s, at[s], c) for s, c in st.items()]
        meta = _meta(entries, pages)
        assert (meta.num_segs > 0) == (max(st.values()) >= 256)
        rows = torch.cat([raws[s][at[s]:at[s] + c] for s, c in st.items()]).to(DEV)
        o = ops.gated_scan(rows, lead, lead + n, lead + 2 * n, fb.to(DEV), lower.to(DEV), state, meta, H, D, P)
        k = 0
        for s, c in st.items():
            got[s].append(o[k:k + c])
            at[s] += c
            k += c
    for s, raw in raws.items():
        r = raw.double()
        q = torch.nn.functional.silu(r[:, lead:lead + n]).view(-1, H, D)
        f = (lower.double() + (1 - lower.double()) * torch.sigmoid(r[:, lead + n:lead + 2 * n] + fb.double())).view(-1, H, D)
        want = gated_recurrence(q, f, r[:, lead + 2 * n:lead + 2 * n + H * P].view(-1, H, P)).reshape(-1, H * P)
        _close(torch.cat(got[s]), want, 2e-5)
    assert (state[2] == 55.0).all() and (state[4] == 55.0).all()


def test_gated_recurrence_keeps_a_long_memory():
    """Forget gates close to 1 (lower bound 0.999) over 1500 tokens in single-token steps after a prompt: what the first token wrote
    is still most of the state at the end, and 1 - f, tiny, is what every later token writes."""
    from oracle.gerupel_ref import gated_recurrence

    ops = _ops()
    g = torch.Generator().manual_seed(1)
    H, D, P, T = 2, 16, 8, 1500
    n = H * D
    lower, fb = torch.full((n,), 0.999), torch.zeros(n)
    raw = torch.randn(T, 2 * n + H * P, generator=g)
    raw[0, 2 * n:] *= 30
    r = raw.double()
    f = (lower.double() + (1 - lower.double()) * torch.sigmoid(r[:, n:2 * n])).view(T, H, D)
    want = gated_recurrence(torch.nn.functional.silu(r[:, :n]).view(T, H, D), f, r[:, 2 * n:].view(T, H, P)).reshape(T, -1)
    state = torch.zeros(2, H, P, D, device=DEV)
    outs, at = [], 0
    for c in [700] + [1] * 100 + [700]:
        outs.append(ops.gated_scan(raw[at:at + c].to(DEV), 0, n, 2 * n, fb.to(DEV), lower.to(DEV), state, _meta([(1, at, c)], {1: list(range(1, 200))}), H, D, P))
        at += c
    _close(torch.cat(outs), want, 2e-5)


# ------------------------------------------------------------------------------------------------ router
@pytest.mark.parametrize("E,top", [(12, 3), (5, 1), (3, 3), (1, 1), (64, 8)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_renormalised_softmax_router_and_experts(E, top, dtype):
    """Scores over all experts, the largest kept and divided by their sum; the experts' outputs weighed in the residual step."""
    from oracle.gerupel_ref import expert_mixture

    ops = _ops()
    g = torch.Generator().manual_seed(E + top)
    T, W, ff, scale = 40, 64, 32, 1.7
    h = _bf16_values(T, W, g=g)
    Wt = {"router": _bf16_values(E, W, g=g, scale=0.6)}
    for e in range(E):
        Wt.update({f"e{e}.gate": _bf16_values(ff, W, g=g, scale=W ** -0.5), f"e{e}.up": _bf16_values(ff, W, g=g, scale=W ** -0.5),
                   f"e{e}.down": _bf16_values(W, ff, g=g, scale=ff ** -0.5)})
    want = expert_mixture(h.double(), {k: v.double() for k, v in Wt.items()}, "",
                          {"router": {"experts": E, "top": top, "scale": scale}})
    logits = (h.double() @ Wt["router"].double().T).float().to(DEV)
    idx, wt = ops.moe_topk(logits, top, mode=ops.ROUTE_SOFTMAX_RENORM)
    s = torch.softmax(logits.double().cpu(), -1)
    val, ref_idx = torch.topk(s, top, dim=-1)
    assert (idx.cpu().long().sort(-1).values == ref_idx.sort(-1).values).all()
    _close(wt.sum(-1), torch.ones(T), 1e-6)
    w_gu = torch.stack([torch.cat([Wt[f"e{e}.gate"], Wt[f"e{e}.up"]]) for e in range(E)]).to(DEV, dtype)
    w_down = torch.stack([Wt[f"e{e}.down"] for e in range(E)]).to(DEV, dtype)
    hd = h.to(DEV, dtype)
    pairs = ops.moe_experts(hd, wt, ops.moe_align(idx, E), w_gu, w_down, top, act=ops.ACT_SILU, scale_input=False)
    x = torch.zeros(T, W, device=DEV)
    ops.scaled_add_rmsnorm2(x, 1e-6, y3=pairs, nsum=top, y3_weight=wt, c3=scale)
    _close(x, want, 1e-5 if dtype == torch.float32 else 1.5e-2)
