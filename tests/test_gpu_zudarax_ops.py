"""GPU: every mechanism of the parallel-branch decoder (Zudarax) alone, against the plain restatement in
oracle/zudarax_ref.py (fp64).  Sizes are awkward on purpose (odd widths, head sizes that are no multiple of a warp, a vector
or a page; pages handed out in reverse), and where random numbers would hide a fault (a chunk's edge, a far key, a weight
that is not normalised) the inputs are made so that it shows."""
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"
NO_WINDOW = 1 << 30


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


# ------------------------------------------------------------------------------------------------ norms and activation
@pytest.mark.parametrize("width,groups", [(60, 1), (60, 3), (264, 4), (7, 7), (2048, 8)])
def test_residual_step_with_grouped_rms_norm(width, groups):
    from oracle.zudarax_ref import group_rms_norm

    ops = _ops()
    g = torch.Generator().manual_seed(width + groups)
    T, eps = 9, 1e-5
    x = torch.randn(T, width, generator=g) * 3
    wide = torch.randn(T, 2 * width + 5, generator=g)            # the branches are column ranges of wider rows
    y1, y2 = wide[:, 3:3 + width], wide[:, width + 5:]
    w = 1 + 0.2 * torch.randn(width, generator=g)
    for branches in (0, 1, 2):
        xd, wd = x.to(DEV), wide.to(DEV)
        d1 = wd[:, 3:3 + width] if branches >= 1 else None
        d2 = wd[:, width + 5:] if branches == 2 else None
        want_x = x.double() + (y1.double() if branches >= 1 else 0) + (y2.double() if branches == 2 else 0)
        for dt, tol in ((torch.float32, 2e-6), (torch.bfloat16, 6e-3)):
            xi = xd.clone()
            h = ops.add_group_rmsnorm(xi, d1, d2, w.to(DEV), groups, eps, dt)
            _close(xi, want_x, 2e-7)
            _close(h, group_rms_norm(want_x, w.double(), groups, eps), tol)
    xi = x.to(DEV)
    assert ops.add_group_rmsnorm(xi, wide.to(DEV)[:, 3:3 + width], None, w.to(DEV), groups, eps, None) is None
    _close(xi, x.double() + y1.double(), 2e-7)


def test_grouped_norm_is_not_the_whole_row_norm():
    """Parts of very different size: one norm over the whole row would leave the small part near zero."""
    from oracle.zudarax_ref import group_rms_norm

    ops = _ops()
    x = torch.cat([torch.full((1, 16), 100.0), torch.full((1, 16), 0.01)], dim=1)
    h = ops.add_group_rmsnorm(x.to(DEV), None, None, torch.ones(32, device=DEV), 2, 1e-12, torch.float32)
    _close(h, group_rms_norm(x.double(), torch.ones(32).double(), 2, 1e-12), 1e-6)
    assert abs(h[0, 20].item() - 1.0) < 1e-4


@pytest.mark.parametrize("ff,col0,pad", [(24, 0, 3), (100, 7, 3), (1536, 64, 3),            # rows off the 16-byte grid: scalar kernel
                                         (24, 0, 4), (36, 120, 0), (1536, 64, 0), (4100, 4, 0),   # the row-in-registers kernel
                                         (20000, 0, 0)])                                          # too long for registers
def test_polynomial_unit_rms_activation(ff, col0, pad):
    from oracle.zudarax_ref import poly_norm

    ops = _ops()
    g = torch.Generator().manual_seed(ff)
    rows = torch.randn(6, col0 + ff + pad, generator=g) * 1.7
    coef = torch.tensor([0.7, -0.4, 0.25, 0.1])
    want = poly_norm(rows[:, col0:col0 + ff].double(), coef.double(), 1e-6)
    _close(ops.poly_norm(rows.to(DEV), col0, ff, coef.to(DEV), 1e-6, torch.float32), want, 3e-6)
    _close(ops.poly_norm(rows.to(DEV), col0, ff, coef.to(DEV), 1e-6, torch.bfloat16), want, 6e-3)
    # each power is normed on its own: with only the cube's coefficient set, the output has unit RMS whatever the input's size
    cube = ops.poly_norm((rows * 50).to(DEV), col0, ff, torch.tensor([0.0, 0.0, 1.0, 0.0], device=DEV), 1e-12, torch.float32)
    assert abs(cube.double().pow(2).mean(-1).sqrt().mean().item() - 1.0) < 1e-4


def test_differential_combine_norm_and_gate():
    from oracle.zudarax_ref import rms_unit

    ops = _ops()
    g = torch.Generator().manual_seed(5)
    T, H, rep, P, lam, diff, eps = 7, 6, 3, 20, 0.37, 0.45, 1e-5
    a = torch.randn(T, 2 * H, P, generator=g)
    rows = torch.randn(T, 11 + H, generator=g) * 2
    # per kv group: the first maps of its `rep` heads, then their second maps
    a1 = torch.stack([a[:, 2 * rep * (h // rep) + h % rep] for h in range(H)], dim=1).double()
    a2 = torch.stack([a[:, 2 * rep * (h // rep) + rep + h % rep] for h in range(H)], dim=1).double()
    want = rms_unit(a1 - lam * a2, eps) * (1 - diff) * torch.sigmoid(rows[:, 11:].double())[:, :, None]
    got = ops.diff_head_norm_gate(a.reshape(T, -1).to(DEV), lam, 1 - diff, rows.to(DEV), 11, eps, H, rep, torch.float32)
    _close(got, want.reshape(T, -1), 3e-6)
    plain = ops.diff_head_norm_gate(a.reshape(T, -1).to(DEV), lam, 1 - diff, None, 0, eps, H, rep, torch.bfloat16)
    _close(plain, (rms_unit(a1 - lam * a2, eps) * (1 - diff)).reshape(T, -1), 6e-3)


# ------------------------------------------------------------------------------------------------ short convolution
@pytest.mark.parametrize("taps", [1, 2, 4])
def test_short_convolution_with_projection_bias_state_and_slot_reuse(taps):
    """No activation; the projection's bias is part of what is convolved (also of the values the state keeps), zeros stand
    before a sequence's start whatever the slot held, and portions of one or two tokens continue from the state."""
    from oracle.zudarax_ref import short_conv

    ops = _ops()
    g = torch.Generator().manual_seed(taps)
    C, col0 = 37, 5
    w = torch.randn(C, taps, generator=g)
    bias = torch.randn(C, generator=g)
    state = torch.full((3, max(taps - 1, 1), C), 7.0, device=DEV)            # stale values in every slot
    seqs = {"a": torch.randn(19, col0 + C + 2, generator=g), "b": torch.randn(6, col0 + C + 2, generator=g),
            "c": torch.randn(9, col0 + C + 2, generator=g)}
    want = {k: short_conv(u[:, col0:col0 + C].double() + bias.double(), w.double()) for k, u in seqs.items()}
    slot = {"a": 2, "b": 0, "c": 0}                                           # c takes over b's slot
    at = {k: 0 for k in seqs}
    for step in ([("a", 1), ("b", 2)], [("a", 2), ("b", 4)], [("a", 1)], [("c", 5), ("a", 13)], [("a", 2), ("c", 1)], [("c", 3)]):
        entries = [(slot[k], at[k], n) for k, n in step]
        rows = torch.cat([seqs[k][at[k]:at[k] + n] for k, n in step])
        meta = _meta(entries, {2: [1, 2, 3], 0: [4, 5]})
        out = ops.causal_conv_silu(rows.to(DEV), col0, C, w.to(DEV), None, state, meta, torch.float32, in_bias=bias.to(DEV),
                                   silu=False)
        _close(out, torch.cat([want[k][at[k]:at[k] + n] for k, n in step]), 3e-6)
        for k, n in step:
            at[k] += n


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps", [2, 3, 4])
def test_short_convolution_over_long_ragged_steps(taps, out_dtype):
    """Channel counts and offsets in multiples of four take the kernel that carries the window in registers along a run of
    tokens: sequences that start in the middle of a run, a one-token sequence between two long ones, and a second step that
    continues all of them from the state."""
    from oracle.zudarax_ref import short_conv

    ops = _ops()
    g = torch.Generator().manual_seed(10 + taps)
    C, col0 = 72, 8
    w = torch.randn(C, taps, generator=g)
    bias = torch.randn(C, generator=g)
    state = torch.full((3, taps - 1, C), -5.0, device=DEV)
    lens = {"a": 700, "b": 2, "c": 900}
    seqs = {k: torch.randn(n, col0 + C + 4, generator=g) for k, n in lens.items()}
    want = {k: short_conv(u[:, col0:col0 + C].double() + bias.double(), w.double()) for k, u in seqs.items()}
    slot = {"a": 1, "b": 0, "c": 2}
    at = {k: 0 for k in seqs}
    for step in ([("a", 301), ("b", 1), ("c", 498)], [("c", 402), ("b", 1), ("a", 399)]):
        entries = [(slot[k], at[k], n) for k, n in step]
        rows = torch.cat([seqs[k][at[k]:at[k] + n] for k, n in step])
        meta = _meta(entries, {0: list(range(1, 40)), 1: list(range(40, 140)), 2: list(range(140, 260))})
        out = ops.causal_conv_silu(rows.to(DEV), col0, C, w.to(DEV), None, state, meta, out_dtype, in_bias=bias.to(DEV), silu=False)
        assert out.dtype == out_dtype
        _close(out, torch.cat([want[k][at[k]:at[k] + n] for k, n in step]), 3e-6 if out_dtype == torch.float32 else 5e-3)
        for k, n in step:
            at[k] += n


# ------------------------------------------------------------------------------------------------ norm + rotation + cache write
@pytest.mark.parametrize("kv_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("half,normed,scaling", [(True, True, None), (True, False, {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 1.0}),
                                                 (False, True, {"factor": 3.0, "original": 32, "fast": 8.0, "slow": 2.0})])
@pytest.mark.parametrize("lead", [3, 4])   # columns before q: 3 puts the rows off the 16-byte grid (scalar kernel), 4 on it
def test_whole_projection_norm_rotation_and_cache_write(kv_dtype, half, normed, scaling, lead):
    from oracle.zudarax_ref import rms_unit, rotate_half
    from vllm_neuron_b200.hybrid import RotSpec

    ops = _ops()
    g = torch.Generator().manual_seed(11)
    H, G, Gv, D, Dv, rot_n, bs, eps = 5, 2, 1, 24, 20, 16, 8, 1e-5
    pos0, n = 37, 13                                                          # positions that cross page borders
    rows = torch.randn(n, lead + H * D + G * D + Gv * Dv, generator=g)
    qn, kn = 1 + 0.3 * torch.randn(H * D, generator=g), 1 + 0.3 * torch.randn(G * D, generator=g)
    rot = {"dims": rot_n, "base": 300.0, "scaling": scaling}
    cos, sin = (t.to(DEV) for t in RotSpec(rot_n, 300.0, scaling).tables(64))
    pages = [6, 5, 4, 3, 2, 1, 7]                                              # not in order
    meta = _meta([(0, pos0, n)], {0: pages}, bs)
    k_pool = torch.zeros(8, G, bs, D, dtype=kv_dtype, device=DEV)
    v_pool = torch.zeros(8, Gv, bs, Dv, dtype=kv_dtype, device=DEV)
    q = ops.qk_norm_rope_kv_write(rows.to(DEV), lead, lead + H * D, lead + H * D + G * D, H, k_pool, v_pool, meta,
                                  q_norm=qn.to(DEV) if normed else None, k_norm=kn.to(DEV) if normed else None, eps=eps, rot_n=rot_n,
                                  rot_half=half, cos=cos, sin=sin)
    r = rows.double()
    rq, rk, rv = r[:, lead:lead + H * D], r[:, lead + H * D:lead + H * D + G * D], r[:, lead + H * D + G * D:]
    if normed:                                                                # over all heads' columns at once
        rq, rk = rms_unit(rq, eps) * qn.double(), rms_unit(rk, eps) * kn.double()

    def turn(u, heads):
        u = torch.cat([u.new_zeros(pos0, heads, D), u.view(n, heads, D)])     # the restatement counts positions from 0
        if half:
            return rotate_half(u, rot)[pos0:]
        # pairs (2i, 2i + 1): the same rotation on a re-ordered head
        perm = torch.cat([torch.arange(0, rot_n, 2), torch.arange(1, rot_n, 2), torch.arange(rot_n, D)])
        out = torch.empty_like(u)
        out[..., perm] = rotate_half(u[..., perm], rot)
        return out[pos0:]

    tol = 3e-6 if kv_dtype == torch.float32 else 5e-3
    _close(q, turn(rq, H).reshape(n, -1), 3e-6)
    wk, wv = turn(rk, G), rv.view(n, Gv, Dv)
    for i in range(n):
        p = pos0 + i
        _close(k_pool[pages[p // bs], :, p % bs], wk[i], tol)
        _close(v_pool[pages[p // bs], :, p % bs], wv[i], tol)


# ------------------------------------------------------------------------------------------------ attention variants over the pools
def _attend(q, k, v, scale, *, kv_dtype, portions, bs=8, **variant):
    """One sequence through the pools: q [T, H, D], k [T, G, D], v [T, Gv, P], cut into `portions`; pages in reverse order, in
    row 1 of the block table.  Each portion is cached and then attended, as a layer does it."""
    ops = _ops()
    T, H, D = q.shape
    G, Gv, P = k.shape[1], v.shape[1], v.shape[2]
    nb = -(-T // bs) + 1
    pages = list(range(nb - 1, 0, -1))
    k_pool = torch.zeros(nb, G, bs, D, dtype=kv_dtype, device=DEV)
    v_pool = torch.zeros(nb, Gv, bs, P, dtype=kv_dtype, device=DEV)
    table = torch.zeros(3, nb, dtype=torch.int32, device=DEV)
    table[1, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
    rows = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1).to(DEV)
    out, at = [], 0
    for n in portions:
        meta = _meta([(1, at, n)], {1: pages}, bs)
        qd = ops.qk_norm_rope_kv_write(rows[at:at + n], 0, H * D, (H + G) * D, H, k_pool, v_pool, meta)
        out.append(ops.swa_sink_attn(qd, H, k_pool, v_pool, table, meta, None, scale, NO_WINDOW, **variant).float().view(n, H, P))
        at += n
    assert at == T
    return torch.cat(out)


def _cuts(T):
    """Whole (the tensor-core kernel in bf16), token by token (the warp kernel), and ragged portions down to two tokens."""
    ragged, k = [], 0
    sizes = [2, 3, 17, 2, 40, 1, 1, 29, 64, 5]
    while sum(ragged) < T:
        ragged.append(min(sizes[k % len(sizes)], T - sum(ragged)))
        k += 1
    return {"whole": [T], "single": [1] * T, "ragged": ragged}


@pytest.mark.parametrize("kv_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("chunk", [1, 7, 24, 64])
def test_chunked_soft_capped_attention_at_the_chunk_edges(kv_dtype, chunk):
    """The keys on both sides of every chunk border are made loud (eight times the others): a mask that is one position off
    lets one in, or leaves one out, and moves the output by its whole size.  The soft cap bites: raw scores reach several
    times the cap."""
    from oracle.zudarax_ref import softmax_attention, visible

    g = torch.Generator().manual_seed(chunk)
    T, H, G, D, P, scale, cap = 150, 4, 2, 32, 48, 0.4, 3.0
    q, k, v = _bf16_values(T, H, D, g=g), _bf16_values(T, G, D, g=g), _bf16_values(T, G, P, g=g)
    for j in range(T):
        if j % chunk in (0, chunk - 1):
            k[j] *= 8
    k = k.to(torch.bfloat16).float()
    want = softmax_attention(q.double(), k.double(), v.double(), scale, visible(T, chunk), cap)
    causal = softmax_attention(q.double(), k.double(), v.double(), scale, visible(T), cap)
    if chunk < T:
        assert _err(causal, want) > 0.05                                      # the mask matters for these inputs
    for name, portions in _cuts(T).items():
        got = _attend(q, k, v, scale, kv_dtype=kv_dtype, portions=portions, chunk=chunk, softcap=cap, split_p=True)
        assert _err(got, want) < (2e-5 if kv_dtype == torch.float32 else 6e-3), (name, _err(got, want))


@pytest.mark.parametrize("kv_dtype", [torch.float32, torch.bfloat16])
def test_a_far_key_among_hundreds_and_the_first_tokens(kv_dtype):
    """Causal softmax over 700 keys; key 2 is made to win for the late queries, so a kernel that loses the first page, or
    starts its walk late, shows.  Odd head sizes in fp32 (no vector loads); 16-multiples in bf16 (tensor cores)."""
    from oracle.zudarax_ref import softmax_attention, visible

    g = torch.Generator().manual_seed(3)
    T, H, G, scale = 700, 6, 3, 0.3
    D, P = (20, 36) if kv_dtype == torch.float32 else (48, 80)
    q, k, v = _bf16_values(T, H, D, g=g), _bf16_values(T, G, D, g=g), _bf16_values(T, G, P, g=g)
    k[2] = 0
    k[2, :, 0] = 8.0
    q[600:, :, 0] = 8.0
    want = softmax_attention(q.double(), k.double(), v.double(), scale, visible(T))
    assert (want[650, 0] - v[2, 0].double()).abs().max() < 0.2 * v[2, 0].abs().max()  # the far key carries the output
    for name, portions in (("whole", [T]), ("prompt then single tokens", [640] + [1] * 60), ("ragged", [3, 2, 250, 1, 300, 144])):
        got = _attend(q, k, v, scale, kv_dtype=kv_dtype, portions=portions, split_p=True)
        assert _err(got, want) < (2e-5 if kv_dtype == torch.float32 else 6e-3), (name, _err(got, want))


@pytest.mark.parametrize("kv_dtype", [torch.float32, torch.bfloat16])
def test_sigmoid_weights_are_not_normalised(kv_dtype):
    """Weights sigmoid(score + bias[head]): the output grows with the number of keys, heads differ by their bias only, and no
    softmax would reproduce either."""
    from oracle.zudarax_ref import sigmoid_attention, softmax_attention, visible

    g = torch.Generator().manual_seed(8)
    T, H, G, D, P, scale = 330, 6, 2, 16, 32, 0.25
    q, k, v = _bf16_values(T, H, D, g=g), _bf16_values(T, G, D, g=g), _bf16_values(T, G, P, g=g) + 0.5
    bias = torch.tensor([-3.0, -1.0, 0.0, 0.5, -6.0, 2.0])
    want = sigmoid_attention(q.double(), k.double(), v.double(), scale, visible(T), bias.double())
    assert want[-1].abs().mean() > 5 * want[3].abs().mean()
    assert _err(softmax_attention(q.double(), k.double(), v.double(), scale, visible(T)), want) > 0.5
    for name, portions in _cuts(T).items():
        got = _attend(q, k, v, scale, kv_dtype=kv_dtype, portions=portions, sigmoid_bias=bias.to(DEV), split_p=True)
        assert _err(got, want) < (2e-5 if kv_dtype == torch.float32 else 6e-3), (name, _err(got, want))


@pytest.mark.parametrize("kv_dtype", [torch.float32, torch.bfloat16])
def test_two_score_maps_over_shared_values_in_fp32(kv_dtype):
    """Twice as many key heads as value heads (key heads 2g and 2g + 1 read value head g), fp32 output rows, and weights that
    go through the tensor cores as two bf16 terms: the bf16 pools give the fp32 result to 1e-4."""
    from oracle.zudarax_ref import softmax_attention, visible

    g = torch.Generator().manual_seed(13)
    T, H, G, Gv, D, P, scale = 200, 12, 4, 2, 16, 32, 0.35
    q, k, v = _bf16_values(T, H, D, g=g), _bf16_values(T, G, D, g=g), _bf16_values(T, Gv, P, g=g)
    want = softmax_attention(q.double(), k.double(), v.double(), scale, visible(T))
    for name, portions in _cuts(T).items():
        got = _attend(q, k, v, scale, kv_dtype=kv_dtype, portions=portions, out_f32=True, split_p=True)
        assert got.dtype == torch.float32 and _err(got, want) < (2e-5 if kv_dtype == torch.float32 else 1e-4), (name, _err(got, want))
    if kv_dtype == torch.bfloat16:                                            # one bf16 term alone is visibly coarser
        coarse = _attend(q, k, v, scale, kv_dtype=kv_dtype, portions=[T], out_f32=True, split_p=False)
        assert 1e-4 < _err(coarse, want) < 6e-3


# ------------------------------------------------------------------------------------------------ long prompt portions (tcgen05 kernel)
def _attend_steps(seqs, steps, scale, *, bs=32, **variant):
    """Several sequences through bf16 pools of 32-token pages.  seqs: name -> (q [T, H, D], k [T, G, D], v [T, Gv, P]); steps:
    lists of (name, n), all entries of a step in one launch.  Pages are dealt out in an interleaved, descending order.
    -> name -> [T, H, P], and the names of the kernels that ran."""
    ops = _ops()
    names = list(seqs)
    q0, k0, v0 = seqs[names[0]]
    H, D, G, Gv, P = q0.shape[1], q0.shape[2], k0.shape[1], v0.shape[1], v0.shape[2]
    need = {s: -(-seqs[s][0].shape[0] // bs) for s in names}
    nb = sum(need.values()) + 1
    free = list(range(nb - 1, 0, -1))
    pages = {i + 1: [] for i in range(len(names))}
    for r in range(max(need.values())):
        for i, s in enumerate(names):
            if r < need[s]:
                pages[i + 1].append(free.pop(0))
    k_pool = torch.zeros(nb, G, bs, D, dtype=torch.bfloat16, device=DEV)
    v_pool = torch.zeros(nb, Gv, bs, P, dtype=torch.bfloat16, device=DEV)
    table = torch.zeros(len(names) + 1, max(need.values()) + 1, dtype=torch.int32, device=DEV)
    for r, pg in pages.items():
        table[r, :len(pg)] = torch.tensor(pg, dtype=torch.int32)
    at = {s: 0 for s in names}
    out = {s: [] for s in names}
    with ops.kernel_timer() as timer:
        for step in steps:
            entries = [(names.index(s) + 1, at[s], n) for s, n in step]
            meta = _meta(entries, pages, bs)
            rows = torch.cat([torch.cat([t[at[s]:at[s] + n].reshape(n, -1) for t in seqs[s]], dim=1) for s, n in step]).to(DEV)
            qd = ops.qk_norm_rope_kv_write(rows, 0, H * D, (H + G) * D, H, k_pool, v_pool, meta)
            a = ops.swa_sink_attn(qd, H, k_pool, v_pool, table, meta, None, scale, NO_WINDOW, **variant).float()
            o = 0
            for s, n in step:
                out[s].append(a[o:o + n].view(n, H, P))
                o, at[s] = o + n, at[s] + n
    assert all(at[s] == seqs[s][0].shape[0] for s in names)
    return {s: torch.cat(v) for s, v in out.items()}, set(timer.summary())


TC_CASES = {
    # name: (H, G, Gv, D, P, variant)
    "softmax 128": (4, 2, 2, 128, 128, {}),
    "softmax 64, odd group": (3, 1, 1, 64, 64, {}),
    "capped chunks of 200": (4, 2, 2, 128, 128, {"chunk": 200, "softcap": 3.0}),
    "capped chunks of 128": (2, 2, 2, 64, 64, {"chunk": 128, "softcap": 5.0}),
    "chunks of 48": (4, 1, 1, 64, 64, {"chunk": 48}),
    "sigmoid 128": (4, 2, 2, 128, 128, {"sigmoid": True}),
    "sigmoid 64": (2, 1, 1, 64, 64, {"sigmoid": True}),
    "two maps, values of 128": (8, 4, 2, 64, 128, {"out_f32": True}),
    "two maps, values of 64": (12, 4, 2, 64, 64, {"out_f32": True}),
    "two maps of 32, values of 64": (8, 4, 2, 32, 64, {"out_f32": True}),
    "two maps of 32, values of 128, one kv group": (6, 2, 1, 32, 128, {"out_f32": True}),
}


@pytest.mark.parametrize("case", list(TC_CASES))
def test_long_prompt_portions_on_the_tcgen05_kernel(case):
    """Portions of 128 tokens and more take the tcgen05 kernel.  Three sequences of unequal length in ragged steps (a long
    portion beside single tokens and short portions, cuts inside pages, key steps and chunks), keys made loud on both sides of
    every chunk border and one far key that wins late, against the restatement; the kernel must really have run."""
    from oracle.zudarax_ref import sigmoid_attention, softmax_attention, visible

    H, G, Gv, D, P, variant = TC_CASES[case]
    variant = dict(variant)
    g = torch.Generator().manual_seed(len(case))
    scale, chunk, cap = 0.5 * D ** -0.5, variant.get("chunk", 0), variant.get("softcap", 0.0)
    lens = {"a": 700, "b": 130, "c": 391}
    seqs, want = {}, {}
    bias = torch.linspace(-3.0, 1.0, H)
    for s, T in lens.items():
        q, k, v = _bf16_values(T, H, D, g=g), _bf16_values(T, G, D, g=g), _bf16_values(T, Gv, P, g=g)
        if chunk:
            for j in range(T):
                if j % chunk in (0, chunk - 1):
                    k[j] *= 4
        k[2] = 0
        k[2, :, 0] = 16.0
        q[T - 60:, :, 0] = 16.0                                              # key 2 wins for the last queries (where it is visible)
        k = k.to(torch.bfloat16).float()
        seqs[s] = (q, k, v)
        if variant.get("sigmoid"):
            want[s] = sigmoid_attention(q.double(), k.double(), v.double(), scale, visible(T), bias.double())
        else:
            want[s] = softmax_attention(q.double(), k.double(), v.double(), scale, visible(T, chunk) if chunk else visible(T), cap or None)
    if variant.pop("sigmoid", False):
        variant["sigmoid_bias"] = bias.to(DEV)
    steps = [[("a", 300), ("b", 1), ("c", 2)], [("a", 129), ("b", 129)], [("c", 260), ("a", 1)], [("a", 270), ("c", 128)], [("c", 1)]]
    got, ran = _attend_steps(seqs, steps, scale, split_p=True, **variant)
    assert any(n.startswith("swa_sink_attn_prefill_tc") for n in ran), ran
    tol = 2e-4 if variant.get("out_f32") else 6e-3
    for s in lens:
        assert _err(got[s], want[s]) < tol, (s, _err(got[s], want[s]))
    whole, _ = _attend_steps({"a": seqs["a"]}, [[("a", 700)]], scale, split_p=True, **variant)
    assert _err(whole["a"], want["a"]) < tol
