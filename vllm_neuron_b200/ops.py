"""Tensor-level wrappers over the C ABI: validate, take raw pointers and the current CUDA stream, call.

Torch is plumbing here (device memory + streams); every op below runs one of the hand-written
sm_100a kernels in libb200_paged.so.  Nothing in this file computes on the host.
"""
from __future__ import annotations

import os

import torch

from . import _cabi
from ._cabi import ACT_GELU_TANH, ACT_SILU, ACT_SWISH_CLAMPED, BF16, F32, FP8_E4M3, INT8, ROUTE_SIGMOID, ROUTE_SOFTMAX_RENORM, ROUTE_SOFTMAX_TOP, check

_QDT = {None: BF16, "bf16": BF16, "fp8": FP8_E4M3, "int8": INT8}
_TORCH_Q = {FP8_E4M3: torch.float8_e4m3fn, INT8: torch.int8}
INT8_WO = 4  # GEMM ab_dtype only: bf16 activations x int8 weights
_DTN = {BF16: "bf16", FP8_E4M3: "fp8", INT8: "int8", INT8_WO: "int8wo"}


def _stream():
    return torch.cuda.current_stream().cuda_stream


# ------------------------------------------------------------------ per-launch device timing (bench.py roofline leg)
_PROF: list | None = None


class kernel_timer:
    """with ops.kernel_timer() as t: ...eager calls...; t.summary() -> {name: (count, mean_ms)}.
    CUDA events are recorded on the launching stream right around each C-ABI call (not usable under graph capture)."""

    def __enter__(self):
        global _PROF
        self.records = _PROF = []
        return self

    def __exit__(self, *exc):
        global _PROF
        _PROF = None
        return False

    def summary(self):
        torch.cuda.synchronize()
        acc: dict[str, list] = {}
        for name, e0, e1 in self.records:
            acc.setdefault(name, []).append(e0.elapsed_time(e1))
        return {k: (len(v), sum(v) / len(v)) for k, v in acc.items()}


class _k:
    __slots__ = ("name", "e0")

    def __init__(self, name):
        self.name = name

    def __enter__(self):
        if _PROF is not None:
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e0.record()
        return self

    def __exit__(self, *exc):
        if _PROF is not None:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record()
            _PROF.append((self.name, self.e0, e1))
        return False


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def _cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise _cabi.B200Error("b200 ops need CUDA tensors (no CPU fallback)")


def device_check(device: int = 0):
    check(_cabi.load().b200_device_check(device), "b200_device_check")


def set_pdl(enabled: bool) -> bool:
    """Programmatic dependent launch on/off for every kernel of the library; returns the previous setting."""
    return bool(_cabi.load().b200_set_pdl(1 if enabled else 0))


def launch_count() -> int:
    """Kernel launches issued through libb200_paged.so by this process so far."""
    return int(_cabi.load().b200_launch_count())


# ------------------------------------------------------------------ index construction
def build_decode_meta(block_table, row_ids, num_tokens, slot_mapping, positions, ctx_lens, block_size: int):
    """block_table int32 [rows, max_blocks]; row_ids int32 [B] or None; num_tokens int32 [rows];
    outputs: slot_mapping int64 [B] (or [B, k]: k consecutive slots per row for speculation, RUNNER:825-830),
    positions int64 [B], ctx_lens int32 [B]."""
    _cuda(block_table, num_tokens, slot_mapping)
    assert block_table.dtype == torch.int32 and num_tokens.dtype == torch.int32
    assert slot_mapping.dtype == torch.int64 and positions.dtype == torch.int64 and ctx_lens.dtype == torch.int32
    b = positions.numel()
    num_spec = 1 if slot_mapping.dim() == 1 else slot_mapping.shape[1]
    assert slot_mapping.is_contiguous() and slot_mapping.numel() == b * num_spec
    with _k("build_decode_meta"):
        check(
            _cabi.load().b200_build_decode_meta(
                _ptr(block_table), block_table.stride(0), _ptr(row_ids), _ptr(num_tokens), _ptr(slot_mapping),
                _ptr(positions), _ptr(ctx_lens), b, block_table.shape[1], block_size, num_spec, _stream(),
            ),
            "b200_build_decode_meta",
        )


def build_prefill_meta(block_table_row, prompt_len: int, num_computed: int, slot_mapping, positions, block_size: int):
    _cuda(block_table_row, slot_mapping, positions)
    assert block_table_row.dtype == torch.int32 and slot_mapping.dtype == torch.int64 and positions.dtype == torch.int64
    check(
        _cabi.load().b200_build_prefill_meta(
            _ptr(block_table_row), prompt_len, num_computed, _ptr(slot_mapping), _ptr(positions),
            slot_mapping.numel(), block_size, _stream(),
        ),
        "b200_build_prefill_meta",
    )


def remask_spec_output(accepted, next_pos, positions):
    """LOADER:308-334: accepted int64 [B, T] 0-padded -> -1 past clamp(next_pos - positions, 0, T) tokens per row."""
    _cuda(accepted, next_pos, positions)
    b, t = accepted.shape
    assert accepted.dtype == next_pos.dtype == positions.dtype == torch.int64 and accepted.is_contiguous()
    out = torch.empty_like(accepted)
    check(_cabi.load().b200_remask_spec_output(_ptr(accepted), _ptr(next_pos), _ptr(positions), _ptr(out), b, t, _stream()),
          "b200_remask_spec_output")
    return out


def block_table_scatter(block_table, updates):
    """updates int32 [n, 3] = (row, col, block_id) on the device."""
    _cuda(block_table, updates)
    assert block_table.dtype == torch.int32 and updates.dtype == torch.int32 and updates.is_contiguous()
    n = updates.shape[0]
    check(
        _cabi.load().b200_block_table_scatter(
            _ptr(block_table), block_table.stride(0), _ptr(updates), n, block_table.shape[0], block_table.shape[1], _stream()
        ),
        "b200_block_table_scatter",
    )


def advance_decode(sampled, tokens_io, num_tokens, row_ids):
    _cuda(sampled, tokens_io, num_tokens)
    check(
        _cabi.load().b200_advance_decode(
            _ptr(sampled), _ptr(tokens_io), _ptr(num_tokens), _ptr(row_ids), sampled.numel(), _stream()
        ),
        "b200_advance_decode",
    )


# ------------------------------------------------------------------ KV cache
def kv_write(k, v, k_pool, v_pool, slot_mapping):
    """k, v [T, Hkv, D] bf16 (last two dims contiguous); pools [num_blocks, Hkv, bs, D]."""
    _cuda(k, v, k_pool, v_pool, slot_mapping)
    t, hkv, d = k.shape
    nb, hkv2, bs, d2 = k_pool.shape
    assert (hkv, d) == (hkv2, d2) and k.stride(2) == 1 and k.stride(1) == d and v.stride(1) == d
    assert k_pool.is_contiguous() and v_pool.is_contiguous() and slot_mapping.dtype == torch.int64
    check(
        _cabi.load().b200_kv_write(
            _ptr(k), _ptr(v), k.stride(0), v.stride(0), _ptr(k_pool), _ptr(v_pool), _ptr(slot_mapping),
            t, hkv, d, bs, nb, _stream(),
        ),
        "b200_kv_write",
    )


def rope_kv_write(qkv, positions, cos, sin, k_pool, v_pool, slot_mapping, num_q_heads: int):
    """qkv [T, (Hq+2Hkv)*D] bf16 contiguous; q is rotated in place, roped k and v go to the pools."""
    _cuda(qkv, positions, cos, sin, k_pool, v_pool, slot_mapping)
    nb, hkv, bs, d = k_pool.shape
    t = qkv.shape[0]
    assert qkv.is_contiguous() and qkv.shape[1] == (num_q_heads + 2 * hkv) * d and qkv.dtype == torch.bfloat16
    assert cos.dtype == torch.float32 and cos.shape[1] == d // 2 and cos.is_contiguous() and sin.is_contiguous()
    assert positions.dtype == torch.int64 and slot_mapping.dtype == torch.int64
    with _k("rope_kv_write"):
        check(
            _cabi.load().b200_rope_kv_write(
                _ptr(qkv), _ptr(positions), _ptr(cos), _ptr(sin), cos.shape[0], _ptr(k_pool), _ptr(v_pool),
                _ptr(slot_mapping), t, num_q_heads, hkv, d, bs, nb, _stream(),
            ),
            "b200_rope_kv_write",
        )


# ------------------------------------------------------------------ paged attention
def paged_attn_decode_workspace_bytes(b, hq, hkv, d, max_blocks, min_quota=0) -> int:
    return int(_cabi.load().b200_paged_attn_decode_workspace_bytes(b, hq, hkv, d, max_blocks, min_quota))


def paged_attn_decode(q, k_pool, v_pool, block_table, ctx_lens, scale, out=None, workspace=None, row_ids=None,
                      max_blocks=None, min_quota=0, quant=None):
    """q [B, Hq, D] bf16 (token stride arbitrary); block_table int32 [rows, max_blocks]; ctx_lens int32 [B].
    quant None -> bf16 out [B, Hq, D]; "fp8"/"int8" -> (q [B, Hq*D], scale [B]) quantised per token in the merge kernel."""
    _cuda(q, k_pool, v_pool, block_table, ctx_lens)
    b, hq, d = q.shape
    nb, hkv, bs, d2 = k_pool.shape
    assert d == d2 and q.stride(2) == 1 and q.stride(1) == d and q.dtype == torch.bfloat16
    assert block_table.dtype == torch.int32 and ctx_lens.dtype == torch.int32
    mb = block_table.shape[1] if max_blocks is None else min(max_blocks, block_table.shape[1])
    qd = _QDT[quant]
    oq = osc = None
    if qd == BF16:
        if out is None:
            out = torch.empty((b, hq, d), dtype=q.dtype, device=q.device)
        assert out.is_contiguous()
    else:
        oq = torch.empty((b, hq * d), dtype=_TORCH_Q[qd], device=q.device)
        osc = torch.empty((b,), dtype=torch.float32, device=q.device)
    if workspace is None:
        workspace = torch.empty(paged_attn_decode_workspace_bytes(b, hq, hkv, d, mb, min_quota), dtype=torch.uint8, device=q.device)
    with _k("paged_attn_decode"):
        check(
            _cabi.load().b200_paged_attn_decode(
                _ptr(q), q.stride(0), _ptr(k_pool), _ptr(v_pool), nb, _ptr(block_table), block_table.stride(0),
                _ptr(row_ids), _ptr(ctx_lens), _ptr(out), _ptr(oq), _ptr(osc), qd, _ptr(workspace),
                workspace.numel() * workspace.element_size(), b, hq, hkv, d, bs, mb, min_quota, float(scale), _stream(),
            ),
            "b200_paged_attn_decode",
        )
    return out if qd == BF16 else (oq, osc)


def paged_attn_prefill(q, k_pool, v_pool, block_table_row, computed_len: int, scale, out=None):
    """q [S_new, Hq, D] bf16; one sequence; K/V of all computed_len + S_new tokens already in the pools."""
    _cuda(q, k_pool, v_pool, block_table_row)
    s_new, hq, d = q.shape
    nb, hkv, bs, _ = k_pool.shape
    assert q.stride(2) == 1 and q.stride(1) == d and block_table_row.dtype == torch.int32
    if out is None:
        out = torch.empty((s_new, hq, d), dtype=q.dtype, device=q.device)
    with _k("paged_attn_prefill"):
        check(
            _cabi.load().b200_paged_attn_prefill(
                _ptr(q), q.stride(0), _ptr(k_pool), _ptr(v_pool), nb, _ptr(block_table_row), _ptr(out), s_new,
                computed_len, hq, hkv, d, bs, float(scale), _stream(),
            ),
            "b200_paged_attn_prefill",
        )
    return out


# ------------------------------------------------------------------ GEMM
def _ab_dtype(t):
    if t.dtype == torch.bfloat16:
        return BF16
    if t.dtype == torch.float8_e4m3fn:
        return FP8_E4M3
    if t.dtype == torch.int8:
        return INT8
    raise _cabi.B200Error(f"unsupported GEMM operand dtype {t.dtype}")


def _gemm_dtype(a, w):
    """ab_dtype code of a GEMM: both operands alike, or bf16 activations x int8 weights (weight-only)."""
    if a.dtype == torch.bfloat16 and w.dtype == torch.int8:
        return INT8_WO
    if a.dtype != w.dtype:
        raise _cabi.B200Error(f"GEMM operand dtypes {a.dtype} x {w.dtype} not supported")
    return _ab_dtype(a)


def gemm_decode_plan(m, n, k, ab_dtype, split_k=0, silu_mul=False, has_residual=False) -> dict:
    """The decode schedule the library picks for this shape on the current device (for benches / DESIGN notes)."""
    import ctypes

    out = (ctypes.c_int * 6)()
    check(_cabi.load().b200_gemm_decode_plan(m, n, k, ab_dtype, split_k, int(silu_mul), int(has_residual), out),
          "b200_gemm_decode_plan")
    return dict(zip(("split", "ctas_per_sm", "w_stages", "a_stages", "cap_ctas", "smem"), list(out)))


def gemm_workspace_bytes(m, n, k, ab_dtype, split_k=0) -> int:
    return int(_cabi.load().b200_gemm_workspace_bytes(m, n, k, ab_dtype, split_k))


def gemm_workspace(m, n, k, ab_dtype, device, split_k=0):
    """Zero-filled workspace (stream-K fix-up counters at its head must start at zero; every call leaves them zeroed).
    The decode schedule (M <= 128) needs none: returns None."""
    nbytes = gemm_workspace_bytes(m, n, k, ab_dtype, split_k)
    return torch.zeros(nbytes, dtype=torch.uint8, device=device) if nbytes else None


def gemm(a, w, a_scale=None, w_scale=None, bias=None, residual=None, out=None, out_dtype=torch.bfloat16, split_k=0,
         workspace=None):
    """out[M,N] = (a[M,K] @ w[N,K]^T) * a_scale[m] * w_scale[n] + bias[n] + residual[m,n]."""
    _cuda(a, w, a_scale, w_scale, bias, residual)
    m, k = a.shape
    n, k2 = w.shape
    assert k == k2 and a.is_contiguous() and w.is_contiguous()
    dt = _gemm_dtype(a, w)
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    assert out.is_contiguous() and out.shape == (m, n)
    odt = F32 if out.dtype == torch.float32 else BF16
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.is_contiguous() and residual.shape == (m, n)
    if workspace is None:
        workspace = gemm_workspace(m, n, k, dt, a.device, split_k)
    with _k(f"gemm_{_DTN[dt]}[{m}x{n}x{k}]"):
        check(
            _cabi.load().b200_gemm(
                _ptr(a), _ptr(w), _ptr(out), _ptr(a_scale), _ptr(w_scale), _ptr(bias), _ptr(residual), m, n, k, dt, odt,
                split_k, _ptr(workspace), 0 if workspace is None else workspace.numel() * workspace.element_size(), _stream(),
            ),
            "b200_gemm",
        )
    return out


def gemm_rope_kv_write(a, w, positions, cos, sin, k_pool, v_pool, slot_mapping, num_q_heads: int, a_scale=None,
                       w_scale=None, bias=None, split_k=0, workspace=None):
    """qkv[M, (Hq+2Hkv)*D] = gemm(a, w, ...) with rope_kv_write fused into the GEMM epilogue when the decode schedule
    allows (one launch), else GEMM + rope_kv_write inside the library (two launches); identical bits.  Returns qkv."""
    _cuda(a, w, a_scale, w_scale, bias, positions, cos, sin, k_pool, v_pool, slot_mapping)
    m, k = a.shape
    n, k2 = w.shape
    nb, hkv, bs, d = k_pool.shape
    assert k == k2 and a.is_contiguous() and w.is_contiguous() and n == (num_q_heads + 2 * hkv) * d
    assert cos.dtype == torch.float32 and cos.shape[1] == d // 2 and cos.is_contiguous() and sin.is_contiguous()
    assert positions.dtype == torch.int64 and slot_mapping.dtype == torch.int64
    dt = _gemm_dtype(a, w)
    out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    if workspace is None:
        workspace = gemm_workspace(m, n, k, dt, a.device, split_k)
    with _k(f"gemm_rope_kv_{_DTN[dt]}[{m}x{n}x{k}]"):
        check(
            _cabi.load().b200_gemm_rope_kv_write(
                _ptr(a), _ptr(w), _ptr(out), _ptr(a_scale), _ptr(w_scale), _ptr(bias), m, n, k, dt, split_k,
                _ptr(workspace), 0 if workspace is None else workspace.numel() * workspace.element_size(),
                _ptr(positions), _ptr(cos), _ptr(sin), cos.shape[0], _ptr(k_pool), _ptr(v_pool), _ptr(slot_mapping),
                num_q_heads, hkv, d, bs, nb, _stream(),
            ),
            "b200_gemm_rope_kv_write",
        )
    return out


def interleave_gate_up(w_gu, *others):
    """Row permutation expected by gemm_silu_mul: [gate(I); up(I)] -> groups of 32 rows = 16 gate rows followed by the
    16 up rows of the same channels.  Applied (load time) to the weight and to every per-row companion (scale, bias)."""
    i = w_gu.shape[0] // 2
    assert i % 16 == 0, "intermediate size must be a multiple of 16"
    idx = torch.arange(i, device=w_gu.device).view(-1, 16)
    perm = torch.cat([idx, idx + i], dim=1).reshape(-1)
    res = [w_gu[perm].contiguous()] + [None if o is None else o[perm].contiguous() for o in others]
    return res[0] if not others else tuple(res)


def gemm_silu_mul(a, w_gu_interleaved, a_scale=None, w_scale=None, bias=None, split_k=0, workspace=None):
    """act[M, I] = bf16(silu(bf16(gate)) * bf16(up)) with gate/up = the two halves of a @ w_gu^T (rows interleaved by
    interleave_gate_up); also returns group_amax [M, 2I/32] for quantize_per_token."""
    _cuda(a, w_gu_interleaved, a_scale, w_scale, bias)
    m, k = a.shape
    n2, k2 = w_gu_interleaved.shape
    assert k == k2 and a.is_contiguous() and w_gu_interleaved.is_contiguous()
    dt = _gemm_dtype(a, w_gu_interleaved)
    act = torch.empty((m, n2 // 2), dtype=torch.bfloat16, device=a.device)
    assert n2 % 32 == 0
    group_amax = torch.empty((m, n2 // 32), dtype=torch.float32, device=a.device)
    if workspace is None:
        workspace = gemm_workspace(m, n2, k, dt, a.device, split_k)
    with _k(f"gemm_silu_mul_{_DTN[dt]}[{m}x{n2}x{k}]"):
        check(
            _cabi.load().b200_gemm_silu_mul(
                _ptr(a), _ptr(w_gu_interleaved), _ptr(act), _ptr(a_scale), _ptr(w_scale), _ptr(bias), _ptr(group_amax),
                m, n2, k, dt, split_k, _ptr(workspace), 0 if workspace is None else workspace.numel() * workspace.element_size(),
                _stream(),
            ),
            "b200_gemm_silu_mul",
        )
    return act, group_amax


_UNSUPPORTED = -4  # B200_ERR_UNSUPPORTED


def gemm_silu_mul_quant(a, w_gu_interleaved, a_scale, w_scale, bias, state, quant: str):
    """gate/up GEMM + SiLU*mul + per-token quantisation in ONE launch (b200_gemm_silu_mul_quant): returns (q [M, I], scale [M])
    or None when the shape does not run as one resident wave of one CTA per weight tile (the caller then uses gemm_silu_mul
    + quantize_per_token, which produce the same bits).  `state`: 1040-byte uint8 device tensor, zeroed once."""
    _cuda(a, w_gu_interleaved, a_scale, w_scale, bias, state)
    m, k = a.shape
    n2, k2 = w_gu_interleaved.shape
    assert k == k2 and a.is_contiguous() and w_gu_interleaved.is_contiguous() and n2 % 32 == 0 and state.numel() >= 1040
    if m > 128:
        return None
    dt = _gemm_dtype(a, w_gu_interleaved)
    qd = _QDT[quant]
    q = torch.empty((m, n2 // 2), dtype=_TORCH_Q[qd], device=a.device)
    sc = torch.empty((m,), dtype=torch.float32, device=a.device)
    with _k(f"gemm_silu_mul_quant_{_DTN[dt]}[{m}x{n2}x{k}]"):
        rc = _cabi.load().b200_gemm_silu_mul_quant(_ptr(a), _ptr(w_gu_interleaved), _ptr(q), _ptr(sc), _ptr(a_scale), _ptr(w_scale),
                                                   _ptr(bias), _ptr(state), m, n2, k, dt, _stream())
    if rc == _UNSUPPORTED:
        return None
    check(rc, "b200_gemm_silu_mul_quant")
    return q, sc


# ------------------------------------------------------------------ glue
def rmsnorm(x, w, eps, quant=None, out_bf16=None, want_bf16=None):
    """Returns bf16 y, or (q, scale) for quant in {"fp8","int8"} (plus y when want_bf16)."""
    _cuda(x, w)
    t, h = x.shape
    assert x.is_contiguous() and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    qd = _QDT[quant]
    if qd == BF16:
        y = out_bf16 if out_bf16 is not None else torch.empty_like(x)
        with _k("rmsnorm"):
            check(_cabi.load().b200_rmsnorm(_ptr(x), _ptr(w), _ptr(y), 0, 0, t, h, float(eps), qd, _stream()), "b200_rmsnorm")
        return y
    q = torch.empty((t, h), dtype=_TORCH_Q[qd], device=x.device)
    s = torch.empty((t,), dtype=torch.float32, device=x.device)
    y = (out_bf16 if out_bf16 is not None else torch.empty_like(x)) if want_bf16 else None
    with _k("rmsnorm_quant"):
        check(_cabi.load().b200_rmsnorm(_ptr(x), _ptr(w), _ptr(y), _ptr(q), _ptr(s), t, h, float(eps), qd, _stream()), "b200_rmsnorm")
    return (q, s, y) if want_bf16 else (q, s)


def silu_mul(gate_up, quant=None):
    _cuda(gate_up)
    t, i2 = gate_up.shape
    i = i2 // 2
    assert gate_up.is_contiguous() and gate_up.dtype == torch.bfloat16
    qd = _QDT[quant]
    if qd == BF16:
        y = torch.empty((t, i), dtype=torch.bfloat16, device=gate_up.device)
        with _k("silu_mul"):
            check(_cabi.load().b200_silu_mul(_ptr(gate_up), _ptr(y), 0, 0, t, i, qd, _stream()), "b200_silu_mul")
        return y
    q = torch.empty((t, i), dtype=_TORCH_Q[qd], device=gate_up.device)
    s = torch.empty((t,), dtype=torch.float32, device=gate_up.device)
    with _k("silu_mul_quant"):
        check(_cabi.load().b200_silu_mul(_ptr(gate_up), 0, _ptr(q), _ptr(s), t, i, qd, _stream()), "b200_silu_mul")
    return q, s


def quantize_per_token(x, quant: str, group_amax=None):
    """x [T, K] bf16 -> (q [T, K], scale [T]).  group_amax [T, n_groups] (from gemm_silu_mul) skips the row scan."""
    _cuda(x, group_amax)
    t, k = x.shape
    assert x.is_contiguous() and x.dtype == torch.bfloat16
    qd = _QDT[quant]
    q = torch.empty((t, k), dtype=_TORCH_Q[qd], device=x.device)
    s = torch.empty((t,), dtype=torch.float32, device=x.device)
    nt = 0
    if group_amax is not None:
        assert group_amax.dtype == torch.float32 and group_amax.is_contiguous() and group_amax.shape[0] == t
        nt = group_amax.shape[1]
    with _k("quantize_per_token"):
        check(_cabi.load().b200_quantize_per_token(_ptr(x), _ptr(q), _ptr(s), _ptr(group_amax), nt, t, k, qd, _stream()),
              "b200_quantize_per_token")
    return q, s


def embedding(tokens, table, out=None):
    _cuda(tokens, table)
    v, h = table.shape
    t = tokens.numel()
    assert tokens.dtype == torch.int64 and table.is_contiguous()
    if out is None:
        out = torch.empty((t, h), dtype=table.dtype, device=table.device)
    with _k("embedding"):
        check(_cabi.load().b200_embedding(_ptr(tokens), _ptr(table), _ptr(out), t, h, v, _stream()), "b200_embedding")
    return out


def argmax(logits, idx_offset: int = 0, want_val: bool = False, out_val=None, out_idx=None):
    _cuda(logits)
    t, v = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    idx = torch.empty((t,), dtype=torch.int64, device=logits.device) if out_idx is None else out_idx[:t]
    val = (torch.empty((t,), dtype=torch.float32, device=logits.device) if out_val is None else out_val[:t]) if want_val else None
    with _k("argmax"):
        check(_cabi.load().b200_argmax(_ptr(logits), logits.stride(0), _ptr(val), _ptr(idx), t, v, idx_offset, _stream()), "b200_argmax")
    return (val, idx) if want_val else idx


def tp_argmax_merge(peer_vals, peer_idxs, peer_flags, epoch, rank, world, b):
    """Greedy merge of the per-shard (max, global index) pairs over peer memory (tp_comm.TpComm.merge_argmax)."""
    out = torch.empty((b,), dtype=torch.int64, device=epoch.device)
    with _k("tp_argmax_merge"):
        check(_cabi.load().b200_tp_argmax_merge(peer_vals, peer_idxs, peer_flags, _ptr(epoch), rank, world, _ptr(out), b,
                                                _stream()), "b200_tp_argmax_merge")
    return out


SAMPLE_K = 256  # candidates per (row, vocab shard); the reference's _MAX_NEURON_SAMPLING_TOP_K (RUNNER:74)


def topk_candidates(logits, idx_offset: int = 0):
    """logits fp32 [B, V] -> (cand_val [B,256] fp32, cand_idx [B,256] int64) sorted by (value desc, index asc)."""
    _cuda(logits)
    b, v = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    val = torch.empty((b, SAMPLE_K), dtype=torch.float32, device=logits.device)
    idx = torch.empty((b, SAMPLE_K), dtype=torch.int64, device=logits.device)
    with _k("topk_candidates"):
        check(_cabi.load().b200_topk_candidates(_ptr(logits), logits.stride(0), _ptr(val), _ptr(idx), b, v, idx_offset,
                                                _stream()), "b200_topk_candidates")
    return val, idx


def sample_candidates(cand_val, cand_idx, params, u, out=None):
    """cand_* [B,256] or [groups,B,256]; params fp32 [B,3] = (top_k, top_p, temperature); u fp32 [B] in [0,1)."""
    _cuda(cand_val, cand_idx, params, u)
    if cand_val.dim() == 2:
        cand_val, cand_idx = cand_val.unsqueeze(0), cand_idx.unsqueeze(0)
    g, b, k = cand_val.shape
    assert k == SAMPLE_K and cand_val.is_contiguous() and cand_idx.is_contiguous() and cand_idx.dtype == torch.int64
    assert params.shape == (b, 3) and params.dtype == torch.float32 and params.is_contiguous()
    assert u.shape == (b,) and u.dtype == torch.float32
    if out is None:
        out = torch.empty((b,), dtype=torch.int64, device=cand_val.device)
    with _k("sample_candidates"):
        check(_cabi.load().b200_sample_candidates(_ptr(cand_val), _ptr(cand_idx), g, b, _ptr(params), _ptr(u), _ptr(out),
                                                  _stream()), "b200_sample_candidates")
    return out


def row_lse(logits):
    """logits fp32 [B, V] -> (row max [B], sum exp(x - max) [B]) of the local vocab shard."""
    _cuda(logits)
    b, v = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    m = torch.empty((b,), dtype=torch.float32, device=logits.device)
    s = torch.empty((b,), dtype=torch.float32, device=logits.device)
    with _k("row_lse"):
        check(_cabi.load().b200_row_lse(_ptr(logits), logits.stride(0), _ptr(m), _ptr(s), b, v, _stream()), "b200_row_lse")
    return m, s


def gather_logprobs(cand_val, cand_idx, sampled, row_max, row_sumexp, num_logprobs: int):
    """cand_* [B,256] or [groups,B,256]; row_max / row_sumexp [B] or [groups,B]; sampled int64 [B].
    -> (ids int32 [B, 1+n], logprobs fp32 [B, 1+n], ranks int32 [B]) in vLLM's LogprobsTensors layout."""
    _cuda(cand_val, cand_idx, sampled, row_max, row_sumexp)
    if cand_val.dim() == 2:
        cand_val, cand_idx, row_max, row_sumexp = cand_val.unsqueeze(0), cand_idx.unsqueeze(0), row_max.unsqueeze(0), row_sumexp.unsqueeze(0)
    g, b, k = cand_val.shape
    assert k == SAMPLE_K and cand_val.is_contiguous() and cand_idx.is_contiguous() and row_max.is_contiguous()
    assert row_max.shape == (g, b) and row_sumexp.shape == (g, b) and row_sumexp.is_contiguous() and sampled.dtype == torch.int64
    ids = torch.empty((b, 1 + num_logprobs), dtype=torch.int32, device=cand_val.device)
    lp = torch.empty((b, 1 + num_logprobs), dtype=torch.float32, device=cand_val.device)
    rk = torch.empty((b,), dtype=torch.int32, device=cand_val.device)
    with _k("gather_logprobs"):
        check(_cabi.load().b200_gather_logprobs(_ptr(cand_val), _ptr(cand_idx), g, b, _ptr(sampled), _ptr(row_max),
                                                _ptr(row_sumexp), num_logprobs, _ptr(ids), _ptr(lp), _ptr(rk), _stream()),
              "b200_gather_logprobs")
    return ids, lp, rk


def allreduce_rmsnorm(peer_bufs, peer_flags, epoch, rank, world, t, h, norm_w, eps, quant=None, want_bf16=False, mc_buf=0):
    """One-shot all-reduce over NVLink peer memory fused with RMSNorm (+ per-token quantisation).
    peer_bufs / peer_flags: ctypes arrays of `world` device pointers (tp_comm.TpComm).  mc_buf != 0: the multicast address
    of the partial -- the sum is then done inside the NVSwitch (b200_allreduce_rmsnorm_nvls).  Returns (x, h_out, h_scale):
    x = the reduced bf16 residual stream; h_out = normed bf16 (quant None) or quantised tensor; h_scale = scales or None."""
    dev = epoch.device
    x = torch.empty((t, h), dtype=torch.bfloat16, device=dev)
    qd = _QDT[quant]
    lib = _cabi.load()
    if mc_buf:
        fn, first, name = lib.b200_allreduce_rmsnorm_nvls, int(mc_buf), "b200_allreduce_rmsnorm_nvls"
    else:
        fn, first, name = lib.b200_allreduce_rmsnorm, peer_bufs, "b200_allreduce_rmsnorm"
    if norm_w is None:
        with _k("allreduce"):
            check(fn(first, peer_flags, _ptr(epoch), rank, world, _ptr(x), 0, 0, 0, 0, t, h, float(eps), BF16, _stream()), name)
        return x, None, None
    if qd == BF16:
        y = torch.empty_like(x)
        with _k("allreduce_rmsnorm"):
            check(fn(first, peer_flags, _ptr(epoch), rank, world, _ptr(x), _ptr(norm_w), _ptr(y), 0, 0, t, h, float(eps), qd,
                     _stream()), name)
        return x, y, None
    q = torch.empty((t, h), dtype=_TORCH_Q[qd], device=dev)
    s = torch.empty((t,), dtype=torch.float32, device=dev)
    y = torch.empty_like(x) if want_bf16 else None
    with _k("allreduce_rmsnorm_quant"):
        check(fn(first, peer_flags, _ptr(epoch), rank, world, _ptr(x), _ptr(norm_w), _ptr(y), _ptr(q), _ptr(s), t, h,
                 float(eps), qd, _stream()), name)
    return x, q, s


# ------------------------------------------------------------------ hybrid decoders (state-space + windowed attention + MoE)
# The residual stream and every norm / recurrence tensor is fp32; tensors that feed a GEMM or live in a KV pool are bf16
# (bf16 serving) or fp32 (32-bit serving).  `meta` is a StepMeta-like object with the ragged-batch index tensors.
def _edt(t):
    if t is torch.bfloat16 or (hasattr(t, "dtype") and t.dtype == torch.bfloat16):
        return BF16
    if t is torch.float32 or (hasattr(t, "dtype") and t.dtype == torch.float32):
        return F32
    raise _cabi.B200Error(f"element type {t} is neither bfloat16 nor float32")


def _f32(*ts):
    for t in ts:
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
            raise _cabi.B200Error("expected a contiguous fp32 tensor")


def embed_scale(tokens, table, scale: float):
    """tokens int32 [T] -> fp32 [T, W] = table[token] * scale."""
    _cuda(tokens, table)
    assert tokens.dtype == torch.int32 and table.is_contiguous()
    t, (v, w) = tokens.numel(), table.shape
    out = torch.empty((t, w), dtype=torch.float32, device=table.device)
    with _k("embed_scale"):
        check(_cabi.load().b200_embed_scale(_ptr(tokens), _ptr(table), _edt(table), _ptr(out), t, w, v, float(scale), _stream()),
              "b200_embed_scale")
    return out


def dyt_norm(x, w, b, alpha: float, out_dtype):
    _cuda(x, w, b)
    _f32(x, w, b)
    t, width = x.shape
    out = torch.empty((t, width), dtype=out_dtype, device=x.device)
    with _k("dyt_norm"):
        check(_cabi.load().b200_dyt_norm(_ptr(x), _ptr(w), _ptr(b), float(alpha), _ptr(out), _edt(out), t, width, _stream()),
              "b200_dyt_norm")
    return out


def dyt_residual(x, y, norm, next_norm=None, out_dtype=torch.bfloat16, y2=None, nsum: int = 1):
    """x += dyt(sum of the nsum consecutive rows of y per token [+ y2]); returns dyt_next(x) in out_dtype (or None).
    norm / next_norm: (w, b, alpha)."""
    _cuda(x, y, y2)
    _f32(x, y, y2)
    t, width = x.shape
    assert y.shape == (t * nsum, width) and (y2 is None or y2.shape == (t, width))
    out2 = torch.empty((t, width), dtype=out_dtype, device=x.device) if next_norm is not None else None
    w2, b2, a2 = next_norm if next_norm is not None else (None, None, 0.0)
    with _k("dyt_residual"):
        check(_cabi.load().b200_dyt_residual(_ptr(x), _ptr(y), nsum, _ptr(y2), _ptr(norm[0]), _ptr(norm[1]), float(norm[2]),
                                             _ptr(w2), _ptr(b2), float(a2), _ptr(out2), _edt(out_dtype), t, width, _stream()),
              "b200_dyt_residual")
    return out2


def gated_group_rmsnorm(y, z_src, w, groups: int, eps: float, out_dtype):
    """y fp32 [T, inner]; z = the first `inner` columns of the fp32 rows z_src (any pitch)."""
    _cuda(y, z_src, w)
    _f32(y, w)
    assert z_src.dtype == torch.float32 and z_src.stride(1) == 1
    t, inner = y.shape
    out = torch.empty((t, inner), dtype=out_dtype, device=y.device)
    with _k("gated_group_rmsnorm"):
        check(_cabi.load().b200_gated_group_rmsnorm(_ptr(y), _ptr(z_src), z_src.stride(0), _ptr(w), _ptr(out), _edt(out), t, inner,
                                                    groups, float(eps), _stream()), "b200_gated_group_rmsnorm")
    return out


def clamped_glu(gate_up, limit: float, out_dtype):
    _cuda(gate_up)
    _f32(gate_up)
    t, ff2 = gate_up.shape
    out = torch.empty((t, ff2 // 2), dtype=out_dtype, device=gate_up.device)
    with _k("clamped_glu"):
        check(_cabi.load().b200_clamped_glu(_ptr(gate_up), _ptr(out), _edt(out), t, ff2 // 2, float(limit), _stream()),
              "b200_clamped_glu")
    return out


def causal_conv_silu(src, col0: int, channels: int, conv_w, conv_b, state, meta, out_dtype, *, in_bias=None, silu: bool = True):
    """Columns [col0, col0 + channels) of the fp32 rows `src` -> SiLU(conv) [T, channels]; `state` [slots, taps-1, channels]
    fp32 is read for continuing sequences and updated for all.  in_bias fp32 [channels]: added to the inputs read from `src`
    (a projection's bias; the state holds biased inputs).  silu False: the convolution alone."""
    _cuda(src, conv_w, conv_b, state, in_bias)  # conv_b may be None (no bias)
    _f32(src, conv_w, conv_b, state, in_bias)
    t, taps = src.shape[0], conv_w.shape[1]
    assert conv_w.shape[0] == channels and state.shape[1:] == (max(taps - 1, 1), channels)  # one unused row when taps == 1
    out = torch.empty((t, channels), dtype=out_dtype, device=src.device)
    assert in_bias is None or in_bias.numel() == channels
    with _k("causal_conv_silu" if silu else "causal_conv"):
        check(_cabi.load().b200_causal_conv(_ptr(src), src.stride(0), col0, _ptr(conv_w), _ptr(conv_b), _ptr(in_bias), 1 if silu else 0,
                                            _ptr(state), _ptr(meta.tok_seq), _ptr(meta.seq_start), _ptr(meta.seq_slot),
                                            _ptr(meta.seq_pos0), _ptr(out), _edt(out), t, meta.num_seqs, channels, taps, _stream()),
              "b200_causal_conv")
    return out


SCAN_SEGMENT = 128  # tokens per parallel segment of a long portion in the selective scan


def ssd_scan(xbc, dt_src, dt_col0: int, a_log, dt_bias, d_skip, state, meta, heads: int, vdim: int, nstate: int, groups: int):
    """xbc [T, H*P + 2*G*N] (bf16 | fp32), raw dt = columns [dt_col0, dt_col0 + H) of the fp32 rows dt_src; state fp32
    [slots, H, P, N] updated in place; returns y fp32 [T, H*P].  When the step carries a segment list (meta.scan_segs: some
    portion is long) the segments run in parallel from scratch states that a combine pass chains together."""
    _cuda(xbc, dt_src, state)
    _f32(dt_src, a_log, dt_bias, d_skip, state)
    assert xbc.is_contiguous() and state.shape[1:] == (heads, vdim, nstate)
    t = xbc.shape[0]
    y = torch.empty((t, heads * vdim), dtype=torch.float32, device=xbc.device)
    segs = getattr(meta, "scan_segs", None)
    nseg = meta.num_segs if segs is not None else 0
    seg_state = seg_dt = None
    if nseg:
        seg_state = torch.empty((nseg + 1, heads, vdim, nstate), dtype=torch.float32, device=xbc.device)
        seg_dt = torch.empty((nseg, heads), dtype=torch.float32, device=xbc.device)
    with _k("ssd_scan"):
        check(_cabi.load().b200_ssd_scan(_ptr(xbc), _edt(xbc), xbc.shape[1], _ptr(dt_src), dt_src.stride(0), dt_col0, _ptr(a_log),
                                         _ptr(dt_bias), _ptr(d_skip), _ptr(state), _ptr(meta.seq_start), _ptr(meta.seq_slot),
                                         _ptr(meta.seq_pos0), _ptr(y), meta.num_seqs, heads, vdim, nstate, groups,
                                         _ptr(segs) if nseg else 0, nseg, _ptr(meta.scan_seq_seg0) if nseg else 0,
                                         _ptr(seg_state), _ptr(seg_dt), _stream()), "b200_ssd_scan")
    return y


def kv_write_vmix(qkv, k_col0: int, v_col0: int, k_pool, v_pool, slot_mapping, *, v_first=None, lam: float = 0.0, mode: int = 0):
    """Pools [num_blocks, G, block_size, D] / [.., Dv].  mode 0 plain, 1 record v_first, 2 mix with v_first before caching."""
    _cuda(qkv, k_pool, v_pool, slot_mapping, v_first)
    _f32(qkv, v_first)
    assert slot_mapping.dtype == torch.int64 and k_pool.dtype == v_pool.dtype and k_pool.is_contiguous() and v_pool.is_contiguous()
    _, g, bs, d = k_pool.shape
    dv = v_pool.shape[3]
    with _k("kv_write_vmix"):
        check(_cabi.load().b200_kv_write_vmix(_ptr(qkv), qkv.stride(0), k_col0, v_col0, _ptr(v_first), float(lam), mode,
                                              _ptr(k_pool), _ptr(v_pool), _edt(k_pool), _ptr(slot_mapping), qkv.shape[0], g, d, dv,
                                              bs, _stream()), "b200_kv_write_vmix")


PREFILL_ATTN_MIN_TOKENS = 16  # longest portion of a step from which the tensor-core attention kernel is used
PREFILL_TC_MIN_TOKENS = 128   # ... and from which the tcgen05 kernel with its 128-row query tiles is
_SWA_PREFILL_LEGACY = bool(os.environ.get("B200_SWA_PREFILL_LEGACY"))


def swa_sink_attn(q_src, num_heads: int, k_pool, v_pool, block_table, meta, sink, scale: float, window: int,
                  latent_values: int = 0, *, chunk: int = 0, softcap: float = 0.0, sigmoid_bias=None, out_f32: bool = False,
                  split_p: bool = False, pooled=None):
    """q = the first num_heads * D columns of the fp32 rows q_src -> [T, num_heads * Dv] in the pools' element type.
    sink None: ordinary softmax.  latent_values = C > 0: v_pool is ignored and the values are the first C columns of the key
    rows (attention over cached latents: one pool holds both).
    chunk > 0: a query sees only the keys of its own chunk of that many positions (counted from position 0).  softcap > 0:
    scaled scores pass through softcap * tanh(s / softcap).  sigmoid_bias fp32 [H]: weights sigmoid(s + bias[h]), not normalised
    over keys.  A value pool with fewer heads than the key pool: consecutive key heads share a value head (two score maps over
    the same values).  out_f32: fp32 rows.  split_p: the tensor-core kernel carries the weights as two bf16 terms.
    pooled = (pooled key pool, pooled value pool, P) with a window: every block of P positions that lies wholly before a query's
    window is seen as one key / value, the block's row of the pooled pools (kv_pool_mean), in the same softmax."""
    _cuda(q_src, k_pool, v_pool, block_table, sink, sigmoid_bias)
    pk, pv, pool = pooled if pooled is not None else (None, None, 0)
    if pool:
        _cuda(pk, pv)
        ppb = -(-k_pool.shape[2] // pool)
        assert not latent_values and window < (1 << 30) and pk.dtype == k_pool.dtype and pv.dtype == k_pool.dtype
        assert pk.is_contiguous() and pv.is_contiguous() and pk.shape == (k_pool.shape[0], k_pool.shape[1], ppb, k_pool.shape[3])
        assert pv.shape == (v_pool.shape[0], v_pool.shape[1], ppb, v_pool.shape[3])
    pool_args = (_ptr(pk), _ptr(pv), int(pool))
    _f32(q_src, sink, sigmoid_bias)
    assert block_table.dtype == torch.int32 and block_table.stride(1) == 1
    _, g, bs, d = k_pool.shape
    if latent_values:
        v_pool, dv, v_pitch = k_pool, int(latent_values), d
        assert g == 1 and dv <= d
    else:
        dv = v_pitch = v_pool.shape[3]
    v_div = g // v_pool.shape[1]
    assert v_pool.shape[1] * v_div == g and v_pool.shape[2] == bs
    t = q_src.shape[0]
    out = torch.empty((t, num_heads * dv), dtype=torch.float32 if out_f32 else k_pool.dtype, device=q_src.device)
    variant = (int(chunk), float(softcap), _ptr(sigmoid_bias), v_div, 1 if out_f32 else 0)
    plain = not chunk and not softcap and sigmoid_bias is None and v_div == 1 and not out_f32
    # the per-launch timer tells the variants apart (their floors differ)
    tag = "" if plain and not pool else "[" + "+".join(n for n, on in (("chunk", chunk), ("cap", softcap), ("sigmoid", sigmoid_bias is not None),
                                                                       ("maps", v_div > 1), ("pool", pool)) if on) + "]"
    # long prompt portions in bf16 serving, head sizes of 64 / 128 with pages of 32 tokens: the tcgen05 kernel (128-row query
    # tiles, accumulators in tensor memory); B200_SWA_PREFILL_LEGACY=1 keeps the mma.sync kernel (A/B aid)
    if (k_pool.dtype == torch.bfloat16 and meta.max_new >= PREFILL_TC_MIN_TOKENS and sink is None and window >= (1 << 30)
            and not latent_values and q_src.stride(0) % 4 == 0 and q_src.data_ptr() % 16 == 0 and not _SWA_PREFILL_LEGACY
            and _cabi.load().b200_swa_sink_attn_prefill_tc_supported(d, dv, bs, v_div, 1 if softcap else 0,
                                                                     0 if sigmoid_bias is None else 1)):
        with _k("swa_sink_attn_prefill_tc" + tag):
            check(_cabi.load().b200_swa_sink_attn_prefill_tc(_ptr(q_src), q_src.stride(0), _ptr(k_pool), _ptr(v_pool), k_pool.shape[0],
                                                             _ptr(block_table), block_table.stride(0), _ptr(meta.seq_start),
                                                             _ptr(meta.seq_slot), _ptr(meta.seq_pos0), meta.num_seqs, meta.max_new,
                                                             float(scale), _ptr(out), num_heads, g, d, dv, bs, *variant,
                                                             1 if split_p else 0, _stream()),
                  "b200_swa_sink_attn_prefill_tc")
        return out
    # shorter prompt portions in bf16 serving: the mma.sync kernel; decode-sized steps, fp32 pools and odd head sizes: one CTA
    # per (token, head) on the CUDA cores
    if (k_pool.dtype == torch.bfloat16 and meta.max_new >= PREFILL_ATTN_MIN_TOKENS and d % 16 == 0 and dv % 16 == 0
            and d <= 512 and dv <= 256 and q_src.stride(0) % 2 == 0):
        with _k("swa_sink_attn_prefill" + tag):
            check(_cabi.load().b200_swa_sink_attn_prefill(_ptr(q_src), q_src.stride(0), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
                                                          block_table.stride(0), _ptr(meta.seq_start), _ptr(meta.seq_slot),
                                                          _ptr(meta.seq_pos0), meta.num_seqs, meta.max_new, _ptr(sink), float(scale),
                                                          int(window), _ptr(out), num_heads, g, d, dv, v_pitch, bs, *variant,
                                                          1 if split_p else 0, *pool_args, _stream()),
                  "b200_swa_sink_attn_prefill")
        return out
    if (plain and latent_values and sink is None and window >= (1 << 30) and k_pool.dtype == torch.bfloat16 and d % 16 == 0 and dv % 16 == 0
            and dv <= 256 and q_src.stride(0) % 2 == 0):
        # attention over cached latents, decode-sized steps: the heads of a token are the rows of a tensor-core tile
        with _k("latent_attn_decode"):
            check(_cabi.load().b200_latent_attn_decode(_ptr(q_src), q_src.stride(0), _ptr(k_pool), _ptr(block_table),
                                                       block_table.stride(0), _ptr(meta.tok_row), _ptr(meta.tok_pos), float(scale),
                                                       _ptr(out), t, num_heads, d, dv, bs, _stream()), "b200_latent_attn_decode")
        return out
    # long contexts at small batch: several CTAs share a (token, kv head)'s keys, so that every SM has its CTAs
    span = min(getattr(meta, "max_end", 0) or 0, int(window), int(chunk) if chunk else 1 << 30)
    if pool:  # the blocks before the window count as keys too
        span += max((getattr(meta, "max_end", 0) or 0) - int(window), 0) // pool
    tc = (k_pool.dtype == torch.bfloat16 and not latent_values and d % 16 == 0 and dv % 16 == 0 and d * v_div <= 512 and dv <= 256
          and q_src.stride(0) % 2 == 0)
    gv = g // v_div
    ctas = t * gv * -(-(num_heads // gv) // 16) if tc else t * g
    splits = max(1, min(8, (148 * (3 if tc else 4)) // max(1, ctas), -(-span // (128 if tc else 512))))
    ws = torch.empty((t * num_heads * splits * (dv + 2),), dtype=torch.float32, device=q_src.device) if splits > 1 else None
    if tc:  # decode-sized steps on bf16 pools: the query heads of a kv head are the rows of a tensor-core tile
        with _k("swa_sink_attn_decode_tc" + tag):
            check(_cabi.load().b200_swa_sink_attn_decode_tc(_ptr(q_src), q_src.stride(0), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
                                                            block_table.stride(0), _ptr(meta.tok_row), _ptr(meta.tok_pos), _ptr(sink),
                                                            float(scale), int(window), _ptr(out), t, num_heads, g, d, dv, v_pitch, bs,
                                                            *variant, 1 if split_p else 0, splits, _ptr(ws), *pool_args, _stream()),
                  "b200_swa_sink_attn_decode_tc")
        return out
    with _k("swa_sink_attn" + tag):
        check(_cabi.load().b200_swa_sink_attn(_ptr(q_src), q_src.stride(0), _ptr(k_pool), _ptr(v_pool), _edt(k_pool),
                                              _ptr(block_table), block_table.stride(0), _ptr(meta.tok_row), _ptr(meta.tok_pos),
                                              _ptr(sink), float(scale), int(window), _ptr(out), t, num_heads, g, d, dv, v_pitch, bs,
                                              *variant, splits, _ptr(ws), *pool_args, _stream()), "b200_swa_sink_attn")
    return out


def moe_topk(logits, top: int, bias=None, mode: int = ROUTE_SIGMOID):
    """fp32 router logits [T, E] (+ bias fp32 [E]) -> (expert ids int32 [T, top], routing weights fp32 [T, top]): the sigmoid of
    each chosen logit (ROUTE_SIGMOID), the softmax over the chosen logits (ROUTE_SOFTMAX_TOP), or the softmax over all experts with
    the chosen scores divided by their sum (ROUTE_SOFTMAX_RENORM)."""
    _cuda(logits, bias)
    _f32(bias)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    t, e = logits.shape
    idx = torch.empty((t, top), dtype=torch.int32, device=logits.device)
    wt = torch.empty((t, top), dtype=torch.float32, device=logits.device)
    with _k("moe_topk"):
        check(_cabi.load().b200_moe_topk(_ptr(logits), logits.stride(0), _ptr(bias), int(mode), _ptr(idx), _ptr(wt), t, e, top,
                                         _stream()), "b200_moe_topk")
    return idx, wt


def moe_tile_rows() -> int:
    return int(_cabi.load().b200_moe_tile_rows())


def moe_align(topk_idx, num_experts: int, tile_rows: int | None = None):
    """-> (sorted pair ids int32 [cap] padded with -1, tile owners int32 [max_tiles], device count of used tiles [1], rows per
    tile).  tile_rows: moe_tile_rows() (default) or four times that for prompt-sized bf16 batches."""
    _cuda(topk_idx)
    assert topk_idx.dtype == torch.int32 and topk_idx.is_contiguous()
    n, bm = topk_idx.numel(), tile_rows or moe_tile_rows()
    max_tiles = -(-n // bm) + num_experts
    dev = topk_idx.device
    sorted_ids = torch.empty(max_tiles * bm, dtype=torch.int32, device=dev)
    tile_expert = torch.empty(max_tiles, dtype=torch.int32, device=dev)
    num_tiles = torch.empty(1, dtype=torch.int32, device=dev)
    with _k("moe_align"):
        check(_cabi.load().b200_moe_align(_ptr(topk_idx), n, num_experts, _ptr(sorted_ids), sorted_ids.numel(), _ptr(tile_expert),
                                          max_tiles, _ptr(num_tiles), bm, _stream()), "b200_moe_align")
    return sorted_ids, tile_expert, num_tiles, bm


def moe_wide_tiles(h, w_gate_up, num_pairs: int) -> int | None:
    """Rows per expert tile for this batch: the wide tile once the experts see about 64 rows each on average and the
    operands suit the tensor-core kernel, else None (the default tile)."""
    e, ff2, width = w_gate_up.shape
    if h.dtype == torch.bfloat16 and width % 8 == 0 and (ff2 // 2) % 8 == 0 and h.stride(0) % 8 == 0 and num_pairs >= 64 * e:
        return 4 * moe_tile_rows()
    return None


def linear_simt(a, w):
    """fp32 [M, N] = a [M, K] @ w [N, K]^T with fp32 accumulation on the CUDA cores: fp32 operands, or shapes the tensor-core
    GEMM does not take."""
    _cuda(a, w)
    assert a.dtype == w.dtype and a.stride(1) == 1 and w.is_contiguous() and a.shape[1] == w.shape[1]
    m, k = a.shape
    n = w.shape[0]
    out = torch.empty((m, n), dtype=torch.float32, device=a.device)
    with _k(f"linear_simt[{m}x{n}x{k}]"):
        check(_cabi.load().b200_grouped_linear(_ptr(a), a.stride(0), 0, 0, 0, _ptr(w), 0, 0, 0, -(-m // moe_tile_rows()), m, n, k,
                                               _edt(a), _ptr(out), n, 0, 0, 0, 0.0, moe_tile_rows(), _stream()), "b200_grouped_linear")
    return out


def batched_linear(a, w, out, *, a_batch_stride: int, out_batch_stride: int, gate=None):
    """out_b = a_b @ w[b]^T for every b of w [batch, N, K] in one launch: a_b = rows of `a` (pitch a.stride(0)) starting at
    column b * a_batch_stride, out_b likewise in `out` (fp32, or the operand type).  gate: fp32 view [M, >= batch] whose
    sigmoid multiplies out_b's rows."""
    _cuda(a, w, out, gate)
    assert a.dtype == w.dtype and a.stride(1) == 1 and out.stride(1) == 1 and w.is_contiguous() and w.dim() == 3
    b, n, k = w.shape
    m = a.shape[0]
    typed = out.dtype == a.dtype and out.dtype != torch.float32
    assert typed or out.dtype == torch.float32
    if gate is not None:
        assert gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape[0] == m
    with _k(f"batched_linear[{b}x{m}x{n}x{k}]"):
        check(_cabi.load().b200_batched_linear(_ptr(a), a.stride(0), a_batch_stride, _ptr(w), n * k, _ptr(out), out.stride(0),
                                               out_batch_stride, b, m, n, k, _edt(a), 1 if typed else 0, _ptr(gate),
                                               gate.stride(0) if gate is not None else 0, _stream()), "b200_batched_linear")
    return out


def moe_experts(h, topk_weight, align, w_gate_up, w_down, top: int, limit: float = 0.0, act: int = ACT_SWISH_CLAMPED,
                scale_input: bool = True):
    """Routed experts: for every (token, choice) pair  W_down glu(W_gate_up (weight * h)) (scale_input), or the unweighted
    expert output (the caller then weighs the outputs).  h [T, W]; w_gate_up [E, 2 ff, W] (gate rows first), w_down
    [E, W, ff]; returns fp32 [T * top, W] in pair order."""
    _cuda(h, topk_weight, w_gate_up, w_down)
    sorted_ids, tile_expert, num_tiles, bm = align
    e, ff2, width = w_gate_up.shape
    ff = ff2 // 2
    tiles = tile_expert.numel()
    hid = torch.empty((sorted_ids.numel(), ff), dtype=h.dtype, device=h.device)
    out = torch.empty((h.shape[0] * top, width), dtype=torch.float32, device=h.device)
    lib = _cabi.load()
    if bm > moe_tile_rows():  # prompt-sized: gather and scale the pairs once, then plain rows into the pipelined kernel
        rows = torch.empty((sorted_ids.numel(), width), dtype=h.dtype, device=h.device)
        with _k("moe_gather_scale"):
            check(lib.b200_moe_gather_scale(_ptr(h), h.stride(0), _ptr(sorted_ids), sorted_ids.numel(), top,
                                            _ptr(topk_weight) if scale_input else 0,
                                            _ptr(num_tiles), bm, _ptr(rows), width, _stream()), "b200_moe_gather_scale")
        a, lda, gdiv, scale = rows, width, 0, 0
    else:
        a, lda, gdiv, scale = h, h.stride(0), top, _ptr(topk_weight) if scale_input else 0
    with _k("moe_gate_up_glu"):
        check(lib.b200_grouped_linear(_ptr(a), lda, _ptr(sorted_ids), gdiv, scale, _ptr(w_gate_up), ff2 * width,
                                      _ptr(tile_expert), _ptr(num_tiles), tiles, 0, ff, width, _edt(h), _ptr(hid), ff, 0, 1,
                                      int(act), float(limit), bm, _stream()), "b200_grouped_linear")
    with _k("moe_down"):
        check(lib.b200_grouped_linear(_ptr(hid), ff, _ptr(sorted_ids), 0, 0, _ptr(w_down), width * ff, _ptr(tile_expert),
                                      _ptr(num_tiles), tiles, 0, width, ff, _edt(h), _ptr(out), width, 1, 0, 0, 0.0, bm, _stream()),
              "b200_grouped_linear")
    return out


# ------------------------------------------------------------------ post-norm hybrid decoders (delta rule + latent attention)
def embed_bigram(tokens, table, scale: float, meta, *, bigram=None, buckets: int = 0, mul_prev: int = 0, mul_cur: int = 0,
                 prev_state=None, want_cast: bool = True):
    """tokens int32 [T] -> (x fp32 [T, W], the same rows in the table's type or None).  x = table[token] * scale + bigram[row]
    with row hashed from (previous token, token); prev_state int32 [slots] carries each sequence's last token across steps."""
    _cuda(tokens, table, bigram, prev_state)
    assert tokens.dtype == torch.int32 and table.is_contiguous() and (bigram is None or (bigram.is_contiguous() and bigram.dtype == table.dtype))
    t, (v, w) = tokens.numel(), table.shape
    out = torch.empty((t, w), dtype=torch.float32, device=table.device)
    cast = torch.empty((t, w), dtype=table.dtype, device=table.device) if want_cast else None
    with _k("embed_bigram"):
        check(_cabi.load().b200_embed_bigram(_ptr(tokens), _ptr(table), _ptr(bigram), _edt(table), int(buckets), int(mul_prev),
                                             int(mul_cur), _ptr(prev_state), _ptr(meta.tok_seq), _ptr(meta.seq_start),
                                             _ptr(meta.seq_slot), _ptr(meta.seq_pos0), _ptr(out), _ptr(cast), t, w, v, float(scale),
                                             _stream()), "b200_embed_bigram")
    return out, cast


def rms_residual(x, y, w, eps: float, *, offset: float = 1.0, nsum: int = 1, y_weight=None, out_dtype=None):
    """x += rmsnorm(sum of the nsum consecutive rows of y per token, weighted by y_weight [T, nsum] when given) * (offset + w);
    returns x in out_dtype (the next GEMM's operand) or None."""
    _cuda(x, y, w, y_weight)
    _f32(x, y, w, y_weight)
    t, width = x.shape
    assert y.shape == (t * nsum, width) and (y_weight is None or y_weight.numel() == t * nsum)
    cast = torch.empty((t, width), dtype=out_dtype, device=x.device) if out_dtype is not None else None
    with _k("rms_residual"):
        check(_cabi.load().b200_rms_residual(_ptr(x), _ptr(y), nsum, _ptr(y_weight), _ptr(w), float(offset), float(eps), _ptr(cast),
                                             _edt(out_dtype) if out_dtype is not None else F32, t, width, _stream()), "b200_rms_residual")
    return cast


def rmsnorm_cols(src, col0: int, n: int, w, eps: float, out_dtype, *, offset: float = 0.0):
    """RMS norm of columns [col0, col0 + n) of the fp32 rows src, times (offset + w) -> [T, n] in out_dtype."""
    _cuda(src, w)
    _f32(w)
    assert src.dtype == torch.float32 and src.stride(1) == 1 and w.numel() == n
    t = src.shape[0]
    out = torch.empty((t, n), dtype=out_dtype, device=src.device)
    with _k("rmsnorm_cols"):
        check(_cabi.load().b200_rmsnorm_cols(_ptr(src), src.stride(0), col0, n, _ptr(w), float(offset), float(eps), _ptr(out),
                                             _edt(out), n, t, _stream()), "b200_rmsnorm_cols")
    return out


def head_rmsnorm_gate(o, gate_src, gate_col0: int, w, eps: float, heads: int, out_dtype):
    """o fp32 [T, H * P]: per head o / rms(o) * w [P] * silu(gate), gate = columns gate_col0.. of the fp32 rows gate_src
    (gate_src None: the norm alone)."""
    _cuda(o, gate_src, w)
    _f32(o, w)
    assert gate_src is None or (gate_src.dtype == torch.float32 and gate_src.stride(1) == 1)
    t, hp = o.shape
    p = hp // heads
    assert w.numel() == p
    out = torch.empty((t, hp), dtype=out_dtype, device=o.device)
    with _k("head_rmsnorm_gate"):
        check(_cabi.load().b200_head_rmsnorm_gate(_ptr(o), _ptr(gate_src), gate_src.stride(0) if gate_src is not None else 0, gate_col0, _ptr(w), float(eps),
                                                  _ptr(out), _edt(out), t, heads, p, _stream()), "b200_head_rmsnorm_gate")
    return out


def glu(gate_up, act: int, out_dtype):
    """fp32 [T, 2 ff] (gate columns first) -> act(gate) * up in out_dtype; act = ACT_SILU | ACT_GELU_TANH."""
    _cuda(gate_up)
    _f32(gate_up)
    t, ff2 = gate_up.shape
    out = torch.empty((t, ff2 // 2), dtype=out_dtype, device=gate_up.device)
    with _k("glu"):
        check(_cabi.load().b200_glu(_ptr(gate_up), _ptr(out), _edt(out), t, ff2 // 2, int(act), _stream()), "b200_glu")
    return out


def delta_rule(qkv, proj, b_col0: int, a_col0: int, a_log, dt_bias, state, meta, heads: int, kv_heads: int, dim: int, vdim: int,
               q_scale: float, unit_eps: float = 1e-6):
    """Gated delta rule over a ragged batch.  qkv fp32 [T, q: G*D | k: G*D | v: H*P] (convolved; q and k are normalised IN
    PLACE); raw beta / decay inputs are columns b_col0.. / a_col0.. of the fp32 rows proj; state fp32 [slots, H, P, D] updated
    in place.  Returns o fp32 [T, H * P]."""
    _cuda(qkv, proj, state)
    _f32(qkv, a_log, dt_bias, state)
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and state.shape[1:] == (heads, vdim, dim)
    assert qkv.shape[1] == 2 * kv_heads * dim + heads * vdim
    t = qkv.shape[0]
    bg = torch.empty((t, 2 * heads), dtype=torch.float32, device=qkv.device)
    kq = torch.empty((t, kv_heads), dtype=torch.float32, device=qkv.device)
    out = torch.empty((t, heads * vdim), dtype=torch.float32, device=qkv.device)
    lib = _cabi.load()
    with _k("delta_prep"):
        check(lib.b200_delta_prep(_ptr(qkv), qkv.stride(0), _ptr(proj), proj.stride(0), b_col0, a_col0, _ptr(a_log), _ptr(dt_bias),
                                  _ptr(bg), _ptr(kq), t, heads, kv_heads, dim, float(q_scale), float(unit_eps), _stream()),
              "b200_delta_prep")
    with _k("delta_scan"):
        check(lib.b200_delta_scan(_ptr(qkv), qkv.stride(0), _ptr(bg), _ptr(kq), _ptr(state), _ptr(meta.seq_start),
                                  _ptr(meta.seq_slot), _ptr(meta.seq_pos0), _ptr(out), meta.num_seqs, int(meta.max_new), heads, kv_heads, dim, vdim,
                                  _stream()), "b200_delta_scan")
    return out


def latent_kv_write(src, col0: int, kv_rank: int, rot_dim: int, rot_n: int, norm_w, eps: float, cos, sin, meta, pool):
    """Columns [col0, col0 + kv_rank + rot_dim) of the fp32 rows src -> pool rows [RMS-normed latent | rotated shared key part]
    at the step's slots.  pool [num_blocks, 1, block_size, kv_rank + rot_dim]; cos / sin fp32 [positions, rot_n / 2]."""
    _cuda(src, norm_w, cos, sin, pool)
    _f32(norm_w, cos, sin)
    assert src.dtype == torch.float32 and src.stride(1) == 1 and pool.is_contiguous() and pool.shape[-1] == kv_rank + rot_dim
    with _k("latent_kv_write"):
        check(_cabi.load().b200_latent_kv_write(_ptr(src), src.stride(0), col0, kv_rank, rot_dim, rot_n, _ptr(norm_w), float(eps),
                                                _ptr(cos), _ptr(sin), _ptr(meta.tok_pos), _ptr(meta.slot_mapping), _ptr(pool),
                                                _edt(pool), src.shape[0], _stream()), "b200_latent_kv_write")


def latent_q_prep(q, heads: int, dim: int, rot_dim: int, rot_n: int, kv_rank: int, cos, sin, meta, nope_dtype):
    """q fp32 [T, H * (dim + rot_dim)] -> (unrotated parts [T, H * dim] in nope_dtype, attention query fp32 [T, H * (kv_rank +
    rot_dim)] whose last rot_dim columns per head hold the rotated part; the first kv_rank are left for the absorbing GEMM)."""
    _cuda(q, cos, sin)
    _f32(q, cos, sin)
    t = q.shape[0]
    nope = torch.empty((t, heads * dim), dtype=nope_dtype, device=q.device)
    q_att = torch.empty((t, heads * (kv_rank + rot_dim)), dtype=torch.float32, device=q.device)
    with _k("latent_q_prep"):
        check(_cabi.load().b200_latent_q_prep(_ptr(q), q.stride(0), heads, dim, rot_dim, rot_n, kv_rank, _ptr(cos), _ptr(sin),
                                              _ptr(meta.tok_pos), _ptr(nope), _edt(nope), _ptr(q_att), t, _stream()),
              "b200_latent_q_prep")
    return nope, q_att


# ------------------------------------------------------------------ parallel-branch decoders (grouped norm, rotating attention variants)
def add_group_rmsnorm(x, y1, y2, w, groups: int, eps: float, out_dtype=None):
    """x += y1 + y2 (fp32 rows, any pitch; y2 or both may be None), in place; returns the grouped RMS norm of x times w in
    out_dtype (each of the `groups` equal consecutive parts of a row divided by its own RMS), or None when out_dtype is None."""
    _cuda(x, y1, y2, w)
    _f32(x, w)
    t, width = x.shape
    for y in (y1, y2):
        assert y is None or (y.dtype == torch.float32 and y.stride(1) == 1 and y.shape == (t, width))
    out = torch.empty((t, width), dtype=out_dtype, device=x.device) if out_dtype is not None else None
    with _k("add_group_rmsnorm"):
        check(_cabi.load().b200_add_group_rmsnorm(_ptr(x), _ptr(y1), y1.stride(0) if y1 is not None else 0, _ptr(y2),
                                                  y2.stride(0) if y2 is not None else 0, _ptr(w), int(groups), float(eps), _ptr(out),
                                                  _edt(out) if out is not None else F32, t, width, _stream()), "b200_add_group_rmsnorm")
    return out


def poly_norm(src, col0: int, n: int, coef, eps: float, out_dtype):
    """Columns [col0, col0 + n) of the fp32 rows src -> a N(z) + b N(z^2) + c N(z^3) + e [T, n] in out_dtype; coef fp32 [4] =
    (a, b, c, e); N divides a row by its RMS."""
    _cuda(src, coef)
    _f32(coef)
    assert src.dtype == torch.float32 and src.stride(1) == 1 and coef.numel() == 4
    t = src.shape[0]
    out = torch.empty((t, n), dtype=out_dtype, device=src.device)
    with _k("poly_norm"):
        check(_cabi.load().b200_poly_norm(_ptr(src), src.stride(0), col0, n, _ptr(coef), float(eps), _ptr(out), _edt(out), n, t,
                                          _stream()), "b200_poly_norm")
    return out


def diff_head_norm_gate(a, lam: float, post: float, gate_src, gate_col0: int, eps: float, heads: int, rep: int, out_dtype):
    """a fp32 [T, 2 * heads * P] (per kv group of `rep` heads: the first maps' rows, then the second maps') ->
    [T, heads * P] = unit-RMS(a1 - lam * a2) * post * sigmoid(gate), gate = columns gate_col0.. of the fp32 rows gate_src
    (None: no gate)."""
    _cuda(a, gate_src)
    _f32(a)
    assert gate_src is None or (gate_src.dtype == torch.float32 and gate_src.stride(1) == 1)
    t = a.shape[0]
    p = a.shape[1] // (2 * heads)
    out = torch.empty((t, heads * p), dtype=out_dtype, device=a.device)
    with _k("diff_head_norm_gate"):
        check(_cabi.load().b200_diff_head_norm_gate(_ptr(a), float(lam), float(post), _ptr(gate_src),
                                                    gate_src.stride(0) if gate_src is not None else 0, gate_col0, float(eps),
                                                    _ptr(out), _edt(out), t, heads, rep, p, _stream()), "b200_diff_head_norm_gate")
    return out


def qk_norm_rope_kv_write(src, q_col0: int, k_col0: int, v_col0: int, heads: int, k_pool, v_pool, meta, *, q_norm=None,
                          k_norm=None, eps: float = 0.0, rot_n: int = 0, rot_half: bool = True, cos=None, sin=None, q_head_scale=None):
    """fp32 rows src = [.. q: heads * D .. k: G * D .. v: Gv * Dv ..] -> q fp32 [T, heads * D] (normed over the whole projection
    when q_norm is given, leading rot_n columns of every head rotated by the token's position), and the step's keys (same
    treatment) and values written into the pools [num_blocks, G, block_size, D] / [num_blocks, Gv, block_size, Dv].
    q_head_scale fp32 [heads]: q of head h is multiplied by it (a per-head temperature of the scores)."""
    _cuda(src, k_pool, v_pool, q_norm, k_norm, cos, sin, q_head_scale)
    _f32(q_norm, k_norm, cos, sin, q_head_scale)
    assert q_head_scale is None or q_head_scale.numel() == heads
    assert src.dtype == torch.float32 and src.stride(1) == 1 and k_pool.dtype == v_pool.dtype
    assert k_pool.is_contiguous() and v_pool.is_contiguous()
    _, g, bs, d = k_pool.shape
    _, gv, _, dv = v_pool.shape
    assert rot_n == 0 or (cos.shape[1] == rot_n // 2 and sin.shape == cos.shape)
    t = src.shape[0]
    q = torch.empty((t, heads * d), dtype=torch.float32, device=src.device)
    with _k("qk_norm_rope_kv_write"):
        check(_cabi.load().b200_qk_norm_rope_kv_write(_ptr(src), src.stride(0), q_col0, k_col0, v_col0, _ptr(q_norm), _ptr(k_norm),
                                                      float(eps), int(rot_n), 1 if rot_half else 0, _ptr(cos), _ptr(sin),
                                                      _ptr(meta.tok_pos), _ptr(meta.slot_mapping), _ptr(q), _ptr(k_pool),
                                                      _ptr(v_pool), _edt(k_pool), t, heads, g, gv, d, dv, bs, _ptr(q_head_scale),
                                                      _stream()),
              "b200_qk_norm_rope_kv_write")
    return q


# ------------------------------------------------------------------ dual-norm parallel decoders (window + pooled-block attention
# beside a gated linear recurrence)
def embed_rmsnorm(tokens, table, w, eps: float):
    """tokens int32 [T] -> fp32 [T, W] = RMS norm of table[token], times w."""
    _cuda(tokens, table, w)
    _f32(w)
    assert tokens.dtype == torch.int32 and table.is_contiguous()
    t, (v, width) = tokens.numel(), table.shape
    out = torch.empty((t, width), dtype=torch.float32, device=table.device)
    with _k("embed_rmsnorm"):
        check(_cabi.load().b200_embed_rmsnorm(_ptr(tokens), _ptr(table), _edt(table), _ptr(w), float(eps), _ptr(out), t, width, v,
                                              _stream()), "b200_embed_rmsnorm")
    return out


def scaled_add_rmsnorm2(x, eps: float, *, y1=None, c1: float = 1.0, y2=None, c2: float = 1.0, y3=None, nsum: int = 1, y3_weight=None,
                        c3: float = 1.0, add_rows=None, add_vec=None, w1=None, w2=None, out_dtype=None):
    """x += c1 y1 + c2 y2 + c3 sum_k y3_weight[t, k] y3[t nsum + k] + add_rows + add_vec, in place (fp32; every term optional);
    returns (RMS norm of x times w1, the same times w2) in out_dtype, None for a weight that is not given."""
    _cuda(x, y1, y2, y3, y3_weight, add_rows, add_vec, w1, w2)
    _f32(x, y3, y3_weight, add_rows, add_vec, w1, w2)
    t, width = x.shape
    for y in (y1, y2):
        assert y is None or (y.dtype == torch.float32 and y.stride(1) == 1 and y.shape == (t, width))
    assert y3 is None or (y3.shape == (t * nsum, width) and (y3_weight is None or y3_weight.numel() == t * nsum))
    assert add_rows is None or add_rows.shape == (t, width)
    assert add_vec is None or add_vec.numel() == width
    o1 = torch.empty((t, width), dtype=out_dtype, device=x.device) if w1 is not None else None
    o2 = torch.empty((t, width), dtype=out_dtype, device=x.device) if w2 is not None else None
    with _k("scaled_add_rmsnorm2"):
        check(_cabi.load().b200_scaled_add_rmsnorm2(_ptr(x), _ptr(y1), y1.stride(0) if y1 is not None else 0, float(c1), _ptr(y2),
                                                    y2.stride(0) if y2 is not None else 0, float(c2), _ptr(y3), int(nsum),
                                                    _ptr(y3_weight), float(c3), _ptr(add_rows), _ptr(add_vec), _ptr(w1), _ptr(o1),
                                                    _ptr(w2), _ptr(o2), float(eps), _edt(out_dtype) if out_dtype is not None else F32,
                                                    t, width, _stream()), "b200_scaled_add_rmsnorm2")
    return o1, o2


def kv_pool_mean(k_pool, v_pool, pk_pool, pv_pool, block_table, meta, pool: int):
    """For every block of `pool` positions that the step's portions close: the mean of the block's cached key rows and value rows
    -> the pooled pools [num_blocks, G, ceil(block_size / pool), D | Dv] (entry of a block: page of its last position)."""
    _cuda(k_pool, v_pool, pk_pool, pv_pool, block_table)
    _, g, bs, d = k_pool.shape
    _, gv, _, dv = v_pool.shape
    ppb = -(-bs // pool)
    assert pk_pool.shape == (k_pool.shape[0], g, ppb, d) and pv_pool.shape == (v_pool.shape[0], gv, ppb, dv)
    assert pk_pool.dtype == k_pool.dtype == v_pool.dtype == pv_pool.dtype and pk_pool.is_contiguous() and pv_pool.is_contiguous()
    assert block_table.dtype == torch.int32 and block_table.stride(1) == 1
    with _k("kv_pool_mean"):
        check(_cabi.load().b200_kv_pool_mean(_ptr(k_pool), _ptr(v_pool), _ptr(pk_pool), _ptr(pv_pool), _edt(k_pool), _ptr(block_table),
                                             block_table.stride(0), _ptr(meta.seq_start), _ptr(meta.seq_slot), _ptr(meta.seq_pos0),
                                             meta.num_seqs, meta.num_tokens, g, gv, d, dv, bs, int(pool), _stream()),
              "b200_kv_pool_mean")


_GATED_SEGS = {"0": False, "1": True}.get(os.environ.get("B200_GATED_SEGS", ""))
GATED_SEGS_MAX_CTAS = 600  # whole-portion CTAs (16 value columns x head x sequence; about four per SM) below which long portions run as segments


def gated_scan(proj, q_col0: int, f_col0: int, v_col0: int, f_bias, lower, state, meta, heads: int, dim: int, vdim: int):
    """Gated linear recurrence S <- diag(f) S + (1 - f) v^T, o = S^T q per head over a ragged batch.  Raw q / f / v are the columns
    q_col0 / f_col0 / v_col0 of the fp32 rows proj; q = silu(raw), f = lower + (1 - lower) sigmoid(raw + f_bias) are written back
    IN PLACE.  state fp32 [slots, H, vdim, dim] (transposed) updated in place; returns o fp32 [T, H * vdim].  When the step
    carries a segment list (meta.scan_segs: some portion is long) the segments run in parallel from start states that an
    elementwise pass chains together."""
    _cuda(proj, f_bias, lower, state)
    _f32(f_bias, lower, state)
    assert proj.dtype == torch.float32 and proj.stride(1) == 1 and state.shape[1:] == (heads, vdim, dim)
    assert f_bias.numel() == heads * dim == lower.numel()
    t = proj.shape[0]
    out = torch.empty((t, heads * vdim), dtype=torch.float32, device=proj.device)
    lib = _cabi.load()
    with _k("gated_scan_prep"):
        check(lib.b200_gated_scan_prep(_ptr(proj), proj.stride(0), q_col0, f_col0, heads * dim, _ptr(f_bias), _ptr(lower), t,
                                       _stream()), "b200_gated_scan_prep")
    segs = getattr(meta, "scan_segs", None)
    nseg = meta.num_segs if segs is not None else 0
    if _GATED_SEGS is not None:  # A/B aid: B200_GATED_SEGS=0 never cuts portions, =1 always does when the step has a list
        nseg = nseg if _GATED_SEGS else 0
    elif -(-vdim // 16) * heads * meta.num_seqs >= GATED_SEGS_MAX_CTAS:
        nseg = 0  # whole portions already give every SM its CTAs: the two passes of the segment scheme would only add work
    seg_state = seg_decay = None
    if nseg:
        seg_state = torch.empty((nseg, heads, vdim, dim), dtype=torch.float32, device=proj.device)
        seg_decay = torch.empty((nseg, heads, dim), dtype=torch.float32, device=proj.device)
    with _k("gated_scan"):
        check(lib.b200_gated_scan(_ptr(proj), proj.stride(0), q_col0, f_col0, v_col0, _ptr(state), _ptr(meta.seq_start),
                                  _ptr(meta.seq_slot), _ptr(meta.seq_pos0), _ptr(out), meta.num_seqs, heads, dim, vdim,
                                  _ptr(segs) if nseg else 0, nseg, _ptr(meta.scan_seq_seg0) if nseg else 0, _ptr(seg_state),
                                  _ptr(seg_decay), _stream()), "b200_gated_scan")
    return out
