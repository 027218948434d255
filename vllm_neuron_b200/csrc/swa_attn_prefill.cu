// Tensor-core prompt-portion kernel of the sliding-window sink attention (bf16 pools): same contract as swa_sink_attn in
// swa_attn.cu -- a query at position i attends keys i - window < j <= i through its block table, the softmax starts
// from the per-head sink (running maximum = sink, denominator = 1, no value; none when sink == NULL) -- computed
// FlashAttention-style.  Value rows have pitch v_pitch (the value pool may alias the leading columns of the key pool).
//   CTA = PF_ROWS (64) consecutive new tokens of one sequence x one query head, a warp per 16 rows.  Keys are walked in tiles of 32
//   from the first key the tile's first row may see to the last key its last row may see; each tile's K and V rows are
//   gathered page by page into shared memory with cp.async, one tile ahead of the MMAs (rows padded by 16 bytes:
//   conflict-free ldmatrix), S = Q K^T and O += P V run
//   on mma.sync m16n8k16 (bf16 in, fp32 accumulate); the mask is applied per element, the online softmax is fp32.
// The variants of the warp kernel are parameters here too: a chunked mask, a soft cap on the scaled score, sigmoid weights with a
// per-head bias (no maximum, no denominator), key heads that share a value head, fp32 output rows.  split_p keeps the weights'
// precision through the tensor cores: P = hi + lo with hi = bf16(P), lo = bf16(P - hi), and O += hi V + lo V (the weights then
// carry 16 mantissa bits instead of 8; the denominators are summed in fp32 either way).
// Needs D % 16 == 0 and Dv % 16 == 0, Dv <= 256; other shapes, fp32 pools and decode-sized steps use the warp kernel.
#include <math.h>

#include "hybrid_common.cuh"

namespace b200 {

constexpr int PF_ROWS = 64;
constexpr int PF_THREADS = PF_ROWS * 2;  // a warp per 16 query rows
constexpr int PF_KEYS = 32;
constexpr int PF_NT = PF_KEYS / 8;  // n8 score tiles per key tile
constexpr int LDT_KEYS = 32;  // keys per warp tile of the decode-sized kernel
constexpr int PF_STAGES = 2;  // ring of K / V tiles: the next tile's cp.async copies run under the current tile's MMAs (a third
                              // stage costs a resident CTA per SM and measured slower)

template <int DV16M>  // accumulator capacity: Dv <= 16 * DV16M
__global__ void __launch_bounds__(PF_THREADS, DV16M <= 8 ? 512 / PF_THREADS : 256 / PF_THREADS)
    swa_sink_prefill_kernel(const float* __restrict__ q, int ldq, const __nv_bfloat16* __restrict__ k_pool,
                            const __nv_bfloat16* __restrict__ v_pool, const int32_t* __restrict__ block_table, int64_t bt_stride,
                            const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_slot,
                            const int32_t* __restrict__ seq_pos0, const float* __restrict__ sink, float scale, int window,
                            void* __restrict__ out, int H, int G, int D, int Dv, int bs, int v_pitch, int chunk, float softcap,
                            const float* __restrict__ sig_bias, int v_div, int out_f32, int split_p, int bs_shift,
                            const __nv_bfloat16* __restrict__ pk_pool, const __nv_bfloat16* __restrict__ pv_pool, int pool, int ppb) {
  griddep_wait();
  // the last rows of a portion see the most keys: their tiles are launched first, so the longest CTAs do not form the tail
  const int sq = blockIdx.z, h = blockIdx.y, i0 = (gridDim.x - 1 - blockIdx.x) * PF_ROWS;
  const int t0 = seq_start[sq], n = seq_start[sq + 1] - t0;
  if (i0 >= n) return;
  extern __shared__ __align__(16) unsigned char smraw[];
  // values that are the leading columns of the key rows (one pool for both) are read from the key tile: no second copy
  const bool v_alias = v_pool == k_pool;
  const int ldk = D + 8, ldv = v_alias ? ldk : Dv + 8;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smraw);  // [64][ldk]
  __nv_bfloat16* Ks0 = Qs + PF_ROWS * ldk;                      // [PF_STAGES][32][ldk]
  __nv_bfloat16* Vs0 = v_alias ? Ks0 : Ks0 + PF_STAGES * PF_KEYS * ldk;  // [PF_STAGES][32][ldv]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = h / (H / G);
  const int Gv = G / v_div, gv = g / v_div;
  const bool sig = sig_bias != nullptr;
  const float sb = sig ? sig_bias[h] : 0.f;
  const float inv_cap = softcap > 0.f ? 1.0f / softcap : 0.f;
  const int pos0 = seq_pos0[sq];
  const int32_t* bt = block_table + (int64_t)seq_slot[sq] * bt_stride;
  // ---- Q tile: fp32 rows -> bf16 shared memory (rows past the portion are zero)
  for (int i = tid; i < PF_ROWS * (D / 2); i += PF_THREADS) {
    const int r = i / (D / 2), d = (i - r * (D / 2)) * 2;
    float2 v = make_float2(0.f, 0.f);
    if (i0 + r < n) v = *reinterpret_cast<const float2*>(q + (int64_t)(t0 + i0 + r) * ldq + (int64_t)h * D + d);
    *reinterpret_cast<__nv_bfloat162*>(Qs + r * ldk + d) = __floats2bfloat162_rn(v.x, v.y);
  }
  // rows of this thread's accumulators: r_lo = 16 warp + lane / 4, r_hi = r_lo + 8
  const int r_lo = 16 * warp + (lane >> 2);
  const int p_lo = pos0 + i0 + r_lo, p_hi = p_lo + 8;
  const bool ok_lo = i0 + r_lo < n, ok_hi = i0 + r_lo + 8 < n;
  // first key a position sees: the window's and the chunk's lower bounds (both grow with the position)
  auto lower = [&](int pos) {
    int lb = pos - window + 1 > 0 ? pos - window + 1 : 0;
    if (chunk > 0 && pos - pos % chunk > lb) lb = pos - pos % chunk;
    return lb;
  };
  const int lb_lo = lower(p_lo), lb_hi = lower(p_hi);
  const int w_first = pos0 + i0 + 16 * warp, w_lb = lower(w_first + 15);  // the warp's first position, its last row's bound
  float m_lo = sig ? 0.f : sink ? sink[h] : -INFINITY, m_hi = m_lo;
  float l_lo = sink && (lane & 3) == 0 ? 1.0f : 0.f, l_hi = l_lo;  // the sink's share of the denominator, counted once per row
  float o[2 * DV16M][4];
#pragma unroll
  for (int j = 0; j < 2 * DV16M; ++j)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[j][c] = 0.f;
  const int first_pos = pos0 + i0;
  const int last_row = (n - i0 < PF_ROWS ? n - i0 : PF_ROWS) - 1;
  int j_lo = first_pos - window + 1 > 0 ? first_pos - window + 1 : 0;
  if (chunk > 0 && first_pos - first_pos % chunk > j_lo) j_lo = first_pos - first_pos % chunk;
  const int j_hi = first_pos + last_row;  // inclusive
  const int kch = D / 8, vch = v_alias ? 0 : Dv / 8;  // 16-byte chunks per row
  // one tile of 32 keys (K and V rows, page by page through the block table) into stage `st`; rows past j_hi are zeros.
  // Four threads share a row and take its 16-byte chunks in turn, so the page look-up happens once per thread and tile.
  constexpr int TPR = PF_THREADS / PF_KEYS;
  const int ir = tid / TPR, ic = tid % TPR;
  // Pooled blocks (pool > 0): block b of `pool` positions is one key / value for the rows that have it wholly before their
  // window, b pool + pool - 1 <= position - window; its row sits in the pooled pools, in the page of the block's last position.
  // The CTA's tile list is the pooled entries its LAST row sees (32 per tile), then the key positions as before; tile `it`
  // of the list is pooled while it < npt.
  const int nb_max = pool > 0 && j_hi - window + 1 > 0 ? (j_hi - window + 1) / pool : 0;
  const int npt = (nb_max + PF_KEYS - 1) / PF_KEYS;
  const int j_first = (j_lo / PF_KEYS) * PF_KEYS;
  const int ntiles = npt + (j_hi - j_first) / PF_KEYS + 1;
  // the page of this thread's row in tile `it` (looked up one tile before the copies that need it are issued)
  auto page_of = [&](int it) -> int64_t {
    if (it < npt) {
      const int b = it * PF_KEYS + ir;
      if (b >= nb_max) return 0;
      const int e = b * pool + pool - 1;
      return bt[bs_shift >= 0 ? e >> bs_shift : e / bs];
    }
    const int j = j_first + (it - npt) * PF_KEYS + ir;
    if (it >= ntiles || j > j_hi) return 0;
    return bt[bs_shift >= 0 ? j >> bs_shift : j / bs];
  };
  auto issue = [&](int it, int st, int64_t blk) {
    if (it < ntiles) {
      const __nv_bfloat16 *kr, *vr;
      bool ok;
      if (it < npt) {
        const int b = it * PF_KEYS + ir;
        ok = b < nb_max;
        const int e = b * pool + pool - 1;
        const int idx = ok ? (bs_shift >= 0 ? e & (bs - 1) : e % bs) / pool : 0;
        kr = pk_pool + ((blk * G + g) * ppb + idx) * D;
        vr = pv_pool + ((blk * Gv + gv) * ppb + idx) * Dv;
      } else {
        const int j = j_first + (it - npt) * PF_KEYS + ir;
        ok = j <= j_hi;
        const int off = ok ? (bs_shift >= 0 ? j & (bs - 1) : j % bs) : 0;
        kr = k_pool + ((blk * G + g) * bs + off) * D;
        vr = v_pool + ((blk * Gv + gv) * bs + off) * v_pitch;
      }
      const uint32_t kd = smem_u32(Ks0 + (st * PF_KEYS + ir) * ldk), vd = smem_u32(Vs0 + (st * PF_KEYS + ir) * ldv);
      for (int c = ic; c < kch; c += TPR) cp_async16(kd + c * 16, kr + c * 8, ok);
      for (int c = ic; c < vch; c += TPR) cp_async16(vd + c * 16, vr + c * 8, ok);
    }
    cp_async_commit();  // an empty group past the last tile keeps the wait counts uniform
  };
  static_assert(PF_STAGES == 2, "the page look-ahead below is written for two stages");
  issue(0, 0, page_of(0));
  int64_t blk_next = page_of(1);
  for (int it = 0; it < ntiles; ++it) {
    const int st = it % PF_STAGES;
    const bool ptile = it < npt;
    // first key position of a window tile, first pooled block of a pooled tile
    const int j0 = ptile ? it * PF_KEYS : j_first + (it - npt) * PF_KEYS;
    // refill the stage that the barrier at the end of the previous tile released, then wait for this tile's group
    issue(it + 1, (it + 1) % PF_STAGES, blk_next);
    blk_next = page_of(it + 2);
    cp_async_wait<PF_STAGES - 1>();
    __syncthreads();  // this tile's copies of every thread have landed (and, first time, Q is written)
    const __nv_bfloat16* Ks = Ks0 + st * PF_KEYS * ldk;
    const __nv_bfloat16* Vs = Vs0 + st * PF_KEYS * ldv;
    // ---- S = Q K^T: 16 rows x 32 keys per warp
    float s[PF_NT][4];
#pragma unroll
    for (int j = 0; j < PF_NT; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[j][c] = 0.f;
#pragma unroll 2
    for (int kk = 0; kk < D; kk += 16) {
      uint32_t af[4];
      ldmatrix_x4(af, smem_u32(Qs + (16 * warp + (lane & 15)) * ldk + kk + (lane >> 4) * 8));
#pragma unroll
      for (int jp = 0; jp < PF_NT / 2; ++jp) {
        uint32_t bf[4];
        const int mi = lane >> 3;
        ldmatrix_x4(bf, smem_u32(Ks + (16 * jp + (mi >> 1) * 8 + (lane & 7)) * ldk + kk + (mi & 1) * 8));
        mma_bf16_16816(s[2 * jp], af, bf[0], bf[1]);
        mma_bf16_16816(s[2 * jp + 1], af, bf[2], bf[3]);
      }
    }
    // ---- mask, online softmax (fp32).  A tile that every row of the warp sees whole (all its keys at or before the warp's
    // first row, none before the lower bound of its last row; the bounds grow with the position) skips the per-element mask
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
    // (a pooled tile: every block of it wholly before the window of the warp's first row)
    const bool whole = ptile ? (j0 + PF_KEYS) * pool - 1 <= w_first - window : j0 + PF_KEYS - 1 <= w_first && j0 >= w_lb;
    if (whole && !sig && softcap <= 0.f) {
#pragma unroll
      for (int j = 0; j < PF_NT; ++j) {
        s[j][0] *= scale, s[j][1] *= scale, s[j][2] *= scale, s[j][3] *= scale;
        mx_lo = fmaxf(mx_lo, fmaxf(s[j][0], s[j][1]));
        mx_hi = fmaxf(mx_hi, fmaxf(s[j][2], s[j][3]));
      }
    } else {
#pragma unroll
      for (int j = 0; j < PF_NT; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int key = j0 + 8 * j + 2 * (lane & 3) + (c & 1);
          const bool hi = c >= 2;
          const int pos = hi ? p_hi : p_lo;
          const bool seen = whole || ((hi ? ok_hi : ok_lo) && (ptile ? key * pool + pool - 1 <= pos - window
                                                                            : key <= pos && key >= (hi ? lb_hi : lb_lo)));
          float v = s[j][c] * scale;
          // tanh(x) = 1 - 2 / (1 + e^(2x)): absolute error ~1e-7, so the capped score is good to ~1e-7 of the cap
          if (softcap > 0.f) v = softcap * (1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * v * inv_cap)));
          if (sig) v = seen ? __fdividef(1.0f, 1.0f + __expf(-(v + sb))) : 0.f;  // the weight itself
          else if (!seen) v = -INFINITY;
          s[j][c] = v;
          if (hi) mx_hi = fmaxf(mx_hi, v); else mx_lo = fmaxf(mx_lo, v);
        }
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float mn_lo = sig ? 0.f : fmaxf(m_lo, mx_lo), mn_hi = sig ? 0.f : fmaxf(m_hi, mx_hi);
    // a row that has seen no key yet (no sink, every key of the tile masked) keeps m = -inf: nothing to rescale
    const float c_lo = mn_lo == -INFINITY ? 1.0f : __expf(m_lo - mn_lo), c_hi = mn_hi == -INFINITY ? 1.0f : __expf(m_hi - mn_hi);
    m_lo = mn_lo;
    m_hi = mn_hi;
    l_lo *= c_lo;
    l_hi *= c_hi;
    uint32_t pf[PF_NT][2], pr[PF_NT][2];  // P as bf16 pairs: [n8 tile][row half]; pr = what bf16 rounding left over (split_p)
#pragma unroll
    for (int j = 0; j < PF_NT; ++j) {
      float p0, p1, p2, p3;
      if (sig) {
        p0 = s[j][0], p1 = s[j][1], p2 = s[j][2], p3 = s[j][3];
      } else {
        p0 = mn_lo == -INFINITY ? 0.f : __expf(s[j][0] - mn_lo), p1 = mn_lo == -INFINITY ? 0.f : __expf(s[j][1] - mn_lo);
        p2 = mn_hi == -INFINITY ? 0.f : __expf(s[j][2] - mn_hi), p3 = mn_hi == -INFINITY ? 0.f : __expf(s[j][3] - mn_hi);
      }
      l_lo += p0 + p1;
      l_hi += p2 + p3;
      pf[j][0] = pack_bf16(p0, p1);
      pf[j][1] = pack_bf16(p2, p3);
      if (split_p) {
        const float2 h0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pf[j][0]));
        const float2 h1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pf[j][1]));
        pr[j][0] = pack_bf16(p0 - h0.x, p1 - h0.y);
        pr[j][1] = pack_bf16(p2 - h1.x, p3 - h1.y);
      }
    }
    if (c_lo != 1.0f || c_hi != 1.0f) {  // a maximum that did not move leaves the accumulators as they are
#pragma unroll
      for (int j = 0; j < 2 * DV16M; ++j) {
        o[j][0] *= c_lo;
        o[j][1] *= c_lo;
        o[j][2] *= c_hi;
        o[j][3] *= c_hi;
      }
    }
    // ---- O += P V: keys are the contraction (two k16 steps), V rows read transposed
#pragma unroll
    for (int ks = 0; ks < PF_NT / 2; ++ks) {
      const uint32_t af[4] = {pf[2 * ks][0], pf[2 * ks][1], pf[2 * ks + 1][0], pf[2 * ks + 1][1]};
      const uint32_t ar[4] = {pr[2 * ks][0], pr[2 * ks][1], pr[2 * ks + 1][0], pr[2 * ks + 1][1]};
#pragma unroll
      for (int jd = 0; jd < DV16M; ++jd) {
        if (jd * 16 < Dv) {
          uint32_t bf[4];
          const int mi = lane >> 3;
          ldmatrix_x4_trans(bf, smem_u32(Vs + (16 * ks + (mi & 1) * 8 + (lane & 7)) * ldv + jd * 16 + (mi >> 1) * 8));
          mma_bf16_16816(o[2 * jd], af, bf[0], bf[1]);
          mma_bf16_16816(o[2 * jd + 1], af, bf[2], bf[3]);
          if (split_p) {
            mma_bf16_16816(o[2 * jd], ar, bf[0], bf[1]);
            mma_bf16_16816(o[2 * jd + 1], ar, bf[2], bf[3]);
          }
        }
      }
    }
    __syncthreads();  // everyone is done with this stage before the tile after next is copied into it
  }
  // the next kernel of the stream may take SM slots from here on: earlier, its waiting CTAs would displace this kernel's own
  griddep_launch();
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  const float inv_lo = sig ? 1.0f : 1.0f / l_lo, inv_hi = sig ? 1.0f : 1.0f / l_hi;
#pragma unroll
  for (int j = 0; j < 2 * DV16M; ++j) {
    const int d = 8 * j + 2 * (lane & 3);
    if (d < Dv) {
      const int64_t a_lo = ((int64_t)(t0 + i0 + r_lo) * H + h) * Dv + d, a_hi = a_lo + (int64_t)8 * H * Dv;
      if (out_f32) {
        if (ok_lo) *reinterpret_cast<float2*>(reinterpret_cast<float*>(out) + a_lo) = make_float2(o[j][0] * inv_lo, o[j][1] * inv_lo);
        if (ok_hi) *reinterpret_cast<float2*>(reinterpret_cast<float*>(out) + a_hi) = make_float2(o[j][2] * inv_hi, o[j][3] * inv_hi);
      } else {
        if (ok_lo)
          *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(out) + a_lo) =
              __floats2bfloat162_rn(o[j][0] * inv_lo, o[j][1] * inv_lo);
        if (ok_hi)
          *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(out) + a_hi) =
              __floats2bfloat162_rn(o[j][2] * inv_hi, o[j][3] * inv_hi);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Decode-sized steps on the tensor cores (bf16 pools): one CTA per (token, kv head, block of up to 16 of its query heads).  The
// query heads that share the kv head are the ROWS of the m16 MMA tile, so a key or value row is fetched once for all of them;
// the CTA's warps take the visible keys in tiles of 32 round-robin, each gathering its tile into its own shared-memory buffer
// with cp.async (a whole tile in flight per warp: the launch is bound by memory latency, not by arithmetic), and merge through
// shared memory.  gridDim.y CTAs may split the keys further; their partial results go to `part` (attn_split_merge_kernel).
// Same variants as the kernels above.
constexpr int DT_WARPS = 4;
constexpr int DT_SLOTS = 3;  // 16-byte chunks per lane and tile row: (512 key + 256 value columns) / 8 / 32

template <int DV16M>
__global__ void __launch_bounds__(DT_WARPS * 32)
    swa_sink_decode_tc_kernel(const float* __restrict__ q, int ldq, const __nv_bfloat16* __restrict__ k_pool,
                              const __nv_bfloat16* __restrict__ v_pool, const int32_t* __restrict__ block_table, int64_t bt_stride,
                              const int32_t* __restrict__ tok_row, const int32_t* __restrict__ tok_pos,
                              const float* __restrict__ sink, float scale, int window, void* __restrict__ out, int H, int G, int D,
                              int Dv, int bs, int v_pitch, int chunk, float softcap, const float* __restrict__ sig_bias, int v_div,
                              int out_f32, int split_p, float* __restrict__ part, const __nv_bfloat16* __restrict__ pk_pool,
                              const __nv_bfloat16* __restrict__ pv_pool, int pool, int ppb) {
  griddep_wait();
  extern __shared__ __align__(16) unsigned char dt_sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.y, splits = gridDim.y;
  // The v_div key heads that share a value head (several score maps over the same values) are served by ONE CTA: a key row of
  // the tile is their rows side by side (width v_div * D) and a query row is zero outside its own key head's columns, so the
  // values are fetched once for all maps.  rep = query heads per VALUE head; they are consecutive heads.
  const int Gv = G / v_div, rep = H / Gv, hbn = (rep + 15) / 16, per_key = H / G;
  const int hb = blockIdx.x % hbn, gv = (blockIdx.x / hbn) % Gv, t = blockIdx.x / (hbn * Gv);
  const int h0 = gv * rep + hb * 16, nrow = rep - hb * 16 < 16 ? rep - hb * 16 : 16;  // this CTA's heads h0 .. h0 + nrow
  const int Dk = v_div * D;
  const bool sig = sig_bias != nullptr;
  const float inv_cap = softcap > 0.f ? 1.0f / softcap : 0.f;
  const int ldk = Dk + 8, ldv = Dv + 8, wbuf = LDT_KEYS * (ldk + ldv);
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(dt_sm);             // [16][ldk]
  __nv_bfloat16* Kt = Qs + 16 * ldk + (size_t)warp * wbuf;                  // this warp's [32][ldk] keys, then [32][ldv] values
  __nv_bfloat16* Vt = Kt + LDT_KEYS * ldk;
  float* ml = reinterpret_cast<float*>(Qs + 16 * ldk + (size_t)DT_WARPS * wbuf);  // [warps][16][2]
  const int pos = tok_pos[t];
  const int32_t* bt = block_table + (int64_t)tok_row[t] * bt_stride;
  for (int i = threadIdx.x; i < 16 * (Dk / 2); i += DT_WARPS * 32) {
    const int r = i / (Dk / 2), d = (i - r * (Dk / 2)) * 2;
    const int mine = (hb * 16 + r) / per_key;  // which of the CTA's key heads row r belongs to
    float2 v = make_float2(0.f, 0.f);
    if (r < nrow && d / D == mine) v = *reinterpret_cast<const float2*>(q + (int64_t)t * ldq + (int64_t)(h0 + r) * D + (d - mine * D));
    *reinterpret_cast<__nv_bfloat162*>(Qs + r * ldk + d) = __floats2bfloat162_rn(v.x, v.y);
  }
  __syncthreads();
  int lo = pos - window + 1 > 0 ? pos - window + 1 : 0;
  if (chunk > 0 && pos - pos % chunk > lo) lo = pos - pos % chunk;
  const int r_lo = lane >> 2;
  const bool ok_lo = r_lo < nrow, ok_hi = r_lo + 8 < nrow;
  const float sb_lo = sig && ok_lo ? sig_bias[h0 + r_lo] : 0.f, sb_hi = sig && ok_hi ? sig_bias[h0 + r_lo + 8] : 0.f;
  float m_lo = sig ? 0.f : sink && ok_lo ? sink[h0 + r_lo] : -INFINITY;
  float m_hi = sig ? 0.f : sink && ok_hi ? sink[h0 + r_lo + 8] : -INFINITY;
  const bool count_sink = sink && warp == 0 && split == 0 && (lane & 3) == 0;  // the sink's 1 in the denominator, once per row
  float l_lo = count_sink && ok_lo ? 1.0f : 0.f, l_hi = count_sink && ok_hi ? 1.0f : 0.f;
  float o[2 * DV16M][4];
#pragma unroll
  for (int j = 0; j < 2 * DV16M; ++j)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[j][c] = 0.f;
  const int kch = D / 8, kcht = v_div * kch, vch = Dv / 8;  // 16-byte chunks per key head's row, per tile row, per value row
  // the 16-byte chunks of a tile row that this lane copies (the same for every row and tile): key chunk c of key head mp comes
  // from that head's row, bs rows after the first head's
  // source offset of a chunk = block * ch_blk + (row of the block) * ch_row + ch_src elements into ch_pool
  // (pooled blocks, pool > 0: the same chunk of a row of the pooled pools, pages of ppb rows: pc_*)
  bool ch_on[DT_SLOTS];
  int ch_blk[DT_SLOTS], ch_row[DT_SLOTS], ch_src[DT_SLOTS], ch_pitch[DT_SLOTS], pc_blk[DT_SLOTS], pc_row[DT_SLOTS], pc_src[DT_SLOTS];
  uint32_t ch_dst[DT_SLOTS];
  const __nv_bfloat16 *ch_pool[DT_SLOTS], *pc_pool[DT_SLOTS];
#pragma unroll
  for (int sl = 0; sl < DT_SLOTS; ++sl) {
    const int c = lane + 32 * sl;
    const bool key = c < kcht;
    const int mp = key ? c / kch : 0;
    ch_on[sl] = c < kcht + vch;
    ch_row[sl] = key ? D : v_pitch;
    ch_blk[sl] = (key ? G : Gv) * bs * ch_row[sl];
    ch_pool[sl] = key ? k_pool : v_pool;
    ch_src[sl] = key ? (gv * v_div + mp) * bs * D + (c - mp * kch) * 8 : gv * bs * v_pitch + (c - kcht) * 8;
    ch_pitch[sl] = (key ? ldk : ldv) * 2;
    ch_dst[sl] = key ? smem_u32(Kt) + c * 16 : smem_u32(Vt) + (c - kcht) * 16;
    pc_row[sl] = key ? D : Dv;
    pc_blk[sl] = (key ? G : Gv) * ppb * pc_row[sl];
    pc_pool[sl] = key ? pk_pool : pv_pool;
    pc_src[sl] = key ? (gv * v_div + mp) * ppb * D + (c - mp * kch) * 8 : gv * ppb * Dv + (c - kcht) * 8;
  }
  // pooled blocks: block b of `pool` positions is one key / value once it lies wholly before the window,
  // b pool + pool - 1 <= pos - window; the tile list is the pooled entries (32 per tile), then the window's keys
  const int nb = pool > 0 && pos - window + 1 > 0 ? (pos - window + 1) / pool : 0;
  const int npt = (nb + LDT_KEYS - 1) / LDT_KEYS, ntt = (pos - lo) / LDT_KEYS + 1;
  for (int ti = warp + DT_WARPS * split; ti < npt + ntt; ti += DT_WARPS * splits) {
    // ---- this warp's 32 key and value rows -> its buffer (rows past the token's position / the last seen block are zeros)
    const bool ptile = ti < npt;
    const int j0 = ptile ? ti * LDT_KEYS : lo + (ti - npt) * LDT_KEYS;  // first pooled block / first key position of the tile
    const int j_end = ptile ? nb - 1 : pos;                            // last visible one
    const int jm = j0 + lane;
    int my_blk = -1, my_off = 0;
    if (jm <= j_end) {
      if (ptile) {
        const int e = jm * pool + pool - 1;
        my_blk = bt[e / bs];
        my_off = (e % bs) / pool;
      } else {
        my_blk = bt[jm / bs];
        my_off = jm % bs;
      }
    }
    for (int r = 0; r < LDT_KEYS; ++r) {
      const int blk = __shfl_sync(0xffffffffu, my_blk, r), off = __shfl_sync(0xffffffffu, my_off, r);
      const bool ok = blk >= 0;
#pragma unroll
      for (int sl = 0; sl < DT_SLOTS; ++sl) {
        if (ch_on[sl]) {
          const __nv_bfloat16* src = ptile ? pc_pool[sl] + ((int64_t)(ok ? blk : 0) * pc_blk[sl] + (off * pc_row[sl] + pc_src[sl]))
                                           : ch_pool[sl] + ((int64_t)(ok ? blk : 0) * ch_blk[sl] + (off * ch_row[sl] + ch_src[sl]));
          cp_async16(ch_dst[sl] + r * ch_pitch[sl], src, ok);
        }
      }
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncwarp();
    // ---- S = Q K^T: 16 heads x 32 keys
    float s[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[j][c] = 0.f;
#pragma unroll 2
    for (int kk = 0; kk < Dk; kk += 16) {
      uint32_t af[4];
      ldmatrix_x4(af, smem_u32(Qs + (lane & 15) * ldk + kk + (lane >> 4) * 8));
#pragma unroll
      for (int jp = 0; jp < 2; ++jp) {
        uint32_t bf[4];
        const int mi = lane >> 3;
        ldmatrix_x4(bf, smem_u32(Kt + (16 * jp + (mi >> 1) * 8 + (lane & 7)) * ldk + kk + (mi & 1) * 8));
        mma_bf16_16816(s[2 * jp], af, bf[0], bf[1]);
        mma_bf16_16816(s[2 * jp + 1], af, bf[2], bf[3]);
      }
    }
    // ---- mask (every row is the same token: keys lo .. pos are visible), weights in fp32
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int key = j0 + 8 * j + 2 * (lane & 3) + (c & 1);
        const bool hi = c >= 2, seen = key <= j_end;
        float v = s[j][c] * scale;
        if (softcap > 0.f) v = softcap * (1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * v * inv_cap)));
        if (sig) v = seen ? __fdividef(1.0f, 1.0f + __expf(-(v + (hi ? sb_hi : sb_lo)))) : 0.f;
        else if (!seen) v = -INFINITY;
        s[j][c] = v;
        if (hi) mx_hi = fmaxf(mx_hi, v); else mx_lo = fmaxf(mx_lo, v);
      }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float mn_lo = sig ? 0.f : fmaxf(m_lo, mx_lo), mn_hi = sig ? 0.f : fmaxf(m_hi, mx_hi);  // finite: key j0 is visible
    const float c_lo = __expf(m_lo - mn_lo), c_hi = __expf(m_hi - mn_hi);
    m_lo = mn_lo;
    m_hi = mn_hi;
    l_lo *= c_lo;
    l_hi *= c_hi;
    uint32_t pf[4][2], pr[4][2];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float p0, p1, p2, p3;
      if (sig) {
        p0 = s[j][0], p1 = s[j][1], p2 = s[j][2], p3 = s[j][3];
      } else {
        p0 = __expf(s[j][0] - mn_lo), p1 = __expf(s[j][1] - mn_lo), p2 = __expf(s[j][2] - mn_hi), p3 = __expf(s[j][3] - mn_hi);
      }
      l_lo += p0 + p1;
      l_hi += p2 + p3;
      pf[j][0] = pack_bf16(p0, p1);
      pf[j][1] = pack_bf16(p2, p3);
      if (split_p) {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pf[j][0]));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pf[j][1]));
        pr[j][0] = pack_bf16(p0 - a.x, p1 - a.y);
        pr[j][1] = pack_bf16(p2 - b.x, p3 - b.y);
      }
    }
    if (c_lo != 1.0f || c_hi != 1.0f) {
#pragma unroll
      for (int j = 0; j < 2 * DV16M; ++j) {
        o[j][0] *= c_lo;
        o[j][1] *= c_lo;
        o[j][2] *= c_hi;
        o[j][3] *= c_hi;
      }
    }
    // ---- O += P V
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      const uint32_t af[4] = {pf[2 * ks][0], pf[2 * ks][1], pf[2 * ks + 1][0], pf[2 * ks + 1][1]};
      const uint32_t ar[4] = {pr[2 * ks][0], pr[2 * ks][1], pr[2 * ks + 1][0], pr[2 * ks + 1][1]};
#pragma unroll
      for (int jd = 0; jd < DV16M; ++jd) {
        if (jd * 16 < Dv) {
          uint32_t bf[4];
          const int mi = lane >> 3;
          ldmatrix_x4_trans(bf, smem_u32(Vt + (16 * ks + (mi & 1) * 8 + (lane & 7)) * ldv + jd * 16 + (mi >> 1) * 8));
          mma_bf16_16816(o[2 * jd], af, bf[0], bf[1]);
          mma_bf16_16816(o[2 * jd + 1], af, bf[2], bf[3]);
          if (split_p) {
            mma_bf16_16816(o[2 * jd], ar, bf[0], bf[1]);
            mma_bf16_16816(o[2 * jd + 1], ar, bf[2], bf[3]);
          }
        }
      }
    }
    __syncwarp();  // every lane has read the tile before the next one is copied over it
  }
  griddep_launch();
  // ---- merge the warps: each leaves (m, l, O) in its own buffer ([16][Dv] fp32 fits where its 32 key + value rows were)
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  float* Os = reinterpret_cast<float*>(Kt);
#pragma unroll
  for (int j = 0; j < 2 * DV16M; ++j) {
    const int d = 8 * j + 2 * (lane & 3);
    if (d < Dv) {
      Os[r_lo * Dv + d] = o[j][0];
      Os[r_lo * Dv + d + 1] = o[j][1];
      Os[(r_lo + 8) * Dv + d] = o[j][2];
      Os[(r_lo + 8) * Dv + d + 1] = o[j][3];
    }
  }
  if ((lane & 3) == 0) {
    ml[(warp * 16 + r_lo) * 2] = m_lo;
    ml[(warp * 16 + r_lo) * 2 + 1] = l_lo;
    ml[(warp * 16 + r_lo + 8) * 2] = m_hi;
    ml[(warp * 16 + r_lo + 8) * 2 + 1] = l_hi;
  }
  __syncthreads();
  const float* O0 = reinterpret_cast<const float*>(Qs + 16 * ldk);
  const size_t wstride = (size_t)wbuf / 2;  // floats between two warps' buffers
  for (int i = threadIdx.x; i < nrow * Dv; i += DT_WARPS * 32) {
    const int r = i / Dv, d = i - r * Dv;
    float mt = -INFINITY;
#pragma unroll
    for (int w = 0; w < DT_WARPS; ++w) mt = fmaxf(mt, ml[(w * 16 + r) * 2]);
    float lt = 0.f, v = 0.f;
#pragma unroll
    for (int w = 0; w < DT_WARPS; ++w) {
      const float f = mt == -INFINITY ? 0.f : expf(ml[(w * 16 + r) * 2] - mt);  // a warp or a split without keys: m = -inf, l = 0, O = 0
      lt += ml[(w * 16 + r) * 2 + 1] * f;
      v += O0[w * wstride + r * Dv + d] * f;
    }
    const int64_t row = (int64_t)t * H + h0 + r;
    if (splits > 1) {
      float* pp = part + (row * splits + split) * (Dv + 2);
      if (d == 0) pp[0] = mt, pp[1] = lt;
      pp[2 + d] = v;
      continue;
    }
    const float res = sig ? v : v / lt;
    if (out_f32) reinterpret_cast<float*>(out)[row * Dv + d] = res;
    else reinterpret_cast<__nv_bfloat16*>(out)[row * Dv + d] = __float2bfloat16_rn(res);
  }
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_swa_sink_attn_prefill(const float* q, int ldq, const void* k_pool, const void* v_pool, const int32_t* block_table,
                               int64_t bt_stride, const int32_t* seq_start, const int32_t* seq_slot, const int32_t* seq_pos0,
                               int B, int max_new, const float* sink, float scale, int window, void* out, int H, int G, int D,
                               int Dv, int v_pitch, int block_size, int chunk, float softcap, const float* sigmoid_bias, int v_div,
                               int out_f32, int split_p, const void* pooled_k, const void* pooled_v, int pool, void* stream) {
  B200_REQUIRE(pool >= 0 && (pool == 0 || (pooled_k && pooled_v && v_pool != k_pool)), "swa_sink_attn_prefill: blocks of %d need pooled pools", pool);
  const int ppb = pool > 0 ? (block_size + pool - 1) / pool : 0;
  B200_REQUIRE(q && k_pool && v_pool && block_table && seq_start && seq_slot && seq_pos0 && out,
               "swa_sink_attn_prefill: null pointer");
  B200_REQUIRE(H > 0 && G > 0 && H % G == 0 && window >= 1, "swa_sink_attn_prefill: %d query heads over %d kv heads", H, G);
  B200_REQUIRE(chunk >= 0 && v_div >= 1 && G % v_div == 0 && (v_div == 1 || v_pool != k_pool) && !(sigmoid_bias && sink),
               "swa_sink_attn_prefill: chunk %d, %d key heads sharing values by %d", chunk, G, v_div);
  if (D % 16 || Dv % 16 || Dv > 256 || D > 512 || v_pitch % 8 || v_pitch < Dv || (ldq & 1) || ((uintptr_t)q & 7)) {
    set_last_error("swa_sink_attn_prefill: head sizes %d / %d need multiples of 16 (<= 512 / 256)", D, Dv);
    return B200_ERR_UNSUPPORTED;
  }
  if (B <= 0 || max_new <= 0) return B200_OK;
  dim3 grid((max_new + PF_ROWS - 1) / PF_ROWS, H, B);
  const size_t smem = ((size_t)(PF_ROWS + PF_STAGES * PF_KEYS) * (D + 8) + (v_pool == k_pool ? 0 : (size_t)PF_STAGES * PF_KEYS * (Dv + 8))) * 2;
  cudaStream_t st = (cudaStream_t)stream;
  int bs_shift = -1;  // pages of a power of two: shifts instead of divisions in the gather
  for (int k = 0; k < 16; ++k)
    if (block_size == 1 << k) bs_shift = k;
  typedef __nv_bfloat16 BT;
#define PF_LAUNCH(M)                                                                                                          \
  do {                                                                                                                        \
    if (smem > 48 * 1024)                                                                                                     \
      B200_CUDA_OK(cudaFuncSetAttribute(swa_sink_prefill_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    B200_CUDA_OK(launch_kernel(swa_sink_prefill_kernel<M>, grid, dim3(PF_THREADS), smem, st, q, ldq, (const BT*)k_pool,              \
                               (const BT*)v_pool, block_table, bt_stride, seq_start, seq_slot, seq_pos0, sink, scale, window, \
                               out, H, G, D, Dv, block_size, v_pitch, chunk, softcap, sigmoid_bias, v_div, out_f32, split_p, bs_shift, \
                               (const BT*)pooled_k, (const BT*)pooled_v, pool, ppb));                                         \
  } while (0)
  if (Dv <= 64) PF_LAUNCH(4);
  else if (Dv <= 128) PF_LAUNCH(8);
  else PF_LAUNCH(16);
#undef PF_LAUNCH
  return B200_OK;
}

int b200_swa_sink_attn_decode_tc(const float* q, int ldq, const void* k_pool, const void* v_pool, const int32_t* block_table,
                                 int64_t bt_stride, const int32_t* tok_row, const int32_t* tok_pos, const float* sink, float scale,
                                 int window, void* out, int T, int H, int G, int D, int Dv, int v_pitch, int block_size, int chunk,
                                 float softcap, const float* sigmoid_bias, int v_div, int out_f32, int split_p, int splits,
                                 float* split_workspace, const void* pooled_k, const void* pooled_v, int pool, void* stream) {
  B200_REQUIRE(pool >= 0 && (pool == 0 || (pooled_k && pooled_v)), "swa_sink_attn_decode_tc: blocks of %d need pooled pools", pool);
  const int ppb = pool > 0 ? (block_size + pool - 1) / pool : 0;
  B200_REQUIRE(q && k_pool && v_pool && block_table && tok_row && tok_pos && out, "swa_sink_attn_decode_tc: null pointer");
  B200_REQUIRE(H > 0 && G > 0 && H % G == 0 && window >= 1 && chunk >= 0, "swa_sink_attn_decode_tc: %d query heads over %d kv heads", H, G);
  B200_REQUIRE(v_div >= 1 && G % v_div == 0 && !(sigmoid_bias && sink), "swa_sink_attn_decode_tc: %d key heads sharing values by %d", G, v_div);
  B200_REQUIRE(splits >= 1 && splits <= 64 && (splits == 1 || split_workspace), "swa_sink_attn_decode_tc: %d key splits need a workspace", splits);
  if (D % 16 || Dv % 16 || Dv > 256 || D > 512 || v_pitch % 8 || v_pitch < Dv || (ldq & 1) || ((uintptr_t)q & 7) || v_pool == k_pool) {
    set_last_error("swa_sink_attn_decode_tc: head sizes %d / %d need multiples of 16 (<= 512 / 256) and a value pool of its own", D, Dv);
    return B200_ERR_UNSUPPORTED;
  }
  if (T <= 0) return B200_OK;
  const int Gv = G / v_div, rep = H / Gv, Dk = v_div * D;  // query heads per value head; width of a tile's key rows
  if (Dk > 512) {
    set_last_error("swa_sink_attn_decode_tc: %d key heads of %d side by side exceed 512 columns", v_div, D);
    return B200_ERR_UNSUPPORTED;
  }
  dim3 grid((unsigned)(T * Gv * ((rep + 15) / 16)), (unsigned)splits);
  const size_t smem = ((size_t)16 * (Dk + 8) + (size_t)DT_WARPS * LDT_KEYS * (Dk + 8 + Dv + 8)) * 2 + (size_t)DT_WARPS * 16 * 2 * 4;
  cudaStream_t st = (cudaStream_t)stream;
  typedef __nv_bfloat16 BT;
#define DT_LAUNCH(M)                                                                                                            \
  do {                                                                                                                          \
    if (smem > 48 * 1024)                                                                                                       \
      B200_CUDA_OK(cudaFuncSetAttribute(swa_sink_decode_tc_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    B200_CUDA_OK(launch_kernel(swa_sink_decode_tc_kernel<M>, grid, dim3(DT_WARPS * 32), smem, st, q, ldq, (const BT*)k_pool,    \
                               (const BT*)v_pool, block_table, bt_stride, tok_row, tok_pos, sink, scale, window, out, H, G, D,  \
                               Dv, block_size, v_pitch, chunk, softcap, sigmoid_bias, v_div, out_f32, split_p,                  \
                               split_workspace, (const BT*)pooled_k, (const BT*)pooled_v, pool, ppb));                          \
  } while (0)
  if (Dv <= 64) DT_LAUNCH(4);
  else if (Dv <= 128) DT_LAUNCH(8);
  else DT_LAUNCH(16);
#undef DT_LAUNCH
  if (splits > 1)
    return b200_attn_split_merge(split_workspace, splits, Dv, sigmoid_bias ? 1 : 0, out_f32, B200_BF16, out, (int64_t)T * H, stream);
  return B200_OK;
}

}  // extern "C"
