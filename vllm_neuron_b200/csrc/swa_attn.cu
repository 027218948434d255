// Sliding-window attention with a softmax sink over the paged KV pools, for layers whose key and value widths differ
// and whose scores carry no positional rotation.
//   * kv_write_vmix: scatters this step's keys and values into the pools by slot; optionally mixes the value with the
//     value the first value-mixing layer produced for the same token, v + lambda (v_first - v), BEFORE it is
//     cached (what is cached is what every later query reads);
//   * swa_sink_attn: ragged batch, one CTA per (token, up to 4 query heads of one kv head).  A query at position i attends keys i - window < j <= i,
//     read through the sequence's block table.  Online softmax in fp32 that STARTS from the sink: running maximum =
//     sink logit, running denominator = 1, accumulator = 0 -- the sink adds exp(sink) to the denominator once, has no key,
//     no value, and is not multiplied by the score scale.
//     Without a sink (sink == NULL) the softmax is the ordinary one over the visible keys.
//     Variants of the same kernel, all parameters: keys confined to the query's CHUNK of positions (counted from position 0),
//     a soft cap on the scaled score (cap tanh(s / cap)), SIGMOID weights sigmoid(s + bias[head]) that are not normalised
//     over the keys (then no sink, no maximum, no denominator), several key heads sharing one value head (v_div: two score
//     maps over the same values), and fp32 output rows;
//   * qk_norm_rope_kv_write: the step between the projections (or their short convolutions) and the attention of layers
//     that norm and rotate: an optional RMS norm over the WHOLE q (and k) projection, rotary positions from cos / sin tables
//     on the leading columns of every head (pairs (i, i + n/2) or (2i, 2i + 1)), q to an fp32 buffer, k and v into the pools.
// Pools: K [num_blocks][G][block_size][D], V [num_blocks][G][block_size][v_pitch] with values in the first Dv columns of a
// row (v_pitch = Dv for a pool of its own; a value pool may alias the key pool, values = the leading columns of the key
// rows, v_pitch = D: attention over cached latents).
#include <math.h>

#include "hybrid_common.cuh"

namespace b200 {

template <typename KT>
__global__ void kv_write_vmix_kernel(const float* __restrict__ qkv, int ld, int k_col0, int v_col0, float* __restrict__ v_first,
                                     float lam, int mode, KT* __restrict__ k_pool, KT* __restrict__ v_pool,
                                     const int64_t* __restrict__ slots, int G, int D, int Dv, int bs) {
  griddep_launch();
  griddep_wait();
  const int t = blockIdx.x;
  const int64_t slot = slots[t];
  if (slot < 0) return;
  const int64_t blk = slot / bs, off = slot % bs;
  const float* row = qkv + (int64_t)t * ld;
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i - g * D;
    stf(k_pool, ((blk * G + g) * bs + off) * D + d, row[k_col0 + i]);
  }
  for (int i = threadIdx.x; i < G * Dv; i += blockDim.x) {
    const int g = i / Dv, d = i - g * Dv;
    float v = row[v_col0 + i];
    if (mode == 1) v_first[(int64_t)t * G * Dv + i] = v;
    if (mode == 2) v = (1.0f - lam) * v + lam * v_first[(int64_t)t * G * Dv + i];
    stf(v_pool, ((blk * G + g) * bs + off) * Dv + d, v);
  }
}

// One CTA per token.  src fp32 rows hold q [H][D] at q_col0, k [G][D] at k_col0 and v [Gv][Dv] at v_col0.  q and k are
// (optionally) divided by the RMS of their whole projection and multiplied by a weight per column, then the first rot_n
// columns of every head turn by the token's position: column pairs (i, i + rot_n / 2) when rot_half, else (2i, 2i + 1); a pair
// (u, v) becomes (u cos - v sin, v cos + u sin) with cos / sin from fp32 tables [positions][rot_n / 2] (any frequency
// scaling and magnitude factor live in the tables).  q goes to q_out fp32 [T][H * D]; k and v to the pools by slot.
template <typename KT>
__global__ void qk_norm_rope_kv_write_kernel(const float* __restrict__ src, int ld, int q_col0, int k_col0, int v_col0,
                                             const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                                             int rot_n, int rot_half, const float* __restrict__ cos_t,
                                             const float* __restrict__ sin_t, const int32_t* __restrict__ tok_pos,
                                             const int64_t* __restrict__ slots, float* __restrict__ q_out, KT* __restrict__ k_pool,
                                             KT* __restrict__ v_pool, int H, int G, int Gv, int D, int Dv, int bs,
                                             const float* __restrict__ q_head_scale) {
  griddep_launch();
  griddep_wait();
  __shared__ float red[2][33];
  const int t = blockIdx.x;
  const float* row = src + (int64_t)t * ld;
  const int nq = H * D, nk = G * D;
  float inv_q = 1.0f, inv_k = 1.0f;
  if (q_norm || k_norm) {  // sums of squares over the whole projections
    float sq = 0.f, sk = 0.f;
    if (q_norm)
      for (int i = threadIdx.x; i < nq; i += blockDim.x) sq += row[q_col0 + i] * row[q_col0 + i];
    if (k_norm)
      for (int i = threadIdx.x; i < nk; i += blockDim.x) sk += row[k_col0 + i] * row[k_col0 + i];
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    if ((threadIdx.x & 31) == 0) {
      red[0][threadIdx.x >> 5] = sq;
      red[1][threadIdx.x >> 5] = sk;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      const int nw = (blockDim.x + 31) >> 5;
      float a = threadIdx.x < nw ? red[0][threadIdx.x] : 0.f, b = threadIdx.x < nw ? red[1][threadIdx.x] : 0.f;
      a = warp_sum(a);
      b = warp_sum(b);
      if (threadIdx.x == 0) {
        red[0][32] = a;
        red[1][32] = b;
      }
    }
    __syncthreads();
    if (q_norm) inv_q = 1.0f / sqrtf(red[0][32] / (float)nq + eps);
    if (k_norm) inv_k = 1.0f / sqrtf(red[1][32] / (float)nk + eps);
  }
  const int pos = tok_pos[t];
  const int half = rot_n >> 1;
  const float* cs = cos_t + (int64_t)pos * half;
  const float* sn = sin_t + (int64_t)pos * half;
  const int64_t slot = slots[t];
  const int64_t blk = slot / bs, off = slot % bs;
  // the value of column i of a projection after its norm
  auto turned = [&](int col0, const float* nw, float inv, int i) -> float {
    const int d = i % D;
    const float u = row[col0 + i] * (nw ? inv * nw[i] : 1.0f);
    if (d >= rot_n) return u;
    int partner, idx;
    bool first;
    if (rot_half) {
      first = d < half;
      idx = first ? d : d - half;
      partner = first ? i + half : i - half;
    } else {
      first = (d & 1) == 0;
      idx = d >> 1;
      partner = i ^ 1;
    }
    const float o = row[col0 + partner] * (nw ? inv * nw[partner] : 1.0f);
    return first ? u * cs[idx] - o * sn[idx] : u * cs[idx] + o * sn[idx];
  };
  for (int i = threadIdx.x; i < nq; i += blockDim.x)
    q_out[(int64_t)t * nq + i] = turned(q_col0, q_norm, inv_q, i) * (q_head_scale ? q_head_scale[i / D] : 1.0f);
  if (slot < 0) return;
  for (int i = threadIdx.x; i < nk; i += blockDim.x) {
    const int g = i / D, d = i - g * D;
    stf(k_pool, ((blk * G + g) * bs + off) * D + d, turned(k_col0, k_norm, inv_k, i));
  }
  for (int i = threadIdx.x; i < Gv * Dv; i += blockDim.x) {
    const int g = i / Dv, d = i - g * Dv;
    stf(v_pool, ((blk * Gv + g) * bs + off) * Dv + d, row[v_col0 + i]);
  }
}

// The same with four columns per thread and step (16-byte loads; 8- or 16-byte stores): needs every column offset, head size
// and the row pitch in multiples of four, a rotating part whose pairs fall into whole groups of four (rot_n % 8 == 0 for the
// half layout, % 4 for neighbours) and 16-byte aligned bases.  One division per four columns.
template <typename KT>
__global__ void qk_norm_rope_kv_write_vec_kernel(const float* __restrict__ src, int ld, int q_col0, int k_col0, int v_col0,
                                                 const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                                                 int rot_n, int rot_half, const float* __restrict__ cos_t,
                                                 const float* __restrict__ sin_t, const int32_t* __restrict__ tok_pos,
                                                 const int64_t* __restrict__ slots, float* __restrict__ q_out,
                                                 KT* __restrict__ k_pool, KT* __restrict__ v_pool, int H, int G, int Gv, int D, int Dv,
                                                 int bs, const float* __restrict__ q_head_scale) {
  griddep_launch();
  griddep_wait();
  __shared__ float red[2][33];
  const int t = blockIdx.x;
  const float* row = src + (int64_t)t * ld;
  const int nq = H * D, nk = G * D;
  auto ld4 = [](const float* p) { return *reinterpret_cast<const float4*>(p); };
  float inv_q = 1.0f, inv_k = 1.0f;
  if (q_norm || k_norm) {
    float sq = 0.f, sk = 0.f;
    if (q_norm)
      for (int i = threadIdx.x * 4; i < nq; i += blockDim.x * 4) {
        const float4 a = ld4(row + q_col0 + i);
        sq += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
      }
    if (k_norm)
      for (int i = threadIdx.x * 4; i < nk; i += blockDim.x * 4) {
        const float4 a = ld4(row + k_col0 + i);
        sk += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
      }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    if ((threadIdx.x & 31) == 0) {
      red[0][threadIdx.x >> 5] = sq;
      red[1][threadIdx.x >> 5] = sk;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      const int nw = (blockDim.x + 31) >> 5;
      float a = threadIdx.x < nw ? red[0][threadIdx.x] : 0.f, b = threadIdx.x < nw ? red[1][threadIdx.x] : 0.f;
      a = warp_sum(a);
      b = warp_sum(b);
      if (threadIdx.x == 0) {
        red[0][32] = a;
        red[1][32] = b;
      }
    }
    __syncthreads();
    if (q_norm) inv_q = 1.0f / sqrtf(red[0][32] / (float)nq + eps);
    if (k_norm) inv_k = 1.0f / sqrtf(red[1][32] / (float)nk + eps);
  }
  const int pos = tok_pos[t];
  const int half = rot_n >> 1;
  const float* cs = cos_t + (int64_t)pos * half;
  const float* sn = sin_t + (int64_t)pos * half;
  const int64_t slot = slots[t];
  const int64_t blk = slot / bs, off = slot % bs;
  // columns i .. i + 3 of a projection after norm and rotation; d = i % D
  auto normed = [&](int col0, const float* nw, float inv, int i) -> float4 {
    float4 u = ld4(row + col0 + i);
    if (nw) {
      const float4 w = ld4(nw + i);
      u.x *= inv * w.x, u.y *= inv * w.y, u.z *= inv * w.z, u.w *= inv * w.w;
    }
    return u;
  };
  auto turned = [&](int col0, const float* nw, float inv, int i, int d) -> float4 {
    const float4 u = normed(col0, nw, inv, i);
    if (d >= rot_n) return u;
    if (rot_half) {
      const bool first = d < half;
      const int idx = first ? d : d - half;
      const float4 o = normed(col0, nw, inv, first ? i + half : i - half);
      const float4 c = ld4(cs + idx), s = ld4(sn + idx);
      if (first) return make_float4(u.x * c.x - o.x * s.x, u.y * c.y - o.y * s.y, u.z * c.z - o.z * s.z, u.w * c.w - o.w * s.w);
      return make_float4(u.x * c.x + o.x * s.x, u.y * c.y + o.y * s.y, u.z * c.z + o.z * s.z, u.w * c.w + o.w * s.w);
    }
    const int idx = d >> 1;
    const float c0 = cs[idx], s0 = sn[idx], c1 = cs[idx + 1], s1 = sn[idx + 1];
    return make_float4(u.x * c0 - u.y * s0, u.y * c0 + u.x * s0, u.z * c1 - u.w * s1, u.w * c1 + u.z * s1);
  };
  auto put = [](KT* p, float4 v) {
    if constexpr (sizeof(KT) == 2) {
      *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
    } else {
      *reinterpret_cast<float4*>(p) = v;
    }
  };
  for (int i = threadIdx.x * 4; i < nq; i += blockDim.x * 4) {
    float4 r = turned(q_col0, q_norm, inv_q, i, i % D);
    if (q_head_scale) {  // D % 4 == 0: the four columns belong to one head
      const float hs = q_head_scale[i / D];
      r.x *= hs, r.y *= hs, r.z *= hs, r.w *= hs;
    }
    *reinterpret_cast<float4*>(q_out + (int64_t)t * nq + i) = r;
  }
  if (slot < 0) return;
  for (int i = threadIdx.x * 4; i < nk; i += blockDim.x * 4) {
    const int g = i / D, d = i - g * D;
    put(k_pool + ((blk * G + g) * bs + off) * D + d, turned(k_col0, k_norm, inv_k, i, d));
  }
  for (int i = threadIdx.x * 4; i < Gv * Dv; i += blockDim.x * 4) {
    const int g = i / Dv, d = i - g * Dv;
    put(v_pool + ((blk * Gv + g) * bs + off) * Dv + d, ld4(row + v_col0 + i));
  }
}

// Block means for attention that sees far-away blocks of `pool` positions as one key / value each.  One CTA per block that the
// step CLOSES (a portion at positions [p0, p0 + n) closes (p0 + n) / pool - p0 / pool blocks; the launch has T / pool + B CTAs,
// an upper bound, and CTA i finds its (sequence, block) by walking the step's sequences); it reads the block's `pool` key and
// value rows back from the pools through the sequence's block table (rows of earlier steps and of this one alike: what is averaged is what
// the cache holds), sums them in fp32, divides by `pool` and writes the mean into the pooled pools
// PK [num_blocks][G][ppb][D], PV [num_blocks][Gv][ppb][Dv], ppb = ceil(block_size / pool): the entry of block b lives in the page
// that holds the block's last position e, at index (e % block_size) / pool.  Runs after the step's keys and values are written.
constexpr int PM_THREADS = 256;
constexpr int PM_ROWS = 64;  // positions whose rows are looked up per round

template <typename KT>
__global__ void __launch_bounds__(PM_THREADS)
    kv_pool_mean_kernel(const KT* __restrict__ k_pool, const KT* __restrict__ v_pool, KT* __restrict__ pk_pool,
                        KT* __restrict__ pv_pool, const int32_t* __restrict__ block_table, int64_t bt_stride,
                        const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_slot,
                        const int32_t* __restrict__ seq_pos0, int B, int G, int Gv, int D, int Dv, int bs, int pool, int ppb) {
  griddep_launch();
  griddep_wait();
  __shared__ int32_t pg[PM_ROWS], po[PM_ROWS];  // page and offset in the page of the round's positions
  int sq = -1, pos = 0;
  for (int s = 0, acc = 0; s < B; ++s) {  // the same walk in every thread
    const int p0 = seq_pos0[s], n = seq_start[s + 1] - seq_start[s];
    const int cnt = (p0 + n) / pool - p0 / pool;
    if ((int)blockIdx.x < acc + cnt) {
      sq = s;
      pos = (p0 / pool + ((int)blockIdx.x - acc)) * pool + pool - 1;  // the block's last position
      break;
    }
    acc += cnt;
  }
  if (sq < 0) return;
  const int32_t* bt = block_table + (int64_t)seq_slot[sq] * bt_stride;
  const int first = pos - pool + 1;
  const int64_t dst_blk = bt[pos / bs];
  const int dst_idx = (pos % bs) / pool;
  const float inv = 1.0f / (float)pool;
  const int cols = G * D + Gv * Dv;
  // a thread owns columns tid, tid + PM_THREADS, ... (up to 8 of them in registers; wider rows take further passes)
  for (int c0 = 0; c0 < cols; c0 += 8 * PM_THREADS) {
    float acc[8];
    int64_t off[8];  // element offset of the column inside a page, without the row: (g * rows_per_page) * W + d
    int width[8];
    const KT* src[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = c0 + u * PM_THREADS + threadIdx.x;
      const bool key = i < G * D;
      const int c = key ? i : i - G * D, W = key ? D : Dv;
      const int g = c / W, d = c - g * W;
      acc[u] = 0.f;
      width[u] = i < cols ? W : 0;
      src[u] = key ? k_pool : v_pool;
      off[u] = ((int64_t)g * bs) * W + d;
    }
    for (int p0 = first; p0 <= pos; p0 += PM_ROWS) {
      const int np = pos + 1 - p0 < PM_ROWS ? pos + 1 - p0 : PM_ROWS;
      __syncthreads();
      if (threadIdx.x < np) {
        const int p = p0 + threadIdx.x;
        pg[threadIdx.x] = bt[p / bs];
        po[threadIdx.x] = p % bs;
      }
      __syncthreads();
      // eight rows of a column in flight at a time (the index is clamped, so every load is unconditional); summed in order
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (!width[u]) continue;
        const int64_t per_page = (int64_t)(src[u] == k_pool ? G : Gv) * bs;
        for (int k0 = 0; k0 < np; k0 += 8) {
          float v[8];
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const int k = k0 + kk < np ? k0 + kk : np - 1;
            v[kk] = ldf(src[u], (pg[k] * per_page + po[k]) * width[u] + off[u]);
          }
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            if (k0 + kk < np) acc[u] += v[kk];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = c0 + u * PM_THREADS + threadIdx.x;
      if (i >= cols) continue;
      const bool key = i < G * D;
      const int c = key ? i : i - G * D, W = key ? D : Dv, N = key ? G : Gv;
      const int g = c / W, d = c - g * W;
      stf(key ? pk_pool : pv_pool, ((dst_blk * N + g) * ppb + dst_idx) * W + d, acc[u] * inv);
    }
  }
}

constexpr int ATT_WARPS = 16;  // the launch is bound by load latency: every warp walks few key tiles, many are in flight

// QH query rows (fp32, shared memory, pitch D) . one k row, with 16-byte loads when the row allows it: the key row is
// fetched once for all the query heads of its group that the CTA serves
template <int QH>
__device__ __forceinline__ void dot_q_rows_f32(const float* __restrict__ qs, int Dp, const float* __restrict__ kr, int D,
                                               float (&dot)[QH]) {
  if ((D & 3) == 0) {
#pragma unroll 4
    for (int d = 0; d < D; d += 4) {
      const float4 k4 = *reinterpret_cast<const float4*>(kr + d);
#pragma unroll
      for (int q = 0; q < QH; ++q) {
        const float4 q4 = *reinterpret_cast<const float4*>(qs + q * Dp + d);
        dot[q] += q4.x * k4.x + q4.y * k4.y + q4.z * k4.z + q4.w * k4.w;
      }
    }
  } else {
    for (int d = 0; d < D; ++d) {
      const float kv = kr[d];
#pragma unroll
      for (int q = 0; q < QH; ++q) dot[q] += qs[q * Dp + d] * kv;
    }
  }
}
template <int QH>
__device__ __forceinline__ void dot_q_rows_bf16(const float* __restrict__ qs, int Dp, const __nv_bfloat16* __restrict__ kr, int D,
                                                float (&dot)[QH]) {
  if ((D & 7) == 0) {
#pragma unroll 4
    for (int d = 0; d < D; d += 8) {
      const uint4 k8 = *reinterpret_cast<const uint4*>(kr + d);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&k8);
      const float2 f0 = __bfloat1622float2(h2[0]), f1 = __bfloat1622float2(h2[1]), f2 = __bfloat1622float2(h2[2]),
                   f3 = __bfloat1622float2(h2[3]);
#pragma unroll
      for (int q = 0; q < QH; ++q) {
        const float4 qa = *reinterpret_cast<const float4*>(qs + q * Dp + d);
        const float4 qb = *reinterpret_cast<const float4*>(qs + q * Dp + d + 4);
        dot[q] += qa.x * f0.x + qa.y * f0.y + qa.z * f1.x + qa.w * f1.y + qb.x * f2.x + qb.y * f2.y + qb.z * f3.x + qb.w * f3.y;
      }
    }
  } else {
    for (int d = 0; d < D; ++d) {
      const float kv = __bfloat162float(kr[d]);
#pragma unroll
      for (int q = 0; q < QH; ++q) dot[q] += qs[q * Dp + d] * kv;
    }
  }
}
template <typename KT, int QH>
struct DotRows;
template <int QH>
struct DotRows<float, QH> {
  static __device__ __forceinline__ void run(const float* qs, int Dp, const float* kr, int D, float (&dot)[QH]) {
    dot_q_rows_f32<QH>(qs, Dp, kr, D, dot);
  }
};
template <int QH>
struct DotRows<__nv_bfloat16, QH> {
  static __device__ __forceinline__ void run(const float* qs, int Dp, const __nv_bfloat16* kr, int D, float (&dot)[QH]) {
    dot_q_rows_bf16<QH>(qs, Dp, kr, D, dot);
  }
};
// two consecutive elements of a value row (pairs: lane l owns columns 2 l, 2 l + 1 of every 64-column slab)
__device__ __forceinline__ float2 ld_pair(const float* r, int d, int Dv, bool vec) {
  if (vec) return *reinterpret_cast<const float2*>(r + d);
  return make_float2(d < Dv ? r[d] : 0.f, d + 1 < Dv ? r[d + 1] : 0.f);
}
__device__ __forceinline__ float2 ld_pair(const __nv_bfloat16* r, int d, int Dv, bool vec) {
  if (vec) return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(r + d));
  return make_float2(d < Dv ? __bfloat162float(r[d]) : 0.f, d + 1 < Dv ? __bfloat162float(r[d + 1]) : 0.f);
}

// One CTA per (token, QH query heads that share a kv head): its 16 warps take the window's 32-key tiles round-robin
// (lane-per-key scores, lanes-over-columns value accumulation, each warp its own running maximum / denominator /
// accumulator per head) and merge through shared memory.  Every K and V row is fetched once for the QH heads.  Warp 0
// carries the sink's 1 in the denominators.  The split depends on the position and the window only.
// Serves decoded tokens and short portions in both element types, and every shape in 32-bit serving.
template <typename KT, int MAXC, int QH>
__global__ void __launch_bounds__(ATT_WARPS * 32)
    swa_sink_attn_kernel(const float* __restrict__ q, int ldq, const KT* __restrict__ k_pool, const KT* __restrict__ v_pool,
                         const int32_t* __restrict__ block_table, int64_t bt_stride, const int32_t* __restrict__ tok_row,
                         const int32_t* __restrict__ tok_pos, const float* __restrict__ sink, float scale, int window,
                         void* __restrict__ out, int T, int H, int G, int D, int Dv, int bs, int v_pitch, int chunk, float softcap,
                         const float* __restrict__ sig_bias, int v_div, int out_f32, float* __restrict__ part,
                         const KT* __restrict__ pk_pool, const KT* __restrict__ pv_pool, int pool, int ppb) {
  griddep_launch();
  griddep_wait();
  extern __shared__ __align__(16) float sm_att[];
  // gridDim.y CTAs split a (token, head block)'s keys: key tiles go round-robin over (split, warp); with more than one
  // split the CTA leaves its maximum, denominator and unnormalised accumulator in `part` for attn_split_merge_kernel
  const int split = blockIdx.y, splits = gridDim.y;
  const int Dp = (D + 3) & ~3;                    // pitch of a query row: 16-byte aligned rows
  float* qs = sm_att;                             // [QH][Dp]
  float* accs = qs + QH * Dp;                     // [ATT_WARPS][QH][64 MAXC]
  float* ml = accs + ATT_WARPS * QH * 64 * MAXC;  // [ATT_WARPS][QH][2]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hb = H / QH;                          // head blocks per token
  const int t = blockIdx.x / hb, h0 = (blockIdx.x - t * hb) * QH;
  const int g = h0 / (H / G);                     // QH divides H / G: the block's heads share this kv head
  const int Gv = G / v_div, gv = g / v_div;       // v_div key heads read one value head
  const bool sig = sig_bias != nullptr;           // sigmoid weights: no maximum, no denominator
  for (int i = threadIdx.x; i < QH * D; i += ATT_WARPS * 32) {
    const int qh = i / D, d = i - qh * D;
    qs[qh * Dp + d] = q[(int64_t)t * ldq + (int64_t)(h0 + qh) * D + d];
  }
  __syncthreads();
  const int pos = tok_pos[t];
  const int32_t* bt = block_table + (int64_t)tok_row[t] * bt_stride;
  int lo = pos - window + 1 > 0 ? pos - window + 1 : 0;
  if (chunk > 0 && pos - pos % chunk > lo) lo = pos - pos % chunk;  // the first position of the query's chunk
  const bool vvec = (Dv & 1) == 0 && (v_pitch & 1) == 0;
  float m[QH], l[QH];  // the sink: exp(sink - m) = 1 in the denominator, nothing in the numerator
  float2 acc[QH][MAXC];
#pragma unroll
  for (int qh = 0; qh < QH; ++qh) {
    m[qh] = sig ? 0.f : sink ? sink[h0 + qh] : -INFINITY;
    l[qh] = sink && warp == 0 && split == 0 ? 1.0f : 0.f;
#pragma unroll
    for (int c = 0; c < MAXC; ++c) acc[qh][c] = make_float2(0.f, 0.f);
  }
  // pooled blocks: block b (positions b pool .. b pool + pool - 1) is seen as one key / value once it lies wholly before the
  // window, b pool + pool - 1 <= pos - window; its row sits in the page of its last position.  The tile list is the pooled
  // entries (32 per tile) followed by the window's keys.
  const int nb = pool > 0 && pos - window + 1 > 0 ? (pos - window + 1) / pool : 0;
  const int npt = (nb + 31) >> 5, ntt = ((pos - lo) >> 5) + 1;
  for (int ti = warp + ATT_WARPS * split; ti < npt + ntt; ti += ATT_WARPS * splits) {
    const bool pooled = ti < npt;
    const int j = pooled ? ti * 32 + lane : lo + (ti - npt) * 32 + lane;  // pooled block, or key position
    const bool valid = pooled ? j < nb : j <= pos;
    const KT* vrow = v_pool;  // lanes past the last key: row 0 of the pool (the null page, finite values) with weight 0
    float p[QH];
#pragma unroll
    for (int qh = 0; qh < QH; ++qh) p[qh] = 0.f;
    if (valid) {
      if (pooled) {
        const int e = j * pool + pool - 1;
        const int64_t blk = bt[e / bs];
        const int idx = (e % bs) / pool;
        vrow = pv_pool + ((blk * Gv + gv) * ppb + idx) * (int64_t)Dv;
        DotRows<KT, QH>::run(qs, Dp, pk_pool + ((blk * G + g) * ppb + idx) * (int64_t)D, D, p);
      } else {
        const int64_t blk = bt[j / bs];
        vrow = v_pool + ((blk * Gv + gv) * bs + (j % bs)) * (int64_t)v_pitch;
        DotRows<KT, QH>::run(qs, Dp, k_pool + ((blk * G + g) * bs + (j % bs)) * (int64_t)D, D, p);
      }
    }
#pragma unroll
    for (int qh = 0; qh < QH; ++qh) {
      float s = p[qh] * scale;
      if (softcap > 0.f) s = softcap * tanhf(s / softcap);
      if (sig) {
        p[qh] = valid ? 1.0f / (1.0f + expf(-(s + sig_bias[h0 + qh]))) : 0.f;
        continue;
      }
      if (!valid) s = -INFINITY;
      const float m_new = fmaxf(m[qh], warp_max(s));
      const float corr = expf(m[qh] - m_new);
      p[qh] = valid ? expf(s - m_new) : 0.f;
      l[qh] = l[qh] * corr + warp_sum(p[qh]);
#pragma unroll
      for (int c = 0; c < MAXC; ++c) {
        acc[qh][c].x *= corr;
        acc[qh][c].y *= corr;
      }
      m[qh] = m_new;
    }
    // all 32 keys of the tile, eight value rows in flight: lanes past the last key hold p = 0 and row 0 of the pools (the
    // null page: finite values), so they add nothing
#pragma unroll 8
    for (int jj = 0; jj < 32; ++jj) {
      const KT* vr = reinterpret_cast<const KT*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(vrow), jj));
      float pj[QH];
#pragma unroll
      for (int qh = 0; qh < QH; ++qh) pj[qh] = __shfl_sync(0xffffffffu, p[qh], jj);
#pragma unroll
      for (int c = 0; c < MAXC; ++c) {
        const int d = 2 * lane + 64 * c;
        if (d < Dv) {
          const float2 v2 = ld_pair(vr, d, Dv, vvec);
#pragma unroll
          for (int qh = 0; qh < QH; ++qh) {
            acc[qh][c].x += pj[qh] * v2.x;
            acc[qh][c].y += pj[qh] * v2.y;
          }
        }
      }
    }
  }
  // ---- merge the warps (fixed order)
#pragma unroll
  for (int qh = 0; qh < QH; ++qh) {
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      accs[((warp * QH + qh) * MAXC + c) * 64 + 2 * lane] = acc[qh][c].x;
      accs[((warp * QH + qh) * MAXC + c) * 64 + 2 * lane + 1] = acc[qh][c].y;
    }
    if (lane == 0) {
      ml[2 * (warp * QH + qh)] = m[qh];
      ml[2 * (warp * QH + qh) + 1] = l[qh];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < QH * Dv; i += ATT_WARPS * 32) {
    const int qh = i / Dv, d = i - qh * Dv;
    float mt = ml[2 * qh];
#pragma unroll
    for (int w = 1; w < ATT_WARPS; ++w) mt = fmaxf(mt, ml[2 * (w * QH + qh)]);
    float lt = 0.f, v = 0.f;
    const int c = d >> 6, e = d & 63;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) {
      const float f = mt == -INFINITY ? 0.f : expf(ml[2 * (w * QH + qh)] - mt);  // a split that saw no key at all
      lt += ml[2 * (w * QH + qh) + 1] * f;
      v += accs[((w * QH + qh) * MAXC + c) * 64 + e] * f;
    }
    if (splits > 1) {
      float* pr = part + (((int64_t)t * H + h0 + qh) * splits + split) * (Dv + 2);
      if (d == 0) pr[0] = mt, pr[1] = lt;
      pr[2 + d] = v;
      continue;
    }
    const float r = sig ? v : v / lt;
    if (out_f32) reinterpret_cast<float*>(out)[((int64_t)t * H + h0 + qh) * Dv + d] = r;
    else stf(reinterpret_cast<KT*>(out), ((int64_t)t * H + h0 + qh) * Dv + d, r);
  }
}

// One warp per (token, head): out = sum_s v_s e^(m_s - M) / sum_s l_s e^(m_s - M) over the key splits' partial results
// [T * H][splits][2 + Dv] = {maximum, denominator, unnormalised accumulator}; sigmoid weights have no denominator.
template <typename KT>
__global__ void attn_split_merge_kernel(const float* __restrict__ part, int splits, int Dv, int sig, int out_f32,
                                        void* __restrict__ out, int64_t rows) {
  griddep_launch();
  griddep_wait();
  const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  const float* p = part + r * splits * (Dv + 2);
  float M = -INFINITY, L = 0.f;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, p[s * (Dv + 2)]);
  for (int s = 0; s < splits; ++s) L += p[s * (Dv + 2) + 1] * expf(p[s * (Dv + 2)] - M);
  for (int d = lane; d < Dv; d += 32) {
    float v = 0.f;
    for (int s = 0; s < splits; ++s) v += p[s * (Dv + 2) + 2 + d] * expf(p[s * (Dv + 2)] - M);
    if (!sig) v /= L;
    if (out_f32) reinterpret_cast<float*>(out)[r * Dv + d] = v;
    else stf(reinterpret_cast<KT*>(out), r * Dv + d, v);
  }
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_kv_write_vmix(const float* qkv, int ld, int k_col0, int v_col0, float* v_first, float lambda, int mode, void* k_pool,
                       void* v_pool, int kv_dtype, const int64_t* slot_mapping, int T, int G, int D, int Dv, int block_size,
                       void* stream) {
  B200_REQUIRE(qkv && k_pool && v_pool && slot_mapping, "kv_write_vmix: null pointer");
  B200_REQUIRE(mode >= 0 && mode <= 2 && (mode == 0 || v_first), "kv_write_vmix: mode %d needs the first-layer value buffer", mode);
  if (T <= 0) return B200_OK;
  B200_DISPATCH_ELEM(kv_dtype, KT,
                     B200_CUDA_OK(launch_kernel(kv_write_vmix_kernel<KT>, dim3(T), dim3(128), 0, (cudaStream_t)stream, qkv, ld,
                                                k_col0, v_col0, v_first, lambda, mode, (KT*)k_pool, (KT*)v_pool, slot_mapping, G, D,
                                                Dv, block_size)));
  return B200_OK;
}

int b200_attn_split_merge(const float* part, int splits, int Dv, int sigmoid, int out_f32, int out_dtype, void* out, int64_t rows,
                          void* stream) {
  B200_REQUIRE(part && out && splits >= 1 && Dv >= 1, "attn_split_merge: null pointer or bad shape");
  if (rows <= 0) return B200_OK;
  B200_DISPATCH_ELEM(out_dtype, KT,
                     B200_CUDA_OK(launch_kernel(attn_split_merge_kernel<KT>, dim3((unsigned)((rows + 3) / 4)), dim3(128), 0,
                                                (cudaStream_t)stream, part, splits, Dv, sigmoid, out_f32, out, rows)));
  return B200_OK;
}

int b200_qk_norm_rope_kv_write(const float* src, int ld, int q_col0, int k_col0, int v_col0, const float* q_norm,
                               const float* k_norm, float eps, int rot_n, int rot_half, const float* cos_table,
                               const float* sin_table, const int32_t* tok_pos, const int64_t* slot_mapping, float* q_out,
                               void* k_pool, void* v_pool, int kv_dtype, int T, int H, int G, int Gv, int D, int Dv, int block_size,
                               const float* q_head_scale, void* stream) {
  B200_REQUIRE(src && tok_pos && slot_mapping && q_out && k_pool && v_pool, "qk_norm_rope_kv_write: null pointer");
  B200_REQUIRE(rot_n >= 0 && rot_n <= D && rot_n % 2 == 0 && (rot_n == 0 || (cos_table && sin_table)),
               "qk_norm_rope_kv_write: %d rotating columns in heads of %d", rot_n, D);
  B200_REQUIRE(H >= 1 && G >= 1 && Gv >= 1 && D >= 1 && Dv >= 1, "qk_norm_rope_kv_write: bad shape");
  if (T <= 0) return B200_OK;
  auto a16 = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  const bool vec = D % 4 == 0 && Dv % 4 == 0 && ld % 4 == 0 && q_col0 % 4 == 0 && k_col0 % 4 == 0 && v_col0 % 4 == 0 &&
                   rot_n % (rot_half ? 8 : 4) == 0 && a16(src) && a16(q_out) && a16(k_pool) && a16(v_pool) && a16(q_norm) &&
                   a16(k_norm) && a16(cos_table) && a16(sin_table);
  if (vec) {
    const int cols = H * D > G * D ? H * D : G * D;
    const int threads = cols >= 1024 ? 256 : cols >= 512 ? 128 : 64;
    B200_DISPATCH_ELEM(kv_dtype, KT,
                       B200_CUDA_OK(launch_kernel(qk_norm_rope_kv_write_vec_kernel<KT>, dim3(T), dim3(threads), 0, (cudaStream_t)stream,
                                                  src, ld, q_col0, k_col0, v_col0, q_norm, k_norm, eps, rot_n, rot_half, cos_table,
                                                  sin_table, tok_pos, slot_mapping, q_out, (KT*)k_pool, (KT*)v_pool, H, G, Gv, D, Dv,
                                                  block_size, q_head_scale)));
    return B200_OK;
  }
  B200_DISPATCH_ELEM(kv_dtype, KT,
                     B200_CUDA_OK(launch_kernel(qk_norm_rope_kv_write_kernel<KT>, dim3(T), dim3(256), 0, (cudaStream_t)stream, src, ld,
                                                q_col0, k_col0, v_col0, q_norm, k_norm, eps, rot_n, rot_half, cos_table, sin_table,
                                                tok_pos, slot_mapping, q_out, (KT*)k_pool, (KT*)v_pool, H, G, Gv, D, Dv, block_size,
                                                q_head_scale)));
  return B200_OK;
}

int b200_kv_pool_mean(const void* k_pool, const void* v_pool, void* pooled_k, void* pooled_v, int kv_dtype,
                      const int32_t* block_table, int64_t bt_stride, const int32_t* seq_start, const int32_t* seq_slot,
                      const int32_t* seq_pos0, int B, int T, int G, int Gv, int D, int Dv, int block_size, int pool, void* stream) {
  B200_REQUIRE(k_pool && v_pool && pooled_k && pooled_v && block_table && seq_start && seq_slot && seq_pos0, "kv_pool_mean: null pointer");
  B200_REQUIRE(pool >= 1 && G >= 1 && Gv >= 1 && D >= 1 && Dv >= 1 && block_size >= 1, "kv_pool_mean: blocks of %d positions", pool);
  if (T <= 0 || B <= 0) return B200_OK;
  const int ppb = (block_size + pool - 1) / pool;
  B200_DISPATCH_ELEM(kv_dtype, KT,
                     B200_CUDA_OK(launch_kernel(kv_pool_mean_kernel<KT>, dim3(T / pool + B), dim3(PM_THREADS), 0, (cudaStream_t)stream,
                                                (const KT*)k_pool, (const KT*)v_pool, (KT*)pooled_k, (KT*)pooled_v, block_table,
                                                bt_stride, seq_start, seq_slot, seq_pos0, B, G, Gv, D, Dv, block_size, pool, ppb)));
  return B200_OK;
}

int b200_swa_sink_attn(const float* q, int ldq, const void* k_pool, const void* v_pool, int kv_dtype, const int32_t* block_table,
                       int64_t bt_stride, const int32_t* tok_row, const int32_t* tok_pos, const float* sink, float scale,
                       int window, void* out, int T, int H, int G, int D, int Dv, int v_pitch, int block_size, int chunk,
                       float softcap, const float* sigmoid_bias, int v_div, int out_f32, int splits, float* split_workspace,
                       const void* pooled_k, const void* pooled_v, int pool, void* stream) {
  B200_REQUIRE(q && k_pool && v_pool && block_table && tok_row && tok_pos && out, "swa_sink_attn: null pointer");
  B200_REQUIRE(pool >= 0 && (pool == 0 || (pooled_k && pooled_v && v_pool != k_pool)), "swa_sink_attn: blocks of %d need pooled pools", pool);
  const int ppb = pool > 0 ? (block_size + pool - 1) / pool : 0;
  B200_REQUIRE(v_pitch >= Dv, "swa_sink_attn: value rows of pitch %d hold %d values", v_pitch, Dv);
  B200_REQUIRE(H > 0 && G > 0 && H % G == 0, "swa_sink_attn: %d query heads over %d kv heads", H, G);
  B200_REQUIRE(window >= 1 && chunk >= 0, "swa_sink_attn: window %d, chunk %d", window, chunk);
  B200_REQUIRE(v_div >= 1 && G % v_div == 0, "swa_sink_attn: %d key heads do not share values %d by %d", G, v_div, v_div);
  B200_REQUIRE(!(sigmoid_bias && sink), "swa_sink_attn: sigmoid weights have no denominator for a sink to join");
  B200_REQUIRE(splits >= 1 && splits <= 64 && (splits == 1 || split_workspace), "swa_sink_attn: %d key splits need a workspace", splits);
  B200_REQUIRE(Dv >= 1 && Dv <= 512 && D >= 1 && D <= 1024, "swa_sink_attn: head sizes %d / %d outside 1..1024 / 1..512", D, Dv);
  if (T <= 0) return B200_OK;
  B200_REQUIRE((int64_t)T * H < (1ll << 31), "swa_sink_attn: %d tokens x %d heads exceed the grid", T, H);
  const int rep = H / G;  // query heads per kv head; the CTA serves 4, 2 or 1 of them with one pass over the keys
  int QHr = rep % 4 == 0 ? 4 : rep % 2 == 0 ? 2 : 1;
  if (Dv > 256 && QHr > 2) QHr = 2;  // accumulator registers: 2 heads x 512 values per lane
  while (QHr > 1 && (int64_t)T * (H / QHr) < 148) QHr /= 2;  // small steps: keep a CTA per SM before sharing key rows
  dim3 grid((unsigned)(T * (H / QHr)), (unsigned)splits);
  cudaStream_t st = (cudaStream_t)stream;
  const int Dp = (D + 3) & ~3;
#define ATT_LAUNCH_Q(MC, QH)                                                                                                 \
  do {                                                                                                                       \
    const size_t smem = (size_t)(QH * Dp + ATT_WARPS * QH * 64 * MC + 2 * ATT_WARPS * QH) * 4;                               \
    if (smem > 48 * 1024)                                                                                                    \
      B200_CUDA_OK(cudaFuncSetAttribute(swa_sink_attn_kernel<KT, MC, QH>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                                        (int)smem));                                                                         \
    B200_CUDA_OK(launch_kernel(swa_sink_attn_kernel<KT, MC, QH>, grid, dim3(ATT_WARPS * 32), smem, st, q, ldq,               \
                               (const KT*)k_pool, (const KT*)v_pool, block_table, bt_stride, tok_row, tok_pos, sink, scale, \
                               window, out, T, H, G, D, Dv, block_size, v_pitch, chunk, softcap, sigmoid_bias, v_div, out_f32,       \
                               split_workspace, (const KT*)pooled_k, (const KT*)pooled_v, pool, ppb));                      \
  } while (0)
#define ATT_LAUNCH(MC)                \
  do {                                \
    if (QHr == 4) ATT_LAUNCH_Q(MC, 4); \
    else if (QHr == 2) ATT_LAUNCH_Q(MC, 2); \
    else ATT_LAUNCH_Q(MC, 1);          \
  } while (0)
  B200_DISPATCH_ELEM(kv_dtype, KT, {
    if (Dv <= 64) ATT_LAUNCH(1);
    else if (Dv <= 128) ATT_LAUNCH(2);
    else if (Dv <= 256) ATT_LAUNCH(4);
    else ATT_LAUNCH(8);
  });
#undef ATT_LAUNCH_Q
#undef ATT_LAUNCH
  if (splits > 1)
    return b200_attn_split_merge(split_workspace, splits, Dv, sigmoid_bias ? 1 : 0, out_f32, kv_dtype, out, (int64_t)T * H, stream);
  return B200_OK;
}

}  // extern "C"
