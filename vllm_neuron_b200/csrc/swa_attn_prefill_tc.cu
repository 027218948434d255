// Prompt attention of the hybrid family's rotating-attention layers on the 5th-generation tensor cores (tcgen05 + TMEM):
// ragged batches of prompt portions over the paged K / V pools, with the layer variants as parameters.
//
//   out[r][h] = sum_k w(q[r][h] . K[k] * scale) V[k],   k <= pos(r), and k >= the start of pos(r)'s chunk when chunk > 0
//   w = softmax over the visible keys | softmax of cap * tanh(. / cap) | sigmoid(. + bias[h]) (not normalised)
//
// The pipeline is the one of paged_attn_prefill_tc.cu (two 128-row query tiles per CTA in tensor memory, S0 | S1 | O0 | O1,
// K / V steps of 128 keys gathered page by page with TMA, one softmax thread per query row, lazy running maximum); what
// differs:
//   * one launch serves every sequence of the step (grid z; start row, position and block-table row come from the step's
//     device arrays), and a tile starts at the key step that holds the first key of its first row's chunk;
//   * q arrives as fp32 rows: the softmax warpgroups round it to bf16 and lay it into the 128-byte-swizzled operand
//     layout themselves;
//   * key size and value size are separate template parameters (keys of 32 columns are 64-byte rows under the 64B swizzle),
//     and with MAPS the two tiles of a CTA are the two score
//     maps of ONE query head: each has its own key head (2g, 2g + 1), both multiply the same value step;
//   * the weights enter the second product as TWO bf16 terms, hi = bf16(p) in the first 64 columns the scores occupied and
//     lo = bf16(p - hi) in the other 64 (16 mantissa bits; the scores sit in registers by then), two MMAs per 16 keys;
//   * sigmoid weights need no maximum and no denominator; rows whose chunk starts after a key step see -inf only, and
//     the maximum stays -inf without producing NaN.
#include "hybrid_common.cuh"

namespace b200 {

// a pool as a 2D bf16 tensor [pages * heads * 32 rows][D], boxes of 64 columns x 32 rows, 128B swizzle (paged_attn.cu)
int kv_pool_tmap(const void* pool, int num_blocks, int Hkv, int D, CUtensorMap* out);

constexpr int TP_BM = 128;   // query rows per tile
constexpr int TP_BN = 128;   // keys per step
constexpr int TP_ST = 2;     // K / V stages
constexpr int TP_THREADS = 384;
constexpr int TP_BLK = 32;   // tokens per page
constexpr int TP_HALF = TP_BN * 128;  // one [128 rows x 128 B] operand half = 16 KB
enum { TP_SOFTMAX = 0, TP_CAPPED = 1, TP_SIGMOID = 2 };

// MN-major, 128B-swizzled operand: 64 contiguous elements of M/N per row, 8 K-rows per 1024 B atom
__device__ __forceinline__ uint64_t tp_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// K-major, 64B-swizzled operand tile: rows of 64 B, 8-row groups 512 B apart
__device__ __forceinline__ uint64_t tp_desc_sw64(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(512 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)4 << 61;  // SWIZZLE_64B
  return d;
}
__device__ __forceinline__ void tp_ld_x32(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]),
        "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]),
        "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tp_st_x16(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16};\n" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
      "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ float tp_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

template <int DK, int DV, int KIND, bool MAPS>
__global__ void __launch_bounds__(TP_THREADS, 1)
    swa_prefill_tc_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                          const float* __restrict__ q, int ldq, const int32_t* __restrict__ block_table, int64_t bt_stride,
                          const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_slot,
                          const int32_t* __restrict__ seq_pos0, void* __restrict__ out, int H, int G, int chunk, float scale,
                          float softcap, const float* __restrict__ sig_bias, int out_f32, int split_p, int ny_tiles) {
  // q / k operand rows: pieces of 64 columns (128 bytes, 128B swizzle), or one piece of 32 columns (64 bytes, 64B swizzle)
  constexpr int KROW = DK >= 64 ? 128 : DK * 2;
  constexpr int NHK = DK >= 64 ? DK / 64 : 1, NHV = DV / 64;
  constexpr int HALFK = TP_BN * KROW;                  // one [128 rows x KROW bytes] piece
  constexpr int TQ = NHK * HALFK;                      // one query tile
  constexpr int TK = (MAPS ? 2 : 1) * NHK * HALFK;     // one key step (both maps' key heads with MAPS)
  constexpr int TV = NHV * TP_HALF;                    // one value step
  constexpr uint32_t IDESC_S = umma_idesc(1, 1, TP_BM, TP_BN);
  constexpr uint32_t IDESC_PV = umma_idesc(1, 1, TP_BM, DV) | (1u << 16);  // B (= V) is MN-major
  constexpr uint32_t TMEM_COLS = 512;

  // ---- which rows, heads and keys this CTA owns (uniform over the CTA; a tile past its sequence's portion leaves at once)
  const int sq = blockIdx.z;
  const int t0 = seq_start[sq], n_new = seq_start[sq + 1] - t0;
  // heaviest tiles first: a causal tile's cost grows with its index; with chunks of several tiles it grows with the tile's
  // place INSIDE its chunk, so all chunks' last tiles go first, then their last but one, ... (grid y covers tiles_per_chunk x
  // chunks >= ny_tiles places; the ones past the end leave)
  const int tpc = chunk / TP_BM;
  int tile = ny_tiles - 1 - (int)blockIdx.y;
  if (tpc >= 2) {
    const int nch = (ny_tiles + tpc - 1) / tpc;
    tile = ((int)blockIdx.y % nch) * tpc + (tpc - 1 - (int)blockIdx.y / nch);
  }
  const int q0 = tile * TP_BM;
  if (tile < 0 || tile >= ny_tiles || q0 >= n_new) return;
  const int pos0 = seq_pos0[sq];
  const int32_t* bt_row = block_table + (int64_t)seq_slot[sq] * bt_stride;
  int qhead[2], khead[2], vhead, ntile, Hv;
  if (MAPS) {
    const int rep = H / G, gv = blockIdx.x / rep, r = blockIdx.x - gv * rep;
    qhead[0] = (2 * gv) * rep + r, qhead[1] = (2 * gv + 1) * rep + r;
    khead[0] = 2 * gv, khead[1] = 2 * gv + 1;
    vhead = gv, ntile = 2, Hv = G / 2;
  } else {
    const int rep = H / G, pairs = (rep + 1) >> 1, kvh = blockIdx.x / pairs, pr = blockIdx.x - kvh * pairs;
    qhead[0] = kvh * rep + 2 * pr, qhead[1] = qhead[0] + 1;
    khead[0] = khead[1] = vhead = kvh;
    ntile = (2 * pr + 1 < rep) ? 2 : 1, Hv = G;
  }
  const int q_hi = q0 + TP_BM < n_new ? q0 + TP_BM : n_new;
  const int kv_end = pos0 + q_hi;                                   // keys [0, kv_end) are visible to some row of the tile
  const int klo_first = chunk > 0 ? ((pos0 + q0) / chunk) * chunk : 0;  // first key the tile's first row sees
  const int j_lo = klo_first / TP_BN;
  const int niter = (kv_end + TP_BN - 1) / TP_BN - j_lo;
  const int nblk_seq = (pos0 + n_new + TP_BLK - 1) / TP_BLK;        // valid entries of bt_row

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;                               // [2 tiles][TQ]
  uint8_t* k_s = q_s + 2 * TQ;                       // [TP_ST][TK]
  uint8_t* v_s = k_s + TP_ST * TK;                   // [TP_ST][TV]
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + TP_ST * TV);
  uint64_t* q_full = bars;                           // 1
  uint64_t* k_full = q_full + 1;                     // TP_ST
  uint64_t* k_empty = k_full + TP_ST;
  uint64_t* v_full = k_empty + TP_ST;
  uint64_t* v_empty = v_full + TP_ST;
  uint64_t* s_full = v_empty + TP_ST;                // 2 (per tile)
  uint64_t* p_ready = s_full + 2;                    // 2
  uint64_t* o_full = p_ready + 2;                    // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 8 && lane == 0) {
    tma_prefetch_desc(&k_map);
    tma_prefetch_desc(&v_map);
    mbar_init(q_full, (uint32_t)ntile * 128u);  // every thread that lays down a part of q arrives once
    for (int s = 0; s < TP_ST; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_ready[t], 4);  // one arrival per softmax warp of the tile
      mbar_init(&o_full[t], 1);
    }
    fence_mbar_init();
    fence_proxy_async();
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  griddep_launch();
  griddep_wait();  // q and the pools were written by the previous kernels of the stream
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;\n");
    if (warp == 9 || warp == 10) {
      // ---------------------------------------------------------------- K (warp 9) / V (warp 10) producer
      if (lane == 0) {
        const bool is_k = warp == 9;
        const CUtensorMap* map = is_k ? &k_map : &v_map;
        uint8_t* ring = is_k ? k_s : v_s;
        uint64_t* full = is_k ? k_full : v_full;
        uint64_t* empty = is_k ? k_empty : v_empty;
        const int tile = is_k ? TK : TV, nh = is_k ? NHK : NHV, heads = is_k ? G : Hv;
        const int piece = is_k ? HALFK : TP_HALF, rowb = is_k ? KROW : 128;
        const int nm = (is_k && MAPS) ? 2 : 1;
        for (int it = 0; it < niter; ++it) {
          const int s = it % TP_ST, j = j_lo + it;
          if (it >= TP_ST) mbar_wait(&empty[s], (uint32_t)(it / TP_ST - 1) & 1u);
          mbar_expect_tx(&full[s], (uint32_t)tile);
          uint8_t* dst = ring + (size_t)s * tile;
#pragma unroll
          for (int b = 0; b < TP_BN / TP_BLK; ++b) {
            const int bi = j * (TP_BN / TP_BLK) + b;
            const int blk = bi < nblk_seq ? __ldg(bt_row + bi) : 0;  // past the sequence: the null page (masked anyway)
            for (int m = 0; m < nm; ++m) {
              const int row = (blk * heads + (is_k ? khead[m] : vhead)) * TP_BLK;
              for (int h = 0; h < nh; ++h)
                tma_load_2d(dst + (m * nh + h) * piece + b * (TP_BLK * rowb), map, &full[s], h * 64, row);
            }
          }
        }
      }
      __syncwarp();
    } else if (warp == 8) {
      // ---------------------------------------------------------------- MMA issuer
      if (lane == 0) {
        auto issue_s = [&](int t, int s) {
          const uint32_t qa = smem_u32(q_s + t * TQ), ka = smem_u32(k_s + (size_t)s * TK + (MAPS ? t * NHK * HALFK : 0));
          constexpr int PER = KROW / 32;  // 16-column MMA steps per row piece
#pragma unroll
          for (int kk = 0; kk < DK / 16; ++kk) {
            const uint32_t off = (uint32_t)(kk / PER) * HALFK + (uint32_t)(kk % PER) * 32;
            if (DK >= 64)
              umma_ss<KIND_F16>(tmem_base + (uint32_t)t * 128u, umma_desc_sw128(qa + off), umma_desc_sw128(ka + off), IDESC_S,
                                (uint32_t)(kk != 0));
            else
              umma_ss<KIND_F16>(tmem_base + (uint32_t)t * 128u, tp_desc_sw64(qa + off), tp_desc_sw64(ka + off), IDESC_S,
                                (uint32_t)(kk != 0));
          }
          tc_commit(&s_full[t]);
        };
        auto issue_pv = [&](int t, int s, int it) {
          const uint32_t va = smem_u32(v_s + (size_t)s * TV);
          const uint32_t o_t = tmem_base + 256u + (uint32_t)t * 128u, p_t = tmem_base + (uint32_t)t * 128u;
#pragma unroll
          for (int kk = 0; kk < TP_BN / 16; ++kk) {  // 16 keys per UMMA_K: two 8-row groups of the [token][d] tile
            const uint64_t vd = tp_desc_mn_sw128(va + kk * 2048, TP_HALF, 1024);
            umma_ts_f16(o_t, p_t + (uint32_t)kk * 8u, vd, IDESC_PV, (uint32_t)((it | kk) != 0));
            if (split_p) umma_ts_f16(o_t, p_t + 64u + (uint32_t)kk * 8u, vd, IDESC_PV, 1u);
          }
        };
        mbar_wait(q_full, 0);
        mbar_wait(&k_full[0], 0);
        tc_fence_after();
        for (int t = 0; t < ntile; ++t) issue_s(t, 0);
        tc_commit(&k_empty[0]);
        for (int it = 0; it < niter; ++it) {
          const int s = it % TP_ST, sn = (it + 1) % TP_ST;
          const bool more = it + 1 < niter;
          mbar_wait(&v_full[s], (uint32_t)(it / TP_ST) & 1u);
          for (int t = 0; t < ntile; ++t) {
            mbar_wait(&p_ready[t], (uint32_t)it & 1u);
            tc_fence_after();
            issue_pv(t, s, it);
            if (t == ntile - 1) tc_commit(&v_empty[s]);
            if (more) {
              if (t == 0) {
                mbar_wait(&k_full[sn], (uint32_t)((it + 1) / TP_ST) & 1u);
                tc_fence_after();
              }
              issue_s(t, sn);
              if (t == ntile - 1) tc_commit(&k_empty[sn]);
            } else {
              tc_commit(&o_full[t]);
            }
          }
        }
      }
      __syncwarp();
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;\n");
    if ((warp >> 2) < ntile) {
      const int t = warp >> 2;
      const int tid = threadIdx.x & 127;
      // ---------------------------------------------------------------- q tile: fp32 rows -> bf16, K-major 128B swizzle
      {
        const float* qsrc = q + (int64_t)(t0 + q0) * ldq + (int64_t)qhead[t] * DK;
        uint8_t* qd = q_s + t * TQ;
#pragma unroll 4
        for (int idx = tid; idx < TP_BM * (DK / 8); idx += 128) {
          const int row = idx / (DK / 8), c = idx - row * (DK / 8);
          uint4 w = make_uint4(0u, 0u, 0u, 0u);
          if (q0 + row < n_new) {
            const float4 a = *reinterpret_cast<const float4*>(qsrc + (int64_t)row * ldq + c * 8);
            const float4 b = *reinterpret_cast<const float4*>(qsrc + (int64_t)row * ldq + c * 8 + 4);
            w.x = pack_bf16(a.x, a.y), w.y = pack_bf16(a.z, a.w), w.z = pack_bf16(b.x, b.y), w.w = pack_bf16(b.z, b.w);
          }
          if (DK >= 64)  // 128B swizzle: 16-byte piece c of row r sits at piece c ^ (r % 8)
            *reinterpret_cast<uint4*>(qd + (c >> 3) * HALFK + row * 128 + (((c & 7) ^ (row & 7)) << 4)) = w;
          else           // 64B swizzle: at piece c ^ ((r / 2) % 4)
            *reinterpret_cast<uint4*>(qd + row * KROW + ((c ^ ((row >> 1) & 3)) << 4)) = w;
        }
        fence_proxy_async();  // the tensor core reads these bytes through the async proxy
        mbar_arrive(q_full);
      }
      // ---------------------------------------------------------------- weights + epilogue of tile t, one row per thread
      const int row = (warp & 3) * 32 + lane;
      const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
      const uint32_t s_addr = lane_base + (uint32_t)t * 128u;  // S_t; the weights' hi terms over its first 64 columns, lo over the rest
      const uint32_t o_addr = lane_base + 256u + (uint32_t)t * 128u;
      const int qpos = pos0 + q0 + row;
      const int klo = chunk > 0 ? (qpos / chunk) * chunk : 0;                             // first key this row sees
      const int klo_last = chunk > 0 ? ((pos0 + q0 + TP_BM - 1) / chunk) * chunk : 0;     // ... and the tile's last row
      constexpr float LOG2E = 1.4426950408889634f;
      const float scale_log2 = scale * LOG2E;
      // capped scores, in log2 units: cap * log2e * tanh(s * scale / cap), tanh(x) = 1 - 2 / (1 + e^(2x))
      const float capl = softcap * LOG2E, cap_arg = KIND == TP_CAPPED ? 2.0f * scale_log2 / softcap : 0.f;
      const float sl = KIND == TP_CAPPED ? 1.0f : scale_log2;
      const float sb_log2 = KIND == TP_SIGMOID ? sig_bias[qhead[t]] * LOG2E : 0.f;
      float m_used = -INFINITY, l = 0.f;
      for (int it = 0; it < niter; ++it) {
        mbar_wait(&s_full[t], (uint32_t)it & 1u);
        tc_fence_after();
        const int k0 = (j_lo + it) * TP_BN;
        const bool masked = k0 + TP_BN - 1 > pos0 + q0 || k0 < klo_last;  // some key of the step is hidden from some row
        uint32_t sv[TP_BN];
        auto load_scores = [&]() {
          tp_ld_x32(s_addr, &sv[0]);
          tp_ld_x32(s_addr + 32, &sv[32]);
          tp_ld_x32(s_addr + 64, &sv[64]);
          tp_ld_x32(s_addr + 96, &sv[96]);
          tmem_ld_wait();
          if (KIND == TP_CAPPED) {
#pragma unroll
            for (int i = 0; i < TP_BN; ++i)
              sv[i] = __float_as_uint(capl - __fdividef(2.0f * capl, 1.0f + tp_ex2(__uint_as_float(sv[i]) * cap_arg)));
          }
          if (masked) {
#pragma unroll
            for (int i = 0; i < TP_BN; ++i)
              if (k0 + i > qpos || k0 + i < klo) sv[i] = 0xff800000u;
          }
        };
        load_scores();
        float neg_m = 0.f;
        if (KIND != TP_SIGMOID) {
          float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int i = 0; i < TP_BN; i += 8) {
            mx4[0] = fmaxf(mx4[0], fmaxf(__uint_as_float(sv[i]), __uint_as_float(sv[i + 1])));
            mx4[1] = fmaxf(mx4[1], fmaxf(__uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3])));
            mx4[2] = fmaxf(mx4[2], fmaxf(__uint_as_float(sv[i + 4]), __uint_as_float(sv[i + 5])));
            mx4[3] = fmaxf(mx4[3], fmaxf(__uint_as_float(sv[i + 6]), __uint_as_float(sv[i + 7])));
          }
          const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
          const float m_new = fmaxf(m_used, mx * sl);
          // lazy maximum: move it (and pay the O read-modify-write) only when it grew by more than 2^8
          const bool grow = m_new > m_used + 8.f;
          if (__any_sync(0xffffffffu, grow)) {
            const float alpha = grow ? tp_ex2(m_used - m_new) : 1.f;  // m_used = -inf -> 0
            if (grow) m_used = m_new;
            l *= alpha;
            if (it > 0) {  // rare after the first steps: the score registers are given up for the O tile and loaded again
#pragma unroll 1
              for (int c = 0; c < DV / 32; ++c) {
                uint32_t v[32];
                tp_ld_x32(o_addr + c * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                tmem_st_32x32b_x32(o_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
              }
              tmem_st_wait();
              load_scores();
            }
          }
          neg_m = m_used == -INFINITY ? 0.f : -m_used;  // a row that has seen no key yet: 2^(-inf) = 0, not NaN
        }
        float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < TP_BN / 32; ++c) {
          uint32_t hi[16], lo[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float s0 = __uint_as_float(sv[c * 32 + i]), s1 = __uint_as_float(sv[c * 32 + i + 1]);
            float p0, p1;
            if (KIND == TP_SIGMOID) {  // 1 / (1 + 2^-(s + b)); a hidden key's -inf gives 1 / inf = 0
              p0 = __fdividef(1.0f, 1.0f + tp_ex2(-fmaf(s0, sl, sb_log2)));
              p1 = __fdividef(1.0f, 1.0f + tp_ex2(-fmaf(s1, sl, sb_log2)));
            } else {
              p0 = tp_ex2(fmaf(s0, sl, neg_m));
              p1 = tp_ex2(fmaf(s1, sl, neg_m));
              l4[(i >> 1) & 3] += p0 + p1;
            }
            const uint32_t h = pack_bf16(p0, p1);
            hi[i >> 1] = h;
            lo[i >> 1] = pack_bf16(p0 - __uint_as_float(h << 16), p1 - __uint_as_float(h & 0xffff0000u));
          }
          tp_st_x16(s_addr + c * 16, hi);
          if (split_p) tp_st_x16(s_addr + 64 + c * 16, lo);
        }
        l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready[t]);
      }
      // epilogue: O (/ l) -> rows of the output
      mbar_wait(&o_full[t], 0);
      tc_fence_after();
      const float inv = KIND == TP_SIGMOID ? 1.f : (l > 0.f ? 1.f / l : 0.f);
      const bool ok = q0 + row < n_new;
      const int64_t o_off = ((int64_t)(t0 + q0 + row) * H + qhead[t]) * DV;
#pragma unroll 1
      for (int c = 0; c < DV / 32; ++c) {
        uint32_t v[32];
        tp_ld_x32(o_addr + c * 32, v);
        tmem_ld_wait();
        if (ok && out_f32) {
          float* dst = reinterpret_cast<float*>(out) + o_off + c * 32;
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<float4*>(dst + i) = make_float4(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv,
                                                              __uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
        } else if (ok) {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out) + o_off + c * 32;
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
            w.y = pack_bf16(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
            w.z = pack_bf16(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv);
            w.w = pack_bf16(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + i) = w;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int DK, int DV, int KIND, bool MAPS>
static int tp_launch(const CUtensorMap& km, const CUtensorMap& vm, const float* q, int ldq, const int32_t* block_table,
                     int64_t bt_stride, const int32_t* seq_start, const int32_t* seq_slot, const int32_t* seq_pos0, int B,
                     int max_new, void* out, int H, int G, int chunk, float scale, float softcap, const float* sig_bias,
                     int out_f32, int split_p, cudaStream_t stream) {
  auto kern = swa_prefill_tc_kernel<DK, DV, KIND, MAPS>;
  // operand tiles + barriers + alignment slack; never less than half an SM's shared memory, so that one CTA (which takes all
  // 512 columns of tensor memory) is resident per SM
  size_t smem = (size_t)(2 + TP_ST * (MAPS ? 2 : 1)) * TP_BN * DK * 2 + (size_t)TP_ST * (DV / 64) * TP_HALF + 256 + 1024;
  if (smem < 120 * 1024) smem = 120 * 1024;
  static bool attr_done = false;
  if (!attr_done) {
    B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_done = true;
  }
  const int rep = H / G;
  const int ny = (max_new + TP_BM - 1) / TP_BM, tpc = chunk / TP_BM;
  const int gy = tpc >= 2 ? ((ny + tpc - 1) / tpc) * tpc : ny;  // the launch order of the kernel's tile map
  dim3 grid(MAPS ? (G / 2) * rep : G * ((rep + 1) / 2), gy, B);
  B200_CUDA_OK(launch_kernel(kern, grid, dim3(TP_THREADS), smem, stream, km, vm, q, ldq, block_table, bt_stride, seq_start,
                             seq_slot, seq_pos0, out, H, G, chunk, scale, softcap, sig_bias, out_f32, split_p, ny));
  return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" {

// 1 when b200_swa_sink_attn_prefill_tc has a kernel for these head sizes and variants
int b200_swa_sink_attn_prefill_tc_supported(int D, int Dv, int block_size, int v_div, int capped, int sigmoid) {
  if (block_size != TP_BLK || (capped && sigmoid)) return 0;
  if (v_div == 1) return (D == 64 && Dv == 64) || (D == 128 && Dv == 128);
  if (v_div == 2) return !capped && !sigmoid && (D == 32 || D == 64) && (Dv == 64 || Dv == 128);
  return 0;
}

int b200_swa_sink_attn_prefill_tc(const float* q, int ldq, const void* k_pool, const void* v_pool, int num_blocks,
                                  const int32_t* block_table, int64_t bt_stride, const int32_t* seq_start,
                                  const int32_t* seq_slot, const int32_t* seq_pos0, int B, int max_new, float scale, void* out,
                                  int H, int G, int D, int Dv, int block_size, int chunk, float softcap,
                                  const float* sigmoid_bias, int v_div, int out_f32, int split_p, void* stream) {
  B200_REQUIRE(q && k_pool && v_pool && block_table && seq_start && seq_slot && seq_pos0 && out,
               "swa_sink_attn_prefill_tc: null pointer");
  B200_REQUIRE(H > 0 && G > 0 && H % G == 0 && chunk >= 0 && v_div >= 1 && G % v_div == 0,
               "swa_sink_attn_prefill_tc: %d query heads over %d key heads, values shared by %d", H, G, v_div);
  if (!b200_swa_sink_attn_prefill_tc_supported(D, Dv, block_size, v_div, softcap > 0.f, sigmoid_bias != nullptr) || (ldq & 3) ||
      ((uintptr_t)q & 15) || ((uintptr_t)out & 15)) {
    set_last_error("swa_sink_attn_prefill_tc: head sizes %d / %d (values shared by %d) or the layout of q have no kernel", D, Dv, v_div);
    return B200_ERR_UNSUPPORTED;
  }
  if (B <= 0 || max_new <= 0) return B200_OK;
  CUtensorMap km, vm;
  // key rows of 32 columns are 64 bytes: boxes of 32 columns x 32 rows under the 64B swizzle
  int rc = D == 32 ? make_tmap_2d_sw64(&km, k_pool, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 32, (uint64_t)num_blocks * G * TP_BLK, 64, 32,
                                       TP_BLK)
                   : kv_pool_tmap(k_pool, num_blocks, G, D, &km);
  if (rc) return rc;
  rc = kv_pool_tmap(v_pool, num_blocks, G / v_div, Dv, &vm);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
#define TP_GO(DK_, DV_, KIND_, MAPS_)                                                                                          \
  return tp_launch<DK_, DV_, KIND_, MAPS_>(km, vm, q, ldq, block_table, bt_stride, seq_start, seq_slot, seq_pos0, B, max_new, \
                                           out, H, G, chunk, scale, softcap, sigmoid_bias, out_f32, split_p, st)
  if (v_div == 2 && D == 32) {
    if (Dv == 64) TP_GO(32, 64, TP_SOFTMAX, true);
    TP_GO(32, 128, TP_SOFTMAX, true);
  }
  if (v_div == 2) {
    if (Dv == 64) TP_GO(64, 64, TP_SOFTMAX, true);
    TP_GO(64, 128, TP_SOFTMAX, true);
  }
  if (D == 64) {
    if (sigmoid_bias) TP_GO(64, 64, TP_SIGMOID, false);
    if (softcap > 0.f) TP_GO(64, 64, TP_CAPPED, false);
    TP_GO(64, 64, TP_SOFTMAX, false);
  }
  if (sigmoid_bias) TP_GO(128, 128, TP_SIGMOID, false);
  if (softcap > 0.f) TP_GO(128, 128, TP_CAPPED, false);
  TP_GO(128, 128, TP_SOFTMAX, false);
#undef TP_GO
}

}  // extern "C"
