// Mixture-of-experts feed-forward over a token batch, and the generic grouped / dense linear kernel it is built on.
//   * moe_topk: over the fp32 router logits (a linear of the layer's input, plus an optional per-expert bias): the `top`
//     largest are chosen (ties go to the lower expert index); the routing weights are either the sigmoid of each chosen
//     logit (no renormalisation) or the softmax over the chosen logits only;
//   * moe_align: counting sort of the (token, choice) pairs by expert into row tiles of MOE_BM, each tile owned by one
//     expert (ragged tails padded with -1), so the expert GEMMs run as one launch without the host knowing the counts;
//   * grouped_linear: out = A W_e^T with fp32 accumulation over K in ascending order (the result of a row does not depend
//     on what else is in the batch).  A rows can be gathered per pair and scaled by the pair's routing weight (the
//     scaling happens on the way INTO the expert, ahead of its nonlinearity), and the epilogue is either a plain fp32 store (optionally scattered back to
//     pair order) or the clamped gated-linear unit over a [gate; up] weight.
// With one expert, no gather and no scatter the same kernel is the dense linear for operand types or shapes the
// tensor-core GEMM does not take (fp32 operands, K not a multiple of 8).
#include "hybrid_common.cuh"

namespace b200 {

constexpr int MOE_BM = 32;
constexpr int MOE_WIDE = 4;  // prompt-sized bf16 batches: tiles of MOE_BM * MOE_WIDE rows (grouped_mma_pipe_kernel)
constexpr int GL_BN = 64;
constexpr int GL_BK = 16;
constexpr int GL_THREADS = 256;

// one thread per token: the `top` largest logits (+ bias; ties to the lower index); weight = sigmoid(logit), or the softmax
// over the chosen logits (mode B200_ROUTE_SOFTMAX_TOP), or the softmax over all experts renormalised over the chosen
// (B200_ROUTE_SOFTMAX_RENORM)
__global__ void moe_topk_kernel(const float* __restrict__ z, int ld, const float* __restrict__ bias, int mode, int E, int top,
                                int32_t* __restrict__ idx, float* __restrict__ wt, int ntok) {
  griddep_launch();
  griddep_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= ntok) return;
  const float* zr = z + (int64_t)t * ld;
  int32_t* out = idx + (int64_t)t * top;
  float* w = wt + (int64_t)t * top;
  for (int c = 0; c < top; ++c) {
    float best = -INFINITY;
    int bi = -1;
    for (int e = 0; e < E; ++e) {
      bool taken = false;
      for (int k = 0; k < c; ++k) taken |= out[k] == e;
      const float v = zr[e] + (bias ? bias[e] : 0.f);
      if (!taken && (bi < 0 || v > best)) {
        best = v;
        bi = e;
      }
    }
    out[c] = bi;
    w[c] = best;
  }
  if (mode == B200_ROUTE_SOFTMAX_RENORM) {
    // scores = softmax over ALL experts; the chosen scores are divided by their own sum (+ 1e-20)
    const float m = w[0];
    float all = 0.f, sum = 0.f;
    for (int e = 0; e < E; ++e) all += expf(zr[e] + (bias ? bias[e] : 0.f) - m);
    for (int c = 0; c < top; ++c) {
      w[c] = expf(w[c] - m) / all;
      sum += w[c];
    }
    for (int c = 0; c < top; ++c) w[c] = w[c] / (sum + 1e-20f);
  } else if (mode == B200_ROUTE_SOFTMAX_TOP) {
    const float m = w[0];  // the first chosen is the largest
    float sum = 0.f;
    for (int c = 0; c < top; ++c) sum += expf(w[c] - m);
    for (int c = 0; c < top; ++c) w[c] = expf(w[c] - m) / sum;
  } else {
    for (int c = 0; c < top; ++c) w[c] = 1.0f / (1.0f + expf(-w[c]));
  }
}

// single CTA: counts -> padded offsets -> tile owners -> scatter of pair ids
__global__ void moe_align_kernel(const int32_t* __restrict__ idx, int npairs, int E, int32_t* __restrict__ sorted_ids, int cap,
                                 int32_t* __restrict__ tile_expert, int max_tiles, int32_t* __restrict__ num_tiles, int bm) {
  griddep_launch();
  griddep_wait();
  extern __shared__ int32_t sm[];
  int32_t* counts = sm;
  int32_t* offs = sm + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
  for (int i = threadIdx.x; i < cap; i += blockDim.x) sorted_ids[i] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < npairs; i += blockDim.x) atomicAdd(&counts[idx[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      offs[e] = o;
      const int tiles = (counts[e] + bm - 1) / bm;
      for (int k = 0; k < tiles && nt < max_tiles; ++k) tile_expert[nt++] = e;
      o += tiles * bm;
    }
    *num_tiles = nt;
  }
  __syncthreads();
  // order inside an expert's rows follows the atomics; every row is computed on its own, so results do not depend on it
  for (int i = threadIdx.x; i < npairs; i += blockDim.x) {
    const int p = atomicAdd(&offs[idx[i]], 1);
    sorted_ids[p] = i;
  }
}

enum { GL_EPI_STORE = 0, GL_EPI_GLU = 1 };

// gated-linear unit on fp32 accumulators: clamped swish (a = min(g, L), b = clip(u, -L, L): (b + 1) a sigmoid(1.702 a)),
// SiLU(g) u, or tanh-GELU(g) u
__device__ __forceinline__ float glu_act(float g, float u, int act, float limit) {
  if (act == B200_ACT_SILU) return g / (1.0f + expf(-g)) * u;
  if (act == B200_ACT_GELU_TANH) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
}

// Row tile `blockIdx.x` (MOE_BM rows), column tile `blockIdx.y` (GL_BN outputs).  256 threads, each 2 rows x 4 columns.
template <typename T, int EPI>
__global__ void __launch_bounds__(GL_THREADS)
    grouped_linear_kernel(const T* __restrict__ a, int lda, const int32_t* __restrict__ sorted_ids, int gather_div,
                          const float* __restrict__ row_scale, const T* __restrict__ w, int64_t w_stride,
                          const int32_t* __restrict__ tile_expert, const int32_t* __restrict__ num_tiles, int M, int N, int K,
                          void* __restrict__ out, int ldo, int scatter, float limit, int act, int64_t a_zs, int64_t o_zs,
                          int store_typed, const float* __restrict__ gate, int gate_ld) {
  griddep_launch();
  griddep_wait();
  constexpr int NW = EPI == GL_EPI_GLU ? 2 : 1;
  __shared__ float As[GL_BK][MOE_BM + 1];
  __shared__ float Ws[NW][GL_BK][GL_BN + 1];
  __shared__ int32_t rid[MOE_BM];     // source row in `a` (or -1)
  __shared__ int32_t oid[MOE_BM];     // destination row in `out` (or -1)
  __shared__ float rsc[MOE_BM];
  const int tile = blockIdx.x;
  if (num_tiles && tile >= *num_tiles) return;
  const int e = tile_expert ? tile_expert[tile] : blockIdx.z;  // z-batched dense launches: one weight per batch index
  const T* we = w + (int64_t)e * w_stride;
  a += (int64_t)blockIdx.z * a_zs;
  const int n0 = blockIdx.y * GL_BN;
  if (threadIdx.x < MOE_BM) {
    const int r = tile * MOE_BM + threadIdx.x;
    int src = -1, dst = -1;
    float sc = 1.0f;
    if (sorted_ids) {
      const int id = sorted_ids[r];
      if (id >= 0) {
        src = gather_div > 0 ? id / gather_div : r;
        dst = scatter ? id : r;
        if (row_scale) sc = row_scale[id];
      }
    } else if (r < M) {
      src = dst = r;
    }
    rid[threadIdx.x] = src;
    oid[threadIdx.x] = dst;
    rsc[threadIdx.x] = sc;
  }
  __syncthreads();
  const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;  // rows 2 ty, 2 ty + 1; columns 4 tx .. 4 tx + 3
  float acc[NW][2][4];
#pragma unroll
  for (int x = 0; x < NW; ++x)
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[x][i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += GL_BK) {
    for (int i = threadIdx.x; i < MOE_BM * GL_BK; i += GL_THREADS) {
      const int r = i / GL_BK, k = i % GL_BK;
      float v = 0.f;
      if (rid[r] >= 0 && k0 + k < K) v = ldf(a, (int64_t)rid[r] * lda + k0 + k) * rsc[r];
      As[k][r] = v;
    }
    for (int i = threadIdx.x; i < NW * GL_BN * GL_BK; i += GL_THREADS) {
      const int x = i / (GL_BN * GL_BK), rem = i % (GL_BN * GL_BK);
      const int n = rem / GL_BK, k = rem % GL_BK;
      float v = 0.f;
      if (n0 + n < N && k0 + k < K) v = ldf(we, ((int64_t)x * N + n0 + n) * K + k0 + k);
      Ws[x][k][n] = v;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < GL_BK; ++k) {
      const float a0 = As[k][2 * ty], a1 = As[k][2 * ty + 1];
#pragma unroll
      for (int x = 0; x < NW; ++x)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float wv = Ws[x][k][4 * tx + j];
          acc[x][0][j] += a0 * wv;
          acc[x][1][j] += a1 * wv;
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int dst = oid[2 * ty + i];
    if (dst < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + 4 * tx + j;
      if (n >= N) continue;
      const int64_t o = (int64_t)blockIdx.z * o_zs + (int64_t)dst * ldo + n;
      if (EPI == GL_EPI_GLU) {
        stf((T*)out, o, glu_act(acc[0][i][j], acc[NW - 1][i][j], act, limit));
      } else {
        float v = acc[0][i][j];
        if (gate) v *= 1.0f / (1.0f + expf(-gate[(int64_t)dst * gate_ld + blockIdx.z]));
        if (store_typed) stf((T*)out, o, v);
        else ((float*)out)[o] = v;
      }
    }
  }
}

// ---------------------------------------------------------------- bf16 operands: the same contract on the tensor cores
// mma.sync m16n8k16 (bf16 x bf16 -> fp32).  CTA = 4 warps, 32 rows x (128 outputs | 64 gate + 64 up outputs), K in steps of
// 32 through shared memory (rows padded to 80 bytes: conflict-free ldmatrix), next tile's global loads in flight during the
// current tile's MMAs.  The routing weight scales the gathered input row in fp32 before it is rounded to the bf16 operand.
// Needs K % 8 == 0 and 16-byte aligned rows (the dispatcher checks; otherwise the CUDA-core kernel above runs).
constexpr int GM_BK = 32;
constexpr int GM_LD = GM_BK + 8;
constexpr int GM_WROWS = 128;

template <int EPI>
__global__ void __launch_bounds__(128)
    grouped_mma_kernel(const __nv_bfloat16* __restrict__ a, int lda, const int32_t* __restrict__ sorted_ids, int gather_div,
                       const float* __restrict__ row_scale, const __nv_bfloat16* __restrict__ w, int64_t w_stride,
                       const int32_t* __restrict__ tile_expert, const int32_t* __restrict__ num_tiles, int M, int N, int K,
                       void* __restrict__ out, int ldo, int scatter, float limit, int act, int64_t a_zs, int64_t o_zs,
                       int store_typed, const float* __restrict__ gate, int gate_ld) {
  griddep_launch();
  griddep_wait();
  constexpr int R = 1;            // 32-row sub-tiles per CTA (prompt-sized batches take grouped_mma_pipe_kernel instead)
  constexpr int BM = MOE_BM * R;  // rows per tile
  __shared__ __align__(16) __nv_bfloat16 As[BM][GM_LD];
  __shared__ __align__(16) __nv_bfloat16 Ws[GM_WROWS][GM_LD];
  __shared__ int32_t rid[BM];
  __shared__ int32_t oid[BM];
  __shared__ float rsc[BM];
  const int tile = blockIdx.x;
  if (num_tiles && tile >= *num_tiles) return;
  const int e = tile_expert ? tile_expert[tile] : blockIdx.z;  // z-batched dense launches: one weight per batch index
  const __nv_bfloat16* we = w + (int64_t)e * w_stride;
  a += (int64_t)blockIdx.z * a_zs;
  constexpr int BN = EPI == GL_EPI_GLU ? 64 : 128;  // outputs per CTA
  const int n0 = blockIdx.y * BN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < BM; i += 128) {
    const int r = tile * BM + i;
    int src = -1, dst = -1;
    float sc = 1.0f;
    if (sorted_ids) {
      const int id = sorted_ids[r];
      if (id >= 0) {
        src = gather_div > 0 ? id / gather_div : r;
        dst = scatter ? id : r;
        if (row_scale) sc = row_scale[id];
      }
    } else if (r < M) {
      src = dst = r;
    }
    rid[i] = src;
    oid[i] = dst;
    rsc[i] = sc;
  }
  __syncthreads();
  // global -> register staging: R 16-byte vectors of A and four of W per thread and K step
  const int a_row = tid >> 2, kc = (tid & 3) * 8;
  int a_src[R];
  float a_sc[R];
#pragma unroll
  for (int rr = 0; rr < R; ++rr) {
    a_src[rr] = rid[a_row + 32 * rr];
    a_sc[rr] = rsc[a_row + 32 * rr];
  }
  const __nv_bfloat16* w_ptr[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = (tid + 128 * i) >> 2;  // 0..127
    int n, grow;
    if (EPI == GL_EPI_GLU) {
      n = n0 + (r & 63);
      grow = (r < 64 ? 0 : N) + n;
    } else {
      n = n0 + r;
      grow = n;
    }
    w_ptr[i] = n < N ? we + (int64_t)grow * K : nullptr;
  }
  uint4 ra[R], rw[4];
  auto fetch = [&](int k0) {
    const bool kin = k0 + kc < K;
#pragma unroll
    for (int rr = 0; rr < R; ++rr) {
      ra[rr] = make_uint4(0, 0, 0, 0);
      if (a_src[rr] >= 0 && kin) {
        ra[rr] = *reinterpret_cast<const uint4*>(a + (int64_t)a_src[rr] * lda + k0 + kc);
        if (a_sc[rr] != 1.0f) {
          __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&ra[rr]);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h2[i]);
            h2[i] = __floats2bfloat162_rn(f.x * a_sc[rr], f.y * a_sc[rr]);
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
      rw[i] = (w_ptr[i] && kin) ? *reinterpret_cast<const uint4*>(w_ptr[i] + k0 + kc) : make_uint4(0, 0, 0, 0);
  };
  float acc[2 * R][4][4];
#pragma unroll
  for (int i = 0; i < 2 * R; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;
  // first shared-memory row of this warp's n8 tile j
  auto nrow = [&](int j) { return EPI == GL_EPI_GLU ? (j < 2 ? 16 * warp + 8 * j : 64 + 16 * warp + 8 * (j - 2)) : 32 * warp + 8 * j; };
  fetch(0);
  for (int k0 = 0; k0 < K; k0 += GM_BK) {
#pragma unroll
    for (int rr = 0; rr < R; ++rr) *reinterpret_cast<uint4*>(&As[a_row + 32 * rr][kc]) = ra[rr];
#pragma unroll
    for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(&Ws[(tid + 128 * i) >> 2][kc]) = rw[i];
    __syncthreads();
    if (k0 + GM_BK < K) fetch(k0 + GM_BK);
#pragma unroll
    for (int kk = 0; kk < GM_BK; kk += 16) {
      uint32_t bf[2][4];
#pragma unroll
      for (int jp = 0; jp < 2; ++jp) {
        const int mi = lane >> 3;  // matrix of the x4 load: tile 2 jp + mi / 2, k half mi % 2
        ldmatrix_x4(bf[jp], smem_u32(&Ws[nrow(2 * jp + (mi >> 1)) + (lane & 7)][kk + (mi & 1) * 8]));
      }
#pragma unroll
      for (int mt = 0; mt < 2 * R; ++mt) {
        uint32_t af[4];
        ldmatrix_x4(af, smem_u32(&As[mt * 16 + (lane & 15)][kk + (lane >> 4) * 8]));
#pragma unroll
        for (int jp = 0; jp < 2; ++jp) {
          mma_bf16_16816(acc[mt][2 * jp], af, bf[jp][0], bf[jp][1]);
          mma_bf16_16816(acc[mt][2 * jp + 1], af, bf[jp][2], bf[jp][3]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int mt = 0; mt < 2 * R; ++mt)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int r = mt * 16 + (lane >> 2) + (c >= 2 ? 8 : 0);
      const int dst = oid[r];
      if (dst < 0) continue;
      const int col = 2 * (lane & 3) + (c & 1);
      if (EPI == GL_EPI_GLU) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int n = n0 + 16 * warp + 8 * j + col;
          if (n >= N) continue;
          ((__nv_bfloat16*)out)[(int64_t)blockIdx.z * o_zs + (int64_t)dst * ldo + n] =
              __float2bfloat16_rn(glu_act(acc[mt][j][c], acc[mt][j + 2][c], act, limit));
        }
      } else {
        const float gt = gate ? 1.0f / (1.0f + expf(-gate[(int64_t)dst * gate_ld + blockIdx.z])) : 1.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int n = n0 + 32 * warp + 8 * j + col;
          if (n >= N) continue;
          const int64_t o = (int64_t)blockIdx.z * o_zs + (int64_t)dst * ldo + n;
          if (store_typed) ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(acc[mt][j][c] * gt);
          else ((float*)out)[o] = acc[mt][j][c] * gt;
        }
      }
    }
}

// Prompt-sized bf16 batches.  moe_gather_scale_kernel lays the (token, choice) pairs out in sorted order ONCE, each row
// scaled by its routing weight in fp32 and rounded to the bf16 operand (padding rows are zeros), so that the expert GEMMs
// read plain contiguous rows; grouped_mma_pipe_kernel then runs 128 rows x 128 weight rows per CTA (8 warps, 64 x 32 each)
// with both operands copied by cp.async through a 3-stage ring of K = 64 slices: no register staging, two slices in
// flight under the MMAs.  Same K order per row as the 32-row kernel: the results are bit-identical.
__global__ void moe_gather_scale_kernel(const __nv_bfloat16* __restrict__ h, int ldh, const int32_t* __restrict__ sorted_ids,
                                        int top, const float* __restrict__ weight, const int32_t* __restrict__ num_tiles,
                                        int tile_rows, __nv_bfloat16* __restrict__ out, int W) {
  griddep_launch();
  griddep_wait();
  const int r = blockIdx.x;
  if (r >= *num_tiles * tile_rows) return;
  const int id = sorted_ids[r];
  const float sc = id >= 0 ? (weight ? weight[id] : 1.0f) : 0.f;
  const __nv_bfloat16* src = h + (int64_t)(id >= 0 ? id / top : 0) * ldh;
  for (int c = threadIdx.x * 8; c < W; c += blockDim.x * 8) {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (id >= 0) {
      v = *reinterpret_cast<const uint4*>(src + c);
      if (sc != 1.0f) {
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h2[i]);
          h2[i] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
        }
      }
    }
    *reinterpret_cast<uint4*>(out + (int64_t)r * W + c) = v;
  }
}

constexpr int GP_BM = MOE_BM * MOE_WIDE;
constexpr int GP_STAGES = 3;
constexpr int GP_THREADS = 256;
constexpr int GP_BK = 64;  // K slice: 128 bytes of every operand row
constexpr int GP_LD = GP_BK + 8;
constexpr int GP_CPT = (GP_BM * GP_BK / 8) / GP_THREADS;  // 16-byte copies per thread, operand and slice
constexpr int GP_STAGE_ELEMS = (GP_BM + GM_WROWS) * GP_LD;

template <int EPI>
__global__ void __launch_bounds__(GP_THREADS)
    grouped_mma_pipe_kernel(const __nv_bfloat16* __restrict__ a, int lda, const int32_t* __restrict__ sorted_ids,
                            const __nv_bfloat16* __restrict__ w, int64_t w_stride, const int32_t* __restrict__ tile_expert,
                            const int32_t* __restrict__ num_tiles, int N, int K, void* __restrict__ out, int ldo, int scatter,
                            float limit, int act) {
  griddep_launch();
  griddep_wait();
  extern __shared__ __align__(16) unsigned char gp_smem[];
  __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(gp_smem);                             // [stages][A 128 | W 128][GP_LD]
  int32_t* oid = reinterpret_cast<int32_t*>(gp_smem + (size_t)GP_STAGES * GP_STAGE_ELEMS * 2);  // [128]
  const int tile = blockIdx.x;
  if (tile >= *num_tiles) return;
  const int e = tile_expert[tile];
  const __nv_bfloat16* we = w + (int64_t)e * w_stride;
  constexpr int BN = EPI == GL_EPI_GLU ? 64 : 128;  // outputs per CTA
  const int n0 = blockIdx.y * BN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp >> 2, wn = warp & 3;  // 2 x 4 warps: 64 rows x (32 outputs | 16 gate + 16 up)
  if (tid < GP_BM) {
    const int id = sorted_ids[tile * GP_BM + tid];
    oid[tid] = id < 0 ? -1 : (scatter ? id : tile * GP_BM + tid);
  }
  // this thread's copies per K slice: GP_CPT of A and GP_CPT of W, 16 bytes each
  const __nv_bfloat16* src[2 * GP_CPT];
  uint32_t dst[2 * GP_CPT];
  const int kc = (tid & (GP_BK / 8 - 1)) * 8;
#pragma unroll
  for (int i = 0; i < 2 * GP_CPT; ++i) {
    const int r = (tid + GP_THREADS * (i % GP_CPT)) / (GP_BK / 8);  // 0..127
    if (i < GP_CPT) {
      src[i] = a + (int64_t)(tile * GP_BM + r) * lda + kc;
      dst[i] = (uint32_t)((r * GP_LD + kc) * 2);
    } else {
      int n, grow;
      if (EPI == GL_EPI_GLU) {
        n = n0 + (r & 63);
        grow = (r < 64 ? 0 : N) + n;
      } else {
        n = n0 + r;
        grow = n;
      }
      src[i] = n < N ? we + (int64_t)grow * K + kc : nullptr;
      dst[i] = (uint32_t)(((GP_BM + r) * GP_LD + kc) * 2);
    }
  }
  const uint32_t ring_u32 = smem_u32(ring);
  auto issue = [&](int kt) {
    const int k0 = kt * GP_BK;
    if (k0 < K) {
      const uint32_t base = ring_u32 + (uint32_t)((kt % GP_STAGES) * GP_STAGE_ELEMS * 2);
      const bool kin = k0 + kc < K;
#pragma unroll
      for (int i = 0; i < 2 * GP_CPT; ++i) {
        const bool ok = kin && src[i] != nullptr;
        cp_async16(base + dst[i], ok ? (const void*)(src[i] + k0) : (const void*)a, ok);
      }
    }
    cp_async_commit();  // an empty group past the end keeps the wait counts uniform
  };
  float acc[4][4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;
  // first shared-memory weight row of this warp's n8 tile j
  auto nrow = [&](int j) { return EPI == GL_EPI_GLU ? (j < 2 ? 16 * wn + 8 * j : 64 + 16 * wn + 8 * (j - 2)) : 32 * wn + 8 * j; };
  const int KT = (K + GP_BK - 1) / GP_BK;
#pragma unroll
  for (int s = 0; s < GP_STAGES - 1; ++s) issue(s);
  for (int kt = 0; kt < KT; ++kt) {
    cp_async_wait<GP_STAGES - 2>();  // slice kt has landed (this thread's part)
    __syncthreads();                 // ... everyone's part; and everyone is done with slice kt - 1, whose stage is refilled next
    issue(kt + GP_STAGES - 1);
    const __nv_bfloat16* As = ring + (kt % GP_STAGES) * GP_STAGE_ELEMS;
    const __nv_bfloat16* Ws = As + GP_BM * GP_LD;
#pragma unroll
    for (int kk = 0; kk < GP_BK; kk += 16) {
      uint32_t bf[2][4];
#pragma unroll
      for (int jp = 0; jp < 2; ++jp) {
        const int mi = lane >> 3;  // matrix of the x4 load: tile 2 jp + mi / 2, k half mi % 2
        ldmatrix_x4(bf[jp], smem_u32(Ws + (nrow(2 * jp + (mi >> 1)) + (lane & 7)) * GP_LD + kk + (mi & 1) * 8));
      }
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        uint32_t af[4];
        ldmatrix_x4(af, smem_u32(As + (64 * wm + mt * 16 + (lane & 15)) * GP_LD + kk + (lane >> 4) * 8));
#pragma unroll
        for (int jp = 0; jp < 2; ++jp) {
          mma_bf16_16816(acc[mt][2 * jp], af, bf[jp][0], bf[jp][1]);
          mma_bf16_16816(acc[mt][2 * jp + 1], af, bf[jp][2], bf[jp][3]);
        }
      }
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int mt = 0; mt < 4; ++mt)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int r = 64 * wm + mt * 16 + (lane >> 2) + (c >= 2 ? 8 : 0);
      const int dstrow = oid[r];
      if (dstrow < 0) continue;
      const int col = 2 * (lane & 3) + (c & 1);
      if (EPI == GL_EPI_GLU) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int n = n0 + 16 * wn + 8 * j + col;
          if (n >= N) continue;
          ((__nv_bfloat16*)out)[(int64_t)dstrow * ldo + n] = __float2bfloat16_rn(glu_act(acc[mt][j][c], acc[mt][j + 2][c], act, limit));
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int n = n0 + 32 * wn + 8 * j + col;
          if (n < N) ((float*)out)[(int64_t)dstrow * ldo + n] = acc[mt][j][c];
        }
      }
    }
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_moe_topk(const float* logits, int ld, const float* bias, int mode, int32_t* topk_idx, float* topk_weight, int T, int E,
                  int top, void* stream) {
  B200_REQUIRE(logits && topk_idx && topk_weight, "moe_topk: null pointer");
  B200_REQUIRE(E >= 1 && top >= 1 && top <= E && ld >= E, "moe_topk: top %d of %d experts", top, E);
  B200_REQUIRE(mode == B200_ROUTE_SIGMOID || mode == B200_ROUTE_SOFTMAX_TOP || mode == B200_ROUTE_SOFTMAX_RENORM,
               "moe_topk: routing mode %d", mode);
  if (T <= 0) return B200_OK;
  B200_CUDA_OK(launch_kernel(moe_topk_kernel, dim3((T + 127) / 128), dim3(128), 0, (cudaStream_t)stream, logits, ld, bias, mode, E,
                             top, topk_idx, topk_weight, T));
  return B200_OK;
}

int b200_moe_tile_rows(void) { return MOE_BM; }

int b200_moe_gather_scale(const void* h, int ldh, const int32_t* sorted_ids, int cap, int top, const float* weight,
                          const int32_t* num_tiles, int tile_rows, void* out, int W, void* stream) {
  B200_REQUIRE(h && sorted_ids && num_tiles && out, "moe_gather_scale: null pointer");
  B200_REQUIRE(top >= 1 && W % 8 == 0 && ldh % 8 == 0 && !((uintptr_t)h & 15) && !((uintptr_t)out & 15),
               "moe_gather_scale: rows of %d bf16 elements (pitch %d) are not 16-byte vectors", W, ldh);
  if (cap <= 0) return B200_OK;
  B200_CUDA_OK(launch_kernel(moe_gather_scale_kernel, dim3(cap), dim3(128), 0, (cudaStream_t)stream, (const __nv_bfloat16*)h, ldh,
                             sorted_ids, top, weight, num_tiles, tile_rows, (__nv_bfloat16*)out, W));
  return B200_OK;
}

int b200_moe_align(const int32_t* topk_idx, int npairs, int E, int32_t* sorted_ids, int cap, int32_t* tile_expert, int max_tiles,
                   int32_t* num_tiles, int tile_rows, void* stream) {
  B200_REQUIRE(topk_idx && sorted_ids && tile_expert && num_tiles, "moe_align: null pointer");
  B200_REQUIRE(E >= 1 && E <= 4096, "moe_align: %d experts", E);
  B200_REQUIRE(tile_rows == MOE_BM || tile_rows == MOE_BM * MOE_WIDE, "moe_align: %d rows per tile", tile_rows);
  B200_REQUIRE(max_tiles >= (npairs + tile_rows - 1) / tile_rows + E && cap >= max_tiles * tile_rows,
               "moe_align: %d tiles / %d rows cannot hold %d pairs of %d experts", max_tiles, cap, npairs, E);
  if (npairs <= 0) return B200_OK;
  B200_CUDA_OK(launch_kernel(moe_align_kernel, dim3(1), dim3(1024), (size_t)2 * E * 4, (cudaStream_t)stream, topk_idx, npairs, E,
                             sorted_ids, cap, tile_expert, max_tiles, num_tiles, tile_rows));
  return B200_OK;
}

int b200_grouped_linear(const void* a, int lda, const int32_t* sorted_ids, int gather_div, const float* row_scale, const void* w,
                        int64_t w_expert_stride, const int32_t* tile_expert, const int32_t* num_tiles, int row_tiles, int M, int N,
                        int K, int dtype, void* out, int ldo, int scatter, int glu, int act, float limit, int tile_rows,
                        void* stream) {
  B200_REQUIRE(a && w && out, "grouped_linear: null pointer");
  B200_REQUIRE(N > 0 && K > 0 && row_tiles >= 0, "grouped_linear: bad shape N=%d K=%d", N, K);
  B200_REQUIRE(sorted_ids || (!tile_expert && !num_tiles && !row_scale), "grouped_linear: expert tiles need the sorted pair list");
  B200_REQUIRE(!glu || act == B200_ACT_SWISH_CLAMPED || act == B200_ACT_SILU || act == B200_ACT_GELU_TANH,
               "grouped_linear: activation %d", act);
  if (row_tiles == 0) return B200_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const bool mma_ok = dtype == B200_BF16 && K % 8 == 0 && lda % 8 == 0 && w_expert_stride % 8 == 0 && !((uintptr_t)a & 15) &&
                      !((uintptr_t)w & 15);
  B200_REQUIRE(tile_rows == MOE_BM || (tile_rows == MOE_BM * MOE_WIDE && mma_ok),
               "grouped_linear: %d rows per tile (32, or 128 for 16-byte aligned bf16 operands)", tile_rows);
  const float* no_gate = nullptr;
  if (mma_ok) {
    using BT = __nv_bfloat16;
#define GM_LAUNCH(EPI, BN)                                                                                                   \
  B200_CUDA_OK(launch_kernel(grouped_mma_kernel<EPI>, dim3(row_tiles, (N + BN - 1) / BN), dim3(128), 0, st, (const BT*)a, lda, \
                             sorted_ids, gather_div, row_scale, (const BT*)w, w_expert_stride, tile_expert, num_tiles, M, N, K, \
                             out, ldo, scatter, limit, act, (int64_t)0, (int64_t)0, 0, no_gate, 0))
    if (tile_rows == MOE_BM) {
      if (glu) GM_LAUNCH(GL_EPI_GLU, 64);
      else GM_LAUNCH(GL_EPI_STORE, 128);
    } else {
      // wide tiles: the operand rows are the gathered, pre-scaled list (one row per sorted pair, no gather and no scale here)
      B200_REQUIRE(sorted_ids && tile_expert && num_tiles && gather_div == 0 && !row_scale,
                   "grouped_linear: 128-row tiles read the gathered pair list (b200_moe_gather_scale)");
      const size_t smem = (size_t)GP_STAGES * GP_STAGE_ELEMS * 2 + GP_BM * 4;
#define GP_LAUNCH(EPI, BN)                                                                                                     \
  do {                                                                                                                         \
    B200_CUDA_OK(cudaFuncSetAttribute(grouped_mma_pipe_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));  \
    B200_CUDA_OK(launch_kernel(grouped_mma_pipe_kernel<EPI>, dim3(row_tiles, (N + BN - 1) / BN), dim3(GP_THREADS), smem, st,   \
                               (const BT*)a, lda, sorted_ids, (const BT*)w, w_expert_stride, tile_expert, num_tiles, N, K, out, \
                               ldo, scatter, limit, act));                                                                     \
  } while (0)
      if (glu) GP_LAUNCH(GL_EPI_GLU, 64);
      else GP_LAUNCH(GL_EPI_STORE, 128);
#undef GP_LAUNCH
    }
#undef GM_LAUNCH
    return B200_OK;
  }
  dim3 grid(row_tiles, (N + GL_BN - 1) / GL_BN);
  B200_DISPATCH_ELEM(dtype, ET, {
    if (glu)
      B200_CUDA_OK(launch_kernel(grouped_linear_kernel<ET, GL_EPI_GLU>, grid, dim3(GL_THREADS), 0, st, (const ET*)a, lda, sorted_ids,
                                 gather_div, row_scale, (const ET*)w, w_expert_stride, tile_expert, num_tiles, M, N, K, out, ldo,
                                 scatter, limit, act, (int64_t)0, (int64_t)0, 0, no_gate, 0));
    else
      B200_CUDA_OK(launch_kernel(grouped_linear_kernel<ET, GL_EPI_STORE>, grid, dim3(GL_THREADS), 0, st, (const ET*)a, lda,
                                 sorted_ids, gather_div, row_scale, (const ET*)w, w_expert_stride, tile_expert, num_tiles, M, N, K,
                                 out, ldo, scatter, limit, act, (int64_t)0, (int64_t)0, 0, no_gate, 0));
  });
  return B200_OK;
}

int b200_batched_linear(const void* a, int lda, int64_t a_batch_stride, const void* w, int64_t w_batch_stride, void* out, int ldo,
                        int64_t out_batch_stride, int batch, int M, int N, int K, int dtype, int out_typed, const float* gate,
                        int gate_ld, void* stream) {
  B200_REQUIRE(a && w && out, "batched_linear: null pointer");
  B200_REQUIRE(N > 0 && K > 0 && batch >= 1 && batch <= 65535, "batched_linear: bad shape N=%d K=%d batch=%d", N, K, batch);
  if (M <= 0) return B200_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int row_tiles = (M + MOE_BM - 1) / MOE_BM;
  const int32_t* none = nullptr;
  const float* no_scale = nullptr;
  const bool mma_ok = dtype == B200_BF16 && K % 8 == 0 && lda % 8 == 0 && a_batch_stride % 8 == 0 && w_batch_stride % 8 == 0 &&
                      !((uintptr_t)a & 15) && !((uintptr_t)w & 15);
  if (mma_ok) {
    using BT = __nv_bfloat16;
    B200_CUDA_OK(launch_kernel(grouped_mma_kernel<GL_EPI_STORE>, dim3(row_tiles, (N + 127) / 128, batch), dim3(128), 0, st,
                               (const BT*)a, lda, none, 0, no_scale, (const BT*)w, w_batch_stride, none, none, M, N, K, out, ldo, 0,
                               0.f, 0, a_batch_stride, out_batch_stride, out_typed, gate, gate_ld));
    return B200_OK;
  }
  dim3 grid(row_tiles, (N + GL_BN - 1) / GL_BN, batch);
  B200_DISPATCH_ELEM(dtype, ET,
                     B200_CUDA_OK(launch_kernel(grouped_linear_kernel<ET, GL_EPI_STORE>, grid, dim3(GL_THREADS), 0, st, (const ET*)a,
                                                lda, none, 0, no_scale, (const ET*)w, w_batch_stride, none, none, M, N, K, out, ldo, 0,
                                                0.f, 0, a_batch_stride, out_batch_stride, out_typed, gate, gate_ld)));
  return B200_OK;
}

}  // extern "C"
