// Gated linear recurrence whose forget gate also decides what is written (the HGRN2 form of linear attention), over a ragged
// batch.  Per head, with a state S [D][P] that starts at zero and lives in fp32 per sequence slot:
//     S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T,     o_t = S_t^T q_t
// where q = silu(raw q), f = lower + (1 - lower) sigmoid(raw f + bias) per channel, and v has P columns per head: the "key" of
// the outer product is 1 - f, there is no other key and no scale.
//   * gated_scan_prep: turns the raw q and f columns of the projection rows into q and f IN PLACE (fp32);
//   * gated_scan: CTA = (16 value columns, head, sequence), 256 threads = 16 slices of the D state rows x 16 columns; a thread
//     keeps its 4 KR state elements in registers (rows 64 k + 4 slice + e: a half-warp reads a token's f and q as conflict-free
//     float4), tokens are staged 16 at a time with cp.async one chunk ahead and taken four at a time (the four row reductions
//     of o, four shuffles each, run under the next tokens' updates), the update is S = v + f (S - v) (one subtraction and one
//     FMA; no 1 - f that would lose digits where f is close to 1).  Launched without programmatic early start: its few
//     long-running CTAs must spread evenly over the SMs.
// The state is stored TRANSPOSED, [slots][H][P][D], so that a warp's loads and stores of it are whole 128-byte lines.
// A sequence whose portion starts at position 0 ignores what its slot held.
#include "hybrid_common.cuh"

namespace b200 {

constexpr int GS_COLS = 16;     // value columns per CTA
constexpr int GS_SLICES = 16;   // lanes that share a column (slices of the state rows)
constexpr int GS_THREADS = GS_COLS * GS_SLICES;
constexpr int GS_CHUNK = 16;    // tokens staged per round

__global__ void gated_scan_prep_kernel(float* __restrict__ proj, int ld, int q_col0, int f_col0, int n,
                                       const float* __restrict__ f_bias, const float* __restrict__ lower, int64_t total) {
  griddep_launch();
  griddep_wait();
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = idx / n;
    const int i = (int)(idx - t * n);
    float* row = proj + t * ld;
    row[q_col0 + i] = silu_f(row[q_col0 + i]);
    const float l = lower[i];
    row[f_col0 + i] = l + (1.0f - l) / (1.0f + expf(-(row[f_col0 + i] + f_bias[i])));
  }
}

__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src, bool ok) {
  const int n = ok ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(dst), "l"(src), "r"(n) : "memory");
}

template <int KR>
__global__ void __launch_bounds__(GS_THREADS)
    gated_scan_kernel(const float* __restrict__ proj, int ld, int q_col0, int f_col0, int v_col0, float* __restrict__ state,
                      const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_slot,
                      const int32_t* __restrict__ seq_pos0, float* __restrict__ out, int H, int D, int P, int vec) {
  griddep_launch();
  griddep_wait();
  constexpr int Dp = 4 * GS_SLICES * KR;
  extern __shared__ __align__(16) float gs_sm[];
  float* qs = gs_sm;                              // [2][GS_CHUNK][Dp]
  float* fs = qs + 2 * GS_CHUNK * Dp;             // [2][GS_CHUNK][Dp]
  float* vs = fs + 2 * GS_CHUNK * Dp;             // [2][GS_CHUNK][GS_COLS]
  float* os = vs + 2 * GS_CHUNK * GS_COLS;        // [GS_CHUNK][GS_COLS]
  const int tid = threadIdx.x, r = tid & (GS_SLICES - 1), c = tid / GS_SLICES;
  const int j0 = blockIdx.x * GS_COLS, h = blockIdx.y, sq = blockIdx.z;
  const int t0 = seq_start[sq], n = seq_start[sq + 1] - t0;
  if (n <= 0) return;
  const int j = j0 + c;
  const bool col_ok = j < P;
  float* st = state + (((int64_t)seq_slot[sq] * H + h) * P + (col_ok ? j : 0)) * D;
  float S[KR][4];
#pragma unroll
  for (int k = 0; k < KR; ++k)
#pragma unroll
    for (int e = 0; e < 4; ++e) S[k][e] = 0.f;
  if (seq_pos0[sq] > 0 && col_ok) {
#pragma unroll
    for (int k = 0; k < KR; ++k) {
      const int i = 4 * GS_SLICES * k + 4 * r;
      if (vec && i + 3 < D) {
        const float4 a = *reinterpret_cast<const float4*>(st + i);
        S[k][0] = a.x, S[k][1] = a.y, S[k][2] = a.z, S[k][3] = a.w;
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (i + e < D) S[k][e] = st[i + e];
      }
    }
  }
  // a chunk of tokens: q and f rows of this head (columns past D are zeros: their state rows stay zero), the CTA's v columns
  auto stage = [&](int ch, int buf) {
    const int tk0 = ch * GS_CHUNK;
    const float* base = proj + (int64_t)(t0 + tk0) * ld;
    if (vec) {  // 16-byte copies: D, ld and the column offsets are multiples of four floats and the rows 16-byte aligned
      for (int idx = tid; idx < GS_CHUNK * (Dp / 4); idx += GS_THREADS) {
        const int tk = idx / (Dp / 4), i = (idx - tk * (Dp / 4)) * 4;
        const bool ok = tk0 + tk < n && i < D;
        const float* src = base + (int64_t)(ok ? tk : 0) * ld + (int64_t)h * D + (ok ? i : 0);
        cp_async16(smem_u32(qs + (buf * GS_CHUNK + tk) * Dp + i), src + q_col0, ok);
        cp_async16(smem_u32(fs + (buf * GS_CHUNK + tk) * Dp + i), src + f_col0, ok);
      }
    } else {
      for (int idx = tid; idx < GS_CHUNK * Dp; idx += GS_THREADS) {
        const int tk = idx / Dp, i = idx - tk * Dp;
        const bool ok = tk0 + tk < n && i < D;
        const float* src = base + (int64_t)(ok ? tk : 0) * ld + (int64_t)h * D + (ok ? i : 0);
        cp_async4(smem_u32(qs + (buf * GS_CHUNK + tk) * Dp + i), src + q_col0, ok);
        cp_async4(smem_u32(fs + (buf * GS_CHUNK + tk) * Dp + i), src + f_col0, ok);
      }
    }
    for (int idx = tid; idx < GS_CHUNK * GS_COLS; idx += GS_THREADS) {
      const int tk = idx / GS_COLS, cc = idx - tk * GS_COLS;
      const bool ok = tk0 + tk < n && j0 + cc < P;
      cp_async4(smem_u32(vs + (buf * GS_CHUNK + tk) * GS_COLS + cc),
                base + (int64_t)(ok ? tk : 0) * ld + v_col0 + (int64_t)h * P + (ok ? j0 + cc : 0), ok);
    }
    cp_async_commit();
  };
  const int nch = (n + GS_CHUNK - 1) / GS_CHUNK;
  stage(0, 0);
  for (int ch = 0; ch < nch; ++ch) {
    const int buf = ch & 1;
    if (ch + 1 < nch) {
      stage(ch + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int cn = n - ch * GS_CHUNK < GS_CHUNK ? n - ch * GS_CHUNK : GS_CHUNK;
    // one token: the thread's state elements, and its share of o = S^T q (two accumulators: half the dependent chain)
    auto token = [&](int tk) -> float {
      const float v = vs[(buf * GS_CHUNK + tk) * GS_COLS + c];
      const float* fr = fs + (buf * GS_CHUNK + tk) * Dp + 4 * r;
      const float* qr = qs + (buf * GS_CHUNK + tk) * Dp + 4 * r;
      float oa = 0.f, ob = 0.f;
#pragma unroll
      for (int k = 0; k < KR; ++k) {
        const float4 f4 = *reinterpret_cast<const float4*>(fr + 4 * GS_SLICES * k);
        const float4 q4 = *reinterpret_cast<const float4*>(qr + 4 * GS_SLICES * k);
        S[k][0] = fmaf(f4.x, S[k][0] - v, v);
        S[k][1] = fmaf(f4.y, S[k][1] - v, v);
        S[k][2] = fmaf(f4.z, S[k][2] - v, v);
        S[k][3] = fmaf(f4.w, S[k][3] - v, v);
        oa = fmaf(S[k][0], q4.x, oa);
        ob = fmaf(S[k][1], q4.y, ob);
        oa = fmaf(S[k][2], q4.z, oa);
        ob = fmaf(S[k][3], q4.w, ob);
      }
      return oa + ob;
    };
    auto reduce = [&](float o) -> float {  // over the 16 lanes that share the column
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      o += __shfl_xor_sync(0xffffffffu, o, 4);
      o += __shfl_xor_sync(0xffffffffu, o, 8);
      return o;
    };
    int tk = 0;
    for (; tk + 4 <= cn; tk += 4) {
      float o0 = token(tk), o1 = token(tk + 1), o2 = token(tk + 2), o3 = token(tk + 3);
      o0 = reduce(o0), o1 = reduce(o1), o2 = reduce(o2), o3 = reduce(o3);
      if (r == 0) {
        os[tk * GS_COLS + c] = o0;
        os[(tk + 1) * GS_COLS + c] = o1;
        os[(tk + 2) * GS_COLS + c] = o2;
        os[(tk + 3) * GS_COLS + c] = o3;
      }
    }
    for (; tk < cn; ++tk) {
      const float o = reduce(token(tk));
      if (r == 0) os[tk * GS_COLS + c] = o;
    }
    __syncthreads();  // the chunk's outputs are complete, and its buffer may be refilled
    for (int idx = tid; idx < cn * GS_COLS; idx += GS_THREADS) {
      const int tk = idx / GS_COLS, cc = idx - tk * GS_COLS;
      if (j0 + cc < P) out[((int64_t)(t0 + ch * GS_CHUNK + tk) * H + h) * P + j0 + cc] = os[idx];
    }
  }
  if (col_ok) {
    // state rows past D were fed f = 0 and hold v: they are not part of the state
#pragma unroll
    for (int k = 0; k < KR; ++k) {
      const int i = 4 * GS_SLICES * k + 4 * r;
      if (vec && i + 3 < D) {
        *reinterpret_cast<float4*>(st + i) = make_float4(S[k][0], S[k][1], S[k][2], S[k][3]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (i + e < D) st[i + e] = S[k][e];
      }
    }
  }
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_gated_scan_prep(float* proj, int ld, int q_col0, int f_col0, int n, const float* f_bias, const float* lower, int T,
                         void* stream) {
  B200_REQUIRE(proj && f_bias && lower && n >= 1, "gated_scan_prep: null pointer");
  if (T <= 0) return B200_OK;
  const int64_t total = (int64_t)T * n;
  int64_t blocks = (total + 255) / 256;
  blocks = blocks > 148 * 16 ? 148 * 16 : blocks;
  B200_CUDA_OK(launch_kernel(gated_scan_prep_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, proj, ld, q_col0,
                             f_col0, n, f_bias, lower, total));
  return B200_OK;
}

int b200_gated_scan(const float* proj, int ld, int q_col0, int f_col0, int v_col0, float* state, const int32_t* seq_start,
                    const int32_t* seq_slot, const int32_t* seq_pos0, float* out, int B, int H, int D, int P, void* stream) {
  B200_REQUIRE(proj && state && seq_start && seq_slot && seq_pos0 && out, "gated_scan: null pointer");
  B200_REQUIRE(H >= 1 && D >= 1 && P >= 1, "gated_scan: bad shape");
  if (D > 512) {
    set_last_error("gated_scan: %d state rows per head exceed 512", D);
    return B200_ERR_UNSUPPORTED;
  }
  if (B <= 0) return B200_OK;
  B200_REQUIRE(B <= 65535 && H <= 65535, "gated_scan: %d sequences x %d heads exceed the grid", B, H);
  const int vec = D % 4 == 0 && ld % 4 == 0 && q_col0 % 4 == 0 && f_col0 % 4 == 0 && ((uintptr_t)proj & 15) == 0 &&
                  ((uintptr_t)state & 15) == 0;
  dim3 grid((P + GS_COLS - 1) / GS_COLS, H, B);
  cudaStream_t st = (cudaStream_t)stream;
#define GS_LAUNCH(KR)                                                                                                     \
  do {                                                                                                                    \
    const size_t smem = (size_t)(4 * GS_CHUNK * 4 * GS_SLICES * KR + 3 * GS_CHUNK * GS_COLS) * 4;                         \
    if (smem > 48 * 1024)                                                                                                 \
      B200_CUDA_OK(cudaFuncSetAttribute(gated_scan_kernel<KR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    B200_CUDA_OK(launch_kernel_serial(gated_scan_kernel<KR>, grid, dim3(GS_THREADS), smem, st, proj, ld, q_col0, f_col0,  \
                                      v_col0, state, seq_start, seq_slot, seq_pos0, out, H, D, P, vec));                 \
  } while (0)
  if (D <= 64) GS_LAUNCH(1);
  else if (D <= 128) GS_LAUNCH(2);
  else if (D <= 256) GS_LAUNCH(4);
  else GS_LAUNCH(8);
#undef GS_LAUNCH
  return B200_OK;
}

}  // extern "C"
