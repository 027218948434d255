// Gated linear recurrence whose forget gate also decides what is written (the HGRN2 form of linear attention), over a ragged
// batch.  Per head, with a state S [D][P] that starts at zero and lives in fp32 per sequence slot:
//     S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T,     o_t = S_t^T q_t
// where q = silu(raw q), f = lower + (1 - lower) sigmoid(raw f + bias) per channel, and v has P columns per head: the "key" of
// the outer product is 1 - f, there is no other key and no scale.
//   * gated_scan_prep: turns the raw q and f columns of the projection rows into q and f IN PLACE (fp32);
//   * gated_scan: CTA = (16 value columns, head, sequence), 128 threads = 16 slices of the D state rows x 8 column PAIRS; a
//     thread keeps 2 x 4 KR state elements in registers (rows 64 k + 4 slice + e of two columns: a half-warp reads a token's f
//     and q as conflict-free float4, once for both columns -- the kernel is bound by shared-memory wavefronts, not arithmetic),
//     tokens are staged 16 at a time with cp.async one chunk ahead and taken four at a time (the row reductions of o, four
//     shuffles per token for both columns, run under the next tokens' updates), the update is S = v + f (S - v) (one subtraction and one
//     FMA; no 1 - f that would lose digits where f is close to 1), issued as packed fp32 pairs (fma.rn.f32x2).  Launched without programmatic early start: its few
//     long-running CTAs must spread evenly over the SMs.
//   * long portions: when the step carries a segment list (some portion has several segments of 128 tokens) the segments run in
//     parallel.  Within a segment that starts from S0, S_t = A_t o S0 + Z_t with A_t the running product of f per state row and
//     Z_t the state reached from zero, so: a PARTIAL pass leaves Z_end and A_end of every segment but a sequence's last, an
//     elementwise pass chains them (start state of segment k + 1 = A_end[k] o start[k] + Z_end[k]), and the FULL pass runs
//     every segment from its true start state and writes the outputs.  The recurrence is linear in S: this is the sequential
//     result up to fp32 rounding.
// The state is stored TRANSPOSED, [slots][H][P][D], so that a warp's loads and stores of it are whole 128-byte lines.
// A sequence whose portion starts at position 0 ignores what its slot held.
#include "hybrid_common.cuh"

namespace b200 {

constexpr int GS_COLS = 16;     // value columns per CTA
constexpr int GS_SLICES = 16;   // lanes that share a column (slices of the state rows)
constexpr int GS_CPT = 2;       // value columns per thread: what is read of a token's f and q serves both (the code pairs them)
constexpr int GS_THREADS = GS_SLICES * GS_COLS / GS_CPT;
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

// MODE 0: grid z = sequence, its whole portion.  MODE 1 / 2: grid z = segment (segs[z] = first token, end token, sequence, 1 =
// first of its sequence | 2 = last): 1 = the partial pass from a zero state (no outputs; Z_end -> seg_state[z], A_end ->
// seg_decay[z]; a sequence's last segment has nothing to hand on and leaves at once), 2 = the full pass from seg_state[z]
// (outputs; a sequence's last segment writes the state back).
template <int KR, int MODE>
__global__ void __launch_bounds__(GS_THREADS)
    gated_scan_kernel(const float* __restrict__ proj, int ld, int q_col0, int f_col0, int v_col0, float* __restrict__ state,
                      const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_slot,
                      const int32_t* __restrict__ seq_pos0, float* __restrict__ out, int H, int D, int P, int vec,
                      const int32_t* __restrict__ segs, float* __restrict__ seg_state, float* __restrict__ seg_decay) {
  griddep_wait();
  constexpr int Dp = 4 * GS_SLICES * KR;
  extern __shared__ __align__(16) float gs_sm[];
  float* qs = gs_sm;                              // [2][GS_CHUNK][Dp]
  float* fs = qs + 2 * GS_CHUNK * Dp;             // [2][GS_CHUNK][Dp]
  float* vs = fs + 2 * GS_CHUNK * Dp;             // [2][GS_CHUNK][GS_COLS]
  float* os = vs + 2 * GS_CHUNK * GS_COLS;        // [GS_CHUNK][GS_COLS]
  // thread = (slice r of the state rows, PAIR c of value columns): a token's f and q, read once, serve both columns
  const int tid = threadIdx.x, r = tid & (GS_SLICES - 1), c = tid / GS_SLICES;
  const int j0 = blockIdx.x * GS_COLS, h = blockIdx.y;
  int sq = blockIdx.z, t0, n, flags = 3;
  if (MODE == 0) {
    t0 = seq_start[sq];
    n = seq_start[sq + 1] - t0;
  } else {
    const int32_t* sg = segs + 4 * blockIdx.z;
    t0 = sg[0], n = sg[1] - t0, sq = sg[2], flags = sg[3];
    if (MODE == 1 && (flags & 2)) return;
  }
  if (n <= 0) return;
  const int j = j0 + GS_CPT * c;  // the thread's first column
  // where the start state comes from and the end state goes to (column j; column j + 1 is D floats further)
  float* seg_st = MODE == 0 ? nullptr : seg_state + (((int64_t)blockIdx.z * H + h) * P + (j < P ? j : 0)) * D;
  float* fin_st = state + (((int64_t)seq_slot[sq] * H + h) * P + (j < P ? j : 0)) * D;
  float S[GS_CPT][KR][4], A[KR][4];  // A: running product of f per state row (partial pass only)
#pragma unroll
  for (int k = 0; k < KR; ++k)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      A[k][e] = 1.f;
#pragma unroll
      for (int u = 0; u < GS_CPT; ++u) S[u][k][e] = 0.f;
    }
  if (MODE == 2 || (MODE == 0 && seq_pos0[sq] > 0)) {
    const float* st = MODE == 2 ? seg_st : fin_st;
#pragma unroll
    for (int u = 0; u < GS_CPT; ++u) {
      if (j + u >= P) continue;
#pragma unroll
      for (int k = 0; k < KR; ++k) {
        const int i = 4 * GS_SLICES * k + 4 * r;
        if (vec && i + 3 < D) {
          const float4 a = *reinterpret_cast<const float4*>(st + (int64_t)u * D + i);
          S[u][k][0] = a.x, S[u][k][1] = a.y, S[u][k][2] = a.z, S[u][k][3] = a.w;
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (i + e < D) S[u][k][e] = st[(int64_t)u * D + i + e];
        }
      }
    }
  }
  const int nch = (n + GS_CHUNK - 1) / GS_CHUNK;
  // a chunk of tokens: q and f rows of this head (columns past D are zeros: their state rows stay zero), the CTA's v columns
  auto stage = [&](int ch, int buf) {
    const int tk0 = ch * GS_CHUNK;
    const float* base = proj + (int64_t)(t0 + tk0) * ld;
    if (vec) {  // 16-byte copies: D, ld and the column offsets are multiples of four floats and the rows 16-byte aligned
      for (int idx = tid; idx < GS_CHUNK * (Dp / 4); idx += GS_THREADS) {
        const int tk = idx / (Dp / 4), i = (idx - tk * (Dp / 4)) * 4;
        const bool ok = tk0 + tk < n && i < D;
        const float* src = base + (int64_t)(ok ? tk : 0) * ld + (int64_t)h * D + (ok ? i : 0);
        if (MODE != 1) cp_async16(smem_u32(qs + (buf * GS_CHUNK + tk) * Dp + i), src + q_col0, ok);
        cp_async16(smem_u32(fs + (buf * GS_CHUNK + tk) * Dp + i), src + f_col0, ok);
      }
    } else {
      for (int idx = tid; idx < GS_CHUNK * Dp; idx += GS_THREADS) {
        const int tk = idx / Dp, i = idx - tk * Dp;
        const bool ok = tk0 + tk < n && i < D;
        const float* src = base + (int64_t)(ok ? tk : 0) * ld + (int64_t)h * D + (ok ? i : 0);
        if (MODE != 1) cp_async4(smem_u32(qs + (buf * GS_CHUNK + tk) * Dp + i), src + q_col0, ok);
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
  const float2 one2 = make_float2(1.f, 1.f);
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
    // one token, both columns.  Packed fp32 pairs: S - v as S * 1 + (-v) (the same rounding as the subtraction), then
    // S = f (S - v) + v and o += S q
    auto update = [&](int tk, float2 (&oa)[GS_CPT], float2 (&ob)[GS_CPT]) {
      const float* fr = fs + (buf * GS_CHUNK + tk) * Dp + 4 * r;
      const float* qr = qs + (buf * GS_CHUNK + tk) * Dp + 4 * r;
      const float2 vv = *reinterpret_cast<const float2*>(vs + (buf * GS_CHUNK + tk) * GS_COLS + GS_CPT * c);
      const float vcol[GS_CPT] = {vv.x, vv.y};
#pragma unroll
      for (int k = 0; k < KR; ++k) {
        const float4 f4 = *reinterpret_cast<const float4*>(fr + 4 * GS_SLICES * k);
        const float2 f01 = make_float2(f4.x, f4.y), f23 = make_float2(f4.z, f4.w);
        float4 q4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (MODE != 1) q4 = *reinterpret_cast<const float4*>(qr + 4 * GS_SLICES * k);
#pragma unroll
        for (int u = 0; u < GS_CPT; ++u) {
          const float2 v2 = make_float2(vcol[u], vcol[u]), nv2 = make_float2(-vcol[u], -vcol[u]);
          float2 s01 = make_float2(S[u][k][0], S[u][k][1]), s23 = make_float2(S[u][k][2], S[u][k][3]);
          s01 = ffma2(f01, ffma2(s01, one2, nv2), v2);
          s23 = ffma2(f23, ffma2(s23, one2, nv2), v2);
          S[u][k][0] = s01.x, S[u][k][1] = s01.y, S[u][k][2] = s23.x, S[u][k][3] = s23.y;
          if (MODE != 1) {
            oa[u] = ffma2(s01, make_float2(q4.x, q4.y), oa[u]);
            ob[u] = ffma2(s23, make_float2(q4.z, q4.w), ob[u]);
          }
        }
        if (MODE == 1) {
          const float2 a01 = fmul2(make_float2(A[k][0], A[k][1]), f01), a23 = fmul2(make_float2(A[k][2], A[k][3]), f23);
          A[k][0] = a01.x, A[k][1] = a01.y, A[k][2] = a23.x, A[k][3] = a23.y;
        }
      }
    };
    // the thread's shares of o for its two columns -> their sums over the 16 row slices: after one exchange the lower eight
    // lanes carry the first column and the upper eight the second, then three steps on one value each
    auto token = [&](int tk) -> float {
      float2 oa[GS_CPT] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)}, ob[GS_CPT] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      update(tk, oa, ob);
      const float o0 = (oa[0].x + oa[0].y) + (ob[0].x + ob[0].y), o1 = (oa[1].x + oa[1].y) + (ob[1].x + ob[1].y);
      const bool up = (r & 8) != 0;
      float o = (up ? o1 : o0) + __shfl_xor_sync(0xffffffffu, up ? o0 : o1, 8);
      o += __shfl_xor_sync(0xffffffffu, o, 4);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      return o;
    };
    if (MODE == 1) {  // states and decay product only
      float2 none[GS_CPT];
      for (int tk = 0; tk < cn; ++tk) update(tk, none, none);
      __syncthreads();  // the chunk's buffer may be refilled
      continue;
    }
    const bool writer = (r & 7) == 0;             // lane 0 of a half holds column 2 c, lane 8 column 2 c + 1
    const int wc = GS_CPT * c + (r >> 3);
    int tk = 0;
    for (; tk + 4 <= cn; tk += 4) {
      const float o0 = token(tk), o1 = token(tk + 1), o2 = token(tk + 2), o3 = token(tk + 3);
      if (writer) {
        os[tk * GS_COLS + wc] = o0;
        os[(tk + 1) * GS_COLS + wc] = o1;
        os[(tk + 2) * GS_COLS + wc] = o2;
        os[(tk + 3) * GS_COLS + wc] = o3;
      }
    }
    for (; tk < cn; ++tk) {
      const float o = token(tk);
      if (writer) os[tk * GS_COLS + wc] = o;
    }
    __syncthreads();  // the chunk's outputs are complete, and its buffer may be refilled
    for (int idx = tid; idx < cn * GS_COLS; idx += GS_THREADS) {
      const int tk2 = idx / GS_COLS, cc = idx - tk2 * GS_COLS;
      if (j0 + cc < P) out[((int64_t)(t0 + ch * GS_CHUNK + tk2) * H + h) * P + j0 + cc] = os[idx];
    }
  }
  // the next kernel of the stream may take SM slots from here on: earlier, its waiting CTAs would displace this kernel's own
  griddep_launch();
  // state rows past D were fed f = 0 and hold v: they are not part of the state
  float* dst = MODE == 1 ? seg_st : fin_st;
  if (MODE != 2 || (flags & 2)) {
#pragma unroll
    for (int u = 0; u < GS_CPT; ++u) {
      if (j + u >= P) continue;
#pragma unroll
      for (int k = 0; k < KR; ++k) {
        const int i = 4 * GS_SLICES * k + 4 * r;
        if (vec && i + 3 < D) {
          *reinterpret_cast<float4*>(dst + (int64_t)u * D + i) = make_float4(S[u][k][0], S[u][k][1], S[u][k][2], S[u][k][3]);
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (i + e < D) dst[(int64_t)u * D + i + e] = S[u][k][e];
        }
      }
    }
  }
  if (MODE == 1 && blockIdx.x == 0 && c == 0) {  // the decay product is the same for every column: one copy per (segment, head)
    float* dd = seg_decay + ((int64_t)blockIdx.z * H + h) * D;
#pragma unroll
    for (int k = 0; k < KR; ++k)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = 4 * GS_SLICES * k + 4 * r + e;
        if (i < D) dd[i] = A[k][e];
      }
  }
}

// Chains the segments of every sequence, one thread per state element: carry = the sequence's state (zero for a sequence that
// starts at position 0); segment k's entry of seg_state (Z_end from the partial pass) is replaced by its START state, and
// carry <- A_end[k] carry + Z_end[k] for the next one.
__global__ void gated_seg_combine_kernel(const float* __restrict__ state, float* __restrict__ seg_state,
                                         const float* __restrict__ seg_decay, const int32_t* __restrict__ seq_seg0,
                                         const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ seq_pos0, int H, int P,
                                         int D, int64_t total) {
  griddep_launch();
  griddep_wait();
  const int64_t per_seq = (int64_t)H * P * D;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int sq = (int)(idx / per_seq);
    const int64_t e = idx - sq * per_seq;       // (h, j, i)
    const int h = (int)(e / ((int64_t)P * D)), i = (int)(e % D);
    const int s0 = seq_seg0[sq], s1 = seq_seg0[sq + 1];
    float carry = seq_pos0[sq] > 0 ? state[(int64_t)seq_slot[sq] * per_seq + e] : 0.f;
    // eight segments' loads are issued before the first store (the stores go to the array the loads read: without the batch
    // every load would wait for the store before it)
    for (int k0 = s0; k0 < s1; k0 += 8) {
      float z[8], a[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int k = k0 + u < s1 ? k0 + u : s1 - 1;
        z[u] = seg_state[(int64_t)k * per_seq + e];
        a[u] = seg_decay[((int64_t)k * H + h) * D + i];
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (k0 + u < s1) {
          seg_state[(int64_t)(k0 + u) * per_seq + e] = carry;
          if (k0 + u + 1 < s1) carry = fmaf(a[u], carry, z[u]);
        }
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
                    const int32_t* seq_slot, const int32_t* seq_pos0, float* out, int B, int H, int D, int P, const int32_t* segs,
                    int num_segs, const int32_t* seq_seg0, float* seg_state, float* seg_decay, void* stream) {
  B200_REQUIRE(proj && state && seq_start && seq_slot && seq_pos0 && out, "gated_scan: null pointer");
  B200_REQUIRE(H >= 1 && D >= 1 && P >= 1, "gated_scan: bad shape");
  B200_REQUIRE(num_segs >= 0 && (num_segs == 0 || (segs && seq_seg0 && seg_state && seg_decay)), "gated_scan: %d segments need their buffers", num_segs);
  if (D > 512) {
    set_last_error("gated_scan: %d state rows per head exceed 512", D);
    return B200_ERR_UNSUPPORTED;
  }
  if (B <= 0) return B200_OK;
  B200_REQUIRE(B <= 65535 && H <= 65535 && num_segs <= 65535, "gated_scan: %d sequences x %d heads exceed the grid", B, H);
  const int vec = D % 4 == 0 && ld % 4 == 0 && q_col0 % 4 == 0 && f_col0 % 4 == 0 && ((uintptr_t)proj & 15) == 0 &&
                  ((uintptr_t)state & 15) == 0 && ((uintptr_t)seg_state & 15) == 0;
  cudaStream_t st = (cudaStream_t)stream;
  // whole portions: few long-running CTAs, launched only when the predecessor has drained; segments: many short ones
#define GS_LAUNCH_M(KR, MODE, LAUNCH, NZ)                                                                                       \
  do {                                                                                                                          \
    const size_t smem = (size_t)(4 * GS_CHUNK * 4 * GS_SLICES * KR + 3 * GS_CHUNK * GS_COLS) * 4;                               \
    if (smem > 48 * 1024)                                                                                                       \
      B200_CUDA_OK(cudaFuncSetAttribute(gated_scan_kernel<KR, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    B200_CUDA_OK(LAUNCH(gated_scan_kernel<KR, MODE>, dim3((P + GS_COLS - 1) / GS_COLS, H, NZ), dim3(GS_THREADS), smem, st, proj, \
                        ld, q_col0, f_col0, v_col0, state, seq_start, seq_slot, seq_pos0, out, H, D, P, vec, segs, seg_state,   \
                        seg_decay));                                                                                            \
  } while (0)
#define GS_LAUNCH(KR)                                                                                                          \
  do {                                                                                                                         \
    if (num_segs == 0) {                                                                                                       \
      GS_LAUNCH_M(KR, 0, launch_kernel_serial, B);                                                                             \
    } else {                                                                                                                   \
      GS_LAUNCH_M(KR, 1, launch_kernel, num_segs);                                                                             \
      const int64_t total = (int64_t)B * H * P * D;                                                                            \
      int64_t blocks = (total + 255) / 256;                                                                                    \
      blocks = blocks > 148 * 16 ? 148 * 16 : blocks;                                                                          \
      B200_CUDA_OK(launch_kernel(gated_seg_combine_kernel, dim3((unsigned)blocks), dim3(256), 0, st, (const float*)state,      \
                                 seg_state, (const float*)seg_decay, seq_seg0, seq_slot, seq_pos0, H, P, D, total));           \
      GS_LAUNCH_M(KR, 2, launch_kernel, num_segs);                                                                             \
    }                                                                                                                          \
  } while (0)
  if (D <= 64) GS_LAUNCH(1);
  else if (D <= 128) GS_LAUNCH(2);
  else if (D <= 256) GS_LAUNCH(4);
  else GS_LAUNCH(8);
#undef GS_LAUNCH
#undef GS_LAUNCH_M
  return B200_OK;
}

}  // extern "C"
