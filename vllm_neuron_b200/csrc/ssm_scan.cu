// State-space (Mamba-2 style) mixer kernels over a ragged batch: every sequence of the step brings n >= 1 new tokens that
// continue from the state its slot holds (a prompt portion and a single decoded token are the same code).
//   * causal depthwise convolution + SiLU over the channels [x | B | C]; the last (taps - 1) inputs of a sequence are
//     part of its state (fp32, [slots][taps - 1][channels], oldest first);
//   * the selective scan  S_t = exp(-exp(A_log) dt_t) S_{t-1} + dt_t B_t x_t^T,  y_t = S_t^T C_t + D x_t  with
//     dt_t = softplus(dt_raw + dt_bias), S in fp32 ([slots][heads][P][N]) and every term of the recurrence in fp32.
// A sequence whose first new token is position 0 starts from zero state whatever its slot held before, so slots can be
// handed to new requests without clearing them.
#include "hybrid_common.cuh"

namespace b200 {

constexpr int CONV_MAX_TAPS = 16;
constexpr int CONV_RUN = 16;  // most consecutive tokens per thread (large steps): the window's earlier inputs and the taps are cache hits

// one thread per (run of `run` tokens, channel); run = 1 for decode-sized steps.  in_bias (or NULL) is added to every input
// taken from `in` (a projection's bias: the state rows hold biased inputs already); silu == 0 leaves the sum as it is.
template <typename OT>
__global__ void causal_conv_silu_kernel(const float* __restrict__ in, int ld, int col0, const float* __restrict__ cw,
                                        const float* __restrict__ cb, const float* __restrict__ in_bias, int silu,
                                        const float* __restrict__ state,
                                        const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ seq_start,
                                        const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ seq_pos0,
                                        OT* __restrict__ out, int T, int C, int taps, int run) {
  griddep_launch();
  griddep_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const float bias = cb ? cb[c] : 0.f;
  const float ib = in_bias ? in_bias[c] : 0.f;
  const float* wc = cw + (int64_t)c * taps;
  const int t_end = min(T, (int)(blockIdx.y + 1) * run);
  for (int t = blockIdx.y * run; t < t_end; ++t) {
    const int s = tok_seq[t];
    const int i = t - seq_start[s];  // index inside this step's portion
    const bool has_state = seq_pos0[s] > 0;
    const float* st = state + (int64_t)seq_slot[s] * (taps - 1) * C;
    float acc = bias;
    for (int j = 0; j < taps; ++j) {
      const int src = i - (taps - 1 - j);  // portion index of the input under tap j (last tap = current token)
      float v;
      if (src >= 0)
        v = in[(int64_t)(t - (taps - 1 - j)) * ld + col0 + c] + ib;
      else if (has_state)
        v = st[(int64_t)(src + taps - 1) * C + c];
      else
        v = 0.f;
      acc += v * wc[j];
    }
    stf(out, (int64_t)t * C + c, silu ? silu_f(acc) : acc);
  }
}

// The same with four channels per thread (16-byte loads and stores) and the window of the last TAPS - 1 inputs carried in
// registers along the run: one load per output instead of TAPS.  The window is filled from the rows before the run (or the
// state, or zeros) at the run's first token and wherever a new sequence starts inside the run.  Sums in the order of the
// kernel above.  Needs C, col0 and ld multiples of 4 and 16-byte aligned bases.
template <typename OT, int TAPS>
__global__ void causal_conv_vec_kernel(const float* __restrict__ in, int ld, int col0, const float* __restrict__ cw,
                                       const float* __restrict__ cb, const float* __restrict__ in_bias, int silu,
                                       const float* __restrict__ state, const int32_t* __restrict__ tok_seq,
                                       const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_slot,
                                       const int32_t* __restrict__ seq_pos0, OT* __restrict__ out, int T, int C, int run) {
  griddep_launch();
  griddep_wait();
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (c >= C) return;
  float w[4][TAPS], bias[4], ib[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    bias[k] = cb ? cb[c + k] : 0.f;
    ib[k] = in_bias ? in_bias[c + k] : 0.f;
#pragma unroll
    for (int j = 0; j < TAPS; ++j) w[k][j] = cw[(int64_t)(c + k) * TAPS + j];
  }
  float win[TAPS > 1 ? TAPS - 1 : 1][4];
  const int t_begin = blockIdx.y * run, t_end = min(T, t_begin + run);
  int prev_s = -1;
  for (int t = t_begin; t < t_end; ++t) {
    const int s = tok_seq[t];
    if (s != prev_s) {
      prev_s = s;
      const int i = t - seq_start[s];
      const bool has_state = seq_pos0[s] > 0;
      const float* st = state + (int64_t)seq_slot[s] * (TAPS - 1) * C;
#pragma unroll
      for (int j = 0; j < TAPS - 1; ++j) {
        const int src = i - (TAPS - 1 - j);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (src >= 0) {
          v = *reinterpret_cast<const float4*>(in + (int64_t)(t - (TAPS - 1 - j)) * ld + col0 + c);
          v.x += ib[0], v.y += ib[1], v.z += ib[2], v.w += ib[3];
        } else if (has_state) {
          v = *reinterpret_cast<const float4*>(st + (int64_t)(src + TAPS - 1) * C + c);
        }
        win[j][0] = v.x, win[j][1] = v.y, win[j][2] = v.z, win[j][3] = v.w;
      }
    }
    const float4 u = *reinterpret_cast<const float4*>(in + (int64_t)t * ld + col0 + c);
    const float cur[4] = {u.x + ib[0], u.y + ib[1], u.z + ib[2], u.w + ib[3]};
    float y[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float acc = bias[k];
#pragma unroll
      for (int j = 0; j < TAPS - 1; ++j) acc += win[j][k] * w[k][j];
      acc += cur[k] * w[k][TAPS - 1];
      y[k] = silu ? silu_f(acc) : acc;
#pragma unroll
      for (int j = 0; j + 1 < TAPS - 1; ++j) win[j][k] = win[j + 1][k];
      if (TAPS > 1) win[TAPS - 2][k] = cur[k];
    }
    if constexpr (sizeof(OT) == 2) {
      *reinterpret_cast<uint2*>(out + (int64_t)t * C + c) = make_uint2(pack_bf16(y[0], y[1]), pack_bf16(y[2], y[3]));
    } else {
      *reinterpret_cast<float4*>(out + (int64_t)t * C + c) = make_float4(y[0], y[1], y[2], y[3]);
    }
  }
}

// new state = the last (taps - 1) inputs of [old state | this step's inputs]; one thread per (sequence, channel) reads
// everything it needs before it writes, so the update is in place.  Runs after causal_conv_silu_kernel on the stream.
__global__ void conv_state_update_kernel(const float* __restrict__ in, int ld, int col0, const float* __restrict__ in_bias,
                                         float* __restrict__ state,
                                         const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_slot,
                                         const int32_t* __restrict__ seq_pos0, int C, int taps) {
  griddep_launch();
  griddep_wait();
  const int s = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int t0 = seq_start[s], n = seq_start[s + 1] - t0, pos0 = seq_pos0[s];
  float* st = state + (int64_t)seq_slot[s] * (taps - 1) * C;
  float keep[CONV_MAX_TAPS];
#pragma unroll
  for (int k = 0; k < CONV_MAX_TAPS - 1; ++k) {
    if (k < taps - 1) {
      const int i = n - (taps - 1) + k;  // portion index of what slot k must hold afterwards
      float v = 0.f;
      if (i >= 0)
        v = in[(int64_t)(t0 + i) * ld + col0 + c] + (in_bias ? in_bias[c] : 0.f);
      else if (pos0 > 0)
        v = st[(int64_t)(i + taps - 1) * C + c];
      keep[k] = v;
    }
  }
#pragma unroll
  for (int k = 0; k < CONV_MAX_TAPS - 1; ++k)
    if (k < taps - 1) st[(int64_t)k * C + c] = keep[k];
}

// Selective scan.  CTA = (32 PP value columns p of one head) x (8 slices of the state dimension); thread (pl, s) keeps
// S[p][n] for p = p0 + pl + 32 q (q < PP) and the pairs n = 2 s + 16 k + {0, 1} (NPT elements) in registers across the tokens it walks, so
// one B / C pair read from shared memory serves PP columns and the update runs on packed fp32 pairs (two state elements
// per issue slot); y is reduced over the 8 slices with shuffles.  Tokens are
// walked in chunks of SCAN_CHUNK: the CTA stages the chunk's B, C and x rows in shared memory with coalesced loads
// (fetched into registers one chunk ahead) and computes each token's step size and decay ONCE (softplus / exp are not
// repeated by every thread), then the recurrence runs out of shared memory.  State layout [slots][H][P][N]: the 8 slices
// of a column read consecutive floats.
//
// Long prompt portions are cut into SEGMENTS of consecutive tokens that run in parallel (`segs` != NULL, blockIdx.z = segment):
//   1. PARTIAL launch: every segment but a sequence's last starts from zero and leaves its end state S_loc and its summed
//      step size in scratch (no y);
//   2. ssd_seg_combine_kernel walks each sequence's segments once, elementwise: S_in[k+1] = exp(-exp(A_log) sum_dt[k]) S_in[k]
//      + S_loc[k], S_in[0] = the slot's state (zero at position 0), and stores S_in[k] over the scratch;
//   3. the full launch starts every segment from its S_in, writes y, and the last segment writes the slot's new state.
// The recurrence is linear in S, so this is the sequential result up to fp32 rounding; everything stays fp32.

constexpr int SCAN_PLANES = 32;
constexpr int SCAN_SLICES = 8;
constexpr int SCAN_CHUNK = 32;
enum { SEG_FIRST = 1, SEG_LAST = 2 };

template <typename XT, int NPT, int PP, bool PARTIAL>
__global__ void __launch_bounds__(SCAN_PLANES* SCAN_SLICES, (NPT * PP <= 32) ? 2 : 1)
    ssd_scan_kernel(const XT* __restrict__ xbc, int C, const float* __restrict__ dt_in, int ld_dt, int dt_col0,
                    const float* __restrict__ A_log, const float* __restrict__ dt_bias, const float* __restrict__ Dskip,
                    float* __restrict__ state, const int32_t* __restrict__ seq_start, const int32_t* __restrict__ seq_slot,
                    const int32_t* __restrict__ seq_pos0, float* __restrict__ y, int H, int P, int N, int G,
                    const int4* __restrict__ segs, float* __restrict__ seg_state, float* __restrict__ seg_dtsum) {
  griddep_launch();
  griddep_wait();
  constexpr int NP = NPT * SCAN_SLICES;  // padded state size: rows of Bs / Cs
  constexpr int PC = SCAN_PLANES * PP;   // value columns per CTA
  extern __shared__ float sm[];
  float* Bs = sm;                               // [SCAN_CHUNK][NP]
  float* Cs = Bs + SCAN_CHUNK * NP;             // [SCAN_CHUNK][NP]
  float* xs = Cs + SCAN_CHUNK * NP;             // [SCAN_CHUNK][PC]
  float* dts = xs + SCAN_CHUNK * PC;            // [SCAN_CHUNK]
  float* dec = dts + SCAN_CHUNK;                // [SCAN_CHUNK]
  const int h = blockIdx.y, tid = threadIdx.x;
  int sq = blockIdx.z, t0, t1, flags = SEG_FIRST | SEG_LAST;
  if (segs) {
    const int4 sd = segs[blockIdx.z];
    t0 = sd.x, t1 = sd.y, sq = sd.z, flags = sd.w;
  } else {
    t0 = seq_start[sq], t1 = seq_start[sq + 1];
  }
  if (PARTIAL && (flags & SEG_LAST)) return;  // nobody continues from a sequence's last segment in this step
  const int s = tid % SCAN_SLICES, pl = tid / SCAN_SLICES;
  const int p0 = blockIdx.x * PC;
  const int g = h / (H / G);
  const int inner = H * P;
  const int64_t head_elems = (int64_t)P * N;
  // where this CTA's state comes from and goes to
  const float* S_in = nullptr;
  float* S_out = nullptr;
  if (PARTIAL) {
    S_out = seg_state + ((int64_t)(blockIdx.z + 1) * H + h) * head_elems;
  } else {
    float* slot = state + ((int64_t)seq_slot[sq] * H + h) * head_elems;
    if (flags & SEG_FIRST) S_in = seq_pos0[sq] > 0 ? slot : nullptr;
    else S_in = seg_state + ((int64_t)blockIdx.z * H + h) * head_elems;
    if (flags & SEG_LAST) S_out = slot;
  }
  // thread (pl, s) owns the state pairs n = 2 s + 16 k + {0, 1}, k < NPT / 2, of each of its columns
  float2 S[PP][NPT / 2];
#pragma unroll
  for (int q = 0; q < PP; ++q) {
    const int p = p0 + pl + SCAN_PLANES * q;
#pragma unroll
    for (int k = 0; k < NPT / 2; ++k) {
      const int n = 2 * s + 2 * SCAN_SLICES * k;
      S[q][k].x = (S_in && p < P && n < N) ? S_in[(int64_t)p * N + n] : 0.f;
      S[q][k].y = (S_in && p < P && n + 1 < N) ? S_in[(int64_t)p * N + n + 1] : 0.f;
    }
  }
  const float negA = -expf(A_log[h]), bias = dt_bias[h], dsk = Dskip[h];
  const int64_t xcol = (int64_t)h * P + p0, bcol = (int64_t)inner + (int64_t)g * N, ccol = bcol + (int64_t)G * N;
  // global -> registers -> shared memory: the next chunk's loads are in flight while the current chunk is applied
  constexpr int NTHR = SCAN_PLANES * SCAN_SLICES;
  constexpr int BC_PER = SCAN_CHUNK * NP / NTHR;
  constexpr int X_PER = SCAN_CHUNK * PC / NTHR;
  float rB[BC_PER], rC[PARTIAL ? 1 : BC_PER], rx[X_PER], rdt = 0.f, dt_sum = 0.f;
  auto fetch = [&](int c0) {
    const int nc = t1 - c0 < SCAN_CHUNK ? t1 - c0 : SCAN_CHUNK;
#pragma unroll
    for (int k = 0; k < BC_PER; ++k) {
      const int i = tid + k * NTHR, tok = i / NP, n = i - tok * NP;
      const bool in = tok < nc && n < N;
      const XT* row = xbc + (int64_t)(c0 + (tok < nc ? tok : 0)) * C;
      rB[k] = in ? ldf(row, bcol + n) : 0.f;
      if (!PARTIAL) rC[k] = in ? ldf(row, ccol + n) : 0.f;
    }
#pragma unroll
    for (int k = 0; k < X_PER; ++k) {
      const int i = tid + k * NTHR, tok = i / PC, pp = i - tok * PC;
      rx[k] = (tok < nc && p0 + pp < P) ? ldf(xbc + (int64_t)(c0 + tok) * C, xcol + pp) : 0.f;
    }
    if (tid < nc) rdt = dt_in[(int64_t)(c0 + tid) * ld_dt + dt_col0 + h];
  };
  if (t0 < t1) fetch(t0);
  for (int c0 = t0; c0 < t1; c0 += SCAN_CHUNK) {
    const int nc = t1 - c0 < SCAN_CHUNK ? t1 - c0 : SCAN_CHUNK;
    __syncthreads();  // the previous chunk has been consumed
#pragma unroll
    for (int k = 0; k < BC_PER; ++k) {
      Bs[tid + k * NTHR] = rB[k];
      if (!PARTIAL) Cs[tid + k * NTHR] = rC[k];
    }
#pragma unroll
    for (int k = 0; k < X_PER; ++k) xs[tid + k * NTHR] = rx[k];
    if (tid < nc) {
      const float z = rdt + bias;
      const float dt = z > 20.f ? z : log1pf(expf(z));  // softplus, no clamp on the step size
      dts[tid] = dt;
      dec[tid] = expf(negA * dt);
      dt_sum += dt;
    }
    __syncthreads();
    if (c0 + SCAN_CHUNK < t1) fetch(c0 + SCAN_CHUNK);
    for (int tok = 0; tok < nc; ++tok) {
      const float a = dec[tok], dtv = dts[tok];
      const float2 a2 = make_float2(a, a);
      float xc[PP];
      float2 dx2[PP], acc2[PP];
#pragma unroll
      for (int q = 0; q < PP; ++q) {
        xc[q] = xs[tok * PC + pl + SCAN_PLANES * q];
        dx2[q] = make_float2(dtv * xc[q], dtv * xc[q]);
        acc2[q] = make_float2(0.f, 0.f);
      }
      const float* Br = Bs + tok * NP + 2 * s;
      const float* Cr = Cs + tok * NP + 2 * s;
#pragma unroll
      for (int k = 0; k < NPT / 2; ++k) {
        const float2 b2 = *reinterpret_cast<const float2*>(Br + 2 * SCAN_SLICES * k);
        const float2 c2 = PARTIAL ? make_float2(0.f, 0.f) : *reinterpret_cast<const float2*>(Cr + 2 * SCAN_SLICES * k);
#pragma unroll
        for (int q = 0; q < PP; ++q) {
          S[q][k] = ffma2(a2, S[q][k], fmul2(b2, dx2[q]));
          if (!PARTIAL) acc2[q] = ffma2(S[q][k], c2, acc2[q]);
        }
      }
      if (!PARTIAL) {
#pragma unroll
        for (int q = 0; q < PP; ++q) {
          float v = acc2[q].x + acc2[q].y;
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          v += __shfl_xor_sync(0xffffffffu, v, 4);
          const int pq = pl + SCAN_PLANES * q;
          if (s == 0 && p0 + pq < P) y[(int64_t)(c0 + tok) * inner + xcol + pq] = v + dsk * xc[q];
        }
      }
    }
  }
  if (S_out) {
#pragma unroll
    for (int q = 0; q < PP; ++q) {
      const int p = p0 + pl + SCAN_PLANES * q;
#pragma unroll
      for (int k = 0; k < NPT / 2; ++k) {
        const int n = 2 * s + 2 * SCAN_SLICES * k;
        if (p < P && n < N) S_out[(int64_t)p * N + n] = S[q][k].x;
        if (p < P && n + 1 < N) S_out[(int64_t)p * N + n + 1] = S[q][k].y;
      }
    }
  }
  if (PARTIAL && blockIdx.x == 0 && tid < 32) {  // the chunk's step sizes live in threads 0..31
    const float tot = warp_sum(dt_sum);
    if (tid == 0) seg_dtsum[(int64_t)blockIdx.z * H + h] = tot;
  }
}

// One thread per state element of a sequence: turns the segments' zero-start end states (scratch entry k + 1 holds segment
// k's) into every segment's true start state, in place.
__global__ void ssd_seg_combine_kernel(const float* __restrict__ state, float* __restrict__ seg_state,
                                       const float* __restrict__ seg_dtsum, const float* __restrict__ A_log,
                                       const int32_t* __restrict__ seq_seg0, const int32_t* __restrict__ seq_slot,
                                       const int32_t* __restrict__ seq_pos0, int H, int64_t head_elems) {
  griddep_launch();
  griddep_wait();
  const int sq = blockIdx.y;
  const int v0 = seq_seg0[sq], nseg = seq_seg0[sq + 1] - v0;
  if (nseg <= 1) return;
  const int64_t per_seq = (int64_t)H * head_elems;
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= per_seq) return;
  const int h = (int)(e / head_elems);
  const float negA = -expf(A_log[h]);
  float S = seq_pos0[sq] > 0 ? state[(int64_t)seq_slot[sq] * per_seq + e] : 0.f;
  for (int k = 1; k < nseg; ++k) {
    const float d = expf(negA * seg_dtsum[(int64_t)(v0 + k - 1) * H + h]);
    float* cell = seg_state + (int64_t)(v0 + k) * per_seq + e;
    S = d * S + *cell;
    *cell = S;
  }
}

template <typename XT, int NPT, int PP>
static int launch_scan(const void* xbc, int C, const float* dt_in, int ld_dt, int dt_col0, const float* A_log,
                       const float* dt_bias, const float* Dskip, float* state, const int32_t* seq_start, const int32_t* seq_slot,
                       const int32_t* seq_pos0, float* y, int B, int H, int P, int N, int G, const int32_t* segs, int num_segs,
                       const int32_t* seq_seg0, float* seg_state, float* seg_dtsum, cudaStream_t stream) {
  constexpr int PC = SCAN_PLANES * PP;
  dim3 grid((P + PC - 1) / PC, H, segs ? num_segs : B);
  const size_t smem = (size_t)(SCAN_CHUNK * (2 * NPT * SCAN_SLICES + PC + 2)) * sizeof(float);
  const int4* sd = reinterpret_cast<const int4*>(segs);
  if (segs) {
    if (smem > 48 * 1024)
      B200_CUDA_OK(cudaFuncSetAttribute(ssd_scan_kernel<XT, NPT, PP, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    B200_CUDA_OK(launch_kernel(ssd_scan_kernel<XT, NPT, PP, true>, grid, dim3(SCAN_PLANES * SCAN_SLICES), smem, stream,
                               (const XT*)xbc, C, dt_in, ld_dt, dt_col0, A_log, dt_bias, Dskip, state, seq_start, seq_slot, seq_pos0,
                               y, H, P, N, G, sd, seg_state, seg_dtsum));
    const int64_t per_seq = (int64_t)H * P * N;
    B200_CUDA_OK(launch_kernel(ssd_seg_combine_kernel, dim3((unsigned)((per_seq + 255) / 256), B), dim3(256), 0, stream,
                               (const float*)state, seg_state, (const float*)seg_dtsum, A_log, seq_seg0, seq_slot, seq_pos0, H,
                               (int64_t)P * N));
  }
  if (smem > 48 * 1024)
    B200_CUDA_OK(cudaFuncSetAttribute(ssd_scan_kernel<XT, NPT, PP, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  B200_CUDA_OK(launch_kernel(ssd_scan_kernel<XT, NPT, PP, false>, grid, dim3(SCAN_PLANES * SCAN_SLICES), smem, stream,
                             (const XT*)xbc, C, dt_in, ld_dt, dt_col0, A_log, dt_bias, Dskip, state, seq_start, seq_slot, seq_pos0, y,
                             H, P, N, G, sd, seg_state, seg_dtsum));
  return B200_OK;
}

// columns per thread: as many as the head has 32-column planes, while the state stays within 32 registers (two CTAs per SM)
template <typename XT, int NPT>
static int pick_scan(const void* xbc, int C, const float* dt_in, int ld_dt, int dt_col0, const float* A_log, const float* dt_bias,
                     const float* Dskip, float* state, const int32_t* seq_start, const int32_t* seq_slot, const int32_t* seq_pos0,
                     float* y, int B, int H, int P, int N, int G, const int32_t* segs, int num_segs, const int32_t* seq_seg0,
                     float* seg_state, float* seg_dtsum, cudaStream_t stream) {
#define PICK_ARGS                                                                                                             \
  xbc, C, dt_in, ld_dt, dt_col0, A_log, dt_bias, Dskip, state, seq_start, seq_slot, seq_pos0, y, B, H, P, N, G, segs, num_segs, \
      seq_seg0, seg_state, seg_dtsum, stream
  if constexpr (NPT * 4 <= 32) {
    if (P > 64) return launch_scan<XT, NPT, 4>(PICK_ARGS);
  }
  if constexpr (NPT * 2 <= 64) {
    if (P > 32) return launch_scan<XT, NPT, 2>(PICK_ARGS);
  }
  return launch_scan<XT, NPT, 1>(PICK_ARGS);
#undef PICK_ARGS
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_causal_conv(const float* in, int ld, int col0, const float* conv_w, const float* conv_b, const float* in_bias, int silu,
                     float* state, const int32_t* tok_seq, const int32_t* seq_start, const int32_t* seq_slot,
                     const int32_t* seq_pos0, void* out, int out_dtype, int T, int B, int C, int taps, void* stream) {
  B200_REQUIRE(in && conv_w && state && tok_seq && seq_start && seq_slot && seq_pos0 && out, "causal_conv: null pointer");
  B200_REQUIRE(taps >= 1 && taps <= CONV_MAX_TAPS, "causal_conv: %d taps (1..%d supported)", taps, CONV_MAX_TAPS);
  if (T <= 0 || B <= 0) return B200_OK;
  const int th = 128;
  const int run = T / 256 < 1 ? 1 : T / 256 > CONV_RUN ? CONV_RUN : T / 256;
  const int oes = out_dtype == B200_BF16 ? 2 : 4;
  const bool vec = taps >= 2 && taps <= 4 && C % 4 == 0 && col0 % 4 == 0 && ld % 4 == 0 && ((uintptr_t)in & 15) == 0 &&
                   ((uintptr_t)state & 15) == 0 && ((uintptr_t)out & (4 * oes - 1)) == 0;
  if (vec) {
    const dim3 grid((C / 4 + th - 1) / th, (T + run - 1) / run);
#define CONV_VEC(TAPS_)                                                                                                          \
  B200_DISPATCH_ELEM(out_dtype, OT,                                                                                              \
                     B200_CUDA_OK(launch_kernel(causal_conv_vec_kernel<OT, TAPS_>, grid, dim3(th), 0, (cudaStream_t)stream, in, ld, \
                                                col0, conv_w, conv_b, in_bias, silu, (const float*)state, tok_seq, seq_start,    \
                                                seq_slot, seq_pos0, (OT*)out, T, C, run)))
    if (taps == 2) CONV_VEC(2);
    else if (taps == 3) CONV_VEC(3);
    else CONV_VEC(4);
#undef CONV_VEC
  } else
  B200_DISPATCH_ELEM(out_dtype, OT,
                     B200_CUDA_OK(launch_kernel(causal_conv_silu_kernel<OT>, dim3((C + th - 1) / th, (T + run - 1) / run), dim3(th), 0,
                                                (cudaStream_t)stream, in, ld, col0, conv_w, conv_b, in_bias, silu, (const float*)state,
                                                tok_seq, seq_start, seq_slot, seq_pos0, (OT*)out, T, C, taps, run)));
  if (taps > 1)
    B200_CUDA_OK(launch_kernel(conv_state_update_kernel, dim3((C + th - 1) / th, B), dim3(th), 0, (cudaStream_t)stream, in, ld,
                               col0, in_bias, state, seq_start, seq_slot, seq_pos0, C, taps));
  return B200_OK;
}

int b200_causal_conv_silu(const float* in, int ld, int col0, const float* conv_w, const float* conv_b, float* state,
                          const int32_t* tok_seq, const int32_t* seq_start, const int32_t* seq_slot, const int32_t* seq_pos0,
                          void* out, int out_dtype, int T, int B, int C, int taps, void* stream) {
  return b200_causal_conv(in, ld, col0, conv_w, conv_b, nullptr, 1, state, tok_seq, seq_start, seq_slot, seq_pos0, out,
                          out_dtype, T, B, C, taps, stream);
}

int b200_ssd_scan(const void* xbc, int x_dtype, int C, const float* dt_in, int ld_dt, int dt_col0, const float* A_log,
                  const float* dt_bias, const float* D, float* state, const int32_t* seq_start, const int32_t* seq_slot,
                  const int32_t* seq_pos0, float* y, int B, int H, int P, int N, int G, const int32_t* segs, int num_segs,
                  const int32_t* seq_seg0, float* seg_state, float* seg_dtsum, void* stream) {
  B200_REQUIRE(xbc && dt_in && A_log && dt_bias && D && state && seq_start && seq_slot && seq_pos0 && y, "ssd_scan: null pointer");
  B200_REQUIRE(H > 0 && G > 0 && H % G == 0, "ssd_scan: %d heads do not split into %d groups", H, G);
  B200_REQUIRE(N >= 1 && N <= 256, "ssd_scan: state size %d (1..256 supported)", N);
  B200_REQUIRE(C == H * P + 2 * G * N, "ssd_scan: %d channels != heads * vdim + 2 * groups * state", C);
  B200_REQUIRE(!segs || (num_segs >= B && seq_seg0 && seg_state && seg_dtsum && !((uintptr_t)segs & 15)),
               "ssd_scan: the segment list needs its per-sequence offsets and scratch");
  if (B <= 0) return B200_OK;
  cudaStream_t st = (cudaStream_t)stream;
#define SCAN_ARGS                                                                                                          \
  xbc, C, dt_in, ld_dt, dt_col0, A_log, dt_bias, D, state, seq_start, seq_slot, seq_pos0, y, B, H, P, N, G, segs, num_segs, \
      seq_seg0, seg_state, seg_dtsum, st
  B200_DISPATCH_ELEM(x_dtype, XT, {
    if (N <= 32) return pick_scan<XT, 4>(SCAN_ARGS);
    if (N <= 64) return pick_scan<XT, 8>(SCAN_ARGS);
    if (N <= 128) return pick_scan<XT, 16>(SCAN_ARGS);
    return pick_scan<XT, 32>(SCAN_ARGS);
  });
#undef SCAN_ARGS
  return B200_OK;
}

}  // extern "C"
