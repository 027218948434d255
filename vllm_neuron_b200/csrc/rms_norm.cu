// Per-row kernels of hybrid decoders with post-norm residual branches (x += N(branch(x)), N an RMS norm whose weight may
// be stored around zero): token + hashed-bigram embedding, the fused "residual += norm(weighted sum of branch rows);
// next operand = cast(residual)" step, an RMS norm over a column range, the per-head RMS norm with an output gate that
// closes a recurrent mixer, and gated-linear-unit activations.  The residual stream and all norm arithmetic are fp32;
// outputs that feed a GEMM are written in the GEMM operand type.
#include "hybrid_common.cuh"

namespace b200 {

// sum over the CTA (every thread gets it); `red` holds 33 floats
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float s = threadIdx.x < ((blockDim.x + 31) >> 5) ? red[threadIdx.x] : 0.f;
    s = warp_sum(s);
    if (threadIdx.x == 0) red[32] = s;
  }
  __syncthreads();
  const float out = red[32];
  __syncthreads();  // `red` may be reused right away
  return out;
}

// x[t] = table[token] * scale + bigram[row];  row = (prev * mul_prev + token * mul_cur) mod buckets, and row `buckets`
// (the table's last) for a sequence's first token.  The token before a portion comes from prev_state[slot]; the CTA of
// a portion's first token reads it and then stores the portion's last token there.
template <typename WT, typename OT>
__global__ void embed_bigram_kernel(const int32_t* __restrict__ tokens, const WT* __restrict__ table, const WT* __restrict__ bigram,
                                    int buckets, int mul_prev, int mul_cur, int32_t* __restrict__ prev_state,
                                    const int32_t* __restrict__ tok_seq, const int32_t* __restrict__ seq_start,
                                    const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ seq_pos0,
                                    float* __restrict__ out, OT* __restrict__ out_cast, int W, int V, float scale) {
  griddep_launch();
  griddep_wait();
  const int t = blockIdx.x;
  int tok = tokens[t];
  tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
  int64_t brow = -1;
  if (bigram) {
    const int s = tok_seq[t];
    const int t0 = seq_start[s];
    if (t > t0) {
      int prev = tokens[t - 1];
      prev = prev < 0 ? 0 : (prev >= V ? V - 1 : prev);
      brow = ((int64_t)prev * mul_prev + (int64_t)tok * mul_cur) % buckets;
    } else {
      const int slot = seq_slot[s];
      brow = seq_pos0[s] > 0 ? ((int64_t)prev_state[slot] * mul_prev + (int64_t)tok * mul_cur) % buckets : buckets;
      __syncthreads();
      if (threadIdx.x == 0) {
        int last = tokens[seq_start[s + 1] - 1];
        prev_state[slot] = last < 0 ? 0 : (last >= V ? V - 1 : last);
      }
    }
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = ldf(table, (int64_t)tok * W + i) * scale;
    if (brow >= 0) v += ldf(bigram, brow * W + i);
    out[(int64_t)t * W + i] = v;
    if (out_cast) stf(out_cast, (int64_t)t * W + i, v);
  }
}

// s = sum_{c < nsum} wt[t * nsum + c] * y[(t * nsum + c)] (wt NULL: plain sum);  x[t] += s / sqrt(mean(s^2) + eps) * (offset + w);
// out_cast[t] = x[t] in the operand type (when given).  One CTA per token; the row is held in shared memory.
template <typename OT>
__global__ void rms_residual_kernel(float* __restrict__ x, const float* __restrict__ y, int nsum, const float* __restrict__ wt,
                                    const float* __restrict__ w, float offset, float eps, OT* __restrict__ out_cast, int W) {
  griddep_launch();
  griddep_wait();
  extern __shared__ float row[];
  __shared__ float red[33];
  const int t = blockIdx.x;
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float s = 0.f;
    for (int c = 0; c < nsum; ++c) {
      const float v = y[((int64_t)t * nsum + c) * W + i];
      s += wt ? wt[(int64_t)t * nsum + c] * v : v;
    }
    row[i] = s;
    ss += s * s;
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float r = x[(int64_t)t * W + i] + row[i] * inv * (offset + w[i]);
    x[(int64_t)t * W + i] = r;
    if (out_cast) stf(out_cast, (int64_t)t * W + i, r);
  }
}

// out[t][0..n) = v / sqrt(mean(v^2) + eps) * (offset + w), v = columns [col0, col0 + n) of the fp32 rows `in`
template <typename OT>
__global__ void rmsnorm_cols_kernel(const float* __restrict__ in, int ld, int col0, int n, const float* __restrict__ w,
                                    float offset, float eps, OT* __restrict__ out, int ldo) {
  griddep_launch();
  griddep_wait();
  __shared__ float red[33];
  const int t = blockIdx.x;
  const float* r = in + (int64_t)t * ld + col0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss += r[i] * r[i];
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) stf(out, (int64_t)t * ldo + i, r[i] * inv * (offset + w[i]));
}

// One warp per (token, head): out = o / sqrt(mean_P(o^2) + eps) * w[0..P) * silu(gate), gate = columns of the fp32 rows gate_src
// (gate NULL: no gate)
template <typename OT>
__global__ void head_rmsnorm_gate_kernel(const float* __restrict__ o, const float* __restrict__ gate, int ldg, int gcol0,
                                         const float* __restrict__ w, float eps, OT* __restrict__ out, int T, int H, int P) {
  griddep_launch();
  griddep_wait();
  const int64_t wid = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wid >= (int64_t)T * H) return;
  const int lane = threadIdx.x & 31;
  const int64_t t = wid / H;
  const int h = (int)(wid - t * H);
  const float* r = o + wid * P;
  float ss = 0.f;
  for (int i = lane; i < P; i += 32) ss += r[i] * r[i];
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)P + eps);
  if (!gate) {  // no output gate: the norm alone
    for (int i = lane; i < P; i += 32) stf(out, wid * P + i, r[i] * inv * w[i]);
    return;
  }
  const float* gr = gate + t * ldg + gcol0 + (int64_t)h * P;
  for (int i = lane; i < P; i += 32) stf(out, wid * P + i, r[i] * inv * w[i] * silu_f(gr[i]));
}

// Parallel-branch residual step: x[t] += y1[t] + y2[t] (either may be absent), then out[t] = the GROUPED RMS norm of x[t]
// times w: the row is cut into `groups` equal consecutive parts and each part is divided by its own sqrt(mean(part^2) + eps).
// One CTA per token, the row in shared memory; warps take the groups round-robin, so the sums do not depend on the batch.
template <typename OT>
__global__ void add_group_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ y1, int ld1, const float* __restrict__ y2,
                                         int ld2, const float* __restrict__ w, int groups, float eps, OT* __restrict__ out, int W) {
  griddep_launch();
  griddep_wait();
  extern __shared__ float row[];  // [W] the row, [groups] 1 / rms per group
  float* inv = row + W;
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float r = x[(int64_t)t * W + i];
    if (y1) r += y2 ? y1[(int64_t)t * ld1 + i] + y2[(int64_t)t * ld2 + i] : y1[(int64_t)t * ld1 + i];
    row[i] = r;
    if (y1) x[(int64_t)t * W + i] = r;
  }
  __syncthreads();
  if (!out) return;
  const int gs = W / groups, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int g = warp; g < groups; g += blockDim.x >> 5) {
    float ss = 0.f;
    for (int i = lane; i < gs; i += 32) ss += row[g * gs + i] * row[g * gs + i];
    ss = warp_sum(ss);
    if (lane == 0) inv[g] = 1.0f / sqrtf(ss / (float)gs + eps);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < W; i += blockDim.x) stf(out, (int64_t)t * W + i, row[i] * inv[i / gs] * w[i]);
}

// Polynomial activation with unit-RMS powers: out = a N(z) + b N(z^2) + c N(z^3) + e, powers elementwise, N(u) = u / sqrt(mean(u^2)
// + eps) over the n columns of the token; coef = {a, b, c, e} on the device.  z = columns [col0, col0 + n) of fp32 rows.
template <typename OT>
__global__ void poly_norm_kernel(const float* __restrict__ in, int ld, int col0, int n, const float* __restrict__ coef, float eps,
                                 OT* __restrict__ out, int ldo) {
  griddep_launch();
  griddep_wait();
  __shared__ float red[33];
  const int t = blockIdx.x;
  const float* r = in + (int64_t)t * ld + col0;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float z2 = r[i] * r[i];
    s2 += z2;
    s4 += z2 * z2;
    s6 += z2 * z2 * z2;
  }
  s2 = block_sum(s2, red);
  s4 = block_sum(s4, red);
  s6 = block_sum(s6, red);
  const float a = coef[0] / sqrtf(s2 / (float)n + eps), b = coef[1] / sqrtf(s4 / (float)n + eps),
              c = coef[2] / sqrtf(s6 / (float)n + eps), e = coef[3];
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float z = r[i];
    stf(out, (int64_t)t * ldo + i, a * z + b * (z * z) + c * (z * z * z) + e);
  }
}

// The same with the row in registers: 16-byte loads, one pass over memory, the three sums reduced in one round, 8- or 16-byte
// stores.  Needs n % 4 == 0, 16-byte aligned rows on both sides and n <= 4 * PN_VEC * blockDim.x.  The sums of a row do not
// depend on what else is in the batch (one CTA per token, fixed order).
constexpr int PN_VEC = 4;
template <typename OT>
__global__ void poly_norm_vec_kernel(const float* __restrict__ in, int ld, int col0, int n, const float* __restrict__ coef,
                                     float eps, OT* __restrict__ out, int ldo) {
  griddep_launch();
  griddep_wait();
  __shared__ float red[3 * 32 + 3];
  const int t = blockIdx.x, nv = n >> 2;
  const float4* r = reinterpret_cast<const float4*>(in + (int64_t)t * ld + col0);
  float4 z[PN_VEC];
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
#pragma unroll
  for (int k = 0; k < PN_VEC; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    z[k] = i < nv ? r[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    const float q[4] = {z[k].x * z[k].x, z[k].y * z[k].y, z[k].z * z[k].z, z[k].w * z[k].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      s2 += q[j];
      s4 += q[j] * q[j];
      s6 += q[j] * q[j] * q[j];
    }
  }
  s2 = warp_sum(s2), s4 = warp_sum(s4), s6 = warp_sum(s6);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) red[warp] = s2, red[32 + warp] = s4, red[64 + warp] = s6;
  __syncthreads();
  if (warp < 3) {
    const float v = warp_sum(lane < nw ? red[warp * 32 + lane] : 0.f);
    if (lane == 0) red[96 + warp] = v;
  }
  __syncthreads();
  const float a = coef[0] / sqrtf(red[96] / (float)n + eps), b = coef[1] / sqrtf(red[97] / (float)n + eps),
              c = coef[2] / sqrtf(red[98] / (float)n + eps), e = coef[3];
  OT* o = out + (int64_t)t * ldo;
#pragma unroll
  for (int k = 0; k < PN_VEC; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i >= nv) continue;
    const float v[4] = {z[k].x, z[k].y, z[k].z, z[k].w};
    float y[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) y[j] = a * v[j] + b * (v[j] * v[j]) + c * (v[j] * v[j] * v[j]) + e;
    if constexpr (sizeof(OT) == 2) {
      *reinterpret_cast<uint2*>(o + 4 * i) = make_uint2(pack_bf16(y[0], y[1]), pack_bf16(y[2], y[3]));
    } else {
      *reinterpret_cast<float4*>(o + 4 * i) = make_float4(y[0], y[1], y[2], y[3]);
    }
  }
}

// Differential attention, closing step.  a fp32 [T][2 H][P] holds both maps' outputs: the kv group of `rep` output heads
// stores its first maps in rows [2 rep g, 2 rep g + rep) and its second maps in the next rep rows.  One warp per (token,
// output head): o = a1 - lambda a2;  out = o / sqrt(mean_P(o^2) + eps) * post * sigmoid(gate[h]).
template <typename OT>
__global__ void diff_head_norm_gate_kernel(const float* __restrict__ a, float lambda, float post, const float* __restrict__ gate,
                                           int ldg, int gcol0, float eps, OT* __restrict__ out, int T, int H, int rep, int P) {
  griddep_launch();
  griddep_wait();
  const int64_t wid = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wid >= (int64_t)T * H) return;
  const int lane = threadIdx.x & 31;
  const int64_t t = wid / H;
  const int h = (int)(wid - t * H);
  const int g = h / rep, j = h - g * rep;
  const float* a1 = a + ((t * 2 * H) + 2 * rep * g + j) * P;
  const float* a2 = a1 + (int64_t)rep * P;
  float ss = 0.f;
  for (int i = lane; i < P; i += 32) {
    const float o = a1[i] - lambda * a2[i];
    ss += o * o;
  }
  ss = warp_sum(ss);
  float f = post / sqrtf(ss / (float)P + eps);
  if (gate) f *= 1.0f / (1.0f + expf(-gate[t * ldg + gcol0 + h]));
  for (int i = lane; i < P; i += 32) stf(out, wid * P + i, (a1[i] - lambda * a2[i]) * f);
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// gu [T, 2 ff] (gate columns first): out = act(g) * u
// x[t] = e / sqrt(mean(e^2) + eps) * w with e = table[token]: a token embedding that is normed before it enters the stream
template <typename WT>
__global__ void embed_rmsnorm_kernel(const int32_t* __restrict__ tokens, const WT* __restrict__ table, const float* __restrict__ w,
                                     float eps, float* __restrict__ out, int W, int V) {
  griddep_launch();
  griddep_wait();
  __shared__ float red[33];
  const int t = blockIdx.x;
  int tok = tokens[t];
  tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = ldf(table, (int64_t)tok * W + i);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) out[(int64_t)t * W + i] = ldf(table, (int64_t)tok * W + i) * inv * w[i];
}

// Residual step of layers whose branches are scaled sums read through TWO norms of the same stream:
//   x[t] += c1 y1[t] + c2 y2[t] + c3 sum_{k < nsum} wt[t][k] y3[t nsum + k] + add_rows[t] + add_vec     (every term optional)
//   out1[t] = x[t] / rms(x[t]) * w1,  out2[t] = x[t] / rms(x[t]) * w2                                    (either may be absent)
// One CTA per token, the row in shared memory, one sum of squares for both norms.
template <typename OT>
__global__ void scaled_add_rmsnorm2_kernel(float* __restrict__ x, const float* __restrict__ y1, int ld1, float c1,
                                           const float* __restrict__ y2, int ld2, float c2, const float* __restrict__ y3, int nsum,
                                           const float* __restrict__ wt, float c3, const float* __restrict__ add_rows,
                                           const float* __restrict__ add_vec, const float* __restrict__ w1, OT* __restrict__ out1,
                                           const float* __restrict__ w2, OT* __restrict__ out2, float eps, int W) {
  griddep_launch();
  griddep_wait();
  extern __shared__ float row[];
  __shared__ float red[33];
  const int t = blockIdx.x;
  const bool touched = y1 || y2 || y3 || add_rows || add_vec;
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float r = x[(int64_t)t * W + i];
    float b = 0.f;
    if (y1) b += c1 * y1[(int64_t)t * ld1 + i];
    if (y2) b += c2 * y2[(int64_t)t * ld2 + i];
    if (y3) {
      float s = 0.f;
      for (int c = 0; c < nsum; ++c) {
        const float v = y3[((int64_t)t * nsum + c) * W + i];
        s += wt ? wt[(int64_t)t * nsum + c] * v : v;
      }
      b += c3 * s;
    }
    r += b;
    if (add_rows) r += add_rows[(int64_t)t * W + i];
    if (add_vec) r += add_vec[i];
    row[i] = r;
    ss += r * r;
    if (touched) x[(int64_t)t * W + i] = r;
  }
  if (!out1 && !out2) return;
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float u = row[i] * inv;
    if (out1) stf(out1, (int64_t)t * W + i, u * w1[i]);
    if (out2) stf(out2, (int64_t)t * W + i, u * w2[i]);
  }
}

template <typename OT>
__global__ void glu_kernel(const float* __restrict__ gu, OT* __restrict__ out, int ff, int act, int64_t total) {
  griddep_launch();
  griddep_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / ff;
    const int c = (int)(i - t * ff);
    const float g = gu[t * 2 * ff + c], u = gu[t * 2 * ff + ff + c];
    stf(out, i, (act == B200_ACT_GELU_TANH ? gelu_tanh_f(g) : silu_f(g)) * u);
  }
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_embed_bigram(const int32_t* tokens, const void* table, const void* bigram, int table_dtype, int buckets, int mul_prev,
                      int mul_cur, int32_t* prev_state, const int32_t* tok_seq, const int32_t* seq_start, const int32_t* seq_slot,
                      const int32_t* seq_pos0, float* out, void* out_cast, int T, int W, int V, float scale, void* stream) {
  B200_REQUIRE(tokens && table && out, "embed_bigram: null pointer");
  B200_REQUIRE(!bigram || (buckets > 0 && prev_state && tok_seq && seq_start && seq_slot && seq_pos0),
               "embed_bigram: the bigram table needs its bucket count, the previous-token state and the step's index tensors");
  if (T <= 0) return B200_OK;
  B200_DISPATCH_ELEM(table_dtype, WT,
                     B200_CUDA_OK(launch_kernel(embed_bigram_kernel<WT, WT>, dim3(T), dim3(256), 0, (cudaStream_t)stream, tokens,
                                                (const WT*)table, (const WT*)bigram, buckets, mul_prev, mul_cur, prev_state, tok_seq,
                                                seq_start, seq_slot, seq_pos0, out, (WT*)out_cast, W, V, scale)));
  return B200_OK;
}

int b200_rms_residual(float* x, const float* y, int nsum, const float* y_weight, const float* w, float offset, float eps,
                      void* out_cast, int out_dtype, int T, int W, void* stream) {
  B200_REQUIRE(x && y && w && nsum >= 1, "rms_residual: null pointer");
  B200_REQUIRE((size_t)W * 4 <= 200 * 1024, "rms_residual: rows of %d do not fit shared memory", W);
  if (T <= 0) return B200_OK;
  const size_t smem = (size_t)W * 4;
  B200_DISPATCH_ELEM(out_dtype, OT, {
    if (smem > 48 * 1024)
      B200_CUDA_OK(cudaFuncSetAttribute(rms_residual_kernel<OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    B200_CUDA_OK(launch_kernel(rms_residual_kernel<OT>, dim3(T), dim3(256), smem, (cudaStream_t)stream, x, y, nsum, y_weight, w,
                               offset, eps, (OT*)out_cast, W));
  });
  return B200_OK;
}

int b200_rmsnorm_cols(const float* in, int ld, int col0, int n, const float* w, float offset, float eps, void* out, int out_dtype,
                      int ldo, int T, void* stream) {
  B200_REQUIRE(in && w && out && n >= 1 && ldo >= n, "rmsnorm_cols: null pointer or bad shape");
  if (T <= 0) return B200_OK;
  B200_DISPATCH_ELEM(out_dtype, OT,
                     B200_CUDA_OK(launch_kernel(rmsnorm_cols_kernel<OT>, dim3(T), dim3(n >= 1024 ? 256 : 128), 0,
                                                (cudaStream_t)stream, in, ld, col0, n, w, offset, eps, (OT*)out, ldo)));
  return B200_OK;
}

int b200_head_rmsnorm_gate(const float* o, const float* gate, int ldg, int gate_col0, const float* w, float eps, void* out,
                           int out_dtype, int T, int H, int P, void* stream) {
  B200_REQUIRE(o && w && out && H >= 1 && P >= 1, "head_rmsnorm_gate: null pointer or bad shape");
  if (T <= 0) return B200_OK;
  const int64_t warps = (int64_t)T * H;
  B200_DISPATCH_ELEM(out_dtype, OT,
                     B200_CUDA_OK(launch_kernel(head_rmsnorm_gate_kernel<OT>, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0,
                                                (cudaStream_t)stream, o, gate, ldg, gate_col0, w, eps, (OT*)out, T, H, P)));
  return B200_OK;
}

int b200_embed_rmsnorm(const int32_t* tokens, const void* table, int table_dtype, const float* w, float eps, float* out, int T,
                       int W, int V, void* stream) {
  B200_REQUIRE(tokens && table && w && out && W >= 1 && V >= 1, "embed_rmsnorm: null pointer or bad shape");
  if (T <= 0) return B200_OK;
  B200_DISPATCH_ELEM(table_dtype, WT,
                     B200_CUDA_OK(launch_kernel(embed_rmsnorm_kernel<WT>, dim3(T), dim3(W >= 1024 ? 256 : 128), 0,
                                                (cudaStream_t)stream, tokens, (const WT*)table, w, eps, out, W, V)));
  return B200_OK;
}

int b200_scaled_add_rmsnorm2(float* x, const float* y1, int ld1, float c1, const float* y2, int ld2, float c2, const float* y3,
                             int nsum, const float* y3_weight, float c3, const float* add_rows, const float* add_vec,
                             const float* w1, void* out1, const float* w2, void* out2, float eps, int out_dtype, int T, int W,
                             void* stream) {
  B200_REQUIRE(x && (!out1 || w1) && (!out2 || w2) && (!y3 || nsum >= 1), "scaled_add_rmsnorm2: null pointer");
  B200_REQUIRE((size_t)W * 4 <= 200 * 1024, "scaled_add_rmsnorm2: rows of %d do not fit shared memory", W);
  if (T <= 0) return B200_OK;
  const size_t smem = (size_t)W * 4;
  B200_DISPATCH_ELEM(out_dtype, OT, {
    if (smem > 48 * 1024)
      B200_CUDA_OK(cudaFuncSetAttribute(scaled_add_rmsnorm2_kernel<OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    B200_CUDA_OK(launch_kernel(scaled_add_rmsnorm2_kernel<OT>, dim3(T), dim3(W >= 1024 ? 256 : 128), smem, (cudaStream_t)stream, x,
                               y1, ld1, c1, y2, ld2, c2, y3, nsum, y3_weight, c3, add_rows, add_vec, w1, (OT*)out1, w2, (OT*)out2,
                               eps, W));
  });
  return B200_OK;
}

int b200_glu(const float* gate_up, void* out, int out_dtype, int T, int ff, int act, void* stream) {
  B200_REQUIRE(gate_up && out, "glu: null pointer");
  B200_REQUIRE(act == B200_ACT_SILU || act == B200_ACT_GELU_TANH, "glu: activation %d", act);
  if (T <= 0) return B200_OK;
  const int64_t total = (int64_t)T * ff;
  int64_t blocks = (total + 255) / 256;
  blocks = blocks > 148 * 16 ? 148 * 16 : blocks;
  B200_DISPATCH_ELEM(out_dtype, OT,
                     B200_CUDA_OK(launch_kernel(glu_kernel<OT>, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, gate_up,
                                                (OT*)out, ff, act, total)));
  return B200_OK;
}

int b200_add_group_rmsnorm(float* x, const float* y1, int ld1, const float* y2, int ld2, const float* w, int groups, float eps,
                           void* out, int out_dtype, int T, int W, void* stream) {
  B200_REQUIRE(x && (out == nullptr || w) && (y1 || !y2), "add_group_rmsnorm: null pointer");
  B200_REQUIRE(groups >= 1 && W % groups == 0, "add_group_rmsnorm: rows of %d do not split into %d equal groups", W, groups);
  B200_REQUIRE((size_t)(W + groups) * 4 <= 200 * 1024, "add_group_rmsnorm: rows of %d do not fit shared memory", W);
  if (T <= 0) return B200_OK;
  const size_t smem = (size_t)(W + groups) * 4;
  B200_DISPATCH_ELEM(out_dtype, OT, {
    if (smem > 48 * 1024)
      B200_CUDA_OK(cudaFuncSetAttribute(add_group_rmsnorm_kernel<OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    B200_CUDA_OK(launch_kernel(add_group_rmsnorm_kernel<OT>, dim3(T), dim3(256), smem, (cudaStream_t)stream, x, y1, ld1, y2, ld2, w,
                               groups, eps, (OT*)out, W));
  });
  return B200_OK;
}

int b200_poly_norm(const float* in, int ld, int col0, int n, const float* coef, float eps, void* out, int out_dtype, int ldo, int T,
                   void* stream) {
  B200_REQUIRE(in && coef && out && n >= 1 && ldo >= n, "poly_norm: null pointer or bad shape");
  if (T <= 0) return B200_OK;
  const int es = out_dtype == B200_BF16 ? 2 : 4;
  const bool vec = n % 4 == 0 && ld % 4 == 0 && col0 % 4 == 0 && ldo % 4 == 0 && ((uintptr_t)in & 15) == 0 &&
                   ((uintptr_t)out & (4 * es - 1)) == 0 && n <= 4 * PN_VEC * 1024;
  if (vec) {  // the row in registers: a CTA of 128 .. 1024 threads (three warps reduce the three sums), four 16-byte loads each at most
    int threads = 128;
    while (threads * 4 * PN_VEC < n) threads *= 2;
    B200_DISPATCH_ELEM(out_dtype, OT,
                       B200_CUDA_OK(launch_kernel(poly_norm_vec_kernel<OT>, dim3(T), dim3(threads), 0, (cudaStream_t)stream, in, ld,
                                                  col0, n, coef, eps, (OT*)out, ldo)));
    return B200_OK;
  }
  B200_DISPATCH_ELEM(out_dtype, OT,
                     B200_CUDA_OK(launch_kernel(poly_norm_kernel<OT>, dim3(T), dim3(n >= 1024 ? 256 : 128), 0, (cudaStream_t)stream,
                                                in, ld, col0, n, coef, eps, (OT*)out, ldo)));
  return B200_OK;
}

int b200_diff_head_norm_gate(const float* a, float lambda, float post, const float* gate, int ldg, int gate_col0, float eps,
                             void* out, int out_dtype, int T, int H, int rep, int P, void* stream) {
  B200_REQUIRE(a && out && H >= 1 && P >= 1 && rep >= 1 && H % rep == 0, "diff_head_norm_gate: null pointer or bad shape");
  if (T <= 0) return B200_OK;
  const int64_t warps = (int64_t)T * H;
  B200_DISPATCH_ELEM(out_dtype, OT,
                     B200_CUDA_OK(launch_kernel(diff_head_norm_gate_kernel<OT>, dim3((unsigned)((warps + 7) / 8)), dim3(256), 0,
                                                (cudaStream_t)stream, a, lambda, post, gate, ldg, gate_col0, eps, (OT*)out, T, H, rep,
                                                P)));
  return B200_OK;
}

}  // extern "C"
