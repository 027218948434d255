/*
 * b200_paged.h -- C ABI of libb200_paged.so: the B200 (sm_100a) replacement for the
 * opaque device call on vllm-neuron's decode hot path.
 *
 * What it replaces.  In the reference every numeric op of a step happens inside ONE call,
 *   self.model(input_ids, position_ids, input_block_ids, slot_mapping, block_tables,
 *              full_context_lens, computed_context_lens, sampling_params, ...)
 *   vllm_neuron/worker/neuronx_distributed_model_runner.py:517-530
 *   -> vllm_neuron/worker/neuronx_distributed_model_loader.py:336-348  (NxDI forward)
 * The entry points below are the pieces of that call, plus the device-side version of the
 * host index construction that feeds it (model_runner.py:739-763, 798-832, 848-936).
 *
 * Conventions.  Plain pointers and sizes only (no torch types).  Every pointer is a DEVICE
 * pointer unless named host_*.  `stream` is a cudaStream_t passed as void*.  No entry point
 * allocates device memory or synchronises the device: scratch is passed in as `workspace`
 * (size from the matching *_workspace_bytes).  Return value 0 = ok; otherwise a B200_ERR_*
 * code (or a cudaError_t for launch failures) and b200_last_error() holds a message.
 * There is no CPU fallback: without an sm_100 device every compute call fails.
 *
 * Block-KV contract (reference: model_runner.py:76-81, platform.py:149-159):
 *   slot = block_id * block_size + offset;  slot == -1 is padding (never written);
 *   block 0 is vLLM's null block;  block tables are right-padded with 0.
 * Device pool layout (ours; NxDI's is not observable): K and V pools are separate arrays
 *   [num_blocks][Hkv][block_size][D] bf16, so one (block, kv head) tile is contiguous.
 */
#ifndef B200_PAGED_H_
#define B200_PAGED_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_ABI_VERSION 12

enum {
  B200_OK = 0,
  B200_ERR_INVALID_ARG = -1,
  B200_ERR_NO_DEVICE = -2,      /* no CUDA device with compute capability 10.x */
  B200_ERR_WORKSPACE = -3,      /* workspace too small */
  B200_ERR_UNSUPPORTED = -4,    /* shape outside what the kernels cover */
  B200_ERR_DRIVER = -5          /* cuTensorMapEncodeTiled / driver entry point failure */
};

/* B200_INT8_WO is only valid as a GEMM `ab_dtype`: bf16 activations x int8 weights (weight-only quantisation) */
enum { B200_BF16 = 0, B200_FP8_E4M3 = 1, B200_INT8 = 2, B200_F32 = 3, B200_INT8_WO = 4 };
/* gate activations of a gated-linear unit, and how a router turns its chosen logits into weights */
enum { B200_ACT_SWISH_CLAMPED = 0, B200_ACT_SILU = 1, B200_ACT_GELU_TANH = 2 };
enum { B200_ROUTE_SIGMOID = 0, B200_ROUTE_SOFTMAX_TOP = 1, B200_ROUTE_SOFTMAX_RENORM = 2 };

int b200_abi_version(void);
const char* b200_last_error(void);
/* 0 iff `device` is an sm_100 part (reference analogue: /dev/neuron* probe, vllm_neuron/__init__.py:8-23) */
int b200_device_check(int device);
/* number of kernel launches issued through this library by the calling process (bench.py's gpu_launches) */
uint64_t b200_launch_count(void);
/* Programmatic dependent launch for every kernel of the library (default on): a kernel may become resident while its
 * predecessor on the stream drains; the GEMM uses that window to prefetch weight tiles.  Returns the previous setting. */
int b200_set_pdl(int enabled);

/* ---------------------------------------------------------------- index construction on device
 * Replaces model_runner.py:765-832 (+ :887-917): per decode row b (persistent row r = row_ids[b]):
 *   position = num_tokens[r] - 1; full_ctx = position + 1;
 *   slot = block_table[r][position / bs] * bs + position % bs.
 * Outputs are int64 like the reference's tensors (ctx_lens int32 for the kernels). */
int b200_build_decode_meta(const int32_t* block_table, int64_t bt_row_stride, const int32_t* row_ids,
                           const int32_t* num_tokens, int64_t* slot_mapping, int64_t* positions, int32_t* ctx_lens,
                           int B, int max_blocks, int block_size, int num_spec, void* stream);
/* num_spec = 1: slot_mapping is [B].  num_spec = k > 1 (EAGLE / fused speculation, model_runner.py:825-830):
 * slot_mapping is [B][k] with slot_mapping[b][i] = slot_mapping[b][0] + i, built exactly like the reference's
 * `slots.append(slots[0] + i)` (not re-derived through the block table); a padded row stays -1.
 *
 * model_loader.py:308-334 (_remask_fused_spec_output): accepted [B][T] int64 is 0-padded; entries past
 * clamp(next_pos[b] - positions[b], 0, T) become -1 in out so that the runner strips them (model_runner.py:306-323). */
int b200_remask_spec_output(const int64_t* accepted, const int64_t* next_pos, const int64_t* positions, int64_t* out, int B,
                            int T, void* stream);
/* Replaces model_runner.py:739-763 (+ :853-885): batch-1 prefill with a prefix-cache hit.
 * slot_mapping_out[i] for i in [0, max_model_len): slot of token (num_computed + i) while that
 * token < prompt_len, else -1 (the reference's slice [num_computed:] right-padded with -1).
 * positions_out[i] = num_computed + i for the same range, else 0. */
int b200_build_prefill_meta(const int32_t* block_table_row, int prompt_len, int num_computed, int64_t* slot_mapping_out,
                            int64_t* positions_out, int max_model_len, int block_size, void* stream);
/* Mirror of InputBatch.block_table.append_row / add_row (model_runner.py:461-471, 484-486):
 * updates = n packed (row, col, block_id) int32 triples already on the device. */
int b200_block_table_scatter(int32_t* block_table, int64_t bt_row_stride, const int32_t* updates, int n, int rows,
                             int max_blocks, void* stream);
/* End of a decode step on device: tokens_io[b] = sampled[b]; num_tokens[row_ids[b]] += 1
 * (the device-side twin of model_runner.py:325-339, so a captured step can be replayed). */
int b200_advance_decode(const int64_t* sampled, int64_t* tokens_io, int32_t* num_tokens, const int32_t* row_ids, int B,
                        void* stream);

/* ---------------------------------------------------------------- KV-cache write
 * Scatter k, v [T][Hkv][D] (token stride in elements) into the pools by slot_mapping; slot < 0 skipped. */
int b200_kv_write(const void* k, const void* v, int64_t k_token_stride, int64_t v_token_stride, void* k_pool, void* v_pool,
                  const int64_t* slot_mapping, int T, int Hkv, int D, int block_size, int num_blocks, void* stream);
/* Fused: rotate q and k of a packed qkv row [T][(Hq+2Hkv)*D] (rotate-half RoPE, fp32 cos/sin tables
 * [max_pos][D/2]), write roped q back in place, and scatter roped k and v into the pools. */
int b200_rope_kv_write(void* qkv, const int64_t* positions, const float* cos_table, const float* sin_table, int max_pos,
                       void* k_pool, void* v_pool, const int64_t* slot_mapping, int T, int Hq, int Hkv, int D,
                       int block_size, int num_blocks, void* stream);

/* ---------------------------------------------------------------- paged attention
 * Decode (q_len = 1): out[b][h][:] = softmax(q K^T scale) V over ctx_lens[b] tokens gathered through
 * block_table[row_ids ? row_ids[b] : b].  Flash-decoding with a BALANCED split: all (sequence, kv head) pairs are laid
 * end to end as one list of 32-token blocks and every warp takes an equal contiguous share (>= min_quota blocks; 0 picks
 * the default), so ragged context lengths cost nothing; per-share partials live in `workspace` and a second kernel merges
 * them.  Outputs: q_dtype == B200_BF16 -> out [B][Hq][D] bf16;  FP8_E4M3 / INT8 -> out_q [B][Hq*D] with the dynamic
 * per-token scale out_scale [B] (same arithmetic as b200_quantize_per_token on the bf16 result), out optional.
 * ctx_lens[b] must be <= max_blocks * 32. */
size_t b200_paged_attn_decode_workspace_bytes(int B, int Hq, int Hkv, int D, int max_blocks, int min_quota);
int b200_paged_attn_decode(const void* q, int64_t q_token_stride, const void* k_pool, const void* v_pool, int num_blocks,
                           const int32_t* block_table, int64_t bt_row_stride, const int32_t* row_ids,
                           const int32_t* ctx_lens, void* out, void* out_q, float* out_scale, int q_dtype, void* workspace,
                           size_t workspace_bytes, int B, int Hq, int Hkv, int D, int block_size, int max_blocks,
                           int min_quota, float scale, void* stream);
/* Decode attention for callers that cannot allocate device memory.  (No counterpart in the reference: NxDI owns all of
 * its device buffers, so vllm-neuron never faces the question.)
 * b200_paged_attn_decode wants a workspace for its flash-decoding partials.  Not every caller can produce one: a binding
 * from a language runtime that may only pass along tensors its framework already holds, a plugin loaded into a serving
 * process after the device-memory budget was handed out (vLLM gives what is left after the weights to the KV pool), or
 * any host that is not allowed to call cudaMalloc.  This variant takes the same inputs and outputs but no workspace: the
 * partials go into an array of B200_DECODE_STATIC_SCRATCH_BYTES that is part of the library image, so EVERY GPU that loads
 * the library gives up that much memory until the process exits, whether or not this entry point is ever called.
 *   - Limit: a shape whose b200_paged_attn_decode_workspace_bytes(...) exceeds the array is refused with
 *     B200_ERR_WORKSPACE (the message gives both numbers) and nothing is launched.  The headline shape (B=64, Hq=32,
 *     Hkv=8, D=128, 64 blocks per sequence) needs 18.1 MB; a larger min_quota shrinks the need.
 *   - It calls no cudaMalloc / cudaFree and no allocating library routine, and does not synchronise.
 *   - First call on each device: the library looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current) and keeps it.  Make that first call on every device you use BEFORE you start capturing a stream.
 *   - There is ONE array per device and every call uses it.  Two calls that can overlap on the same GPU (different
 *     streams, or different host threads feeding different streams) corrupt each other's partials; keep them on one
 *     stream or order them with events.  The array keeps whatever the last call left there; nothing in it needs to be
 *     zero, the kernels overwrite every entry they later read.
 * Results are bit-identical to b200_paged_attn_decode with the same arguments. */
#define B200_DECODE_STATIC_SCRATCH_BYTES (32u << 20)
size_t b200_paged_attn_decode_static_max_bytes(void);
int b200_paged_attn_decode_static(const void* q, int64_t q_token_stride, const void* k_pool, const void* v_pool,
                                  int num_blocks, const int32_t* block_table, int64_t bt_row_stride, const int32_t* row_ids,
                                  const int32_t* ctx_lens, void* out, void* out_q, float* out_scale, int q_dtype, int B,
                                  int Hq, int Hkv, int D, int block_size, int max_blocks, int min_quota, float scale,
                                  void* stream);
/* Prefix-cached prefill, one sequence: queries for absolute positions computed_len .. computed_len+S_new-1,
 * causal over cached prefix + new tokens, all K/V already in the pools. */
int b200_paged_attn_prefill(const void* q, int64_t q_token_stride, const void* k_pool, const void* v_pool, int num_blocks,
                            const int32_t* block_table_row, void* out, int S_new, int computed_len, int Hq, int Hkv,
                            int D, int block_size, float scale, void* stream);

/* ---------------------------------------------------------------- per-channel-scaled GEMM (tcgen05 / TMEM / TMA)
 * out[M][N] = (sum_k a[m][k] * w[n][k]) * a_scale[m] * w_scale[n] + bias[n] + residual[m][n]
 * a: [M][K], w: [N][K], both `ab_dtype` (BF16 | FP8_E4M3 | INT8); scales fp32 (NULL = 1), bias bf16 [N] or NULL,
 * residual bf16 [M][N] or NULL; out_dtype BF16 | F32.
 * M <= 128 (decode): one CTA per (128-row weight tile, K split); the `split_k` CTAs (0 = auto; 1, 2, 4 or 8) of a tile
 *   form a thread-block cluster and are summed through distributed shared memory in fixed rank order; needs no workspace.
 *   Weights stream through a deep TMA ring (up to 176 KB per SM in flight, issued before the previous kernel of the
 *   stream has finished), activations through a shallow one; the schedule (S, CTAs per SM, ring depths) is picked per
 *   shape from occupancy queries and a latency/bandwidth model (b200_gemm_decode_plan reports it).
 * M > 128 (prefill): persistent stream-K over min(split_k, #SM) CTAs (0 = one per SM), each an equal share of the
 *   (tile, k-block) space; tiles cut by a share boundary are summed in fixed order by the last contributor.
 *   `workspace` (b200_gemm_workspace_bytes) holds the fix-up counters in its first 4 KiB: it must be ZERO-FILLED before
 *   its first use and is left zeroed by every call; one workspace may serve all GEMMs issued on one stream. */
size_t b200_gemm_workspace_bytes(int M, int N, int K, int ab_dtype, int split_k);
/* The decode schedule (M <= 128) chosen on the current device for a shape: out6 = {cluster size S, CTAs per SM, weight
 * ring depth, activation ring depth, CTAs the chip holds at once, dynamic shared memory bytes}.  Needs a device.
 * silu_mul selects the epilogue variant planned for: 0 linear, 1 SiLU*mul (b200_gemm_silu_mul), 2 RoPE + KV write
 * (b200_gemm_rope_kv_write). */
int b200_gemm_decode_plan(int M, int N, int K, int ab_dtype, int split_k, int silu_mul, int has_residual, int* out6);
/* Profiling aid: with a non-NULL device buffer ([#CTAs][8] uint64) every decode-schedule GEMM CTA records %globaltimer
 * at its phase boundaries (tools/gemm_trace.py); NULL (default) switches it off. */
void b200_gemm_set_trace(void* device_buf);
int b200_gemm(const void* a, const void* w, void* out, const float* a_scale, const float* w_scale, const void* bias,
              const void* residual, int M, int N, int K, int ab_dtype, int out_dtype, int split_k, void* workspace,
              size_t workspace_bytes, void* stream);
/* INT8 weight-only linear (SURVEY 8(b) `b200_gemm_int8_wo`; reference config keys quantized / quantization_dtype=int8 with
 * bf16 activations, model_loader.py:885-898): out = (a_bf16 . w_int8^T) * w_scale[n] + bias + residual.  The int8 rows are
 * streamed from HBM as int8 (half the bytes of bf16) and widened to bf16 operand tiles in shared memory by the CTA's
 * epilogue warps (exact), then multiplied with kind::f16.  Same as b200_gemm with ab_dtype = B200_INT8_WO. */
int b200_gemm_int8_wo(const void* a_bf16, const void* w_int8, void* out, const float* w_scale, const void* bias,
                      const void* residual, int M, int N, int K, int out_dtype, int split_k, void* workspace,
                      size_t workspace_bytes, void* stream);
/* gate/up projection with SiLU(gate)*up fused into the epilogue.  w_gu [2I][K] holds, per group of 32 rows, 16 gate rows
 * followed by the 16 up rows of the same channels (w_scale / bias permuted alike); out_act [M][I] bf16 =
 * bf16(silu(bf16(gate)) * bf16(up)) exactly as b200_gemm + b200_silu_mul produce; group_amax [M][2I/32] fp32 receives
 * max|act| over the 16 channels of every row group, for the per-token quantisation that follows
 * (b200_quantize_per_token).  split_k as b200_gemm, at most 4 in the decode schedule. */
int b200_gemm_silu_mul(const void* a, const void* w_gu, void* out_act, const float* a_scale, const float* w_scale,
                       const void* bias, float* group_amax, int M, int N2, int K, int ab_dtype, int split_k,
                       void* workspace, size_t workspace_bytes, void* stream);
/* The same gate/up GEMM + SiLU*mul with the dynamic per-token quantisation of its result (the down_proj input) done in the
 * SAME launch: out_q [M][N2/2] e4m3 / int8, out_scale [M].  The CTAs agree on each token's amax through a grid-wide
 * barrier; `state` is 1040 bytes of device memory, zero-initialised ONCE and then owned by the library (any number of
 * launches on one stream).  Bit-identical to b200_gemm_silu_mul + b200_quantize_per_token.  Decode schedule only:
 * returns B200_ERR_UNSUPPORTED (nothing launched) when M > 128 or when the shape does not run as one resident wave of
 * one CTA per weight tile -- the caller then uses the two-call form.  "Resident" is worked out from the occupancy
 * query for a GPU that runs nothing else: if another stream or process holds SM slots while this kernel starts, CTAs wait
 * at the barrier for peers that cannot be scheduled and the kernel traps after about 2 s.  Use it only where this library's
 * stream owns the GPU; the product path keeps it off (B200_FUSE_SILU_QUANT unset) and uses the two-call form. */
int b200_gemm_silu_mul_quant(const void* a, const void* w_gu, void* out_q, float* out_scale, const float* a_scale,
                             const float* w_scale, const void* bias, void* state, int M, int N2, int K, int ab_dtype,
                             void* stream);

/* qkv projection with RoPE and the KV-cache write fused into its epilogue: b200_gemm (bf16 out, no residual) followed by
 * b200_rope_kv_write on its output, in ONE launch when the decode schedule splits K over a cluster (the token's owner
 * holds whole heads; rotate-half partner = lane ^ D/8), else as the two launches.  Same bits either way: qkv_out keeps
 * rotated q, un-rotated k and v; rotated k and v land in the pools at slot_mapping[t] (slot < 0 skipped).
 * Replaces the qkv linear + rotary + KV scatter inside NxDI's decoder layer (model_loader.py:336-348). */
int b200_gemm_rope_kv_write(const void* a, const void* w, void* qkv_out, const float* a_scale, const float* w_scale,
                            const void* bias, int M, int N, int K, int ab_dtype, int split_k, void* workspace,
                            size_t workspace_bytes, const int64_t* positions, const float* cos_table,
                            const float* sin_table, int max_pos, void* k_pool, void* v_pool, const int64_t* slot_mapping,
                            int Hq, int Hkv, int D, int block_size, int num_blocks, void* stream);

/* ---------------------------------------------------------------- glue kernels of the decoder step */
/* y = x * rsqrt(mean(x^2)+eps) * w (fp32 math).  Writes any of: out_bf16 [T][H]; out_q [T][H] (q_dtype FP8/INT8)
 * with dynamic per-token scale out_scale [T] (scale = amax/qmax, q = rn(y_bf16 / scale)). */
int b200_rmsnorm(const void* x, const void* w, void* out_bf16, void* out_q, float* out_scale, int T, int H, float eps,
                 int q_dtype, void* stream);
/* act = silu(gate) * up from gate_up [T][2I] (gate columns first); same output options as rmsnorm. */
int b200_silu_mul(const void* gate_up, void* out_bf16, void* out_q, float* out_scale, int T, int I, int q_dtype,
                  void* stream);
/* Dynamic per-token quantisation of x [T][K] bf16.  group_amax [T][n_groups] (optional, from b200_gemm_silu_mul)
 * supplies partial row maxima so rows can be cut across CTAs without a scan; NULL = scan the row. */
int b200_quantize_per_token(const void* x, void* out_q, float* out_scale, const float* group_amax, int n_groups, int T, int K,
                            int q_dtype, void* stream);
int b200_embedding(const int64_t* tokens, const void* table, void* out, int T, int H, int V, void* stream);
/* ---------------------------------------------------------------- on-device sampling (top-k / top-p / temperature)
 * Replaces NxDI's on-device sampler behind `self.model.sample(...)` (model_runner.py:1084-1098, model_loader.py:367-382)
 * fed by the [B][3] (top_k, top_p, temperature) tensor of get_nxd_sampling_params (model_runner.py:1106-1140).
 * b200_topk_candidates: per row the 256 (= _MAX_NEURON_SAMPLING_TOP_K, model_runner.py:74) largest fp32 logits of the
 *   local vocab shard, sorted by (value desc, index asc): cand_val [B][256] fp32, cand_idx [B][256] int64 (global token id
 *   = idx_offset + column; -inf / -1 padding when V < 256).  Exact (radix select), ties towards the lower index.
 * b200_sample_candidates: cand_* laid out [groups][B][256] (groups = TP shards, all-gathered by the caller); merges the
 *   groups, keeps top_k (1..256), w_j = exp((v_j - v_0)/temperature), keeps the shortest prefix with cumulative weight
 *   >= top_p * Z, and draws by inverse CDF with the caller's uniform u[b] in [0,1).  top_k == 1 is greedy (== b200_argmax).
 *   fp32, sequential, fixed order: the result is a pure function of (logits, params, u). */
int b200_topk_candidates(const float* logits, int64_t row_stride, float* cand_val, int64_t* cand_idx, int B, int V,
                         int64_t idx_offset, void* stream);
int b200_sample_candidates(const float* cand_val, const int64_t* cand_idx, int groups, int B, const float* params,
                           const float* u, int64_t* out_ids, void* stream);
/* Log-probabilities on device (the reference returns them from its CPU sampling path, model_runner.py:347-356, 1142-1239:
 * vLLM's Sampler = raw log-softmax of the logits, the sampled token's rank, the top-n tokens).
 * b200_row_lse: per row of the local vocab shard, out_max[b] = max_v logits[b][v], out_sumexp[b] = sum_v exp(logits - max)
 *   (fixed reduction tree: bit-reproducible).  TP: one (max, sumexp) pair per shard, laid out [groups][B] for the gather.
 * b200_gather_logprobs: with the sorted candidate lists of b200_topk_candidates ([groups][B][256]) and the sampled ids:
 *   out_ids / out_logprobs [B][1 + num_logprobs] (int32 / fp32; column 0 = the sampled token, then the num_logprobs most
 *   likely tokens, value desc / index asc), out_rank[b] = #tokens whose logit is >= the sampled token's (itself included). */
int b200_row_lse(const float* logits, int64_t row_stride, float* out_max, float* out_sumexp, int B, int V, void* stream);
int b200_gather_logprobs(const float* cand_val, const int64_t* cand_idx, int groups, int B, const int64_t* sampled,
                         const float* row_max, const float* row_sumexp, int num_logprobs, int32_t* out_ids,
                         float* out_logprobs, int32_t* out_rank, void* stream);
/* Greedy sampling (reference: top_k=1, temperature=1.0 for temperature 0, model_runner.py:1126-1128).
 * out_idx[t] = idx_offset + first index of the row maximum; out_val[t] = that maximum (for TP merges). */
int b200_argmax(const float* logits, int64_t row_stride, float* out_val, int64_t* out_idx, int T, int V,
                int64_t idx_offset, void* stream);

/* ---------------------------------------------------------------- tensor-parallel exchange (NVLink peer memory)
 * All-reduce (sum over `world` ranks, bf16) of the row-parallel GEMM outputs fused with the RMSNorm (+ dynamic per-token
 * quantisation) that consumes it; replaces the Neuron-runtime collectives NxDI issues after o_proj / down_proj
 * (tp_degree, model_loader.py:752-753).  host_peer_bufs[p] / host_peer_flags[p] are HOST arrays of `world` DEVICE
 * pointers: rank p's partial [T][H] bf16 and rank p's flag area ([>= T][8] uint32, zero-initialised once), both inside
 * peer-mapped (symmetric) memory.  epoch [>= T] uint32 is local, zero-initialised once.  Every rank must issue the same
 * sequence of calls; consecutive calls must alternate between two partial buffers (see csrc/tp_allreduce.cu).
 * Outputs (local): x_out [T][H] bf16 = the sum (ranks added in rank order, identical bits on every rank); with norm_w:
 * out_bf16 and/or out_q + out_scale as b200_rmsnorm.  norm_w == NULL: plain all-reduce. */
int b200_allreduce_rmsnorm(const void* const* host_peer_bufs, void* const* host_peer_flags, uint32_t* epoch, int rank,
                           int world, void* x_out, const void* norm_w, void* out_bf16, void* out_q, float* out_scale, int T,
                           int H, float eps, int q_dtype, void* stream);
/* Same exchange with the sum done INSIDE the NVSwitch (NVLS): mc_buf is the MULTICAST device address of the partial
 * [T][H] bf16 (the address that maps every rank's replica; torch symmetric memory: handle.multicast_ptr + offset); the
 * kernel issues one multimem.ld_reduce (bf16x2 add, fp32 accumulate) per 16 bytes, so a rank receives T*H*2 bytes
 * instead of (world-1) x that.  Flags, epoch, outputs and the alternation rule as above.  The order of the additions is
 * the switch's: identical bits on every rank, but not necessarily those of the rank-order sum (last bf16 bit). */
int b200_allreduce_rmsnorm_nvls(const void* mc_buf, void* const* host_peer_flags, uint32_t* epoch, int rank, int world,
                                void* x_out, const void* norm_w, void* out_bf16, void* out_q, float* out_scale, int T,
                                int H, float eps, int q_dtype, void* stream);

/* Greedy merge over the vocabulary shards of a TP group (the reference leaves sampling of the sharded logits to NxDI's
 * on-device sampler, model_loader.py:367-382).  host_peer_vals[p] / host_peer_idxs[p]: rank p's [B] fp32 local maxima and
 * [B] int64 GLOBAL indices inside peer-mapped memory, written by b200_argmax earlier on the stream; host_peer_flags[p]:
 * rank p's [8] uint32 flag words (zero-initialised once); epoch: one local uint32 (zero-initialised once).
 * out_ids[b] = index of the largest value over all ranks, ties to the lowest index; identical on every rank. */
int b200_tp_argmax_merge(const void* const* host_peer_vals, const void* const* host_peer_idxs,
                         void* const* host_peer_flags, uint32_t* epoch, int rank, int world, int64_t* out_ids, int B,
                         void* stream);

/* ---------------------------------------------------------------- hybrid decoders (state-space + windowed attention + MoE)
 * Kernels for decoders that mix state-space layers, sliding-window attention with a softmax sink, Dynamic-Tanh norms and
 * a mixture-of-experts feed-forward.  The residual stream, norms, softmax, router and recurrences are fp32; `*_dtype`
 * arguments (B200_BF16 or B200_F32) name the type of GEMM operands, weights and KV pools.
 * A step is a RAGGED batch: B sequences, sequence s brings tokens [seq_start[s], seq_start[s+1]) of the flattened batch,
 * continues at position seq_pos0[s] and owns state slot seq_slot[s]; tok_seq[t] is the sequence of token t.  A sequence
 * with seq_pos0 == 0 starts from zero state whatever its slot held. */

/* out[t][:] = table[tokens[t]][:] * scale (fp32 residual stream) */
int b200_embed_scale(const int32_t* tokens, const void* table, int table_dtype, float* out, int T, int W, int V, float scale,
                     void* stream);
/* Dynamic Tanh: out[i] = gain[i] * tanh(a * x[i]) + shift[i] (a: one scalar per norm); x fp32 [T][W], gain `w` / shift `b` fp32 [W],
 * out in out_dtype */
int b200_dyt_norm(const float* x, const float* w, const float* b, float alpha, void* out, int out_dtype, int T, int W,
                  void* stream);
/* x[t] += dyt1(sum_{c < nsum} y[t * nsum + c] + y2[t]);  out2[t] = dyt2(x[t]) when out2 != NULL.  y fp32 [T * nsum][W],
 * y2 fp32 [T][W] or NULL. */
int b200_dyt_residual(float* x, const float* y, int nsum, const float* y2, const float* w1, const float* b1, float alpha1,
                      const float* w2, const float* b2, float alpha2, void* out2, int out_dtype, int T, int W, void* stream);
/* r = y * silu(z) first, then each of the `groups` equal slices r_k of a row becomes r_k * rsqrt(mean(r_k^2) + eps), times w.
 * y fp32 [T][inner]; z fp32 rows of pitch ldz. */
int b200_gated_group_rmsnorm(const float* y, const float* z, int ldz, const float* w, void* out, int out_dtype, int T,
                             int inner, int groups, float eps, void* stream);
/* gate_up fp32 [T][2 ff] (gate first): a = min(gate, L), b = max(-L, min(up, L)), out = (b + 1) * a / (1 + exp(-1.702 a)) */
int b200_clamped_glu(const float* gate_up, void* out, int out_dtype, int T, int ff, float limit, void* stream);
/* Causal depthwise convolution + SiLU over columns [col0, col0 + C) of `in` (fp32, pitch ld); conv_w fp32 [C][taps] with
 * the LAST tap on the current token; conv_b fp32 [C] or NULL; state fp32 [slots][taps - 1][C] holds each sequence's last
 * inputs and is updated. */
int b200_causal_conv_silu(const float* in, int ld, int col0, const float* conv_w, const float* conv_b, float* state,
                          const int32_t* tok_seq, const int32_t* seq_start, const int32_t* seq_slot, const int32_t* seq_pos0,
                          void* out, int out_dtype, int T, int B, int C, int taps, void* stream);
/* The same convolution with two more choices: in_bias fp32 [C] (or NULL) is added to every input read from `in` (the bias of
 * the projection that produced it; the state keeps biased inputs), and silu == 0 leaves the convolution's sum as it is. */
int b200_causal_conv(const float* in, int ld, int col0, const float* conv_w, const float* conv_b, const float* in_bias, int silu,
                     float* state, const int32_t* tok_seq, const int32_t* seq_start, const int32_t* seq_slot,
                     const int32_t* seq_pos0, void* out, int out_dtype, int T, int B, int C, int taps, void* stream);
/* Selective state-space scan: xbc [T][C] = [x: H*P | B: G*N | C: G*N] (x_dtype); dt_raw = dt_in[t][dt_col0 + h] (fp32);
 * dt = softplus(dt_raw + dt_bias[h]); S = exp(-exp(A_log[h]) dt) S + dt B x^T; y = S^T C + D[h] x.
 * state fp32 [slots][H][P][N], updated; y fp32 [T][H*P].  Head h reads group h / (H / G).  N <= 256.
 * segs (or NULL): int32 [num_segs][4] = {first token, end token, sequence, 1 (first of its sequence) | 2 (last)}, 16-byte
 * aligned, a sequence's segments consecutive; seq_seg0 int32 [B + 1] = first segment of each sequence; scratch seg_state
 * fp32 [num_segs][H][P][N] and seg_dtsum fp32 [num_segs][H].  Segments then run in parallel (three launches). */
int b200_ssd_scan(const void* xbc, int x_dtype, int C, const float* dt_in, int ld_dt, int dt_col0, const float* A_log,
                  const float* dt_bias, const float* D, float* state, const int32_t* seq_start, const int32_t* seq_slot,
                  const int32_t* seq_pos0, float* y, int B, int H, int P, int N, int G, const int32_t* segs, int num_segs,
                  const int32_t* seq_seg0, float* seg_state, float* seg_dtsum, void* stream);
/* Scatter keys [G][D] (columns k_col0..) and values [G][Dv] (columns v_col0..) of the fp32 rows `qkv` into the pools
 * K [num_blocks][G][block_size][D], V [num_blocks][G][block_size][Dv] by slot (slot < 0: skipped).
 * mode 0: plain; 1: also keep the unmixed values in v_first fp32 [T][G*Dv]; 2: cache v + lambda * (v_first - v) instead of v. */
int b200_kv_write_vmix(const float* qkv, int ld, int k_col0, int v_col0, float* v_first, float lambda, int mode, void* k_pool,
                       void* v_pool, int kv_dtype, const int64_t* slot_mapping, int T, int G, int D, int Dv, int block_size,
                       void* stream);
/* Sliding-window attention with a per-head sink logit in the softmax denominator (sink NULL: ordinary softmax), scores
 * taken as they are (a rotation, if any, is already in q and the cached keys).
 * q fp32 rows (pitch ldq, head h at column h * D); token t is position tok_pos[t] of the sequence whose block-table row is
 * tok_row[t] and sees keys j with 0 <= pos - j < window, all already in the pools.  Value rows have pitch v_pitch >= Dv
 * (v_pool may be k_pool itself, with the values in the leading columns of the key rows).  out [T][H][Dv] in kv_dtype.
 * Dv <= 512.
 * Variants: chunk > 0 also hides keys before the first position of the query's chunk, pos - pos % chunk; softcap > 0 replaces
 * the scaled score s by softcap * tanh(s / softcap); sigmoid_bias fp32 [H] (or NULL) makes the weight of a visible key
 * sigmoid(s + sigmoid_bias[h]) with no normalisation over keys (no sink then); v_div >= 1: key head g reads value head
 * g / v_div of a value pool with G / v_div heads; out_f32: fp32 output rows whatever kv_dtype.
 * splits > 1: that many CTAs share a (token, head block)'s keys and a second launch merges their partial results from
 * split_workspace fp32 [T * H * splits * (Dv + 2)] (long contexts at small batch: more CTAs than one per token and head block).
 * pool > 0 (with a window): beside the window's keys a query at position i sees ONE key / value for every block b of `pool`
 * positions that lies wholly before its window, b pool + pool - 1 <= i - window -- the block's rows of pooled_k / pooled_v
 * (b200_kv_pool_mean); blocks and keys share the softmax. */
int b200_swa_sink_attn(const float* q, int ldq, const void* k_pool, const void* v_pool, int kv_dtype, const int32_t* block_table,
                       int64_t bt_stride, const int32_t* tok_row, const int32_t* tok_pos, const float* sink, float scale,
                       int window, void* out, int T, int H, int G, int D, int Dv, int v_pitch, int block_size, int chunk,
                       float softcap, const float* sigmoid_bias, int v_div, int out_f32, int splits, float* split_workspace,
                       const void* pooled_k, const void* pooled_v, int pool, void* stream);
/* Means of the key / value blocks that the step completes: sequence s brings tokens [seq_start[s], seq_start[s+1]) at positions
 * seq_pos0[s].. (block-table row seq_slot[s]); for every block of `pool` positions whose last position is among them the block's
 * `pool` key and value rows are read back from the pools, summed in fp32, divided by `pool` and written to
 * pooled_k [num_blocks][G][ppb][D] / pooled_v [num_blocks][Gv][ppb][Dv], ppb = ceil(block_size / pool): the entry of a block lives
 * in the page of the block's last position e, at index (e % block_size) / pool.  T = tokens of the step (sizes the launch).
 * Run it after the step's keys are written. */
int b200_kv_pool_mean(const void* k_pool, const void* v_pool, void* pooled_k, void* pooled_v, int kv_dtype,
                      const int32_t* block_table, int64_t bt_stride, const int32_t* seq_start, const int32_t* seq_slot,
                      const int32_t* seq_pos0, int B, int T, int G, int Gv, int D, int Dv, int block_size, int pool, void* stream);
/* The same attention for prompt portions on the tensor cores (bf16 pools; D and Dv multiples of 16, Dv <= 256, else
 * B200_ERR_UNSUPPORTED): sequence s brings tokens [seq_start[s], seq_start[s+1]) at positions seq_pos0[s].., block-table row
 * seq_slot[s]; max_new = the longest portion of the step.  q is rounded to bf16; softmax and accumulation are fp32.
 * chunk / softcap / sigmoid_bias / v_div / out_f32 as above; split_p: the weights enter the tensor cores as two bf16 terms
 * (rounded value + remainder) instead of one. */
int b200_swa_sink_attn_prefill(const float* q, int ldq, const void* k_pool, const void* v_pool, const int32_t* block_table,
                               int64_t bt_stride, const int32_t* seq_start, const int32_t* seq_slot, const int32_t* seq_pos0,
                               int B, int max_new, const float* sink, float scale, int window, void* out, int H, int G, int D,
                               int Dv, int v_pitch, int block_size, int chunk, float softcap, const float* sigmoid_bias, int v_div,
                               int out_f32, int split_p, const void* pooled_k, const void* pooled_v, int pool, void* stream);
/* Prompt portions on the 5th-generation tensor cores (tcgen05, accumulators in tensor memory): same ragged step arguments as
 * b200_swa_sink_attn_prefill, no sink and no window.  Kernels exist for pages of 32 tokens and D = Dv = 64 or 128 (softmax,
 * capped softmax, sigmoid weights) and, with v_div = 2, D = 32 or 64 with Dv = 64 or 128 (softmax); q rows must be 16-byte aligned.
 * b200_swa_sink_attn_prefill_tc_supported says whether a combination has one; the launch returns B200_ERR_UNSUPPORTED
 * otherwise.  num_blocks = pages of the pools. */
int b200_swa_sink_attn_prefill_tc_supported(int D, int Dv, int block_size, int v_div, int capped, int sigmoid);
int b200_swa_sink_attn_prefill_tc(const float* q, int ldq, const void* k_pool, const void* v_pool, int num_blocks,
                                  const int32_t* block_table, int64_t bt_stride, const int32_t* seq_start,
                                  const int32_t* seq_slot, const int32_t* seq_pos0, int B, int max_new, float scale, void* out,
                                  int H, int G, int D, int Dv, int block_size, int chunk, float softcap,
                                  const float* sigmoid_bias, int v_div, int out_f32, int split_p, void* stream);
/* The same attention for decode-sized steps on the tensor cores (bf16 pools with a value pool of its own; D and Dv multiples of
 * 16, Dv <= 256, else B200_ERR_UNSUPPORTED): the query heads of a kv head are the rows of one MMA tile, each key and value row
 * is fetched once for all of them.  Arguments as b200_swa_sink_attn (+ split_p as in the prompt kernel). */
int b200_swa_sink_attn_decode_tc(const float* q, int ldq, const void* k_pool, const void* v_pool, const int32_t* block_table,
                                 int64_t bt_stride, const int32_t* tok_row, const int32_t* tok_pos, const float* sink, float scale,
                                 int window, void* out, int T, int H, int G, int D, int Dv, int v_pitch, int block_size, int chunk,
                                 float softcap, const float* sigmoid_bias, int v_div, int out_f32, int split_p, int splits,
                                 float* split_workspace, const void* pooled_k, const void* pooled_v, int pool, void* stream);
/* Merge of key splits: part fp32 [rows][splits][2 + Dv] = {maximum, denominator, unnormalised accumulator} per split ->
 * out [rows][Dv] (fp32 when out_f32, else out_dtype); sigmoid: plain sums, no denominator. */
int b200_attn_split_merge(const float* part, int splits, int Dv, int sigmoid, int out_f32, int out_dtype, void* out, int64_t rows,
                          void* stream);
/* Between the projections and the attention of layers that norm and rotate: fp32 rows `src` (pitch ld) hold q [H][D] at
 * q_col0, k [G][D] at k_col0, v [Gv][Dv] at v_col0.  q_norm / k_norm fp32 [H * D] / [G * D] (or NULL): RMS norm over the WHOLE
 * projection, times the weight.  The first rot_n columns of every q and k head turn by tok_pos[t]: pairs (i, i + rot_n / 2) when
 * rot_half, else (2i, 2i + 1); (u, v) -> (u cos - v sin, v cos + u sin), cos / sin fp32 tables [positions][rot_n / 2].
 * q -> q_out fp32 [T][H * D], head h times q_head_scale[h] when given (a per-head temperature of the scores);
 * k, v -> pools K [num_blocks][G][block_size][D], V [num_blocks][Gv][block_size][Dv] by slot. */
int b200_qk_norm_rope_kv_write(const float* src, int ld, int q_col0, int k_col0, int v_col0, const float* q_norm,
                               const float* k_norm, float eps, int rot_n, int rot_half, const float* cos_table,
                               const float* sin_table, const int32_t* tok_pos, const int64_t* slot_mapping, float* q_out,
                               void* k_pool, void* v_pool, int kv_dtype, int T, int H, int G, int Gv, int D, int Dv, int block_size,
                               const float* q_head_scale, void* stream);
/* Router decision over fp32 logits [T] rows of pitch ld (+ bias fp32 [E] when given): the `top` largest (ties to the lower
 * index); weights = sigmoid of each chosen logit, no renormalisation (B200_ROUTE_SIGMOID), or the softmax over the chosen
 * logits only (B200_ROUTE_SOFTMAX_TOP), or the softmax over ALL experts with the chosen scores divided by their sum + 1e-20
 * (B200_ROUTE_SOFTMAX_RENORM). */
int b200_moe_topk(const float* logits, int ld, const float* bias, int mode, int32_t* topk_idx, float* topk_weight, int T, int E,
                  int top, void* stream);
/* rows per expert tile of b200_moe_align / b200_grouped_linear; four times as many (tile_rows = 4 x this) are taken for
 * prompt-sized batches of 16-byte aligned bf16 operands, where every weight tile then serves 128 rows */
int b200_moe_tile_rows(void);
/* Sort the npairs (token, choice) pairs by expert into tiles: sorted_ids [cap] (pair id or -1), tile_expert [max_tiles],
 * *num_tiles.  Needs max_tiles >= ceil(npairs / tile_rows) + E and cap >= max_tiles * tile_rows. */
int b200_moe_align(const int32_t* topk_idx, int npairs, int E, int32_t* sorted_ids, int cap, int32_t* tile_expert, int max_tiles,
                   int32_t* num_tiles, int tile_rows, void* stream);
/* Prompt-sized bf16 batches: out[r][:] = bf16(weight[pair] * h[pair / top][:]) for row r of the sorted list (pair =
 * sorted_ids[r]; padding rows become zeros; weight NULL: plain copies), for the rows of the *num_tiles used tiles of
 * tile_rows rows.  out [cap][W]. */
int b200_moe_gather_scale(const void* h, int ldh, const int32_t* sorted_ids, int cap, int top, const float* weight,
                          const int32_t* num_tiles, int tile_rows, void* out, int W, void* stream);
/* out = A W_e^T, fp32 accumulation.  Dense (sorted_ids NULL): rows 0..M-1, one weight.  Grouped: row tile i belongs to
 * expert tile_expert[i]; row r of the tile list is pair sorted_ids[r]; its A row is pair / gather_div (gather_div > 0,
 * scaled by row_scale[pair] when given) or r itself; its out row is the pair id (scatter) or r.  glu: w_e = [gate; up] of N
 * rows each and out (dtype) = the gated-linear unit with gate activation `act` (B200_ACT_*; `limit` for the clamped one);
 * else out is fp32.  row_tiles = grid size (tiles beyond *num_tiles exit).  With tile_rows = 4 x b200_moe_tile_rows() the
 * rows of A are the list b200_moe_gather_scale wrote (gather_div 0, no row_scale). */
int b200_grouped_linear(const void* a, int lda, const int32_t* sorted_ids, int gather_div, const float* row_scale, const void* w,
                        int64_t w_expert_stride, const int32_t* tile_expert, const int32_t* num_tiles, int row_tiles, int M, int N,
                        int K, int dtype, void* out, int ldo, int scatter, int glu, int act, float limit, int tile_rows,
                        void* stream);
/* `batch` dense linears in one launch: out_b [M][N] = A_b [M][K] W_b [N][K]^T with A_b = a + b * a_batch_stride (pitch lda),
 * W_b = w + b * w_batch_stride, out_b = out + b * out_batch_stride (pitch ldo); fp32 accumulation.  The result is
 * multiplied by sigmoid(gate[row * gate_ld + b]) when gate != NULL and stored as fp32, or in `dtype` when out_typed. */
int b200_batched_linear(const void* a, int lda, int64_t a_batch_stride, const void* w, int64_t w_batch_stride, void* out, int ldo,
                        int64_t out_batch_stride, int batch, int M, int N, int K, int dtype, int out_typed, const float* gate,
                        int gate_ld, void* stream);

/* ---------------------------------------------------------------- post-norm hybrid decoders (delta rule + latent attention)
 * x = table[token] * scale (+ bigram[row] when a bigram table is given: row = (prev * mul_prev + token * mul_cur) mod buckets,
 * row `buckets` for a sequence's first token; the token before a portion is prev_state[slot], which is then set to the
 * portion's last token).  out fp32 [T][W]; out_cast (or NULL): the same rows in table_dtype. */
int b200_embed_bigram(const int32_t* tokens, const void* table, const void* bigram, int table_dtype, int buckets, int mul_prev,
                      int mul_cur, int32_t* prev_state, const int32_t* tok_seq, const int32_t* seq_start, const int32_t* seq_slot,
                      const int32_t* seq_pos0, float* out, void* out_cast, int T, int W, int V, float scale, void* stream);
/* s = sum_{c < nsum} y_weight[t * nsum + c] * y[t * nsum + c] (y_weight NULL: plain sum);
 * x[t] += s / sqrt(mean(s^2) + eps) * (offset + w);  out_cast[t] = x[t] in out_dtype (when given). */
int b200_rms_residual(float* x, const float* y, int nsum, const float* y_weight, const float* w, float offset, float eps,
                      void* out_cast, int out_dtype, int T, int W, void* stream);
/* out[t][0..n) = v / sqrt(mean(v^2) + eps) * (offset + w), v = columns [col0, col0 + n) of the fp32 rows `in` (pitch ld) */
int b200_rmsnorm_cols(const float* in, int ld, int col0, int n, const float* w, float offset, float eps, void* out, int out_dtype,
                      int ldo, int T, void* stream);
/* o fp32 [T][H][P]: out = o / sqrt(mean_P(o^2) + eps) * w[0..P) * silu(gate), gate = columns gate_col0.. of fp32 rows (pitch ldg);
 * gate NULL: the norm alone */
int b200_head_rmsnorm_gate(const float* o, const float* gate, int ldg, int gate_col0, const float* w, float eps, void* out,
                           int out_dtype, int T, int H, int P, void* stream);
/* Parallel-branch residual step with a grouped RMS norm: x[t] += y1[t] + y2[t] (fp32 rows of pitch ld1 / ld2; y2 or both may be
 * NULL); out[t] (or NULL) = x[t] cut into `groups` equal consecutive parts, each divided by its own sqrt(mean(part^2) + eps), the
 * whole times w.  x fp32 [T][W]. */
int b200_add_group_rmsnorm(float* x, const float* y1, int ld1, const float* y2, int ld2, const float* w, int groups, float eps,
                           void* out, int out_dtype, int T, int W, void* stream);
/* out[t][0..n) = a N(z) + b N(z^2) + c N(z^3) + e with elementwise powers, N(u) = u / sqrt(mean(u^2) + eps) over the n columns,
 * z = columns [col0, col0 + n) of the fp32 rows `in` (pitch ld), coef = {a, b, c, e} fp32 on the device */
int b200_poly_norm(const float* in, int ld, int col0, int n, const float* coef, float eps, void* out, int out_dtype, int ldo, int T,
                   void* stream);
/* Differential attention, closing step: a fp32 [T][2 H][P], the kv group of `rep` output heads storing its first maps in rows
 * [2 rep g, 2 rep g + rep) and its second maps in the next rep rows.  o = a1 - lambda a2;
 * out[t][h] = o / sqrt(mean_P(o^2) + eps) * post * sigmoid(gate[t * ldg + gate_col0 + h]) (gate NULL: no gate). */
int b200_diff_head_norm_gate(const float* a, float lambda, float post, const float* gate, int ldg, int gate_col0, float eps,
                             void* out, int out_dtype, int T, int H, int rep, int P, void* stream);
/* ---------------------------------------------------------------- dual-norm parallel decoders (window + pooled-block attention
 * beside a gated linear recurrence)
 * x[t] = e / sqrt(mean(e^2) + eps) * w, e = table[token]: out fp32 [T][W] */
int b200_embed_rmsnorm(const int32_t* tokens, const void* table, int table_dtype, const float* w, float eps, float* out, int T,
                       int W, int V, void* stream);
/* x[t] += c1 y1[t] + c2 y2[t] + c3 sum_{k < nsum} y3_weight[t][k] y3[t nsum + k] + add_rows[t] + add_vec (fp32; y1 / y2 rows of
 * pitch ld1 / ld2, y3 [T nsum][W], add_rows [T][W], add_vec [W]; every term may be NULL, y3_weight NULL: plain sum), then
 * out1[t] = x[t] / sqrt(mean(x[t]^2) + eps) * w1 and out2[t] = the same times w2, in out_dtype (either may be NULL). */
int b200_scaled_add_rmsnorm2(float* x, const float* y1, int ld1, float c1, const float* y2, int ld2, float c2, const float* y3,
                             int nsum, const float* y3_weight, float c3, const float* add_rows, const float* add_vec,
                             const float* w1, void* out1, const float* w2, void* out2, float eps, int out_dtype, int T, int W,
                             void* stream);
/* Gated linear recurrence, preparation, IN PLACE on the fp32 rows proj (pitch ld): columns [q_col0, q_col0 + n) become silu(z),
 * columns [f_col0, f_col0 + n) become lower + (1 - lower) sigmoid(z + f_bias); f_bias, lower fp32 [n]. */
int b200_gated_scan_prep(float* proj, int ld, int q_col0, int f_col0, int n, const float* f_bias, const float* lower, int T,
                         void* stream);
/* Gated linear recurrence over a ragged batch: per head S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t with q, f [H][D]
 * and v [H][P] the columns q_col0 / f_col0 / v_col0 of the fp32 rows proj.  state fp32 [slots][H][P][D] (transposed), read for
 * sequences with seq_pos0 > 0 and written back for all; out fp32 [T][H * P].  D <= 512, else B200_ERR_UNSUPPORTED.
 * num_segs > 0: the step's portions cut into segments that run in parallel -- segs int32 [num_segs][4] = (first token, end token,
 * sequence, 1 = first of its sequence | 2 = last), seq_seg0 int32 [B + 1] first segment per sequence, scratch seg_state fp32
 * [num_segs][H][P][D] and seg_decay fp32 [num_segs][H][D]: a partial pass from zero states, an elementwise pass that chains
 * the segments with the per-row products of f, and the full pass from every segment's start state. */
int b200_gated_scan(const float* proj, int ld, int q_col0, int f_col0, int v_col0, float* state, const int32_t* seq_start,
                    const int32_t* seq_slot, const int32_t* seq_pos0, float* out, int B, int H, int D, int P, const int32_t* segs,
                    int num_segs, const int32_t* seq_seg0, float* seg_state, float* seg_decay, void* stream);
/* gate_up fp32 [T][2 ff] (gate first): out = act(gate) * up, act = B200_ACT_SILU or B200_ACT_GELU_TANH */
int b200_glu(const float* gate_up, void* out, int out_dtype, int T, int ff, int act, void* stream);
/* Gated delta rule, preparation: qkv fp32 rows [q: G*D | k: G*D | v: H*P] (pitch ldc) are the convolved activations; q and k
 * become unit vectors per key head IN PLACE (x / sqrt(sum x^2 + unit_eps), q also times q_scale); beta_decay fp32 [T][2 H] =
 * [sigmoid(raw_b) | exp(-exp(A_log) softplus(raw_a + dt_bias))] with raw_b / raw_a = columns b_col0 / a_col0 of the fp32
 * rows proj; kq fp32 [T][G] = k . q. */
int b200_delta_prep(float* qkv, int ldc, const float* proj, int ldp, int b_col0, int a_col0, const float* A_log,
                    const float* dt_bias, float* beta_decay, float* kq, int T, int H, int G, int D, float q_scale, float unit_eps,
                    void* stream);
/* Gated delta rule over the prepared rows: per head  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.
 * state fp32 [slots][H][P][D] (read when seq_pos0 > 0, zero otherwise, updated); out fp32 [T][H][P].  Head h reads key
 * head h / (H / G).  D <= 1024.  max_new: the longest portion of the step (picks the thread layout; any value is correct). */
int b200_delta_scan(const float* qkv, int ldc, const float* beta_decay, const float* kq, float* state, const int32_t* seq_start,
                    const int32_t* seq_slot, const int32_t* seq_pos0, float* out, int B, int max_new, int H, int G, int D, int P,
                    void* stream);
/* Latent attention, cache write: columns [col0, col0 + C) of the fp32 rows `in` are RMS-normed (weight norm_w) into
 * pool[slot][0..C); the next R columns are the shared rotated key part: pairs (2i, 2i+1) of its first rot_n columns turn by
 * the token's position with cos / sin from tables [positions][rot_n / 2], the rest is copied.  pool [slots][C + R]. */
int b200_latent_kv_write(const float* in, int ld, int col0, int C, int R, int rot_n, const float* norm_w, float eps,
                         const float* cos_table, const float* sin_table, const int32_t* tok_pos, const int64_t* slot_mapping,
                         void* pool, int kv_dtype, int T, void* stream);
/* Latent attention, query side: q fp32 rows [H][D + R] (pitch ldq).  q_nope [T][H * D] (nope_dtype) = the unrotated parts;
 * q_att fp32 [T][H][C + R]: columns [C, C + R) = the rotated part, turned like the key's. */
int b200_latent_q_prep(const float* q, int ldq, int H, int D, int R, int rot_n, int C, const float* cos_table,
                       const float* sin_table, const int32_t* tok_pos, void* q_nope, int nope_dtype, float* q_att, int T,
                       void* stream);
/* Latent attention for single tokens and short portions, bf16 pools, on the tensor cores: token t (position tok_pos[t], block
 * table row tok_row[t]) attends cache rows 0..pos; q fp32 [T][H][D] (pitch ldq), rows [D] with the values in the first Dv
 * columns; out bf16 [T][H][Dv].  D and Dv multiples of 16, Dv <= 256, else B200_ERR_UNSUPPORTED. */
int b200_latent_attn_decode(const float* q, int ldq, const void* pool, const int32_t* block_table, int64_t bt_stride,
                            const int32_t* tok_row, const int32_t* tok_pos, float scale, void* out, int T, int H, int D, int Dv,
                            int block_size, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_PAGED_H_ */
