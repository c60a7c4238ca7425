/*
 * b200.h — C ABI of libb200.so, the sm_100a kernel library behind the engine.
 *
 * GPUStack has no in-process engine ABI: its engine boundary is process + CLI + HTTP
 * (reference: gpustack/worker/backends/custom.py:141-159, gpustack/worker/serve_manager.py:1000-1048,
 * gpustack/routes/openai.py:92-181).  That boundary is implemented by gpustack_b200/{cli,server}.py.
 * This header is the INTERNAL boundary the north star asks for ("Python over PyTorch tensors
 * calling the kernels through a thin C-ABI extension"): one entry point per operator on the
 * decoder hot path, each citing the operator of the reference's vLLM backend it replaces
 * ($VLLM = site-packages/vllm 0.22.0, the engine gpustack/worker/backends/vllm.py:403-407 launches).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its name ends in _host; the caller owns all memory;
 *   - kernels never allocate and never synchronise; `stream` is a cudaStream_t passed as void*;
 *   - return 0 on success, negative on error (B200_ERR_*), message via b200_last_error();
 *   - bf16 tensors are row-major, innermost dimension contiguous, 16-byte aligned rows.
 */
#ifndef B200_H_
#define B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_ABI_VERSION 1

#define B200_ERR_INVALID (-1)
#define B200_ERR_CUDA (-2)
#define B200_ERR_UNSUPPORTED (-3)

/* ---- runtime ------------------------------------------------------------------------------ */
int b200_abi_version(void);
const char* b200_last_error(void);
/* sm count, compute capability and L2 size of the current device. */
int b200_device_info(int* sm_count, int* cc_major, int* cc_minor, int* l2_bytes);

/* ---- normalisation: $VLLM/model_executor/layers/layernorm.py:104-150,
 *      math $VLLM/ir/ops/layernorm.py:10-58 ------------------------------------------------- */
/* y = bf16(bf16(x * rsqrt(mean(x^2) + eps)) * w); x,y [T,H] bf16, w [H] bf16. */
int b200_rms_norm(const void* x, const void* w, void* y, int T, int H, float eps, void* stream);
/* z = x + residual (fp32); residual_out = bf16(z); y = rmsnorm(z) as above.
 * y may alias x, residual_out may alias residual (the reference op is in-place). */
int b200_fused_add_rms_norm(const void* x, const void* residual, const void* w, void* y,
                            void* residual_out, int T, int H, float eps, void* stream);
/* Same, but x arrives as `splits` fp32 partial sums [splits][T][H] (split-K GEMM output);
 * the partials are summed in fp32 before the residual add.  residual may be NULL (first layer). */
int b200_fused_add_rms_norm_partials(const float* partials, int splits, const void* residual,
                                     const void* w, void* y, void* residual_out, int T, int H,
                                     float eps, void* stream);

/* ---- rotary embedding + KV-cache write:
 *      $VLLM/model_executor/layers/rotary_embedding/base.py:150-215 (neox style) and
 *      $VLLM/_custom_ops.py:2591-2610 (reshape_and_cache_flash) -------------------------------- */
/* qkv [T, (Hq+2*Hkv)*D] bf16: q and k heads are rotated in place; rotated k and v are scattered
 * into k_cache/v_cache laid out [num_blocks][Hkv][block_size][D] at slot_mapping[t]
 * (= block*block_size + offset; negative = skip).  cos_sin [max_pos][D] bf16 = cos | sin halves. */
int b200_rope_kv_write(void* qkv, const int32_t* positions, const void* cos_sin, void* k_cache,
                       void* v_cache, const int32_t* slot_mapping, int T, int Hq, int Hkv, int D,
                       int block_size, void* stream);

/* Same, with the QKV projection arriving as `splits` fp32 split-K partial sums
 * [splits][T][(Hq+2Hkv)*D]: they are summed, the optional QKV bias [(Hq+2Hkv)*D] bf16 (Qwen2) is added
 * in fp32, the result is rounded to bf16 (what the un-split GEMM would have stored), rotated,
 * written to qkv_out (bf16, same layout) and scattered into the cache. */
int b200_rope_kv_write_partials(const float* partials, int splits, const void* qkv_bias, void* qkv_out,
                                const int32_t* positions, const void* cos_sin, void* k_cache,
                                void* v_cache, const int32_t* slot_mapping, int T, int Hq, int Hkv,
                                int D, int block_size, void* stream);

/* ---- activation: $VLLM/model_executor/layers/activation.py:133-143 ----------------------- */
/* out[t, i] = bf16(bf16(silu(x[t, i])) * x[t, I + i]);  x [T, 2I] bf16, out [T, I] bf16. */
int b200_silu_and_mul(const void* x, void* out, int T, int I, void* stream);

/* ---- embedding + greedy sampler:
 *      $VLLM/model_executor/layers/vocab_parallel_embedding.py, $VLLM/v1/sample/sampler.py -- */
/* out[t] = table[ids[t] - vocab_start] if vocab_start <= ids[t] < vocab_end else 0. */
int b200_embedding(const int32_t* ids, const void* table, void* out, int T, int H, int vocab_start,
                   int vocab_end, void* stream);
/* out_idx[b] = lowest index of the row maximum of logits[b, :V] (fp32, row stride ld);
 * out_val[b] (optional) = that maximum. */
int b200_argmax_f32(const float* logits, int64_t ld, int32_t* out_idx, float* out_val, int B, int V,
                    void* stream);
/* Sampler, one pass over the logits: row b is greedy when temps[b] == 0 (or temps is NULL), otherwise an
 * exact softmax(logits / temps[b]) sample by the Gumbel-max trick with the counter-based noise
 * u = hash(seeds[b], vocab_offset + column) -- deterministic per (seed, position), and composable with
 * vocabulary-parallel shards (the cross-rank (max, argmax) exchange of greedy picks the sample).
 * out_val (optional): the winning key of each row. */
int b200_sample_f32(const float* logits, int64_t ld, const float* temps, const uint32_t* seeds,
                    int vocab_offset, int32_t* out_idx, float* out_val, int B, int V, void* stream);
/* gather rows: out[i] = x[rows[i]]; x [*,H] bf16 (used to pick each sequence's last token). */
int b200_gather_rows(const void* x, const int32_t* rows, void* out, int n, int H, void* stream);

/* ---- dense projection (tcgen05/TMEM, TMA-fed):
 *      $VLLM/model_executor/layers/utils.py:92-98 (F.linear of QKV/O/gate_up/down/lm_head) ---- */
/* Y[M,N] = X[M,K] * W[N,K]^T.  X,W bf16 (K contiguous, ldx/ldw in elements), fp32 accumulate.
 *   out_f32 == 0: Y bf16 [M, ldy];  out_f32 == 1: Y fp32 [M, ldy].
 *   splits > 1 : K is cut into `splits` equal ranges and Y must be fp32 [splits][M][ldy]
 *                partial sums (reduced by b200_fused_add_rms_norm_partials / b200_splitk_reduce).
 * K % 64 == 0 required.  M, N arbitrary (tails are zero-filled by TMA and masked on store). */
int b200_gemm_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int64_t ldx,
                   int64_t ldw, int64_t ldy, int out_f32, int splits, void* stream);
/* Same with an explicit activation-tile width block_x in {16,32,64,128,256} (0 = pick from M, see
 * b200_gemm_pick_block_x); used by the tuning sweep in tools/gemm_sweep.py. */
int b200_gemm_bf16_ex(const void* X, const void* W, void* Y, int M, int N, int K, int64_t ldx,
                      int64_t ldw, int64_t ldy, int out_f32, int splits, int block_x, void* stream);
int b200_gemm_pick_block_x(int M, int N, int K);
/* gate_up projection with the SiLU*mul activation ($VLLM activation.py:133-143) fused into the
 * epilogue.  W [N=2I, K] holds gate and up rows INTERLEAVED (row 2i = gate_i, row 2i+1 = up_i);
 * Y [M, ldy >= I] bf16 = bf16(bf16(silu(bf16(g))) * bf16(u)): bit-identical to
 * b200_gemm_bf16 followed by b200_silu_and_mul. */
int b200_gemm_bf16_silu_mul(const void* X, const void* W, void* Y, int M, int N, int K, int64_t ldx,
                            int64_t ldw, int64_t ldy, void* stream);
/* W8A8 fp8 (e4m3) projection -- the linear layers of the fp8 checkpoints GPUStack deploys
 * (BASELINE config "Llama-3-70B fp8"; reference operator: cutlass_scaled_mm behind
 * Fp8LinearMethod.apply, $VLLM/model_executor/layers/quantization/fp8.py:437-470):
 *   Y[m,n] = (sum_k Xq[m,k] * Wq[n,k]) * xscale[m] * wscale[n * wscale_stride]
 * Xq [M,K], Wq [N,K] e4m3 bytes (K-major, K % 128 == 0, N > 128); xscale [M] fp32 dynamic
 * per-token scales (b200_quant_fp8_per_token); wscale fp32, stride 0 = per-tensor, 1 = per output
 * channel.  out_f32/splits as b200_gemm_bf16.  silu_mul != 0: W rows are interleaved gate/up and
 * Y [M, N/2] bf16 gets SiLU*mul of the dequantised, bf16-rounded pair (as b200_gemm_bf16_silu_mul). */
int b200_gemm_fp8(const void* X, const void* W, void* Y, int M, int N, int K, int64_t ldx, int64_t ldw,
                  int64_t ldy, const float* xscale, const float* wscale, int wscale_stride, int out_f32,
                  int splits, int silu_mul, void* stream);
/* Dynamic per-token e4m3 quantisation of bf16 activations (QuantFP8.forward_native,
 * $VLLM/model_executor/layers/quantization/input_quant_fp8.py:188-235):
 *   scales[t] = max(absmax(x[t,:]) / 448, 1/(448*512));  q[t,k] = e4m3(x[t,k] * (1/scales[t])), RNE, saturating. */
int b200_quant_fp8_per_token(const void* x, int64_t ldx, void* q, int64_t ldq, float* scales, int T, int K,
                             void* stream);
/* ---- mixture of experts (Mixtral family): MixtralMoE -> FusedMoE, $VLLM/model_executor/models/
 * mixtral.py, $VLLM/model_executor/layers/fused_moe/ (topk_softmax, moe_align_block_size,
 * fused_experts, moe_sum).  Everything stays on the device; tile counts are read by the grouped
 * GEMM from device memory, so a MoE layer is CUDA-graph capturable. ---- */
/* topk_w[t,:] = (renormalised) top-K of softmax(float(router_logits[t,:E])), router_logits bf16 with row
 * stride ld >= E; topk_ids int32 [T,K]; ties go to the lowest expert index.  E <= 64, K <= 8. */
int b200_moe_route(const void* router_logits, int64_t ld, int32_t* topk_ids, float* topk_w, int T, int E,
                   int K, int renormalize, void* stream);
/* Rows the permuted space can need for n_pairs (token,k) pairs: every expert is padded to whole
 * tiles of block_x rows. */
int b200_moe_capacity_rows(int n_pairs, int E, int block_x);
/* Group the pairs by expert.  pair_row [n_pairs] = row of each pair; row_pair [capacity_rows] = pair of
 * each row (-1 = padding); row_weight [capacity_rows] = routing weight (0 = padding); tile_expert
 * [capacity_rows / block_x] = owner of each tile; num_tiles[0] = tiles in use, [1] = rows in use. */
int b200_moe_align(const int32_t* topk_ids, const float* topk_w, int n_pairs, int E, int block_x,
                   int capacity_rows, int32_t* pair_row, int32_t* row_pair, float* row_weight,
                   int32_t* tile_expert, int32_t* num_tiles, void* stream);
/* xp[row,:] = x[row_pair[row] / K, :] (zeros for padding rows) for the rows in use. */
int b200_moe_gather(const void* x, const int32_t* row_pair, const int32_t* num_tiles, void* xp, int H, int K,
                    int capacity_rows, void* stream);
/* Grouped tcgen05 GEMM over the permuted rows: Y[row,:] = X[row,:] * W[tile_expert[row / block_x]]^T.
 * W [num_experts * N, K] bf16 (experts stacked, N % 256 == 0, K % 64 == 0).  row_scale (optional)
 * multiplies each row's fp32 accumulator (routing weight); silu_mul != 0: W rows are interleaved
 * gate/up and Y is [capacity_rows, N/2] (as b200_gemm_bf16_silu_mul). */
int b200_moe_grouped_gemm(const void* X, const void* W, void* Y, int capacity_rows, int N, int K,
                          int num_experts, int64_t ldx, int64_t ldw, int64_t ldy, const float* row_scale,
                          const int32_t* tile_expert, const int32_t* num_tiles, int block_x, int silu_mul,
                          void* stream);
/* out[t,:] = bf16(sum_j float(yp[pair_row[t*K+j], :]))  (moe_sum). */
int b200_moe_combine(const void* yp, const int32_t* pair_row, void* out, int T, int H, int K, void* stream);
/* Y[m,n] = bf16(sum_s partials[s][m][n]). */
int b200_splitk_reduce(const float* partials, int splits, void* Y, int M, int N, int64_t ldy,
                       void* stream);
/* Heuristic used by the engine: how many K-splits b200_gemm_bf16 should use for this shape. */
int b200_gemm_suggest_splits(int M, int N, int K);

/* ---- paged-KV attention: $VLLM/v1/attention/backends/flashinfer.py:1095-1230 -------------- */
/* Decode: one query token per sequence.  q [B, Hq, D] bf16 with row stride q_stride (elements),
 * out [B, Hq*D] bf16, block_table [B, max_blocks] int32, seq_lens [B] int32 (incl. the new
 * token).  workspace: b200_attn_decode_workspace_bytes() bytes, ZEROED ONCE by the caller before its
 * first use (it starts with the self-resetting arrival counters of the in-kernel split merge; a
 * buffer sized for a larger batch may be reused for smaller ones); num_splits from
 * b200_attn_decode_splits() or caller-chosen (>=1). */
int b200_attn_decode_splits(int B, int Hkv, int max_seq_len, int block_size);
size_t b200_attn_decode_workspace_bytes(int B, int Hq, int D, int num_splits);
int b200_paged_attn_decode(const void* q, int64_t q_stride, const void* k_cache,
                           const void* v_cache, const int32_t* block_table, int max_blocks,
                           const int32_t* seq_lens, void* out, void* workspace, int num_splits,
                           int B, int Hq, int Hkv, int D, int block_size, float scale,
                           void* stream);
/* Prefill / chunked prefill: ragged batch of query chunks.  Sequence s contributes tokens
 * [cu_q[s], cu_q[s+1]) of q; its chunk starts at context position ctx_lens[s] (tokens already in
 * the cache) and attends causally to cache positions [0, ctx_lens[s] + i].  K/V of the chunk must
 * already be in the cache (b200_rope_kv_write runs first).  tile_seq/tile_q0 [num_tiles] list the
 * (sequence, first query offset) of each 32-token query tile, built on the host.  num_tokens = rows
 * of q, num_blocks = pages of the cache tensors (bounds of the TMA tensor maps of the tcgen05 kernel
 * that serves head_dim 128 with GQA groups of 4 or 8; other shapes run the mma.sync kernel). */
/* query-tile size (tokens) the prefill kernel uses for this head grouping: 32 (group <= 4),
 * 16 (group <= 8), 0 = unsupported. */
int b200_attn_prefill_tile(int Hq, int Hkv);
int b200_paged_attn_prefill(const void* q, int64_t q_stride, int num_tokens, const void* k_cache,
                            const void* v_cache, int num_blocks, const int32_t* block_table, int max_blocks,
                            const int32_t* cu_q, const int32_t* ctx_lens, const int32_t* tile_seq,
                            const int32_t* tile_q0, int num_tiles, void* out, int Hq, int Hkv, int D,
                            int block_size, float scale, void* stream);

/* ---- tensor-parallel all-reduce over NVLink peer memory:
 *      $VLLM/distributed/device_communicators/cuda_communicator.py:241-290 (custom all-reduce) */
/* Zero-filled device allocation made directly with cudaMalloc (so that it has its own IPC handle;
 * framework allocators sub-allocate) and its release. */
int b200_dev_malloc(size_t bytes, void** dev_ptr_out);
int b200_dev_free(void* dev_ptr);
int b200_ipc_get_handle(void* dev_ptr, void* handle_out_host /* 64 bytes */);
int b200_ipc_open_handle(const void* handle_host /* 64 bytes */, void** dev_ptr_out);
int b200_ipc_close_handle(void* dev_ptr);
/* uint32 words each rank's flag buffer must hold (zero-initialised once, peer-mapped). */
int b200_allreduce_flag_words(int world);
/* One-shot all-reduce(sum) of bf16 [T,H] fused with residual add + RMSNorm of the reduced rows:
 * peers[r] = rank r's staging buffer (already filled by that rank's row-parallel GEMM);
 * flags[r] = rank r's flag words.  Every rank reduces all rows (redundantly, in rank order, so
 * results are bit-identical across ranks) -- no second exchange.  w == NULL: plain all-reduce
 * into y.  Arrival epochs live on the device (CUDA-graph replays stay valid); `epoch` is unused.
 * The caller alternates between two staging buffers on consecutive calls. */
int b200_allreduce_add_rms_norm(void* const* peers_host, void* const* flags_host, int world,
                                int rank, uint32_t epoch, const void* residual, const void* w,
                                void* y, void* residual_out, int T, int H, float eps, void* stream);

/* Two-shot, sequence-parallel form for large messages (prefill chunks, big decode batches): ONE
 * kernel = barrier, reduce-scatter by token rows over peer loads, residual add + RMSNorm on this
 * rank's rows only, all-gather of the normalised rows by peer stores, barrier.
 * stage_host[r] / xn_host[r] / flags_host[r]: rank r's GEMM-partial staging buffer [T,H] bf16, its
 * gathered-output buffer [T,H] bf16 (every rank's copy is complete when the kernel ends) and its
 * flag buffer (b200_allreduce_twoshot_flag_words() zero-initialised uint32 words), as mapped in the
 * calling process.  The residual stream is sharded by rows between calls: only rows
 * [rank*ceil(T/world), (rank+1)*ceil(T/world)) of residual / residual_out are read / written. */
int b200_allreduce_twoshot_flag_words(void);
/* Greedy sampling over vocabulary-parallel logits: rank r holds, for each of n sequences, the max
 * (val) and LOCAL argmax (idx) of its lm_head shard in peer-mapped arrays; one CTA per rank reads
 * every rank's pair over NVLink and writes the global argmax (idx + r * vocab_per_rank; ties -> the
 * lowest vocabulary index) to out_idx.  flags_host[r]: >= 32 zero-initialised uint32 words. */
int b200_tp_argmax_select(void* const* val_host, void* const* idx_host, void* const* flags_host,
                          int world, int rank, int vocab_per_rank, int32_t* out_idx, int n, void* stream);
int b200_allreduce_rs_norm_ag(void* const* stage_host, void* const* xn_host, void* const* flags_host,
                              int world, int rank, const void* residual, const void* w,
                              void* residual_out, int T, int H, float eps, void* stream);

/* ---- layer-list decoders: norm-after-sum residual stream in fp32, attention with a softmax sink,
 *      matrix-memory recurrence.  `f32` flags select the element type of activations and caches:
 *      0 = bf16, 1 = fp32 (a model served in true 32-bit).  Weights are always bf16. ------------- */
/* y = x W^T (+ bias) on the CUDA cores, fp32 accumulation, no shape or alignment rule. */
int b200_linear_simt(const void* X, int x_f32, const void* W, const void* bias, void* Y, int y_f32, int M,
                     int N, int K, int64_t ldx, int64_t ldw, int64_t ldy, void* stream);
/* z = alpha * x_in[src] + y[r] (z = x_in[src] when y == NULL; src = rows[r] or r), then
 * o = (z - mean) / sqrt(var + eps) * w * out_scale; x_out (fp32) and xb_out (bf16 / fp32) receive o;
 * either may be NULL; x_out may alias x_in when rows == NULL. */
int b200_sum_layer_norm(const void* y, int y_f32, int64_t ldy, const float* x_in, const int32_t* rows,
                        const void* w, float* x_out, void* xb_out, int xb_f32, int T, int D, float alpha,
                        float eps, float out_scale, void* stream);
/* x_out[t] = table[ids[t]] as fp32 (zeros for an id outside [0, V)); xb_out: the same rows as bf16 / fp32. */
int b200_embed_rows_f32(const int32_t* ids, const void* table, float* x_out, void* xb_out, int xb_f32,
                        int T, int D, int V, void* stream);
/* out = max(u, 0)^2 over n elements. */
int b200_relu2(const void* u, void* out, int f32, int64_t n, void* stream);
/* Fused projection row = [q: H*dk | k: G*dk | v: G*dv | ...] (q only when has_kv == 0): adds the bias,
 * RMS-normalises every q and k head (a NULL weight: that side is not normalised), multiplies q by its position's temperature
 * 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) (temp_every <= 0: none), writes q back in place
 * and scatters k / v into the paged caches K [blocks][G][page][dk], V [blocks][G][page][dv]. */
int b200_attn_prep(void* proj, int f32, int64_t ld, const void* bias, const void* qnorm_w,
                   const void* knorm_w, const int32_t* positions, const int32_t* slots, void* k_cache,
                   void* v_cache, int T, int H, int G, int dk, int dv, int page, int has_kv, float eps,
                   float temp_coef, int temp_every, void* stream);
int b200_attn_sink_prefill_tile(void);
/* Causal attention of prompt portions over the paged cache, tiles of tile_rows rows (a multiple of
 * b200_attn_sink_prefill_tile()); sink [H] fp32 or NULL; gate_col >= 0:
 * the output is multiplied by sigmoid(proj[t, gate_col + h*dv + d]).  v_ld: elements between value rows
 * (0 = dv); v_cache == k_cache with v_ld == dk reads the values from the first dv entries of the key rows. */
int b200_attn_sink_prefill(const void* proj, int f32, int64_t ld, int gate_col, const void* k_cache,
                           const void* v_cache, const int32_t* block_table, int max_blocks,
                           const int32_t* cu_q, const int32_t* ctx_lens, const int32_t* tile_seq,
                           const int32_t* tile_q0, int n_tiles, int tile_rows, const float* sink, void* out,
                           int64_t ldo, int H, int G, int dk, int dv, int page, float scale, int64_t v_ld,
                           void* stream);
/* The same for one new row per sequence (row b of proj / out sees keys [0, seq_lens[b])). */
int b200_attn_sink_decode(const void* proj, int f32, int64_t ld, int gate_col, const void* k_cache,
                          const void* v_cache, const int32_t* block_table, int max_blocks,
                          const int32_t* seq_lens, int B, const float* sink, void* out, int64_t ldo, int H,
                          int G, int dk, int dv, int page, float scale, int64_t v_ld, void* stream);
/* The tensor-core kernels of the Llama-class models with the same two options, for mixers whose key and
 * value widths are equal and a tile size (decode: D 64 / 128; prefill: D 128, group of 4 or 8, tiles of
 * b200_attn_prefill_tile rows): sink [Hq] fp32 or NULL joins the softmax denominator, gate (bf16,
 * [rows][gate_stride], columns h*D + d) or NULL multiplies the output by its sigmoid. */
int b200_attn_prefill_tc_covers(int Hq, int Hkv, int D);
int b200_paged_attn_prefill_ex(const void* q, int64_t q_stride, int num_tokens, const void* k_cache,
                               const void* v_cache, int num_blocks, const int32_t* block_table,
                               int max_blocks, const int32_t* cu_q, const int32_t* ctx_lens,
                               const int32_t* tile_seq, const int32_t* tile_q0, int num_tiles, void* out,
                               int Hq, int Hkv, int D, int block_size, float scale, const float* sink,
                               const void* gate, int64_t gate_stride, void* stream);
int b200_paged_attn_decode_ex(const void* q, int64_t q_stride, const void* k_cache,
                              const void* v_cache, const int32_t* block_table,
                              int max_blocks, const int32_t* seq_lens, void* out,
                              void* workspace, int num_splits, int B, int Hq, int Hkv,
                              int D, int block_size, float scale, const float* sink,
                              const void* gate, int64_t gate_stride, void* stream);
/* y = max(x W^T, 0)^2 in the tcgen05 GEMM's epilogue (bf16 in and out; same shape rules as b200_gemm_bf16). */
int b200_gemm_bf16_relu2(const void* X, const void* W, void* Y, int M, int N, int K, int64_t ldx,
                         int64_t ldw, int64_t ldy, void* stream);
/* Column slices Z of a head's state (n and m are kept once per slice). */
int b200_mlstm_state_slices(int dv);
/* Stabilised matrix-memory recurrence over each sequence's new rows [cu_seq[s], cu_seq[s+1]); gates
 * [T][2H] fp32 raw (input | forget) projections, gate_bias [2H] bf16; state of slot state_slots[s]
 * (S [slots][H][dv][dk], n [slots][H][Z][dk], m [slots][H][Z], fp32) is read unless ctx_lens[s] == 0
 * and written back; o_raw [T][H*dv] fp32.  Negative slot: the sequence is skipped.  max_len: an upper bound of
 * the sequences' new rows (>= 4 selects the chunk form for prompt portions, else the serial form). */
int b200_mlstm_scan(const void* proj, int f32, int64_t ld, int q_col, int k_col, int v_col,
                    const float* gates, const void* gate_bias, const int32_t* cu_seq,
                    const int32_t* ctx_lens, const int32_t* state_slots, float* S_state, float* n_state,
                    float* m_state, float* o_raw, int n_seq, int H, int dk, int dv, float cap, float qscale,
                    int max_len, void* stream);
/* out = o_raw / rms_head(o_raw) * norm_w * sigmoid(gate). */
int b200_mlstm_out(const float* o_raw, const void* proj, int f32, int64_t ld, int gate_col,
                   const void* norm_w, void* out, int64_t ldo, int T, int H, int dv, float eps,
                   void* stream);

/* ---- latent attention, residual streams, gated / routed feed-forward (layer-list decoders) ------------- */
/* X [T][S][D] fp32 streams.  y != NULL: X_t <- sum_s mix[s][t] X_s + mult * out[t] * y  (hc_write = [in: S | out: S |
 * mix: S*S, (from, to)]).  Then u = sum_t hc_read[t] X_t (hc_read NULL: the plain sum) and, when xb_out != NULL,
 * xb_out[r] = tanh(alpha[0] * u) * w + b.  rows != NULL (only without y): row r reads X[rows[r]]. */
int b200_streams_step(const void* y, int y_f32, int64_t ldy, float* X, const int32_t* rows, const float* hc_write,
                      float mult, const float* hc_read, const float* alpha, const void* w, const void* b,
                      void* xb_out, int xb_f32, int T, int S, int D, void* stream);
/* X[t][s] = table[ids[t]] * scale for every stream s. */
int b200_embed_streams(const int32_t* ids, const void* table, float* X, int T, int S, int D, int V, float scale,
                       void* stream);
/* out[t, :n] = x[t, :n] / sqrt(mean(x^2) + eps) * w, rows ldx / ldo apart. */
int b200_rms_rows(const void* x, int f32, int64_t ldx, const void* w, void* out, int64_t ldo, int T, int n, float eps,
                  void* stream);
/* Per token: RMS norm of the latent proj[t, kv_col : kv_col + R] into cache row slots[t] ([.., R + dr]), the
 * rotated key part proj[t, kv_col + R : + dr] behind it, and every head's rotated query part q[t, h, dn : dn + dr]
 * into qa[t, h, R : R + dr].  Rotation of the first `dims` entries at positions[t] with freq[dims / 2] (fp64),
 * pairs (2i, 2i+1) or, half_layout, (i, i + dims/2); cos and sin times mag. */
int b200_latent_prep(const void* proj, int f32, int64_t ld, int kv_col, const void* q, int64_t ldq,
                     const void* kv_norm_w, const int32_t* positions, const int32_t* slots, void* cache, void* qa,
                     int64_t ldqa, int T, int H, int dn, int dr, int R, int dims, int half_layout, const double* freq,
                     float mag, float eps, void* stream);
/* Latent attention on the tensor cores (bf16; csrc/latent_attention_mma.cu): qa [rows][H][R + dr] absorbed queries,
 * cache [blocks][page][R + dr], out [rows][H][R]; sink [H] fp32 or NULL.  covers(): W = R + dr a multiple of 16 and
 * R in {64, 128, 192, 256, 384, 512}.  prefill: tile list as b200_attn_sink_prefill; decode: one row per sequence. */
int b200_latent_attn_covers(int H, int R, int dr);
int b200_latent_attn_prefill(const void* qa, int64_t ldq, const void* cache, int page, const int32_t* block_table,
                             int max_blocks, const int32_t* cu_q, const int32_t* ctx_lens, const int32_t* tile_seq,
                             const int32_t* tile_q0, int n_tiles, int tile_rows, const float* sink, void* out,
                             int64_t ldo, int H, int R, int dr, float scale, void* stream);
/* decode: nsplit > 1 cuts every row's keys into that many ranges (more CTAs for small batches of long sequences) and
 * merges them in a second launch; workspace of b200_latent_attn_decode_workspace_bytes(), contents irrelevant. */
int b200_latent_attn_decode_splits(int B, int H, int max_len);
size_t b200_latent_attn_decode_workspace_bytes(int B, int H, int R, int nsplit);
int b200_latent_attn_decode(const void* qa, int64_t ldq, const void* cache, int page, const int32_t* block_table,
                            int max_blocks, const int32_t* seq_lens, int B, const float* sink, void* out, int64_t ldo,
                            int H, int R, int dr, float scale, int nsplit, void* workspace, void* stream);
/* Batched / grouped / gated linear on the CUDA cores (see gemm_simt_grouped.cu).  act: 0 plain, 1 gelu_tanh(g) u,
 * 2 clamped g sigmoid(1.702 g) (u + 1) with `limit`, 3 silu(g) u; act != 0: W rows interleaved gate / up, N pairs. */
int b200_linear_simt_grouped(const void* X, int x_f32, const void* W, void* Y, int y_f32, int M, int N, int K,
                             int64_t ldx, int64_t ldw, int64_t ldy, int batch, int64_t bsx, int64_t bsw, int64_t bsy,
                             const int32_t* row_pair, int top_k, const int32_t* tile_expert, const int32_t* num_tiles,
                             int n_real, int64_t w_expert, const float* row_scale, int act, float limit, void* stream);
int b200_simt_group_rows(void);
/* H GEMMs over strided views: Y[:, h*y_head : +N] = X[:, h*x_head : +K] W_h^T, W_h the h-th contiguous [N, K] matrix. */
int b200_gemm_bf16_heads(const void* X, const void* W, void* Y, int M, int N, int K, int64_t ldx, int64_t ldy, int H,
                         int64_t x_head, int64_t y_head, int out_f32, void* stream);
/* The tcgen05 GEMM with a gated epilogue over interleaved gate / up rows (bf16 Y [M, N/2], K % 64 == 0):
 * act 0 silu(g) u (factors rounded to bf16), 1 gelu_tanh(g) u, 2 clamped g sigmoid(1.702 g) (u + 1). */
int b200_gemm_bf16_gated(const void* X, const void* W, void* Y, int M, int N, int K, int64_t ldx, int64_t ldw,
                         int64_t ldy, int act, float limit, void* stream);
/* b200_moe_grouped_gemm with those activations (gated != 0) or an fp32 output (out_f32 != 0, with row_scale). */
int b200_moe_grouped_gemm_ex(const void* X, const void* W, void* Y, int capacity_rows, int N, int K, int num_experts,
                             int64_t ldx, int64_t ldw, int64_t ldy, const float* row_scale, const int32_t* tile_expert,
                             const int32_t* num_tiles, int block_x, int gated, int act, float limit, int out_f32,
                             void* stream);
/* Softmax over E fp32 router outputs, top K of score + correction, weights score / (sum + 1e-20) * scale. */
int b200_moe_route_biased(const float* logits, int64_t ld, const float* correction, int32_t* topk_ids, float* topk_w,
                          int T, int E, int K, float scale, void* stream);
/* out[t] = sum_j (topk_ids[t, j] < n_real ? yp[pair_row[t K + j]] : topk_w[t, j] * x[t]) (+ shared[t]); fp32 out. */
int b200_moe_combine_mixed(const void* yp, int p_f32, int64_t ldp, const int32_t* pair_row, const int32_t* topk_ids,
                           const float* topk_w, const void* x, int x_f32, int64_t ldx, const void* shared, int64_t lds,
                           float* out, int64_t ldo, int T, int D, int K, int n_real, void* stream);

/* ---- pre-norm fp32 residual, per-head preparation with rotation, decayed linear attention ---------------------- */
/* z = x_in + a + b + c (a, b, c optional fp32 rows); x_out = z; xb_out = z / sqrt(mean(z^2) + eps) * w (bf16 or fp32).
 * rows != NULL: gather (row r reads source row rows[r]; x_out must be NULL).  w == NULL: the sum only. */
int b200_add_rms_norm_f32(const float* x_in, const float* a, const float* b, const float* c, const int32_t* rows,
                          const void* w, float* x_out, void* xb_out, int xb_f32, int T, int D, float eps, void* stream);
/* Per (token, head): feature map (0 none, 1 silu), rotation of the first `dims` entries (pairs (2i, 2i+1) or,
 * half_layout, (i, i + dims/2); angle position * freq[i], fp64 freq), unit RMS norm (no weight), factors q_mul / k_mul.
 * Queries to q_out rows; keys / values to cache pages at slots[t] (paged) or to row buffers; v_col < 0: the values
 * are the keys as projected (written to v_out when it is not NULL).  src bf16 | fp32, dst the same or fp32. */
int b200_rot_prep(const void* proj, int src_f32, int64_t ld, int q_col, int k_col, int v_col, const int32_t* positions,
                  const int32_t* slots, void* q_out, int64_t ldq, void* k_out, int64_t ldk, void* v_out, int64_t ldv,
                  int dst_f32, int paged, int page, int T, int H, int G, int dk, int dv, int feature, int dims,
                  int half_layout, const double* freq, int unit_norm, float eps, float q_mul, float k_mul, void* stream);
/* S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t over every sequence's new rows [cu_seq[s], cu_seq[s+1]) of the fp32
 * rows x (q / k / v at their columns); state S [slots][H][dv][dk] fp32 in and out, zero start when ctx_lens[s] == 0;
 * o_raw [T][H*dv] fp32.  max_len: an upper bound of the new rows per sequence (> 2: the chunk form). */
int b200_linattn_scan(const float* x, int64_t ld, int q_col, int k_col, int v_col, const float* decay,
                      const int32_t* cu_seq, const int32_t* ctx_lens, const int32_t* state_slots, float* S, float* o_raw,
                      int n_seqs, int H, int dk, int dv, int max_len, void* stream);
/* out = o_raw / rms * (w) * act(gate): all_heads: one RMS over the H*dv entries and w [H*dv]; else per head, w [dv] or
 * NULL.  gate = proj[t, gate_col : gate_col + H*dv]; gate_act 0 sigmoid, 1 silu. */
int b200_linattn_out(const float* o_raw, const void* proj, int f32, int64_t ld, int gate_col, const void* w, void* out,
                     int64_t ldo, int T, int H, int dv, int all_heads, int gate_act, float eps, void* stream);
/* The generic attention kernels with a sliding window (position i sees j with 0 <= i - j < window; 0 = none). */
int b200_attn_sink_prefill_ex(const void* proj, int f32, int64_t ld, int gate_col, const void* k_cache,
                              const void* v_cache, const int32_t* block_table, int max_blocks, const int32_t* cu_q,
                              const int32_t* ctx_lens, const int32_t* tile_seq, const int32_t* tile_q0, int n_tiles,
                              int tile_rows, const float* sink, void* out, int64_t ldo, int H, int G, int dk, int dv,
                              int page, float scale, int64_t v_ld, int window, void* stream);
int b200_attn_sink_decode_ex(const void* proj, int f32, int64_t ld, int gate_col, const void* k_cache, const void* v_cache,
                             const int32_t* block_table, int max_blocks, const int32_t* seq_lens, int B, const float* sink,
                             void* out, int64_t ldo, int H, int G, int dk, int dv, int page, float scale, int64_t v_ld,
                             int window, void* stream);
/* The tensor-core attention kernels (tcgen05 prefill, split-KV decode) with a sliding window (0 = none). */
int b200_paged_attn_prefill_win(const void* q, int64_t q_stride, int num_tokens, const void* k_cache, const void* v_cache,
                                int num_blocks, const int32_t* block_table, int max_blocks, const int32_t* cu_q,
                                const int32_t* ctx_lens, const int32_t* tile_seq, const int32_t* tile_q0, int num_tiles,
                                void* out, int Hq, int Hkv, int D, int block_size, float scale, const float* sink,
                                const void* gate, int64_t gate_stride, int window, void* stream);
int b200_paged_attn_decode_win(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                               const int32_t* block_table, int max_blocks, const int32_t* seq_lens, void* out,
                               void* workspace, int num_splits, int B, int Hq, int Hkv, int D, int block_size, float scale,
                               const float* sink, const void* gate, int64_t gate_stride, int window, void* stream);
/* b200_moe_route_biased with sigmoid scores (sigmoid_scores != 0) and / or weights that are not renormalised. */
int b200_moe_route_scored(const float* logits, int64_t ld, const float* correction, int32_t* topk_ids, float* topk_w, int T,
                          int E, int K, float scale, int sigmoid_scores, int renormalize, void* stream);
/* b200_linear_simt_grouped whose row_scale multiplies the rows' input (before the activation) when scale_in != 0. */
int b200_linear_simt_grouped_ex(const void* X, int x_f32, const void* W, void* Y, int y_f32, int M, int N, int K,
                                int64_t ldx, int64_t ldw, int64_t ldy, int batch, int64_t bsx, int64_t bsw, int64_t bsy,
                                const int32_t* row_pair, int top_k, const int32_t* tile_expert, const int32_t* num_tiles,
                                int n_real, int64_t w_expert, const float* row_scale, int act, float limit, int scale_in,
                                void* stream);
/* b200_moe_gather whose gathered rows are multiplied by row_scale[row] (fp32 product, one rounding). */
int b200_moe_gather_scaled(const void* x, const int32_t* row_pair, const int32_t* num_tiles, void* xp, int H, int K,
                           int capacity_rows, const float* row_scale, void* stream);

/* ---- residual stream with a norm before and after every sublayer; short causal convolutions; pooled KV blocks ---- */
/* x[t] = table[ids[t]] + pos_table[positions[t]] (fp32). */
int b200_embed_pos_f32(const int32_t* ids, const int32_t* positions, const void* table, const void* pos_table, float* x,
                       int T, int D, int vocab, int max_pos, void* stream);
/* v = ya*y (+ yb*y2); z = x_in + mult * v / rms(v) * wb (y == NULL: z = x_in); x_out = z; h_out = z / rms(z) * wa.
 * zero_centred: the stored weights enter as 1 + w.  rows: gather (h_out only). */
int b200_sandwich_join(const float* x_in, const float* y, const float* y2, float ya, float yb, const void* wb, float mult,
                       const int32_t* rows, const void* wa, float* x_out, void* h_out, int h_f32, int T, int D, float eps,
                       int zero_centred, void* stream);
/* out_t = (in_t if add_input) + bias + sum_j w[c][j] in_(t - taps + 1 + j) over every sequence's new rows; older inputs
 * come from ring [slots][taps - 1][C] (entry = position mod (taps - 1)); in_bias is added to every input. */
int b200_causal_conv(const void* in, int in_f32, int64_t ld_in, const float* in_bias, const float* w, const float* bias,
                     int add_input, const float* ring, const int32_t* cu_seq, const int32_t* ctx_lens,
                     const int32_t* state_slots, int n_seqs, void* out, int out_f32, int64_t ld_out, int T, int C, int taps,
                     void* stream);
/* The last taps - 1 inputs of every sequence's new rows go to its ring (run after b200_causal_conv). */
int b200_conv_commit(const void* in, int in_f32, int64_t ld_in, const float* in_bias, float* ring, const int32_t* cu_seq,
                     const int32_t* ctx_lens, const int32_t* state_slots, int n_seqs, int C, int taps, void* stream);
/* Mean key / value (fp32) of every block of `pool` tokens that this step completes.  cu_q == NULL: one new row per
 * sequence and ctx_lens counts it. */
int b200_kv_pool_update(const void* k_cache, const void* v_cache, int f32, float* pool_k, float* pool_v,
                        const int32_t* block_table, int max_blocks, const int32_t* cu_q, const int32_t* ctx_lens, int n_seqs,
                        int max_new, int G, int dk, int dv, int page, int pool, int per_page, void* stream);
/* b200_attn_sink_prefill_ex / _decode_ex with a gate of one number per head, a score factor per head and pooled blocks. */
int b200_attn_sink_prefill_pool(const void* proj, int f32, int64_t ld, int gate_col, const void* k_cache, const void* v_cache,
                                const int32_t* block_table, int max_blocks, const int32_t* cu_q, const int32_t* ctx_lens,
                                const int32_t* tile_seq, const int32_t* tile_q0, int n_tiles, int tile_rows, const float* sink,
                                void* out, int64_t ldo, int H, int G, int dk, int dv, int page, float scale, int64_t v_ld,
                                int window, int gate_per_head, const float* head_scale, const float* pool_k,
                                const float* pool_v, int pool, int per_page, void* stream);
int b200_attn_sink_decode_pool(const void* proj, int f32, int64_t ld, int gate_col, const void* k_cache, const void* v_cache,
                               const int32_t* block_table, int max_blocks, const int32_t* seq_lens, int B, const float* sink,
                               void* out, int64_t ldo, int H, int G, int dk, int dv, int page, float scale, int64_t v_ld,
                               int window, int gate_per_head, const float* head_scale, const float* pool_k,
                               const float* pool_v, int pool, int per_page, void* stream);
/* The tensor-core attention kernels with an output gate of ONE number per head (gate[token][head]) when
 * gate_per_head != 0; otherwise as b200_paged_attn_prefill_win / _decode_win. */
int b200_paged_attn_prefill_hg(const void* q, int64_t q_stride, int num_tokens, const void* k_cache, const void* v_cache,
                               int num_blocks, const int32_t* block_table, int max_blocks, const int32_t* cu_q,
                               const int32_t* ctx_lens, const int32_t* tile_seq, const int32_t* tile_q0, int num_tiles,
                               void* out, int Hq, int Hkv, int D, int block_size, float scale, const float* sink,
                               const void* gate, int64_t gate_stride, int window, int gate_per_head, void* stream);
/* ... and lse_out [T][Hq] (fp32, may be NULL): every row's log-sum-exp, for a caller that continues the softmax over
 * more keys (b200_attn_sink_prefill_more). */
int b200_paged_attn_prefill_lse(const void* q, int64_t q_stride, int num_tokens, const void* k_cache, const void* v_cache,
                                int num_blocks, const int32_t* block_table, int max_blocks, const int32_t* cu_q,
                                const int32_t* ctx_lens, const int32_t* tile_seq, const int32_t* tile_q0, int num_tiles,
                                void* out, int Hq, int Hkv, int D, int block_size, float scale, const float* sink,
                                const void* gate, int64_t gate_stride, int window, int gate_per_head, float* lse_out,
                                void* stream);
int b200_paged_attn_decode_hg(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                              const int32_t* block_table, int max_blocks, const int32_t* seq_lens, void* out,
                              void* workspace, int num_splits, int B, int Hq, int Hkv, int D, int block_size, float scale,
                              const float* sink, const void* gate, int64_t gate_stride, int window, int gate_per_head,
                              void* stream);
/* ... and lse_out [B][Hq] (fp32, may be NULL): every row's log-sum-exp over the keys it attended, for a caller that
 * continues the softmax over more keys (b200_attn_sink_decode_more). */
int b200_paged_attn_decode_lse(const void* q, int64_t q_stride, const void* k_cache, const void* v_cache,
                               const int32_t* block_table, int max_blocks, const int32_t* seq_lens, void* out,
                               void* workspace, int num_splits, int B, int Hq, int Hkv, int D, int block_size, float scale,
                               const float* sink, const void* gate, int64_t gate_stride, int window, int gate_per_head,
                               float* lse_out, void* stream);
/* b200_attn_sink_decode_pool that CONTINUES a softmax over the pooled blocks alone: `out` holds the normalised attention
 * over the window's tokens (another kernel's) and init_lse [B][H] its log-sum-exp; `out` is rewritten. */
int b200_attn_sink_decode_more(const void* proj, int f32, int64_t ld, const int32_t* block_table, int max_blocks,
                               const int32_t* seq_lens, int B, void* out, int64_t ldo, int H, int G, int dk, int dv, int page,
                               float scale, int window, const float* head_scale, const float* pool_k, const float* pool_v,
                               int pool, int per_page, const float* init_lse, void* stream);
/* b200_attn_sink_prefill_pool that CONTINUES a softmax: the window's tokens have been attended by another kernel, which
 * left its normalised output in `out` and every row's log-sum-exp in init_lse [T][H]; only the pooled blocks are read
 * here and `out` is rewritten with the joint result. */
int b200_attn_sink_prefill_more(const void* proj, int f32, int64_t ld, const void* k_cache, const int32_t* block_table,
                                int max_blocks, const int32_t* cu_q, const int32_t* ctx_lens, const int32_t* tile_seq,
                                const int32_t* tile_q0, int n_tiles, int tile_rows, void* out, int64_t ldo, int H, int G, int dk,
                                int dv, int page, float scale, int window, const float* head_scale, const float* pool_k,
                                const float* pool_v, int pool, int per_page, const float* init_lse, void* stream);
/* b200_rot_prep with one more factor per query head (q_head_mul [H] fp32, may be NULL). */
int b200_rot_prep_hm(const void* proj, int src_f32, int64_t ld, int q_col, int k_col, int v_col, const int32_t* positions,
                     const int32_t* slots, void* q_out, int64_t ldq, void* k_out, int64_t ldk, void* v_out, int64_t ldv,
                     int dst_f32, int paged, int page, int T, int H, int G, int dk, int dv, int feature, int dims,
                     int half_layout, const double* freq, int unit_norm, float eps, float q_mul, float k_mul,
                     const float* q_head_mul, void* stream);
/* Gated diagonal recurrence over every sequence's new rows: u [T][W], gates [T][2W] (recurrence | input gate
 * pre-activations), S [slots][W]; out = S_t * gelu_tanh(proj[t][y_col + c] + y_bias[c]). */
int b200_gated_recurrence_scan(const float* u, const float* gates, const float* gate_bias, const float* lam, const void* proj,
                               int f32, int64_t ld, int y_col, const float* y_bias, const int32_t* cu_seq,
                               const int32_t* ctx_lens, const int32_t* state_slots, float* S, void* out, int64_t ldo,
                               int n_seqs, int W, float gate_c, void* stream);
/* The same for prompt portions, in chunks of b200_gated_recurrence_chunk_rows() rows that run side by side
 * (workspace: 2 * (T / chunk + n_seqs + 1) * W floats; max_len: the longest portion). */
int b200_gated_recurrence_chunk_rows(void);
int b200_gated_recurrence_scan_chunked(const float* u, const float* gates, const float* gate_bias, const float* lam,
                                       const void* proj, int f32, int64_t ld, int y_col, const float* y_bias,
                                       const int32_t* cu_seq, const int32_t* ctx_lens, const int32_t* state_slots, float* S,
                                       void* out, int64_t ldo, int n_seqs, int W, float gate_c, int T, int max_len,
                                       float* workspace, int64_t workspace_floats, void* stream);
/* Linear attention with a decay per key channel and token, alpha = sigmoid(z)^inv_tau: S [slots][H][dv][dk]. */
int b200_gla_scan(const float* x, int64_t ld, int q_col, int k_col, int v_col, const float* z, int64_t ldz, float inv_tau,
                  const int32_t* cu_seq, const int32_t* ctx_lens, const int32_t* state_slots, float* S, float* o_raw,
                  int n_seqs, int H, int dk, int dv, void* stream);
/* ... with max_len, an upper bound of the new rows per sequence (0: unknown): single rows take the kernel that reads and
 * writes the state in whole lines. */
int b200_gla_scan_rows(const float* x, int64_t ld, int q_col, int k_col, int v_col, const float* z, int64_t ldz, float inv_tau,
                  const int32_t* cu_seq, const int32_t* ctx_lens, const int32_t* state_slots, float* S, float* o_raw,
                  int n_seqs, int H, int dk, int dv, int max_len, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_H_ */
