// Softmax attention over the paged KV cache for mixers whose key and value widths differ and are
// not a tensor-core tile size, with the options such mixers combine:
//   * per-head RMS norm of queries and keys (one weight vector of the head width, shared by heads),
//   * no rotation; instead a query temperature  1 + c * ln(floor((p + 1) / n) + 1)  at position p,
//   * a learned per-head SINK: exp(sink_h) is added to the softmax denominator (a virtual key whose
//     score is sink_h, unscaled, and whose value is zero),
//   * a sigmoid output gate read from the same fused projection as the queries,
//   * keys / values that belong to an earlier layer's cache (the caller passes that cache),
//   * a sliding window (position i sees j with 0 <= i - j < window; 0 = every earlier key): key blocks that lie
//     wholly before the window are never read.
//   * pooled blocks beside a window: one (mean key, mean value) per block of `pool` tokens that lies wholly before
//     the window -- block b is seen by position i when (b + 1) pool - 1 <= i - window -- in the same softmax as the
//     window's tokens; the means are fp32 entries of a second cache addressed through the same block table
//     (sandwich.cu: kv_pool_update),
//   * an output gate with ONE number per head, and a learned factor per head on the score.
// Three kernels: `attn_prep` (bias + norms + temperature, in place for q, scatter of k and v into
// the pages), `prefill` (a tile of 16 query rows of one sequence per CTA, keys staged in shared
// memory 32 at a time, online softmax) and `decode` (one query row per CTA, the four warps take
// 32-key blocks in turn and merge).  Scores, softmax statistics and the accumulator are fp32; the element
// type TA of the projection, the cache and the output is bf16, or fp32 for a model served in 32-bit.
// Cache layout: K [blocks][G][page][dk], V [blocks][G][page][dv]; v_ld (value row pitch) lets the values be a
// slice of another array with wider rows -- the first dv entries of the key rows when v_cache == k_cache and
// v_ld == dk, which is how a latent cache (one shared row per token, G = 1) is read.
#include "common.cuh"
#include "runtime.h"
#include "../../include/b200.h"

#include <math_constants.h>

namespace b200 {

__device__ __forceinline__ float as_f32(float v) { return v; }
__device__ __forceinline__ float as_f32(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void as_store(float* p, float v) { *p = v; }
__device__ __forceinline__ void as_store(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

constexpr int kMaxDvLanes = 16;    // value width <= 512: kernels are built for 8 (<= 256) and 16 columns per lane

// ----------------------------------------------------------------------------------------- prep
// One warp per (token, head slot): slots [0, H) are query heads, [H, H + G) key heads, [H + G, H + 2G) value
// heads (a layer that reuses another layer's keys and values has query slots only).  8 warps per CTA.  Each
// lane keeps its elements (two neighbours per step) in registers between the sum of squares and the
// store, so the row is read once.  Widths up to 512.
constexpr int kPrepWarps = 8, kPrepPairs = 8;

__device__ __forceinline__ float2 ld_pair(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 ld_pair(const bf16* p) {
  return __bfloat1622float2(*reinterpret_cast<const bf162*>(p));
}
__device__ __forceinline__ void st_pair(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void st_pair(bf16* p, float a, float b) {
  *reinterpret_cast<bf162*>(p) = __floats2bfloat162_rn(a, b);
}

// PAIR: every width, column offset and leading dimension is even (2-element loads and stores)
template <typename TA, bool PAIR>
__global__ void __launch_bounds__(kPrepWarps * 32)
attn_prep_kernel(TA* proj, int64_t ld, const bf16* __restrict__ bias, const bf16* __restrict__ qnorm_w,
                 const bf16* __restrict__ knorm_w, const int32_t* __restrict__ positions,
                 const int32_t* __restrict__ slots, TA* k_cache, TA* v_cache, int H, int G, int dk, int dv, int page,
                 int n_slots, float eps, float temp_coef, int temp_every) {
  const int t = blockIdx.x, hs = blockIdx.y * kPrepWarps + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (hs >= n_slots) return;
  TA* row = proj + (size_t)t * ld;
  const bool is_q = hs < H, is_k = !is_q && hs < H + G;
  const int width = (is_q || is_k) ? dk : dv;
  const int col0 = (is_q || is_k) ? hs * dk : (H + G) * dk + (hs - H - G) * dv;
  TA* dst = row + col0;
  if (!is_q) {
    const int slot = slots[t];
    if (slot < 0) return;
    const int g = is_k ? hs - H : hs - H - G;
    dst = (is_k ? k_cache : v_cache) + (((size_t)(slot / page) * G + g) * page + (slot % page)) * width;
  }
  constexpr int STEP = PAIR ? 64 : 32;
  float x0[kPrepPairs], x1[kPrepPairs];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kPrepPairs; ++i) {
    const int d = (PAIR ? 2 * lane : lane) + STEP * i;
    x0[i] = x1[i] = 0.f;
    if (d < width) {
      if (PAIR) {
        const float2 v = ld_pair(row + col0 + d);
        x0[i] = v.x;
        x1[i] = v.y;
        if (bias != nullptr) {
          x0[i] += __bfloat162float(bias[col0 + d]);
          x1[i] += __bfloat162float(bias[col0 + d + 1]);
        }
      } else {
        x0[i] = as_f32(row[col0 + d]);
        if (bias != nullptr) x0[i] += __bfloat162float(bias[col0 + d]);
      }
      ss = fmaf(x0[i], x0[i], fmaf(x1[i], x1[i], ss));
    }
  }
  const bf16* w = is_q ? qnorm_w : (is_k ? knorm_w : nullptr);
  float mul = 1.0f;
  if (is_q || is_k) {
    ss = warp_sum(ss);
    if (w != nullptr) mul = 1.0f / sqrtf(ss / (float)dk + eps);            // no weight = no head norm
    if (is_q && temp_every > 0) {
      const int steps = (positions[t] + 1) / temp_every;
      mul *= 1.0f + temp_coef * logf((float)steps + 1.0f);
    }
  }
#pragma unroll
  for (int i = 0; i < kPrepPairs; ++i) {
    const int d = (PAIR ? 2 * lane : lane) + STEP * i;
    if (d < width) {
      const float w0 = w != nullptr ? __bfloat162float(w[d]) : 1.0f;
      if (PAIR) {
        const float w1 = w != nullptr ? __bfloat162float(w[d + 1]) : 1.0f;
        st_pair(dst + d, x0[i] * mul * w0, x1[i] * mul * w1);
      } else {
        as_store(dst + d, x0[i] * mul * w0);
      }
    }
  }
}

// The same step with 16-byte loads and stores, for widths that are multiples of 16 bytes (every real head
// size): LPH lanes share a head (LPH = a power of two >= width / VEC), a warp covers 32 / LPH head slots of one
// token, each lane moves one 16-byte piece of the row, of the bias and of the norm weight.
template <typename TA>
__global__ void __launch_bounds__(kPrepWarps * 32)
attn_prep_vec_kernel(TA* proj, int64_t ld, const bf16* __restrict__ bias, const bf16* __restrict__ qnorm_w,
                     const bf16* __restrict__ knorm_w, const int32_t* __restrict__ positions,
                     const int32_t* __restrict__ slots, TA* k_cache, TA* v_cache, int H, int G, int dk, int dv, int page,
                     int n_slots, int lph, float eps, float temp_coef, int temp_every) {
  constexpr int VEC = 16 / (int)sizeof(TA);
  const int t = blockIdx.x, lane = threadIdx.x & 31, per_warp = 32 / lph;
  const int hs = (blockIdx.y * kPrepWarps + (threadIdx.x >> 5)) * per_warp + lane / lph;
  const int li = lane % lph;
  const bool live = hs < n_slots;
  const bool is_q = live && hs < H, is_k = live && !is_q && hs < H + G;
  const int width = (is_q || is_k) ? dk : dv;
  const int col0 = !live ? 0 : ((is_q || is_k) ? hs * dk : (H + G) * dk + (hs - H - G) * dv);
  const int d = li * VEC;
  const bool act = live && d < width;
  TA* row = proj + (size_t)t * ld;
  float x[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) x[i] = 0.f;
  if (act) {
    const uint4 raw = *reinterpret_cast<const uint4*>(row + col0 + d);
    const TA* rv = reinterpret_cast<const TA*>(&raw);
#pragma unroll
    for (int i = 0; i < VEC; ++i) x[i] = as_f32(rv[i]);
    if (bias != nullptr) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) x[i] += __bfloat162float(bias[col0 + d + i]);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) ss = fmaf(x[i], x[i], ss);
  for (int o = lph >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);   // all lanes take part
  if (!act) return;
  const bf16* w = is_q ? qnorm_w : (is_k ? knorm_w : nullptr);
  float mul = 1.0f;
  if (is_q || is_k) {
    if (w != nullptr) mul = 1.0f / sqrtf(ss / (float)dk + eps);
    if (is_q && temp_every > 0) {
      const int steps = (positions[t] + 1) / temp_every;
      mul *= 1.0f + temp_coef * logf((float)steps + 1.0f);
    }
  }
  TA* dst = row + col0;
  if (!is_q) {
    const int slot = slots[t];
    if (slot < 0) return;
    const int g = is_k ? hs - H : hs - H - G;
    dst = (is_k ? k_cache : v_cache) + (((size_t)(slot / page) * G + g) * page + (slot % page)) * width;
  }
  uint4 outv;
  TA* ov = reinterpret_cast<TA*>(&outv);
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const float wv = w != nullptr ? __bfloat162float(w[d + i]) : 1.0f;
    as_store(ov + i, x[i] * mul * wv);
  }
  *reinterpret_cast<uint4*>(dst + d) = outv;
}

// -------------------------------------------------------------------------------------- prefill
constexpr int kPfRows = 16, kPfKeys = 32, kPfWarps = 4, kPfRowsPerWarp = kPfRows / kPfWarps;

// grid (tiles, H, tile_rows / 16).  Tile i = rows [tile_q0[i], +tile_rows) of sequence tile_seq[i], cut into
// 16-row pieces along z; the sequence's new rows are [cu_q[s], cu_q[s+1]) of the projection and sit at
// positions ctx_lens[s] + row.
template <typename TA, int kMaxDvPerLane>
__global__ void __launch_bounds__(kPfWarps * 32)
attn_sink_prefill_kernel(const TA* __restrict__ proj, int64_t ld, int gate_col, const TA* __restrict__ k_cache,
                         const TA* __restrict__ v_cache, const int32_t* __restrict__ block_table, int max_blocks,
                         const int32_t* __restrict__ cu_q, const int32_t* __restrict__ ctx_lens,
                         const int32_t* __restrict__ tile_seq, const int32_t* __restrict__ tile_q0,
                         const float* __restrict__ sink, TA* out, int64_t ldo, int H, int G, int dk, int dv, int page,
                         float scale, int64_t v_ld, int window, int gate_per_head, const float* __restrict__ head_scale,
                         const float* __restrict__ pool_k, const float* __restrict__ pool_v, int pool, int per_page,
                         const float* __restrict__ init_lse) {
  extern __shared__ float smem[];
  float* Qs = smem;                                   // [16][dk]
  float* Ks = Qs + kPfRows * dk;                      // [32][dk + 1]
  float* Vs = Ks + kPfKeys * (dk + 1);                // [32][dv]
  float* Ps = Vs + kPfKeys * dv;                      // [4 warps][4 rows][32]
  const int tile = blockIdx.x, h = blockIdx.y, g = h / (H / G);
  const int s = tile_seq[tile], q0 = tile_q0[tile] + kPfRows * blockIdx.z;
  const int row0 = cu_q[s], qlen = cu_q[s + 1] - row0, ctx = ctx_lens[s];
  if (q0 >= qlen) return;                             // a piece beyond the end of a short last tile
  const int nrows = min(kPfRows, qlen - q0);
  // a continued softmax whose last row sees no pooled block yet: the first part's rows stand as they are
  if (init_lse != nullptr && (pool_k == nullptr || window <= 0 || (ctx + q0 + nrows - window) / pool <= 0)) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int32_t* bt = block_table + (size_t)s * max_blocks;
  if (head_scale != nullptr) scale *= head_scale[h];

  for (int i = threadIdx.x; i < kPfRows * dk; i += blockDim.x) {
    const int r = i / dk, d = i - r * dk;
    Qs[i] = r < nrows ? as_f32(proj[(size_t)(row0 + q0 + r) * ld + h * dk + d]) : 0.f;
  }
  float m[kPfRowsPerWarp], l[kPfRowsPerWarp], acc[kPfRowsPerWarp][kMaxDvPerLane];
#pragma unroll
  for (int r = 0; r < kPfRowsPerWarp; ++r) {
    // the sink opens the running softmax: a key with score sink_h and a zero value
    m[r] = sink != nullptr ? sink[h] : -CUDART_INF_F;
    l[r] = sink != nullptr ? 1.f : 0.f;
#pragma unroll
    for (int j = 0; j < kMaxDvPerLane; ++j) acc[r][j] = 0.f;
  }
  if (init_lse != nullptr) {
    // the softmax is CONTINUED: another kernel has attended the window's tokens, `out` holds its normalised rows and
    // init_lse their log-sum-exp -- a running state with maximum lse, denominator 1 and the output as accumulator
#pragma unroll
    for (int r = 0; r < kPfRowsPerWarp; ++r) {
      const int qr = warp * kPfRowsPerWarp + r;
      if (qr >= nrows) continue;
      const size_t t = (size_t)(row0 + q0 + qr);
      m[r] = init_lse[t * H + h];
      l[r] = m[r] > -CUDART_INF_F ? 1.f : 0.f;
#pragma unroll
      for (int c = 0; c < kMaxDvPerLane; ++c) {
        const int d = lane + 32 * c;
        if (d < dv) acc[r][c] = as_f32(out[t * ldo + h * dv + d]);
      }
    }
  }
  const int kv_end = ctx + q0 + nrows;                // keys this tile can see: [kv_begin, kv_end)
  // a sliding window: position i sees j with 0 <= i - j < window, so nothing before the first row's window is read
  const int kv_begin = window > 0 ? max(0, ctx + q0 - window + 1) : 0;
  // pooled blocks first (entries [0, blocks the tile's last row sees)), then the tokens; one running softmax
  const int n_pool = (pool_k != nullptr && window > 0) ? max(0, (kv_end - 1 - window + 1) / pool) : 0;
  const int pool_span = (n_pool + kPfKeys - 1) & ~(kPfKeys - 1);
  const int tok_begin = kv_begin & ~(kPfKeys - 1);
  const int it_end = init_lse != nullptr ? 0 : kv_end - tok_begin;      // a continued softmax reads the pooled blocks only
  for (int it = -pool_span; it < it_end; it += kPfKeys) {
    const bool pooled = it < 0;
    const int k0 = pooled ? it + pool_span : tok_begin + it;
    __syncthreads();                                  // previous block's K / V fully consumed (and Qs written)
    // each warp stages 8 keys
#pragma unroll 2
    for (int jj = 0; jj < kPfKeys / kPfWarps; ++jj) {
      const int j = warp * (kPfKeys / kPfWarps) + jj;
      const int key = k0 + j;
      if (pooled && key < n_pool) {
        const int pj = (key * pool) / page;
        const size_t base = ((size_t)bt[pj] * G + g) * per_page + (key - (pj * page + pool - 1) / pool);
        const float* kp = pool_k + base * dk;
        const float* vp = pool_v + base * dv;
#pragma unroll 4
        for (int d = lane; d < dk; d += 32) Ks[j * (dk + 1) + d] = kp[d];
#pragma unroll 4
        for (int d = lane; d < dv; d += 32) Vs[j * dv + d] = vp[d];
      } else if (!pooled && key < kv_end) {
        const size_t base = ((size_t)bt[key / page] * G + g) * page + (key % page);
        const TA* kp = k_cache + base * dk;
        const TA* vp = v_cache + base * v_ld;
#pragma unroll 4
        for (int d = lane; d < dk; d += 32) Ks[j * (dk + 1) + d] = as_f32(kp[d]);
#pragma unroll 4
        for (int d = lane; d < dv; d += 32) Vs[j * dv + d] = as_f32(vp[d]);
      } else {
        for (int d = lane; d < dk; d += 32) Ks[j * (dk + 1) + d] = 0.f;
        for (int d = lane; d < dv; d += 32) Vs[j * dv + d] = 0.f;
      }
    }
    __syncthreads();
    // scores of this warp's rows against key k0 + lane
    float sc[kPfRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kPfRowsPerWarp; ++r) sc[r] = 0.f;
    const float* kr = Ks + lane * (dk + 1);
    const float* qr = Qs + warp * kPfRowsPerWarp * dk;
    for (int d = 0; d < dk; ++d) {
      const float kv = kr[d];
#pragma unroll
      for (int r = 0; r < kPfRowsPerWarp; ++r) sc[r] = fmaf(qr[r * dk + d], kv, sc[r]);
    }
    float* pw = Ps + warp * kPfRowsPerWarp * 32;
#pragma unroll
    for (int r = 0; r < kPfRowsPerWarp; ++r) {
      const int qpos = ctx + q0 + warp * kPfRowsPerWarp + r;
      const bool seen = pooled ? (k0 + lane) < (qpos - window + 1) / pool      // (negative numerators: nothing seen)
                               : ((k0 + lane) <= qpos && (k0 + lane) < kv_end && (window <= 0 || qpos - (k0 + lane) < window));
      const float sv = seen ? sc[r] * scale : -CUDART_INF_F;
      const float mn = fmaxf(m[r], warp_max(sv));
      float p = 0.f, corr = 1.f;
      if (mn > -CUDART_INF_F) {
        p = seen ? expf(sv - mn) : 0.f;
        corr = expf(m[r] - mn);                       // m = -inf before the first key: exp(-inf) = 0
      }
      l[r] = l[r] * corr + warp_sum(p);
      m[r] = mn;
#pragma unroll
      for (int j = 0; j < kMaxDvPerLane; ++j) acc[r][j] *= corr;
      pw[r * 32 + lane] = p;
    }
    __syncwarp();
    for (int j = 0; j < kPfKeys; ++j) {
      float p[kPfRowsPerWarp];
#pragma unroll
      for (int r = 0; r < kPfRowsPerWarp; ++r) p[r] = pw[r * 32 + j];
#pragma unroll
      for (int c = 0; c < kMaxDvPerLane; ++c) {
        const int d = lane + 32 * c;
        if (d < dv) {
          const float vv = Vs[j * dv + d];
#pragma unroll
          for (int r = 0; r < kPfRowsPerWarp; ++r) acc[r][c] = fmaf(p[r], vv, acc[r][c]);
        }
      }
    }
    __syncwarp();
  }
#pragma unroll
  for (int r = 0; r < kPfRowsPerWarp; ++r) {
    const int qr = warp * kPfRowsPerWarp + r;
    if (qr >= nrows) continue;
    const size_t t = (size_t)(row0 + q0 + qr);
    const float inv = l[r] > 0.f ? 1.0f / l[r] : 0.f;
#pragma unroll
    for (int c = 0; c < kMaxDvPerLane; ++c) {
      const int d = lane + 32 * c;
      if (d < dv) {
        float o = acc[r][c] * inv;
        if (gate_col >= 0) {
          const float gv = as_f32(proj[t * ld + gate_col + (gate_per_head ? h : h * dv + d)]);
          o *= 1.0f / (1.0f + expf(-gv));
        }
        as_store(out + t * ldo + h * dv + d, o);
      }
    }
  }
}

// --------------------------------------------------------------------------------------- decode
constexpr int kDecWarps = 4;

// grid (B, H): sequence b's single new row is row b of proj / out; it sees keys [0, seq_lens[b]).  The four warps
// take 32-key blocks in turn.  Scores: lane = key, the (scaled) query is broadcast from shared memory and every
// lane walks its own key row (16-byte loads when VEC); one max / sum reduction per 32 keys.  Values: lane = column,
// the 32 probabilities and page offsets go round by shuffle, value rows are read contiguously.
template <typename TA, bool VEC, int kMaxDvPerLane>
__global__ void __launch_bounds__(kDecWarps * 32)
attn_sink_decode_kernel(const TA* __restrict__ proj, int64_t ld, int gate_col, const TA* __restrict__ k_cache,
                        const TA* __restrict__ v_cache, const int32_t* __restrict__ block_table, int max_blocks,
                        const int32_t* __restrict__ seq_lens, const float* __restrict__ sink, TA* out, int64_t ldo,
                        int H, int G, int dk, int dv, int page, float scale, int64_t v_ld, int window, int gate_per_head,
                        const float* __restrict__ head_scale, const float* __restrict__ pool_k,
                        const float* __restrict__ pool_v, int pool, int per_page, const float* __restrict__ init_lse) {
  __shared__ float sm_m[kDecWarps], sm_l[kDecWarps];
  extern __shared__ __align__(16) float sm_dyn[];      // [dk (padded to 8)] query, then [warps][dv] partial outputs
  constexpr int E = 16 / (int)sizeof(TA);               // elements per 16-byte load
  const int dkp = (dk + 7) & ~7;
  float* qsm = sm_dyn;
  float* sm_acc = sm_dyn + dkp;
  const int b = blockIdx.x, h = blockIdx.y, g = h / (H / G);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = seq_lens[b];
  const int32_t* bt = block_table + (size_t)b * max_blocks;
  if (head_scale != nullptr) scale *= head_scale[h];
  for (int d = threadIdx.x; d < dkp; d += blockDim.x)
    qsm[d] = d < dk ? as_f32(proj[(size_t)b * ld + h * dk + d]) * scale : 0.f;
  __syncthreads();
  float m = -CUDART_INF_F, l = 0.f, acc[kMaxDvPerLane];
  if (warp == 0 && sink != nullptr) { m = sink[h]; l = 1.f; }
#pragma unroll
  for (int c = 0; c < kMaxDvPerLane; ++c) acc[c] = 0.f;
  if (init_lse != nullptr && warp == 0) {
    // the softmax is CONTINUED: another kernel has attended the window's tokens, `out` holds its normalised row and
    // init_lse its log-sum-exp -- a running state with maximum lse, denominator 1 and the output as accumulator
    m = init_lse[(size_t)b * H + h];
    l = m > -CUDART_INF_F ? 1.f : 0.f;
#pragma unroll
    for (int c = 0; c < kMaxDvPerLane; ++c) {
      const int d = lane + 32 * c;
      if (d < dv && l > 0.f) acc[c] = as_f32(out[(size_t)b * ldo + h * dv + d]);
    }
  }
  // a sliding window: the row at position n - 1 sees keys [n - window, n); the first block read is the one that holds
  // the window's first key
  const int first = window > 0 ? max(0, n - window) : 0;
  // pooled blocks: the row at position n - 1 sees the blocks that end at or before n - 1 - window
  const int n_pool = (pool_k != nullptr && window > 0) ? max(0, (n - window) / pool) : 0;
  for (int k0 = warp * 32; k0 < n_pool; k0 += kDecWarps * 32) {
    const int key = k0 + lane;
    const bool live = key < n_pool;
    size_t base = 0;
    float sc = -CUDART_INF_F;
    if (live) {
      const int pj = (key * pool) / page;
      base = ((size_t)bt[pj] * G + g) * per_page + (key - (pj * page + pool - 1) / pool);
      const float* kp = pool_k + base * dk;
      float a = 0.f;
      if ((dk & 3) == 0) {                  // entries are 16-byte aligned: dk * 4 bytes each from an aligned base
#pragma unroll 8                            // (several loads in flight: a lane walks its own row)
        for (int d = 0; d < dk; d += 4) {
          const float4 kv = *reinterpret_cast<const float4*>(kp + d);
          a = fmaf(qsm[d], kv.x, a); a = fmaf(qsm[d + 1], kv.y, a); a = fmaf(qsm[d + 2], kv.z, a); a = fmaf(qsm[d + 3], kv.w, a);
        }
      } else {
        for (int d = 0; d < dk; ++d) a = fmaf(qsm[d], kp[d], a);
      }
      sc = a;
    }
    const float mn = fmaxf(m, warp_max(sc));
    const float corr = expf(m - mn), p = live ? expf(sc - mn) : 0.f;
    l = l * corr + warp_sum(p);
    m = mn;
#pragma unroll
    for (int c = 0; c < kMaxDvPerLane; ++c) acc[c] *= corr;
    const int cnt = min(32, n_pool - k0);
#pragma unroll 8
    for (int j = 0; j < cnt; ++j) {
      const float pj_ = __shfl_sync(0xffffffffu, p, j);
      const unsigned long long bj = __shfl_sync(0xffffffffu, (unsigned long long)base, j);
      const float* vp = pool_v + (size_t)bj * dv;
#pragma unroll
      for (int c = 0; c < kMaxDvPerLane; ++c) {
        const int d = lane + 32 * c;
        if (d < dv) acc[c] = fmaf(pj_, vp[d], acc[c]);
      }
    }
  }
  const int tok_end = init_lse != nullptr ? 0 : n;      // a continued softmax reads the pooled blocks only
  for (int k0 = (first & ~31) + warp * 32; k0 < tok_end; k0 += kDecWarps * 32) {
    const int key = k0 + lane;
    const bool live = key < n && key >= first;
    size_t base = 0;
    float sc = -CUDART_INF_F;
    if (live) {
      base = ((size_t)bt[key / page] * G + g) * page + (key % page);
      const TA* kp = k_cache + base * dk;
      float a = 0.f;
      if (VEC) {
#pragma unroll 8
        for (int d = 0; d < dk; d += E) {
          const uint4 raw = *reinterpret_cast<const uint4*>(kp + d);
          const TA* kv = reinterpret_cast<const TA*>(&raw);
#pragma unroll
          for (int i = 0; i < E; ++i) a = fmaf(qsm[d + i], as_f32(kv[i]), a);
        }
      } else {
        for (int d = 0; d < dk; ++d) a = fmaf(qsm[d], as_f32(kp[d]), a);
      }
      sc = a;
    }
    const float mn = fmaxf(m, warp_max(sc));            // finite: some key of this block is live
    const float corr = expf(m - mn), p = live ? expf(sc - mn) : 0.f;
    l = l * corr + warp_sum(p);
    m = mn;
#pragma unroll
    for (int c = 0; c < kMaxDvPerLane; ++c) acc[c] *= corr;
    const int cnt = min(32, n - k0);
#pragma unroll 8
    for (int j = max(0, first - k0); j < cnt; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const unsigned long long bj = __shfl_sync(0xffffffffu, (unsigned long long)base, j);
      const TA* vp = v_cache + (size_t)bj * v_ld;
#pragma unroll
      for (int c = 0; c < kMaxDvPerLane; ++c) {
        const int d = lane + 32 * c;
        if (d < dv) acc[c] = fmaf(pj, as_f32(vp[d]), acc[c]);
      }
    }
  }
  if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
  __syncthreads();
  float mt = -CUDART_INF_F;
#pragma unroll
  for (int w = 0; w < kDecWarps; ++w) mt = fmaxf(mt, sm_m[w]);
  const float mine = mt > -CUDART_INF_F && m > -CUDART_INF_F ? expf(m - mt) : 0.f;
#pragma unroll
  for (int c = 0; c < kMaxDvPerLane; ++c) {
    const int d = lane + 32 * c;
    if (d < dv) sm_acc[warp * dv + d] = acc[c] * mine;
  }
  __syncthreads();
  float lt = 0.f;
#pragma unroll
  for (int w = 0; w < kDecWarps; ++w) lt += sm_m[w] > -CUDART_INF_F ? sm_l[w] * expf(sm_m[w] - mt) : 0.f;
  const float inv = lt > 0.f ? 1.0f / lt : 0.f;
  for (int d = threadIdx.x; d < dv; d += blockDim.x) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) o += sm_acc[w * dv + d];
    o *= inv;
    if (gate_col >= 0) {
      const float gv = as_f32(proj[(size_t)b * ld + gate_col + (gate_per_head ? h : h * dv + d)]);
      o *= 1.0f / (1.0f + expf(-gv));
    }
    as_store(out + (size_t)b * ldo + h * dv + d, o);
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_attn_prep(void* proj, int f32, int64_t ld, const void* bias, const void* qnorm_w,
                              const void* knorm_w, const int32_t* positions, const int32_t* slots, void* k_cache,
                              void* v_cache, int T, int H, int G, int dk, int dv, int page, int has_kv, float eps,
                              float temp_coef, int temp_every, void* stream) {
  B200_REQUIRE(T >= 0 && H > 0 && G > 0 && H % G == 0 && dk > 0 && dv > 0 && page > 0, "attn_prep: bad shape");
  if (T == 0) return B200_OK;
  const int n_slots = has_kv ? H + 2 * G : H;
  dim3 grid(T, (n_slots + kPrepWarps - 1) / kPrepWarps);
  cudaStream_t s = (cudaStream_t)stream;
  const int esz = f32 ? 4 : 2;
  const bool pair = dk % 2 == 0 && dv % 2 == 0 && ld % 2 == 0 && (reinterpret_cast<uintptr_t>(proj) % (2 * esz)) == 0 &&
                    (!has_kv || ((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) % (2 * esz)) == 0);
  {
    // 16-byte path: widths, offsets and pitches that are multiples of 16 bytes, at most 32 pieces per head
    const int vec = 16 / esz, wmax = dk > dv ? dk : dv;
    const bool al = ((reinterpret_cast<uintptr_t>(proj) | (has_kv ? reinterpret_cast<uintptr_t>(k_cache) |
                                                            reinterpret_cast<uintptr_t>(v_cache) : 0)) & 15) == 0;
    if (al && dk % vec == 0 && dv % vec == 0 && ld % vec == 0 && wmax / vec <= 32) {
      int lph = 1;
      while (lph < wmax / vec) lph <<= 1;
      const int per_block = kPrepWarps * (32 / lph);
      dim3 vgrid(T, (n_slots + per_block - 1) / per_block);
      if (f32)
        attn_prep_vec_kernel<float><<<vgrid, kPrepWarps * 32, 0, s>>>(
            (float*)proj, ld, (const bf16*)bias, (const bf16*)qnorm_w, (const bf16*)knorm_w, positions, slots,
            (float*)k_cache, (float*)v_cache, H, G, dk, dv, page, n_slots, lph, eps, temp_coef, temp_every);
      else
        attn_prep_vec_kernel<bf16><<<vgrid, kPrepWarps * 32, 0, s>>>(
            (bf16*)proj, ld, (const bf16*)bias, (const bf16*)qnorm_w, (const bf16*)knorm_w, positions, slots,
            (bf16*)k_cache, (bf16*)v_cache, H, G, dk, dv, page, n_slots, lph, eps, temp_coef, temp_every);
      return b200_check_launch("b200_attn_prep");
    }
  }
  B200_REQUIRE(dk <= (pair ? 64 : 32) * kPrepPairs && dv <= (pair ? 64 : 32) * kPrepPairs,
               "attn_prep: head widths %d / %d exceed %d", dk, dv, (pair ? 64 : 32) * kPrepPairs);
#define B200_PREP(TA, P)                                                                                         \
  attn_prep_kernel<TA, P><<<grid, kPrepWarps * 32, 0, s>>>((TA*)proj, ld, (const bf16*)bias, (const bf16*)qnorm_w, \
                                                           (const bf16*)knorm_w, positions, slots, (TA*)k_cache,  \
                                                           (TA*)v_cache, H, G, dk, dv, page, n_slots, eps,        \
                                                           temp_coef, temp_every)
  if (f32) { if (pair) B200_PREP(float, true); else B200_PREP(float, false); }
  else { if (pair) B200_PREP(bf16, true); else B200_PREP(bf16, false); }
#undef B200_PREP
  return b200_check_launch("b200_attn_prep");
}

extern "C" int b200_attn_sink_prefill_tile(void) { return kPfRows; }

static int attn_sink_prefill_launch(const void* proj, int f32, int64_t ld, int gate_col, const void* k_cache,
                                    const void* v_cache, const int32_t* block_table, int max_blocks,
                                    const int32_t* cu_q, const int32_t* ctx_lens, const int32_t* tile_seq,
                                    const int32_t* tile_q0, int n_tiles, int tile_rows, const float* sink, void* out,
                                    int64_t ldo, int H, int G, int dk, int dv, int page, float scale, int64_t v_ld,
                                    int window, int gate_per_head, const float* head_scale, const float* pool_k,
                                    const float* pool_v, int pool, int per_page, const float* init_lse, void* stream) {
  if (v_ld <= 0) v_ld = dv;
  B200_REQUIRE(pool_k == nullptr || (pool_v != nullptr && window > 0 && pool > 0 && per_page == (page + pool - 1) / pool),
               "attn_sink_prefill: pooled blocks need a window, both caches and ceil(page / pool) entries per page");
  B200_REQUIRE(v_ld >= dv, "attn_sink_prefill: value row pitch %lld < dv=%d", (long long)v_ld, dv);
  B200_REQUIRE(tile_rows > 0 && tile_rows % kPfRows == 0, "attn_sink_prefill: tiles of %d rows (multiples of %d)",
               tile_rows, kPfRows);
  B200_REQUIRE(H > 0 && G > 0 && H % G == 0 && dk > 0 && dv > 0 && dv <= 32 * kMaxDvLanes && page > 0,
               "attn_sink_prefill: bad shape H=%d G=%d dk=%d dv=%d", H, G, dk, dv);
  if (n_tiles <= 0) return B200_OK;
  const size_t smem = sizeof(float) * ((size_t)kPfRows * dk + (size_t)kPfKeys * (dk + 1) + (size_t)kPfKeys * dv +
                                       (size_t)kPfWarps * kPfRowsPerWarp * 32);
  B200_REQUIRE(smem <= 200 * 1024, "attn_sink_prefill: head widths %d / %d exceed shared memory", dk, dv);
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(n_tiles, H, tile_rows / kPfRows);
#define B200_PF(TA, L)                                                                                             \
  do {                                                                                                             \
    if (smem > 48 * 1024)                                                                                          \
      cudaFuncSetAttribute(attn_sink_prefill_kernel<TA, L>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    attn_sink_prefill_kernel<TA, L><<<grid, kPfWarps * 32, smem, s>>>(                                             \
        (const TA*)proj, ld, gate_col, (const TA*)k_cache, (const TA*)v_cache, block_table, max_blocks, cu_q,       \
        ctx_lens, tile_seq, tile_q0, sink, (TA*)out, ldo, H, G, dk, dv, page, scale, v_ld, window, gate_per_head,   \
        head_scale, pool_k, pool_v, pool, per_page, init_lse);                                                     \
  } while (0)
  const bool wide = dv > 256;
  if (f32) { if (wide) B200_PF(float, 16); else B200_PF(float, 8); }
  else { if (wide) B200_PF(bf16, 16); else B200_PF(bf16, 8); }
#undef B200_PF
  return b200_check_launch("b200_attn_sink_prefill");
}

extern "C" int b200_attn_sink_prefill_pool(const void* proj, int f32, int64_t ld, int gate_col, const void* k_cache,
                                           const void* v_cache, const int32_t* block_table, int max_blocks,
                                           const int32_t* cu_q, const int32_t* ctx_lens, const int32_t* tile_seq,
                                           const int32_t* tile_q0, int n_tiles, int tile_rows, const float* sink, void* out,
                                           int64_t ldo, int H, int G, int dk, int dv, int page, float scale, int64_t v_ld,
                                           int window, int gate_per_head, const float* head_scale, const float* pool_k,
                                           const float* pool_v, int pool, int per_page, void* stream) {
  return attn_sink_prefill_launch(proj, f32, ld, gate_col, k_cache, v_cache, block_table, max_blocks, cu_q, ctx_lens, tile_seq,
                                  tile_q0, n_tiles, tile_rows, sink, out, ldo, H, G, dk, dv, page, scale, v_ld, window,
                                  gate_per_head, head_scale, pool_k, pool_v, pool, per_page, nullptr, stream);
}

extern "C" int b200_attn_sink_prefill_more(const void* proj, int f32, int64_t ld, const void* k_cache,
                                           const int32_t* block_table, int max_blocks, const int32_t* cu_q,
                                           const int32_t* ctx_lens, const int32_t* tile_seq, const int32_t* tile_q0, int n_tiles,
                                           int tile_rows, void* out, int64_t ldo, int H, int G, int dk, int dv, int page,
                                           float scale, int window, const float* head_scale, const float* pool_k,
                                           const float* pool_v, int pool, int per_page, const float* init_lse, void* stream) {
  B200_REQUIRE(init_lse != nullptr && pool_k != nullptr, "attn_sink_prefill_more: needs the first part's log-sum-exp and pooled blocks");
  return attn_sink_prefill_launch(proj, f32, ld, -1, k_cache, k_cache, block_table, max_blocks, cu_q, ctx_lens, tile_seq,
                                  tile_q0, n_tiles, tile_rows, nullptr, out, ldo, H, G, dk, dv, page, scale, 0, window, 0,
                                  head_scale, pool_k, pool_v, pool, per_page, init_lse, stream);
}

extern "C" int b200_attn_sink_prefill_ex(const void* proj, int f32, int64_t ld, int gate_col, const void* k_cache,
                                         const void* v_cache, const int32_t* block_table, int max_blocks,
                                         const int32_t* cu_q, const int32_t* ctx_lens, const int32_t* tile_seq,
                                         const int32_t* tile_q0, int n_tiles, int tile_rows, const float* sink, void* out,
                                         int64_t ldo, int H, int G, int dk, int dv, int page, float scale, int64_t v_ld,
                                         int window, void* stream) {
  return b200_attn_sink_prefill_pool(proj, f32, ld, gate_col, k_cache, v_cache, block_table, max_blocks, cu_q, ctx_lens,
                                     tile_seq, tile_q0, n_tiles, tile_rows, sink, out, ldo, H, G, dk, dv, page, scale, v_ld,
                                     window, 0, nullptr, nullptr, nullptr, 0, 0, stream);
}

extern "C" int b200_attn_sink_prefill(const void* proj, int f32, int64_t ld, int gate_col, const void* k_cache,
                                      const void* v_cache, const int32_t* block_table, int max_blocks,
                                      const int32_t* cu_q, const int32_t* ctx_lens, const int32_t* tile_seq,
                                      const int32_t* tile_q0, int n_tiles, int tile_rows, const float* sink, void* out,
                                      int64_t ldo, int H, int G, int dk, int dv, int page, float scale, int64_t v_ld,
                                      void* stream) {
  return b200_attn_sink_prefill_ex(proj, f32, ld, gate_col, k_cache, v_cache, block_table, max_blocks, cu_q, ctx_lens,
                                   tile_seq, tile_q0, n_tiles, tile_rows, sink, out, ldo, H, G, dk, dv, page, scale, v_ld, 0,
                                   stream);
}

static int attn_sink_decode_launch(const void* proj, int f32, int64_t ld, int gate_col, const void* k_cache,
                                   const void* v_cache, const int32_t* block_table, int max_blocks,
                                   const int32_t* seq_lens, int B, const float* sink, void* out, int64_t ldo, int H,
                                   int G, int dk, int dv, int page, float scale, int64_t v_ld, int window,
                                   int gate_per_head, const float* head_scale, const float* pool_k,
                                   const float* pool_v, int pool, int per_page, const float* init_lse, void* stream) {
  if (v_ld <= 0) v_ld = dv;
  B200_REQUIRE(pool_k == nullptr || (pool_v != nullptr && window > 0 && pool > 0 && per_page == (page + pool - 1) / pool),
               "attn_sink_decode: pooled blocks need a window, both caches and ceil(page / pool) entries per page");
  B200_REQUIRE(v_ld >= dv, "attn_sink_decode: value row pitch %lld < dv=%d", (long long)v_ld, dv);
  B200_REQUIRE(H > 0 && G > 0 && H % G == 0 && dk > 0 && dv > 0 && dv <= 32 * kMaxDvLanes && page > 0,
               "attn_sink_decode: bad shape H=%d G=%d dk=%d dv=%d", H, G, dk, dv);
  if (B <= 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const size_t smem = sizeof(float) * (((dk + 7) & ~7) + (size_t)kDecWarps * dv);
  B200_REQUIRE(smem <= 48 * 1024, "attn_sink_decode: key width %d exceeds shared memory", dk);
  const int esz = f32 ? 4 : 2;
  const bool vec = (dk * esz) % 16 == 0 && (reinterpret_cast<uintptr_t>(k_cache) & 15) == 0;
  dim3 grid(B, H);
#define B200_DEC(TA, V)                                                                                          \
  if (dv > 256)                                                                                                  \
    attn_sink_decode_kernel<TA, V, 16><<<grid, kDecWarps * 32, smem, s>>>(                                       \
        (const TA*)proj, ld, gate_col, (const TA*)k_cache, (const TA*)v_cache, block_table, max_blocks, seq_lens, \
        sink, (TA*)out, ldo, H, G, dk, dv, page, scale, v_ld, window, gate_per_head, head_scale, pool_k, pool_v,  \
        pool, per_page, init_lse);                                                                               \
  else                                                                                                           \
    attn_sink_decode_kernel<TA, V, 8><<<grid, kDecWarps * 32, smem, s>>>(                                        \
      (const TA*)proj, ld, gate_col, (const TA*)k_cache, (const TA*)v_cache, block_table, max_blocks, seq_lens,   \
      sink, (TA*)out, ldo, H, G, dk, dv, page, scale, v_ld, window, gate_per_head, head_scale, pool_k, pool_v,    \
      pool, per_page, init_lse)
  if (f32) { if (vec) B200_DEC(float, true); else B200_DEC(float, false); }
  else { if (vec) B200_DEC(bf16, true); else B200_DEC(bf16, false); }
#undef B200_DEC
  return b200_check_launch("b200_attn_sink_decode");
}

extern "C" int b200_attn_sink_decode_pool(const void* proj, int f32, int64_t ld, int gate_col, const void* k_cache,
                                          const void* v_cache, const int32_t* block_table, int max_blocks,
                                          const int32_t* seq_lens, int B, const float* sink, void* out, int64_t ldo, int H,
                                          int G, int dk, int dv, int page, float scale, int64_t v_ld, int window,
                                          int gate_per_head, const float* head_scale, const float* pool_k,
                                          const float* pool_v, int pool, int per_page, void* stream) {
  return attn_sink_decode_launch(proj, f32, ld, gate_col, k_cache, v_cache, block_table, max_blocks, seq_lens, B, sink, out, ldo,
                                 H, G, dk, dv, page, scale, v_ld, window, gate_per_head, head_scale, pool_k, pool_v, pool,
                                 per_page, nullptr, stream);
}

extern "C" int b200_attn_sink_decode_more(const void* proj, int f32, int64_t ld, const int32_t* block_table, int max_blocks,
                                          const int32_t* seq_lens, int B, void* out, int64_t ldo, int H, int G, int dk, int dv,
                                          int page, float scale, int window, const float* head_scale, const float* pool_k,
                                          const float* pool_v, int pool, int per_page, const float* init_lse, void* stream) {
  B200_REQUIRE(init_lse != nullptr && pool_k != nullptr, "attn_sink_decode_more: needs the first part's log-sum-exp and pooled blocks");
  // no token is read: the caches' pointers only pass the alignment test of the vector path
  return attn_sink_decode_launch(proj, f32, ld, -1, pool_k, pool_k, block_table, max_blocks, seq_lens, B, nullptr, out, ldo, H, G,
                                 dk, dv, page, scale, 0, window, 0, head_scale, pool_k, pool_v, pool, per_page, init_lse, stream);
}

extern "C" int b200_attn_sink_decode_ex(const void* proj, int f32, int64_t ld, int gate_col, const void* k_cache,
                                        const void* v_cache, const int32_t* block_table, int max_blocks,
                                        const int32_t* seq_lens, int B, const float* sink, void* out, int64_t ldo, int H,
                                        int G, int dk, int dv, int page, float scale, int64_t v_ld, int window,
                                        void* stream) {
  return b200_attn_sink_decode_pool(proj, f32, ld, gate_col, k_cache, v_cache, block_table, max_blocks, seq_lens, B, sink, out,
                                    ldo, H, G, dk, dv, page, scale, v_ld, window, 0, nullptr, nullptr, nullptr, 0, 0, stream);
}

extern "C" int b200_attn_sink_decode(const void* proj, int f32, int64_t ld, int gate_col, const void* k_cache,
                                     const void* v_cache, const int32_t* block_table, int max_blocks,
                                     const int32_t* seq_lens, int B, const float* sink, void* out, int64_t ldo, int H,
                                     int G, int dk, int dv, int page, float scale, int64_t v_ld, void* stream) {
  return b200_attn_sink_decode_ex(proj, f32, ld, gate_col, k_cache, v_cache, block_table, max_blocks, seq_lens, B, sink, out,
                                  ldo, H, G, dk, dv, page, scale, v_ld, 0, stream);
}
