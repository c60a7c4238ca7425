// Residual stream with a norm before AND after every sublayer, short causal convolutions with per-sequence state,
// learned positions, and the block means of a KV cache.  The stream, every statistic and every sum is fp32.
//
//   embed_pos        x = table[id] + pos_table[position]                                   (fp32 stream)
//   sandwich_join    v = ya * y (+ yb * y2)            the sublayer output(s), fp32
//                    z = x + mult * v / rms(v) * (wb)  the stream takes the NORMED output        (y == null: z = x)
//                    h = z / rms(z) * (wa)             the next sublayer's normed input, fp32 or rounded once
//                    rms(v) = sqrt(mean(v^2) + eps); a weight stored around zero enters as 1 + w (zero_centred).
//                    With a row list it gathers: row r reads row rows[r] and writes h only (the rows whose logits are
//                    wanted).  One CTA per row, the row staged in shared memory between statistic and product.
//   causal_conv      out_t = (in_t if add_input) + bias + sum_j w[:, j] in_(t - taps + 1 + j),  zeros before position 0.
//                    A step brings every sequence's NEW rows; inputs older than the step come from the sequence's
//                    ring: ring[slot][p mod (taps - 1)][c] holds the input at position p for the last taps - 1
//                    positions.  A sequence whose context is empty never reads the ring, so a slot needs no clearing.
//   conv_commit      after the convolution has run: the last taps - 1 inputs of every sequence's new rows go to the
//                    ring (a separate launch: the convolution's first rows read what the last rows replace).
//   kv_pool_update   mean key and mean value of every block of `pool` tokens that a step completes, summed in
//                    position order in fp32 from the cache as it holds them.  Entry b of a sequence lives in the page
//                    of its first token: pool_k [blocks][G][per_page][dk], entry index b - ceil(first token's page *
//                    page / pool) -- the sequence's own block table addresses it, and pages that are handed to
//                    another sequence are overwritten before they are read.
#include "common.cuh"
#include "runtime.h"
#include "../../include/b200.h"

namespace b200 {

__device__ __forceinline__ float sw_f32(float v) { return v; }
__device__ __forceinline__ float sw_f32(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void sw_store(float* p, float v) { *p = v; }
__device__ __forceinline__ void sw_store(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__global__ void __launch_bounds__(256)
embed_pos_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ positions, const bf16* __restrict__ table,
                 const bf16* __restrict__ pos_table, float* __restrict__ x, int D, int vocab, int max_pos) {
  const int t = blockIdx.x;
  int id = ids[t], p = positions[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  p = p < 0 ? 0 : (p >= max_pos ? max_pos - 1 : p);
  const bf16* e = table + (size_t)id * D;
  const bf16* q = pos_table + (size_t)p * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x)
    x[(size_t)t * D + i] = __bfloat162float(e[i]) + __bfloat162float(q[i]);
}

__device__ __forceinline__ float block_sum_256(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();                                    // red may still be read from the call before
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.f;
  return warp_sum(t);
}

// 4-entry loads and stores (VEC: D a multiple of 4, 16-byte aligned fp32 rows, 8-byte aligned bf16 rows)
__device__ __forceinline__ float4 sw_ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 sw_ld4(const bf16* p) {
  const uint2 r = *reinterpret_cast<const uint2*>(p);
  return make_float4(bf16_lo(r.x), bf16_hi(r.x), bf16_lo(r.y), bf16_hi(r.y));
}
__device__ __forceinline__ void sw_st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void sw_st4(bf16* p, float4 v) {
  *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
}

template <typename TO, int V>
__global__ void __launch_bounds__(256)
sandwich_join_kernel(const float* x_in, const float* __restrict__ y, const float* __restrict__ y2, float ya, float yb,
                     const bf16* __restrict__ wb, float mult, const int32_t* __restrict__ rows,
                     const bf16* __restrict__ wa, float* x_out, TO* h_out, int D, float eps, float w_base) {
  extern __shared__ __align__(16) float zrow[];       // [D] the output row, then the new stream row
  __shared__ float red[32];
  const int r = blockIdx.x;
  const size_t src = (size_t)(rows != nullptr ? rows[r] : r) * D;
  const int i0 = threadIdx.x * V, step = blockDim.x * V;
  if (y != nullptr) {
    float ss = 0.f;
    for (int i = i0; i < D; i += step) {
      if (V == 4) {
        float4 v = sw_ld4(y + src + i);
        v.x *= ya; v.y *= ya; v.z *= ya; v.w *= ya;
        if (y2 != nullptr) {
          const float4 b = sw_ld4(y2 + src + i);
          v.x = fmaf(yb, b.x, v.x); v.y = fmaf(yb, b.y, v.y); v.z = fmaf(yb, b.z, v.z); v.w = fmaf(yb, b.w, v.w);
        }
        sw_st4(zrow + i, v);
        ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
      } else {
        float v = ya * y[src + i];
        if (y2 != nullptr) v = fmaf(yb, y2[src + i], v);
        zrow[i] = v;
        ss = fmaf(v, v, ss);
      }
    }
    const float rstd = 1.0f / sqrtf(block_sum_256(ss, red) / (float)D + eps);
    for (int i = i0; i < D; i += step) {
      if (V == 4) {
        const float4 v = sw_ld4(zrow + i), x = sw_ld4(x_in + src + i), w = sw_ld4(wb + i);
        sw_st4(zrow + i, make_float4(fmaf(mult, v.x * rstd * (w_base + w.x), x.x), fmaf(mult, v.y * rstd * (w_base + w.y), x.y),
                                     fmaf(mult, v.z * rstd * (w_base + w.z), x.z), fmaf(mult, v.w * rstd * (w_base + w.w), x.w)));
      } else {
        zrow[i] = fmaf(mult, zrow[i] * rstd * (w_base + __bfloat162float(wb[i])), x_in[src + i]);
      }
    }
  } else {
    for (int i = i0; i < D; i += step) {
      if (V == 4) sw_st4(zrow + i, sw_ld4(x_in + src + i));
      else zrow[i] = x_in[src + i];
    }
  }
  float ss = 0.f;
  for (int i = i0; i < D; i += step) {                 // every thread reads back what it staged itself
    if (V == 4) {
      const float4 z = sw_ld4(zrow + i);
      if (x_out != nullptr) sw_st4(x_out + (size_t)r * D + i, z);
      ss = fmaf(z.x, z.x, fmaf(z.y, z.y, fmaf(z.z, z.z, fmaf(z.w, z.w, ss))));
    } else {
      const float z = zrow[i];
      if (x_out != nullptr) x_out[(size_t)r * D + i] = z;
      ss = fmaf(z, z, ss);
    }
  }
  if (wa == nullptr || h_out == nullptr) return;
  const float rstd = 1.0f / sqrtf(block_sum_256(ss, red) / (float)D + eps);
  for (int i = i0; i < D; i += step) {
    if (V == 4) {
      const float4 z = sw_ld4(zrow + i), w = sw_ld4(wa + i);
      sw_st4(h_out + (size_t)r * D + i, make_float4(z.x * rstd * (w_base + w.x), z.y * rstd * (w_base + w.y),
                                                    z.z * rstd * (w_base + w.z), z.w * rstd * (w_base + w.w)));
    } else {
      sw_store(h_out + (size_t)r * D + i, zrow[i] * rstd * (w_base + __bfloat162float(wa[i])));
    }
  }
}

// Row t belongs to the sequence s with cu_seq[s] <= t < cu_seq[s + 1]
__device__ __forceinline__ int seq_of_row(const int32_t* __restrict__ cu_seq, int n_seqs, int t) {
  int lo = 0, hi = n_seqs - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_seq[mid] <= t) lo = mid; else hi = mid - 1;
  }
  return lo;
}

constexpr int kConvMaxTaps = 8;

// grid (ceil(T / RB), ceil(C / (256 V))); TI input element, TO output element; a thread takes V neighbouring channels of RB
// rows in turn, the taps' weights staying in registers (RB = 1 for small steps, which need the CTAs more than the reuse)
template <typename TI, typename TO, int V, int RB>
__global__ void __launch_bounds__(256)
causal_conv_kernel(const TI* __restrict__ in, int64_t ld_in, const float* __restrict__ in_bias,
                   const float* __restrict__ w, const float* __restrict__ bias, int add_input,
                   const float* __restrict__ ring, const int32_t* __restrict__ cu_seq,
                   const int32_t* __restrict__ ctx_lens, const int32_t* __restrict__ state_slots, int n_seqs, TO* out,
                   int64_t ld_out, int T, int C, int taps) {
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
  // the rows' sequences, looked up once per CTA: context length, position and ring slot of each row
  __shared__ int sh_ctx[RB], sh_p[RB], sh_slot[RB], sh_seq[RB];
  if (threadIdx.x < RB) {
    const int t = blockIdx.x * RB + threadIdx.x;
    if (t < T) {
      const int s = seq_of_row(cu_seq, n_seqs, t);
      sh_seq[threadIdx.x] = s;
      sh_ctx[threadIdx.x] = ctx_lens[s];
      sh_p[threadIdx.x] = ctx_lens[s] + (t - cu_seq[s]);
      sh_slot[threadIdx.x] = state_slots[s];
    }
  }
  __syncthreads();
  if (c >= C) return;
  const int R = taps - 1;
  // wd[d]: the weight of the input d positions back (d = 0: the current token, the LAST tap)
  float wd[kConvMaxTaps][V], ib[V], ob[V];
#pragma unroll
  for (int d = 0; d < kConvMaxTaps; ++d)
#pragma unroll
    for (int v = 0; v < V; ++v) wd[d][v] = d <= R ? w[(size_t)(c + v) * taps + (R - d)] : 0.f;
#pragma unroll
  for (int v = 0; v < V; ++v) {
    ib[v] = in_bias != nullptr ? in_bias[c + v] : 0.f;
    ob[v] = bias != nullptr ? bias[c + v] : 0.f;
  }
  auto load_row = [&](int t, float (&x)[V]) {           // row t of the input, with its bias
    if (V == 4) {
      const float4 q = sw_ld4(in + (size_t)t * ld_in + c);
      x[0] = q.x + ib[0]; x[V > 1 ? 1 : 0] = q.y + ib[V > 1 ? 1 : 0]; x[V > 2 ? 2 : 0] = q.z + ib[V > 2 ? 2 : 0];
      x[V > 3 ? 3 : 0] = q.w + ib[V > 3 ? 3 : 0];
    } else {
      x[0] = sw_f32(in[(size_t)t * ld_in + c]) + ib[0];
    }
  };
  // all of the CTA's rows first (independent loads in flight); earlier taps then come from registers
  float cur[RB][V];
#pragma unroll
  for (int i = 0; i < RB; ++i) {
    const int t = blockIdx.x * RB + i;
    if (t < T) {
      load_row(t, cur[i]);
    } else {
#pragma unroll
      for (int v = 0; v < V; ++v) cur[i][v] = 0.f;
    }
  }
  // the common case of a prompt step: all rows of one sequence and every tap among this step's rows -- no ring, no
  // per-tap position arithmetic
  const int n_rows = min(RB, T - (int)blockIdx.x * RB);
  if (RB > 1 && sh_seq[0] == sh_seq[n_rows - 1] && sh_p[0] - R >= sh_ctx[0]) {
#pragma unroll
    for (int i = 0; i < RB; ++i) {
      const int t = blockIdx.x * RB + i;
      if (i >= n_rows) break;
      float acc[V];
#pragma unroll
      for (int v = 0; v < V; ++v) acc[v] = fmaf(wd[0][v], cur[i][v], add_input ? ob[v] + cur[i][v] : ob[v]);
#pragma unroll
      for (int d = 1; d < kConvMaxTaps; ++d) {
        if (d > R) break;
        float val[V];
        if (i - d >= 0) {
#pragma unroll
          for (int v = 0; v < V; ++v) val[v] = cur[i - d >= 0 ? i - d : 0][v];
        } else {
          load_row(t - d, val);                        // a row of the CTA before
        }
#pragma unroll
        for (int v = 0; v < V; ++v) acc[v] = fmaf(wd[d][v], val[v], acc[v]);
      }
      if (V == 4) sw_st4(out + (size_t)t * ld_out + c, make_float4(acc[0], acc[V > 1 ? 1 : 0], acc[V > 2 ? 2 : 0], acc[V > 3 ? 3 : 0]));
      else sw_store(out + (size_t)t * ld_out + c, acc[0]);
    }
    return;
  }
#pragma unroll
  for (int i = 0; i < RB; ++i) {
    const int t = blockIdx.x * RB + i;
    if (t >= T) break;
    const int ctx = sh_ctx[i], p = sh_p[i];
    float acc[V];
#pragma unroll
    for (int v = 0; v < V; ++v) acc[v] = fmaf(wd[0][v], cur[i][v], add_input ? ob[v] + cur[i][v] : ob[v]);
#pragma unroll
    for (int d = 1; d < kConvMaxTaps; ++d) {
      const int sp = p - d;                            // the position this tap multiplies
      if (d > R || sp < 0) continue;
      float val[V];
      if (sp >= ctx) {                                 // one of this step's rows of the same sequence
        if (i - d >= 0) {
#pragma unroll
          for (int v = 0; v < V; ++v) val[v] = cur[i - d >= 0 ? i - d : 0][v];
        } else {
          load_row(t - d, val);
        }
      } else {                                         // an earlier step's: the sequence's ring
        const float* rp = ring + ((size_t)sh_slot[i] * R + (sp % R)) * C + c;
        if (V == 4) {
          const float4 q = sw_ld4(rp);
          val[0] = q.x; val[V > 1 ? 1 : 0] = q.y; val[V > 2 ? 2 : 0] = q.z; val[V > 3 ? 3 : 0] = q.w;
        } else {
          val[0] = rp[0];
        }
      }
#pragma unroll
      for (int v = 0; v < V; ++v) acc[v] = fmaf(wd[d][v], val[v], acc[v]);
    }
    if (V == 4) sw_st4(out + (size_t)t * ld_out + c, make_float4(acc[0], acc[V > 1 ? 1 : 0], acc[V > 2 ? 2 : 0], acc[V > 3 ? 3 : 0]));
    else sw_store(out + (size_t)t * ld_out + c, acc[0]);
  }
}

// grid (n_seqs, taps - 1, ceil(C / 256))
template <typename TI>
__global__ void __launch_bounds__(256)
conv_commit_kernel(const TI* __restrict__ in, int64_t ld_in, const float* __restrict__ in_bias, float* ring,
                   const int32_t* __restrict__ cu_seq, const int32_t* __restrict__ ctx_lens,
                   const int32_t* __restrict__ state_slots, int C, int taps) {
  const int s = blockIdx.x, r = blockIdx.y, c = blockIdx.z * blockDim.x + threadIdx.x;
  const int slot = state_slots[s];
  const int t0 = cu_seq[s], t1 = cu_seq[s + 1];
  if (c >= C || slot < 0 || r >= t1 - t0) return;      // an older input stays where it is
  const int R = taps - 1;
  const int p = ctx_lens[s] + (t1 - t0) - 1 - r;
  const float ib = in_bias != nullptr ? in_bias[c] : 0.f;
  ring[((size_t)slot * R + (p % R)) * C + c] = sw_f32(in[(size_t)(t1 - 1 - r) * ld_in + c]) + ib;
}

// grid (n_seqs, most blocks a sequence completes in this step, G); cu_q == null: one new row per sequence whose
// context is ctx_lens[s] - 1 tokens (ctx_lens then counts the new row, as a decode step's lengths do)
template <typename TA, int V>
__global__ void __launch_bounds__(128)
kv_pool_update_kernel(const TA* __restrict__ k_cache, const TA* __restrict__ v_cache, float* pool_k, float* pool_v,
                      const int32_t* __restrict__ block_table, int max_blocks, const int32_t* __restrict__ cu_q,
                      const int32_t* __restrict__ ctx_lens, int G, int dk, int dv, int page, int pool, int per_page) {
  const int s = blockIdx.x, g = blockIdx.z;
  const int ctx = cu_q != nullptr ? ctx_lens[s] : ctx_lens[s] - 1;
  const int n = cu_q != nullptr ? cu_q[s + 1] - cu_q[s] : 1;
  if (n <= 0 || ctx < 0) return;
  const int b = ctx / pool + blockIdx.y;               // blocks whose last token is among the new rows
  if (b >= (ctx + n) / pool) return;
  const int32_t* bt = block_table + (size_t)s * max_blocks;
  const int first = b * pool, pj = first / page;
  const int idx = b - (pj * page + pool - 1) / pool;
  const size_t dst = ((size_t)bt[pj] * G + g) * per_page + idx;
  const float inv = 1.0f / (float)pool;
  // a thread takes V neighbouring columns (V = 4: one 8- or 16-byte load per token); tokens are added in order
  const int nk = dk / V, nv = dv / V;
  for (int c = threadIdx.x; c < nk + nv; c += blockDim.x) {
    const bool is_k = c < nk;
    const int cc = (is_k ? c : c - nk) * V, w = is_k ? dk : dv;
    const TA* cache = is_k ? k_cache : v_cache;
    float sum[V];
#pragma unroll
    for (int v = 0; v < V; ++v) sum[v] = 0.f;
#pragma unroll 4
    for (int i = 0; i < pool; ++i) {
      const int tok = first + i;
      const TA* src = cache + (((size_t)bt[tok / page] * G + g) * page + (tok % page)) * w + cc;
      if (V == 4) {
        const float4 t = sw_ld4(src);
        sum[0] += t.x; sum[V > 1 ? 1 : 0] += t.y; sum[V > 2 ? 2 : 0] += t.z; sum[V > 3 ? 3 : 0] += t.w;
      } else {
        sum[0] += sw_f32(src[0]);
      }
    }
    float* out = (is_k ? pool_k : pool_v) + dst * w + cc;
    if (V == 4) sw_st4(out, make_float4(sum[0] * inv, sum[V > 1 ? 1 : 0] * inv, sum[V > 2 ? 2 : 0] * inv, sum[V > 3 ? 3 : 0] * inv));
    else out[0] = sum[0] * inv;
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_embed_pos_f32(const int32_t* ids, const int32_t* positions, const void* table, const void* pos_table,
                                  float* x, int T, int D, int vocab, int max_pos, void* stream) {
  B200_REQUIRE(T >= 0 && D > 0 && vocab > 0 && max_pos > 0, "embed_pos: bad shape");
  if (T == 0) return B200_OK;
  embed_pos_kernel<<<T, 256, 0, (cudaStream_t)stream>>>(ids, positions, (const bf16*)table, (const bf16*)pos_table, x, D,
                                                        vocab, max_pos);
  return b200_check_launch("b200_embed_pos_f32");
}

extern "C" int b200_sandwich_join(const float* x_in, const float* y, const float* y2, float ya, float yb, const void* wb,
                                  float mult, const int32_t* rows, const void* wa, float* x_out, void* h_out, int h_f32,
                                  int T, int D, float eps, int zero_centred, void* stream) {
  B200_REQUIRE(T >= 0 && D > 0 && x_in != nullptr, "sandwich_join: bad arguments T=%d D=%d", T, D);
  B200_REQUIRE(y == nullptr || wb != nullptr, "sandwich_join: a sublayer output needs the weight of its norm");
  B200_REQUIRE(rows == nullptr || x_out == nullptr, "sandwich_join: the gather form writes the normed rows only");
  if (T == 0) return B200_OK;
  const size_t smem = (size_t)D * sizeof(float);
  B200_REQUIRE(smem <= 48 * 1024, "sandwich_join: D=%d exceeds the staged row (12288)", D);
  cudaStream_t s = (cudaStream_t)stream;
  const float base = zero_centred ? 1.0f : 0.0f;
  auto al = [](const void* p, int n) { return (reinterpret_cast<uintptr_t>(p) & (n - 1)) == 0; };
  const bool vec = D % 4 == 0 && al(x_in, 16) && al(y, 16) && al(y2, 16) && al(x_out, 16) && al(wb, 8) && al(wa, 8) &&
                   al(h_out, h_f32 ? 16 : 8);
#define B200_SJ(TO, V)                                                                                                  \
  sandwich_join_kernel<TO, V><<<T, 256, smem, s>>>(x_in, y, y2, ya, yb, (const bf16*)wb, mult, rows, (const bf16*)wa, x_out, \
                                                   (TO*)h_out, D, eps, base)
  if (h_f32) { if (vec) B200_SJ(float, 4); else B200_SJ(float, 1); }
  else { if (vec) B200_SJ(bf16, 4); else B200_SJ(bf16, 1); }
#undef B200_SJ
  return b200_check_launch("b200_sandwich_join");
}

extern "C" int b200_causal_conv(const void* in, int in_f32, int64_t ld_in, const float* in_bias, const float* w,
                                const float* bias, int add_input, const float* ring, const int32_t* cu_seq,
                                const int32_t* ctx_lens, const int32_t* state_slots, int n_seqs, void* out, int out_f32,
                                int64_t ld_out, int T, int C, int taps, void* stream) {
  B200_REQUIRE(T >= 0 && C > 0 && taps >= 1 && taps <= kConvMaxTaps && n_seqs >= 0, "causal_conv: bad shape C=%d taps=%d", C,
               taps);
  B200_REQUIRE(taps == 1 || ring != nullptr, "causal_conv: more than one tap needs the sequences' rings");
  if (T == 0 || n_seqs == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  auto al = [](const void* p, int n) { return (reinterpret_cast<uintptr_t>(p) & (n - 1)) == 0; };
  const bool vec = C % 4 == 0 && ld_in % 4 == 0 && ld_out % 4 == 0 && al(in, in_f32 ? 16 : 8) && al(out, out_f32 ? 16 : 8) &&
                   al(in_bias, 16) && al(bias, 16) && al(ring, 16);
  const int V = vec ? 4 : 1;
  const int rb = T >= 2048 ? 8 : 1;
  dim3 grid((T + rb - 1) / rb, (C + 256 * V - 1) / (256 * V));
#define B200_CC2(TI, TO, VV, RB)                                                                                      \
  causal_conv_kernel<TI, TO, VV, RB><<<grid, 256, 0, s>>>((const TI*)in, ld_in, in_bias, w, bias, add_input, ring, cu_seq, \
                                                          ctx_lens, state_slots, n_seqs, (TO*)out, ld_out, T, C, taps)
#define B200_CC(TI, TO)                                                                                               \
  do {                                                                                                                \
    if (vec) { if (rb == 8) B200_CC2(TI, TO, 4, 8); else B200_CC2(TI, TO, 4, 1); }                                    \
    else { if (rb == 8) B200_CC2(TI, TO, 1, 8); else B200_CC2(TI, TO, 1, 1); }                                        \
  } while (0)
  if (in_f32) { if (out_f32) B200_CC(float, float); else B200_CC(float, bf16); }
  else { if (out_f32) B200_CC(bf16, float); else B200_CC(bf16, bf16); }
#undef B200_CC
#undef B200_CC2
  return b200_check_launch("b200_causal_conv");
}

extern "C" int b200_conv_commit(const void* in, int in_f32, int64_t ld_in, const float* in_bias, float* ring,
                                const int32_t* cu_seq, const int32_t* ctx_lens, const int32_t* state_slots, int n_seqs,
                                int C, int taps, void* stream) {
  B200_REQUIRE(C > 0 && taps >= 1 && taps <= kConvMaxTaps && n_seqs >= 0, "conv_commit: bad shape C=%d taps=%d", C, taps);
  if (n_seqs == 0 || taps == 1) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(n_seqs, taps - 1, (C + 255) / 256);
  if (in_f32)
    conv_commit_kernel<float><<<grid, 256, 0, s>>>((const float*)in, ld_in, in_bias, ring, cu_seq, ctx_lens, state_slots, C, taps);
  else
    conv_commit_kernel<bf16><<<grid, 256, 0, s>>>((const bf16*)in, ld_in, in_bias, ring, cu_seq, ctx_lens, state_slots, C, taps);
  return b200_check_launch("b200_conv_commit");
}

extern "C" int b200_kv_pool_update(const void* k_cache, const void* v_cache, int f32, float* pool_k, float* pool_v,
                                   const int32_t* block_table, int max_blocks, const int32_t* cu_q, const int32_t* ctx_lens,
                                   int n_seqs, int max_new, int G, int dk, int dv, int page, int pool, int per_page,
                                   void* stream) {
  B200_REQUIRE(n_seqs >= 0 && G > 0 && dk > 0 && dv > 0 && page > 0 && pool > 0 && per_page == (page + pool - 1) / pool,
               "kv_pool_update: bad shape page=%d pool=%d per_page=%d", page, pool, per_page);
  if (n_seqs == 0 || max_new <= 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(n_seqs, max_new / pool + 1, G);
  auto al = [](const void* p, int n) { return (reinterpret_cast<uintptr_t>(p) & (n - 1)) == 0; };
  const bool vec = dk % 4 == 0 && dv % 4 == 0 && al(k_cache, 16) && al(v_cache, 16) && al(pool_k, 16) && al(pool_v, 16);
  const int threads = vec ? 64 : 128;
#define B200_KP(TA, V)                                                                                             \
  kv_pool_update_kernel<TA, V><<<grid, threads, 0, s>>>((const TA*)k_cache, (const TA*)v_cache, pool_k, pool_v, block_table, \
                                                        max_blocks, cu_q, ctx_lens, G, dk, dv, page, pool, per_page)
  if (f32) { if (vec) B200_KP(float, 4); else B200_KP(float, 1); }
  else { if (vec) B200_KP(bf16, 4); else B200_KP(bf16, 1); }
#undef B200_KP
  return b200_check_launch("b200_kv_pool_update");
}
