// Per-head preparation of queries, keys and values between a fused input projection and a mixer's core kernel:
// the element-wise steps that different mixers combine, in one launch.
//
//   feature map   silu(x) on the head's entries (queries, keys and values alike), or none;
//   rotation      the first `dims` entries of a query / key head are rotated by the angle position * freq[i] of
//                 pair i -- pairs (2i, 2i+1) ("interleaved") or (i, i + dims/2) ("half"); the rest pass unchanged.
//                 The angle is formed and reduced to [-pi, pi] in fp64, cos / sin of the remainder in fp32;
//   unit norm     the rotated head over its root mean square, x / sqrt(mean(x^2) + eps), no weight;
//   factor        a constant on the queries and one on the keys (after rotation and norm); optionally one more factor
//                 per query head.
//
// Where the results go:
//   queries       q_out rows (the projection itself = in place, or a separate fp32 buffer);
//   keys, values  either the pages of a KV cache (K [blocks][G][page][dk], V [blocks][G][page][dv]) at slots[t]
//                 (a softmax-attention mixer), or rows of a separate buffer (a recurrent mixer reads them once);
//   values        come from their own columns, or are the keys AS PROJECTED (before feature map, rotation and
//                 norm) when the mixer has no value projection.
//   A mixer that reads another layer's keys and values passes no key destination: only its queries are prepared.
// One warp per (token, head slot): slots [0, H) queries, [H, H + G) keys, [H + G, H + 2G) values (absent when the
// values are the keys).  Each lane keeps its entries in registers between the sum of squares and the store.
// Source type TA (bf16 | fp32), destination type TD (the same, or fp32 for recurrent mixers).
#include "common.cuh"
#include "runtime.h"
#include "../../include/b200.h"

namespace b200 {

__device__ __forceinline__ float rp_f32(float v) { return v; }
__device__ __forceinline__ float rp_f32(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void rp_store(float* p, float v) { *p = v; }
__device__ __forceinline__ void rp_store(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

constexpr int kRpWarps = 8, kRpPairs = 8, kRpTail = 16;     // rotated width <= 512, unrotated rest <= 512

struct RotPrepArgs {
  const void* proj;
  int64_t ld;
  int q_col, k_col, v_col;          // first column of the q / k / v heads in a projection row (v_col < 0: values are keys)
  const int32_t* positions;
  const int32_t* slots;             // cache slot of every token (cache destinations only)
  void* q_out;
  int64_t ldq;
  void* k_out;                      // k_cache, or a row buffer with leading dimension ldk
  int64_t ldk;
  void* v_out;
  int64_t ldv;
  int paged;                        // 1: k_out / v_out are pages
  int page;
  int H, G, dk, dv;
  int feature;                      // 0 none, 1 silu
  int dims, half_layout;            // dims == 0: no rotation
  const double* freq;
  int unit_norm;
  float eps, q_mul, k_mul;
  const float* q_head_mul;          // optional [H]: one more factor per query head (a learned temperature)
};

template <typename TA, typename TD>
__global__ void __launch_bounds__(kRpWarps * 32)
rot_prep_kernel(RotPrepArgs a) {
  const int t = blockIdx.x, lane = threadIdx.x & 31;
  const int hs = blockIdx.y * kRpWarps + (threadIdx.x >> 5);
  const int H = a.H, G = a.G, dk = a.dk, dv = a.dv;
  const bool has_v = a.v_col >= 0;
  if (hs >= (a.k_out == nullptr ? H : H + G + (has_v ? G : 0))) return;   // no key destination: queries only
  const bool is_q = hs < H, is_k = !is_q && hs < H + G;
  const int g = is_q ? hs : (is_k ? hs - H : hs - H - G);
  const TA* src = reinterpret_cast<const TA*>(a.proj) + (size_t)t * a.ld +
                  (is_q ? a.q_col + g * dk : (is_k ? a.k_col + g * dk : a.v_col + g * dv));
  const int width = (is_q || is_k) ? dk : dv;
  size_t cache_row = 0;
  if (!is_q && a.paged) {
    const int slot = a.slots[t];
    if (slot < 0) return;
    cache_row = ((size_t)(slot / a.page) * G + g) * a.page + (slot % a.page);
  }
  TD* dst;
  if (is_q) dst = reinterpret_cast<TD*>(a.q_out) + (size_t)t * a.ldq + g * dk;
  else if (is_k) dst = reinterpret_cast<TD*>(a.k_out) + (a.paged ? cache_row * dk : (size_t)t * a.ldk + g * dk);
  else dst = reinterpret_cast<TD*>(a.v_out) + (a.paged ? cache_row * dv : (size_t)t * a.ldv + g * dv);

  if (!is_q && !is_k) {             // a value head: feature map only
    for (int d = lane; d < dv; d += 32) {
      float x = rp_f32(src[d]);
      if (a.feature == 1) x = x / (1.0f + expf(-x));
      rp_store(dst + d, x);
    }
    return;
  }
  const int dims = a.dims, half = dims >> 1;
  TD* vdst = nullptr;               // values are the keys as projected
  if (is_k && !has_v && a.v_out != nullptr)
    vdst = reinterpret_cast<TD*>(a.v_out) + (a.paged ? cache_row * dv : (size_t)t * a.ldv + g * dv);
  float u[kRpPairs], v[kRpPairs], rest[kRpTail];
  float ss = 0.f;
  const int pos = a.positions[t];
#pragma unroll
  for (int i = 0; i < kRpPairs; ++i) {
    const int j = lane + 32 * i;
    u[i] = v[i] = 0.f;
    if (j < half) {
      const int d0 = a.half_layout ? j : 2 * j, d1 = a.half_layout ? j + half : 2 * j + 1;
      float x0 = rp_f32(src[d0]), x1 = rp_f32(src[d1]);
      if (vdst != nullptr) { rp_store(vdst + d0, x0); rp_store(vdst + d1, x1); }
      if (a.feature == 1) { x0 = x0 / (1.0f + expf(-x0)); x1 = x1 / (1.0f + expf(-x1)); }
      const double ang = (double)pos * a.freq[j];
      const float rem = (float)(ang - 6.283185307179586 * rint(ang * 0.15915494309189535));
      float sn, cs;
      sincosf(rem, &sn, &cs);
      u[i] = x0 * cs - x1 * sn;
      v[i] = x1 * cs + x0 * sn;
      ss = fmaf(u[i], u[i], fmaf(v[i], v[i], ss));
    }
  }
#pragma unroll
  for (int i = 0; i < kRpTail; ++i) {
    const int d = dims + lane + 32 * i;
    rest[i] = 0.f;
    if (d < width) {
      float x = rp_f32(src[d]);
      if (vdst != nullptr) rp_store(vdst + d, x);
      if (a.feature == 1) x = x / (1.0f + expf(-x));
      rest[i] = x;
      ss = fmaf(x, x, ss);
    }
  }
  float mul = is_q ? a.q_mul : a.k_mul;
  if (is_q && a.q_head_mul != nullptr) mul *= a.q_head_mul[g];
  if (a.unit_norm) mul *= 1.0f / sqrtf(warp_sum(ss) / (float)width + a.eps);
#pragma unroll
  for (int i = 0; i < kRpPairs; ++i) {
    const int j = lane + 32 * i;
    if (j < half) {
      rp_store(dst + (a.half_layout ? j : 2 * j), u[i] * mul);
      rp_store(dst + (a.half_layout ? j + half : 2 * j + 1), v[i] * mul);
    }
  }
#pragma unroll
  for (int i = 0; i < kRpTail; ++i) {
    const int d = dims + lane + 32 * i;
    if (d < width) rp_store(dst + d, rest[i] * mul);
  }
}

// The same steps with 16-byte accesses, one CTA per token: the token's cos / sin are computed ONCE (dims / 2 angles)
// into shared memory and used by every head.  A head is cut into items of VEC = 16 bytes / sizeof(TA) entries: an
// interleaved rotation turns the pairs inside an item; a half-split rotation makes an item of the piece [d, d + VEC)
// and its partner [d + dims/2, ...); the unrotated rest are plain items.  LPH lanes (a power of two >= items per
// head) share a head, a warp covers 32 / LPH head slots at a time, the sum of squares is reduced inside the group.
constexpr int kRvThreads = 256;

template <typename TA, typename TD>
__global__ void __launch_bounds__(kRvThreads)
rot_prep_vec_kernel(RotPrepArgs a, int lph, int items_q, int items_v) {
  constexpr int VEC = 16 / (int)sizeof(TA);
  extern __shared__ float2 cs[];                      // [dims / 2] (cos, sin) of this token
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int H = a.H, G = a.G, dk = a.dk, dv = a.dv, dims = a.dims, half = dims >> 1;
  if (dims > 0) {
    const int pos = a.positions[t];
    for (int j = threadIdx.x; j < half; j += kRvThreads) {
      const double ang = (double)pos * a.freq[j];
      const float rem = (float)(ang - 6.283185307179586 * rint(ang * 0.15915494309189535));
      float sn, c;
      sincosf(rem, &sn, &c);
      cs[j] = make_float2(c, sn);
    }
    __syncthreads();
  }
  const bool has_v = a.v_col >= 0;
  const int n_slots = a.k_out == nullptr ? H : H + G + (has_v ? G : 0);    // no key destination: queries only
  const int per_warp = 32 / lph, sub = lane / lph, li = lane % lph;
  const int slot = a.paged ? a.slots[t] : 0;
  const TA* row = reinterpret_cast<const TA*>(a.proj) + (size_t)t * a.ld;
  const int n_rot = dims == 0 ? 0 : (a.half_layout ? half / VEC : dims / VEC);
  for (int hs0 = warp * per_warp; hs0 < n_slots; hs0 += (kRvThreads / 32) * per_warp) {
    const int hs = hs0 + sub;
    const bool live = hs < n_slots;
    const bool is_q = live && hs < H, is_k = live && !is_q && hs < H + G, is_v = live && !is_q && !is_k;
    const int g = is_q ? hs : (is_k ? hs - H : hs - H - G);
    const bool act = live && li < (is_v ? items_v : items_q) && (is_q || !a.paged || slot >= 0);
    float x0[VEC], x1[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) x0[i] = x1[i] = 0.f;
    int d0 = 0, d1 = -1;
    float ss = 0.f;
    TD* dst = nullptr;
    if (act) {
      const size_t cache_row = a.paged ? ((size_t)(slot / a.page) * G + g) * a.page + (slot % a.page) : 0;
      const TA* src = row + (is_q ? a.q_col + g * dk : (is_k ? a.k_col + g * dk : a.v_col + g * dv));
      if (is_q) dst = reinterpret_cast<TD*>(a.q_out) + (size_t)t * a.ldq + g * dk;
      else if (is_k) dst = reinterpret_cast<TD*>(a.k_out) + (a.paged ? cache_row * dk : (size_t)t * a.ldk + g * dk);
      else dst = reinterpret_cast<TD*>(a.v_out) + (a.paged ? cache_row * dv : (size_t)t * a.ldv + g * dv);
      const bool rot = !is_v && li < n_rot;
      d0 = is_v ? li * VEC : (rot ? li * VEC : dims + (li - n_rot) * VEC);
      if (rot && a.half_layout) d1 = d0 + half;
      {
        const uint4 raw = *reinterpret_cast<const uint4*>(src + d0);
        const TA* rv = reinterpret_cast<const TA*>(&raw);
#pragma unroll
        for (int i = 0; i < VEC; ++i) x0[i] = rp_f32(rv[i]);
      }
      if (d1 >= 0) {
        const uint4 raw = *reinterpret_cast<const uint4*>(src + d1);
        const TA* rv = reinterpret_cast<const TA*>(&raw);
#pragma unroll
        for (int i = 0; i < VEC; ++i) x1[i] = rp_f32(rv[i]);
      }
      if (is_k && !has_v && a.v_out != nullptr) {      // the values are the keys as projected
        TD* vdst = reinterpret_cast<TD*>(a.v_out) + (a.paged ? cache_row * dv : (size_t)t * a.ldv + g * dv);
#pragma unroll
        for (int i = 0; i < VEC; ++i) rp_store(vdst + d0 + i, x0[i]);
        if (d1 >= 0) {
#pragma unroll
          for (int i = 0; i < VEC; ++i) rp_store(vdst + d1 + i, x1[i]);
        }
      }
      if (a.feature == 1) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          x0[i] = x0[i] / (1.0f + expf(-x0[i]));
          if (d1 >= 0) x1[i] = x1[i] / (1.0f + expf(-x1[i]));
        }
      }
      if (rot && a.half_layout) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          const float2 c = cs[d0 + i];
          const float u = x0[i], v = x1[i];
          x0[i] = u * c.x - v * c.y;
          x1[i] = v * c.x + u * c.y;
        }
      } else if (rot) {
#pragma unroll
        for (int i = 0; i < VEC; i += 2) {
          const float2 c = cs[(d0 + i) >> 1];
          const float u = x0[i], v = x0[i + 1];
          x0[i] = u * c.x - v * c.y;
          x0[i + 1] = v * c.x + u * c.y;
        }
      }
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        ss = fmaf(x0[i], x0[i], ss);
        if (d1 >= 0) ss = fmaf(x1[i], x1[i], ss);
      }
    }
    float mul = is_q ? a.q_mul : a.k_mul;
    if (is_q && a.q_head_mul != nullptr) mul *= a.q_head_mul[g];
    if (a.unit_norm) {                                 // every lane takes part in the shuffles
      for (int o = lph >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      mul *= 1.0f / sqrtf(ss / (float)dk + a.eps);
    }
    if (!act) continue;
    if (is_v) mul = 1.0f;
    // 16-byte stores whatever the destination type: VEC fp32 entries are VEC / 4 pieces, VEC bf16 entries one
    if constexpr (sizeof(TD) == 4) {
#pragma unroll
      for (int i = 0; i < VEC; i += 4) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + d0 + i) =
            make_float4(x0[i] * mul, x0[i + 1] * mul, x0[i + 2] * mul, x0[i + 3] * mul);
        if (d1 >= 0)
          *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + d1 + i) =
              make_float4(x1[i] * mul, x1[i + 1] * mul, x1[i + 2] * mul, x1[i + 3] * mul);
      }
    } else {
      uint32_t w0[VEC / 2], w1[VEC / 2];
#pragma unroll
      for (int i = 0; i < VEC; i += 2) {
        w0[i / 2] = pack_bf16(x0[i] * mul, x0[i + 1] * mul);
        w1[i / 2] = pack_bf16(x1[i] * mul, x1[i + 1] * mul);
      }
      *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(dst) + d0) = *reinterpret_cast<uint4*>(w0);
      if (d1 >= 0) *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(dst) + d1) = *reinterpret_cast<uint4*>(w1);
    }
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_rot_prep(const void* proj, int src_f32, int64_t ld, int q_col, int k_col, int v_col,
                             const int32_t* positions, const int32_t* slots, void* q_out, int64_t ldq, void* k_out,
                             int64_t ldk, void* v_out, int64_t ldv, int dst_f32, int paged, int page, int T, int H, int G,
                             int dk, int dv, int feature, int dims, int half_layout, const double* freq, int unit_norm,
                             float eps, float q_mul, float k_mul, void* stream) {
  return b200_rot_prep_hm(proj, src_f32, ld, q_col, k_col, v_col, positions, slots, q_out, ldq, k_out, ldk, v_out, ldv, dst_f32,
                          paged, page, T, H, G, dk, dv, feature, dims, half_layout, freq, unit_norm, eps, q_mul, k_mul, nullptr,
                          stream);
}

extern "C" int b200_rot_prep_hm(const void* proj, int src_f32, int64_t ld, int q_col, int k_col, int v_col,
                                const int32_t* positions, const int32_t* slots, void* q_out, int64_t ldq, void* k_out,
                                int64_t ldk, void* v_out, int64_t ldv, int dst_f32, int paged, int page, int T, int H, int G,
                                int dk, int dv, int feature, int dims, int half_layout, const double* freq, int unit_norm,
                                float eps, float q_mul, float k_mul, const float* q_head_mul, void* stream) {
  B200_REQUIRE(T >= 0 && H > 0 && G > 0 && dk > 0 && dv > 0, "rot_prep: bad shape");
  B200_REQUIRE(dims >= 0 && dims % 2 == 0 && dims <= dk && dims <= 64 * kRpPairs && dk - dims <= 32 * kRpTail,
               "rot_prep: %d rotated of %d entries (rotated <= %d, rest <= %d)", dims, dk, 64 * kRpPairs, 32 * kRpTail);
  B200_REQUIRE(dims == 0 || (freq != nullptr && positions != nullptr), "rot_prep: a rotation needs frequencies and positions");
  B200_REQUIRE(feature == 0 || feature == 1, "rot_prep: unknown feature map %d", feature);
  B200_REQUIRE(!paged || (slots != nullptr && page > 0), "rot_prep: cache destinations need slots");
  B200_REQUIRE(v_col >= 0 || v_out == nullptr || dv == dk, "rot_prep: values that are keys have the keys' width");
  B200_REQUIRE(src_f32 ? dst_f32 : 1, "rot_prep: fp32 rows are not rounded to bf16 here");
  if (T == 0) return B200_OK;
  RotPrepArgs a{proj, ld, q_col, k_col, v_col, positions, slots, q_out, ldq, k_out, ldk, v_out, ldv, paged, page, H, G, dk, dv,
                feature, dims, half_layout, freq, unit_norm, eps, q_mul, k_mul, q_head_mul};
  const int n_slots = k_out == nullptr ? H : H + G + (v_col >= 0 ? G : 0);
  dim3 grid(T, (n_slots + kRpWarps - 1) / kRpWarps);
  cudaStream_t s = (cudaStream_t)stream;
  {
    // 16-byte path: every width, column offset, leading dimension and base address a multiple of 16 bytes on both
    // sides, rotated part a whole number of items, at most 32 items per head
    const int esz = src_f32 ? 4 : 2, dsz = dst_f32 ? 4 : 2, vec = 16 / esz;
    auto al = [](const void* p_) { return (reinterpret_cast<uintptr_t>(p_) & 15) == 0; };
    const bool has_v = v_col >= 0;
    const int rot_items = dims == 0 ? 0 : (half_layout ? (dims / 2) / vec : dims / vec);
    const int items_q = rot_items + (dk - dims) / vec, items_v = dv / vec;
    const int items = items_q > items_v ? items_q : items_v;
    bool ok = dk % vec == 0 && dv % vec == 0 && dims % vec == 0 && (!half_layout || (dims / 2) % vec == 0) && items <= 32 &&
              ld % vec == 0 && q_col % vec == 0 && k_col % vec == 0 && (!has_v || v_col % vec == 0) && al(proj) && al(q_out) &&
              al(k_out) && al(v_out) && (ldq * dsz) % 16 == 0 && (paged || ((ldk * dsz) % 16 == 0 && (ldv * dsz) % 16 == 0)) &&
              (size_t)(dims / 2) * sizeof(float2) <= 40 * 1024 && !(src_f32 && !dst_f32);
    if (ok) {
      int lph = 1;
      while (lph < items) lph <<= 1;
      const size_t smem = (size_t)(dims / 2) * sizeof(float2);
      if (src_f32) rot_prep_vec_kernel<float, float><<<T, kRvThreads, smem, s>>>(a, lph, items_q, items_v);
      else if (dst_f32) rot_prep_vec_kernel<bf16, float><<<T, kRvThreads, smem, s>>>(a, lph, items_q, items_v);
      else rot_prep_vec_kernel<bf16, bf16><<<T, kRvThreads, smem, s>>>(a, lph, items_q, items_v);
      return b200_check_launch("b200_rot_prep");
    }
  }
  if (src_f32) rot_prep_kernel<float, float><<<grid, kRpWarps * 32, 0, s>>>(a);
  else if (dst_f32) rot_prep_kernel<bf16, float><<<grid, kRpWarps * 32, 0, s>>>(a);
  else rot_prep_kernel<bf16, bf16><<<grid, kRpWarps * 32, 0, s>>>(a);
  return b200_check_launch("b200_rot_prep");
}
