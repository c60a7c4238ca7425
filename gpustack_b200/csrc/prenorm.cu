// Pre-norm residual stream kept in fp32, for layers whose branches are summed into the stream un-normalised.
//
//   add_rms_norm_f32:  z = x_in + a + b + c   (each of a, b, c optional: the branch outputs of the layer before --
//                      a mixer and a feed-forward that ran side by side on one normed input -- and a third
//                      addend such as the embedding output that a repeated span of layers takes in again),
//                      x_out = z  (the new fp32 stream),   xb_out = z / sqrt(mean(z^2) + eps) * w  (the next
//                      layer's input, rounded once to bf16, or fp32).
//                      The sum, the statistic and the product are fp32 in a fixed order (x, a, b, c).
//                      With a row list it gathers: row r reads x_in / a / b / c at rows[r] and writes row r of
//                      xb_out only (final norm of the rows whose logits are wanted).  Without w nothing is normed
//                      (the sum alone is written).
// One CTA per row; the summed row is staged in shared memory between the statistic and the product.
#include "common.cuh"
#include "runtime.h"
#include "../../include/b200.h"

namespace b200 {

__device__ __forceinline__ void prn_store(float* p, float v) { *p = v; }
__device__ __forceinline__ void prn_store(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

template <typename TO, bool VEC>
__global__ void __launch_bounds__(256)
add_rms_norm_f32_kernel(const float* x_in, const float* __restrict__ a, const float* __restrict__ b,
                        const float* __restrict__ c, const int32_t* __restrict__ rows, const bf16* __restrict__ w,
                        float* x_out, TO* xb_out, int D, float eps) {
  extern __shared__ __align__(16) float zrow[];
  __shared__ float red[32];
  const int r = blockIdx.x;
  const size_t src = (size_t)(rows != nullptr ? rows[r] : r) * D;
  float ss = 0.f;
  if (VEC) {
    for (int i = threadIdx.x * 4; i < D; i += blockDim.x * 4) {
      float4 z = *reinterpret_cast<const float4*>(x_in + src + i);
      if (a != nullptr) { const float4 v = *reinterpret_cast<const float4*>(a + src + i); z.x += v.x; z.y += v.y; z.z += v.z; z.w += v.w; }
      if (b != nullptr) { const float4 v = *reinterpret_cast<const float4*>(b + src + i); z.x += v.x; z.y += v.y; z.z += v.z; z.w += v.w; }
      if (c != nullptr) { const float4 v = *reinterpret_cast<const float4*>(c + src + i); z.x += v.x; z.y += v.y; z.z += v.z; z.w += v.w; }
      *reinterpret_cast<float4*>(zrow + i) = z;
      if (x_out != nullptr) *reinterpret_cast<float4*>(x_out + (size_t)r * D + i) = z;
      ss = fmaf(z.x, z.x, fmaf(z.y, z.y, fmaf(z.z, z.z, fmaf(z.w, z.w, ss))));
    }
  } else {
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
      float z = x_in[src + i];
      if (a != nullptr) z += a[src + i];
      if (b != nullptr) z += b[src + i];
      if (c != nullptr) z += c[src + i];
      zrow[i] = z;
      if (x_out != nullptr) x_out[(size_t)r * D + i] = z;
      ss = fmaf(z, z, ss);
    }
  }
  if (w == nullptr || xb_out == nullptr) return;
  ss = warp_sum(ss);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.f;
  t = warp_sum(t);
  const float rstd = 1.0f / sqrtf(t / (float)D + eps);
  // every thread reads back only what it staged itself: no barrier between the passes beyond the one above
  if (VEC) {
    for (int i = threadIdx.x * 4; i < D; i += blockDim.x * 4) {
      const float4 z = *reinterpret_cast<const float4*>(zrow + i);
      const uint2 wr = *reinterpret_cast<const uint2*>(w + i);
      const float o0 = z.x * rstd * bf16_lo(wr.x), o1 = z.y * rstd * bf16_hi(wr.x);
      const float o2 = z.z * rstd * bf16_lo(wr.y), o3 = z.w * rstd * bf16_hi(wr.y);
      TO* dst = xb_out + (size_t)r * D + i;
      if (sizeof(TO) == 4) {
        *reinterpret_cast<float4*>(dst) = make_float4(o0, o1, o2, o3);
      } else {
        *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(o0, o1), pack_bf16(o2, o3));
      }
    }
  } else {
    for (int i = threadIdx.x; i < D; i += blockDim.x)
      prn_store(xb_out + (size_t)r * D + i, zrow[i] * rstd * __bfloat162float(w[i]));
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_add_rms_norm_f32(const float* x_in, const float* a, const float* b, const float* c,
                                     const int32_t* rows, const void* w, float* x_out, void* xb_out, int xb_f32, int T,
                                     int D, float eps, void* stream) {
  B200_REQUIRE(T >= 0 && D > 0 && x_in != nullptr, "add_rms_norm_f32: bad arguments T=%d D=%d", T, D);
  B200_REQUIRE(rows == nullptr || x_out == nullptr, "add_rms_norm_f32: the gather form writes the normed rows only");
  if (T == 0) return B200_OK;
  const size_t smem = (size_t)D * sizeof(float);
  B200_REQUIRE(smem <= 48 * 1024, "add_rms_norm_f32: D=%d exceeds the staged row (12288)", D);
  cudaStream_t s = (cudaStream_t)stream;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vec = D % 4 == 0 && al(x_in) && al(a) && al(b) && al(c) && al(x_out) && al(xb_out) &&
                   (reinterpret_cast<uintptr_t>(w) & 7) == 0;
#define B200_ARN(TO, V)                                                                                            \
  add_rms_norm_f32_kernel<TO, V><<<T, 256, smem, s>>>(x_in, a, b, c, rows, (const bf16*)w, x_out, (TO*)xb_out, D, eps)
  if (xb_f32) { if (vec) B200_ARN(float, true); else B200_ARN(float, false); }
  else { if (vec) B200_ARN(bf16, true); else B200_ARN(bf16, false); }
#undef B200_ARN
  return b200_check_launch("b200_add_rms_norm_f32");
}
