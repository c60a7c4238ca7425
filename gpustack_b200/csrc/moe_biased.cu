// Routing with a choice correction and identity experts, and the combine that closes such a layer.
//
//   moe_route_biased:  s = softmax(z) over all E router outputs (fp32 logits); the K outputs with the largest
//                      s + correction are chosen (ties: the lowest index); their weights are
//                      s / (sum of the chosen s + 1e-20) * scale -- the correction steers the choice only.
//   moe_route_scored:  the same with two options: s = sigmoid(z) per output instead of the softmax, and weights that
//                      are the chosen scores as they are (times scale), not renormalised.
//   moe_combine_mixed: out[t] = sum_j ( id_j < n_real ? yp[pair_row[t K + j]] : w_j * x[t] ) (+ shared[t]).
//                      Routed rows arrive already multiplied by their weight (the down projection's row
//                      scale); an identity expert returns the layer input itself times the weight.  fp32 sum in a
//                      fixed order (j = 0 .. K-1, then the shared expert), fp32 output: it enters the residual.
// The pair bookkeeping between the two (moe_align: pairs grouped by expert into whole tiles) is shared with the
// other routed models; identity experts are ordinary ids there, their tiles are skipped by the expert GEMMs.
#include "common.cuh"
#include "runtime.h"
#include "../../include/b200.h"

#include <math_constants.h>

namespace b200 {

constexpr int kRbPerLane = 8;        // E <= 256
constexpr int kRbMaxTop = 16;

__device__ __forceinline__ float rb_f32(float v) { return v; }
__device__ __forceinline__ float rb_f32(bf16 v) { return __bfloat162float(v); }

// one warp per token, lane l holds outputs l, l + 32, ...
__global__ void __launch_bounds__(128)
moe_route_biased_kernel(const float* __restrict__ logits, int64_t ld, const float* __restrict__ correction,
                        int32_t* __restrict__ topk_ids, float* __restrict__ topk_w, int T, int E, int K, float scale,
                        int sigmoid_scores, int renormalize) {
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  float s[kRbPerLane], c[kRbPerLane];
  float mx = -CUDART_INF_F;
#pragma unroll
  for (int i = 0; i < kRbPerLane; ++i) {
    const int e = lane + 32 * i;
    s[i] = e < E ? logits[(size_t)t * ld + e] : -CUDART_INF_F;
    mx = fmaxf(mx, s[i]);
  }
  mx = warp_max(mx);
  if (sigmoid_scores) {
    // every output scored on its own; without a correction the choice is made on the logits themselves (the
    // sigmoid is monotone, and two large logits must not tie where it saturates)
#pragma unroll
    for (int i = 0; i < kRbPerLane; ++i) {
      const int e = lane + 32 * i;
      const float z = s[i];
      s[i] = e < E ? 1.0f / (1.0f + expf(-z)) : 0.f;
      c[i] = e < E ? (correction != nullptr ? s[i] + correction[e] : z) : -CUDART_INF_F;
    }
  } else {
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kRbPerLane; ++i) {
      const int e = lane + 32 * i;
      s[i] = e < E ? expf(s[i] - mx) : 0.f;
      sum += s[i];
    }
    const float inv = 1.0f / warp_sum(sum);
#pragma unroll
    for (int i = 0; i < kRbPerLane; ++i) {
      const int e = lane + 32 * i;
      s[i] *= inv;
      c[i] = e < E ? s[i] + (correction != nullptr ? correction[e] : 0.f) : -CUDART_INF_F;
    }
  }
  float wsum = 0.f, mine_w = 0.f;
  int mine_id = 0;
  for (int j = 0; j < K; ++j) {
    float bv = -CUDART_INF_F, bs = 0.f;
    int be = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kRbPerLane; ++i) {
      const int e = lane + 32 * i;
      if (e < E && c[i] > bv) { bv = c[i]; be = e; bs = s[i]; }       // ascending e: the lowest index wins a tie
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o), os = __shfl_xor_sync(0xffffffffu, bs, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; bs = os; }
    }
    if (be >= E) { be = j; bs = 0.f; }                                 // logits that are not numbers: still a valid id
#pragma unroll
    for (int i = 0; i < kRbPerLane; ++i)
      if (lane + 32 * i == be) c[i] = -CUDART_INF_F;                   // taken
    wsum += bs;
    if (lane == j) { mine_id = be; mine_w = bs; }
  }
  if (lane < K) {
    topk_ids[(size_t)t * K + lane] = mine_id;
    topk_w[(size_t)t * K + lane] = (renormalize ? mine_w / (wsum + 1e-20f) : mine_w) * scale;
  }
}

template <typename TX, typename TP>
__global__ void __launch_bounds__(256)
moe_combine_mixed_kernel(const TP* __restrict__ yp, int64_t ldp, const int32_t* __restrict__ pair_row,
                         const int32_t* __restrict__ topk_ids, const float* __restrict__ topk_w,
                         const TX* __restrict__ x, int64_t ldx, const TP* __restrict__ shared, int64_t lds,
                         float* __restrict__ out, int64_t ldo, int T, int D, int K, int n_real) {
  const size_t total = (size_t)T * D;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(i / D), d = (int)(i % D);
    float acc = 0.f;
    for (int j = 0; j < K; ++j) {
      const int id = topk_ids[(size_t)t * K + j];
      if (id < n_real) acc += rb_f32(yp[(size_t)pair_row[(size_t)t * K + j] * ldp + d]);
      else acc += topk_w[(size_t)t * K + j] * rb_f32(x[(size_t)t * ldx + d]);
    }
    if (shared != nullptr) acc += rb_f32(shared[(size_t)t * lds + d]);
    out[(size_t)t * ldo + d] = acc;
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_moe_route_scored(const float* logits, int64_t ld, const float* correction, int32_t* topk_ids,
                                     float* topk_w, int T, int E, int K, float scale, int sigmoid_scores,
                                     int renormalize, void* stream) {
  B200_REQUIRE(ld >= E, "moe_route_biased: row stride %lld < E=%d", (long long)ld, E);
  B200_REQUIRE(T >= 0 && E >= 1 && E <= 32 * kRbPerLane && K >= 1 && K <= kRbMaxTop && K <= E,
               "moe_route_biased: unsupported E=%d K=%d (E <= %d, K <= %d)", E, K, 32 * kRbPerLane, kRbMaxTop);
  if (T == 0) return B200_OK;
  moe_route_biased_kernel<<<(T + 3) / 4, 128, 0, (cudaStream_t)stream>>>(logits, ld, correction, topk_ids, topk_w, T, E, K,
                                                                       scale, sigmoid_scores, renormalize);
  return b200_check_launch("b200_moe_route_biased");
}

extern "C" int b200_moe_route_biased(const float* logits, int64_t ld, const float* correction, int32_t* topk_ids,
                                     float* topk_w, int T, int E, int K, float scale, void* stream) {
  return b200_moe_route_scored(logits, ld, correction, topk_ids, topk_w, T, E, K, scale, 0, 1, stream);
}

extern "C" int b200_moe_combine_mixed(const void* yp, int p_f32, int64_t ldp, const int32_t* pair_row,
                                      const int32_t* topk_ids, const float* topk_w, const void* x, int x_f32, int64_t ldx,
                                      const void* shared, int64_t lds, float* out, int64_t ldo, int T, int D, int K,
                                      int n_real, void* stream) {
  B200_REQUIRE(T >= 0 && D > 0 && K >= 1, "moe_combine_mixed: bad shape");
  if (T == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  size_t blocks = ((size_t)T * D + 255) / 256;
  if (blocks > 8192) blocks = 8192;
#define B200_CM(TX, TP)                                                                                             \
  moe_combine_mixed_kernel<TX, TP><<<(int)blocks, 256, 0, s>>>((const TP*)yp, ldp, pair_row, topk_ids, topk_w,     \
                                                               (const TX*)x, ldx, (const TP*)shared, lds, out, ldo, T, D, \
                                                               K, n_real)
  if (x_f32 && p_f32) B200_CM(float, float);
  else if (x_f32) B200_CM(float, bf16);
  else if (p_f32) B200_CM(bf16, float);
  else B200_CM(bf16, bf16);
#undef B200_CM
  return b200_check_launch("b200_moe_combine_mixed");
}
