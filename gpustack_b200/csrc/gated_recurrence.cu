// Gated diagonal linear recurrence (a real-gated linear recurrent unit), state in fp32.
//
// Per channel c, with the convolved input u_t (fp32), the gate pre-activations r~_t, i~_t (block-diagonal
// projections of u_t, fp32) and their biases:
//     r = sigmoid(r~ + b_r),  i = sigmoid(i~ + b_i)
//     log a = -gate_c * r * softplus(lam_c),   a = exp(log a)
//     S_t = a S_(t-1) + sqrt(1 - a^2) * i * u_t          (S = 0 before a sequence's first token, also for that token)
//     out_t = S_t * gelu_tanh(y_t + b_y)                 (the second branch, read from the fused projection)
// Everything above is fp32; 1 - a^2 is formed as -expm1(2 log a), which keeps its digits when a is close to one.
// One thread per (sequence, channel) walks the sequence's new rows in order; the state of slot s is S [slots][W].
// A sequence whose context is empty starts from zero, whatever the slot held before.
#include "common.cuh"
#include "runtime.h"
#include "../../include/b200.h"

namespace b200 {

__device__ __forceinline__ float gr_f32(float v) { return v; }
__device__ __forceinline__ float gr_f32(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void gr_store(float* p, float v) { *p = v; }
__device__ __forceinline__ void gr_store(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// grid (n_seqs, ceil(W / 128))
template <typename TA>
__global__ void __launch_bounds__(128)
gated_recurrence_scan_kernel(const float* __restrict__ u, const float* __restrict__ gates, const float* __restrict__ gate_bias,
                             const float* __restrict__ lam, const TA* __restrict__ proj, int64_t ld, int y_col,
                             const float* __restrict__ y_bias, const int32_t* __restrict__ cu_seq,
                             const int32_t* __restrict__ ctx_lens, const int32_t* __restrict__ state_slots, float* S_state,
                             TA* out, int64_t ldo, int W, float gate_c) {
  const int s = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  const int slot = state_slots[s];
  if (c >= W || slot < 0) return;
  const int t0 = cu_seq[s], t1 = cu_seq[s + 1];
  if (t1 <= t0) return;
  float* Sp = S_state + (size_t)slot * W + c;
  float S = ctx_lens[s] == 0 ? 0.f : *Sp;
  const float l = lam[c];
  const float sp = gate_c * (l > 20.f ? l : log1pf(expf(l)));       // gate_c * softplus(lam)
  const float br = gate_bias[c], bi = gate_bias[W + c], by = y_bias[c];
  for (int t = t0; t < t1; ++t) {
    const float ut = u[(size_t)t * W + c];
    const float r = 1.0f / (1.0f + expf(-(gates[(size_t)t * 2 * W + c] + br)));
    const float i = 1.0f / (1.0f + expf(-(gates[(size_t)t * 2 * W + W + c] + bi)));
    const float la = -sp * r;
    const float a = expf(la);
    S = fmaf(a, S, sqrtf(-expm1f(2.0f * la)) * i * ut);
    const float y = gelu_tanh_f(gr_f32(proj[(size_t)t * ld + y_col + c]) + by);
    gr_store(out + (size_t)t * ldo + c, S * y);
  }
  *Sp = S;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_gated_recurrence_scan(const float* u, const float* gates, const float* gate_bias, const float* lam,
                                          const void* proj, int f32, int64_t ld, int y_col, const float* y_bias,
                                          const int32_t* cu_seq, const int32_t* ctx_lens, const int32_t* state_slots, float* S,
                                          void* out, int64_t ldo, int n_seqs, int W, float gate_c, void* stream) {
  B200_REQUIRE(n_seqs >= 0 && W > 0, "gated_recurrence_scan: bad shape");
  if (n_seqs == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(n_seqs, (W + 127) / 128);
  if (f32)
    gated_recurrence_scan_kernel<float><<<grid, 128, 0, s>>>(u, gates, gate_bias, lam, (const float*)proj, ld, y_col, y_bias,
                                                             cu_seq, ctx_lens, state_slots, S, (float*)out, ldo, W, gate_c);
  else
    gated_recurrence_scan_kernel<bf16><<<grid, 128, 0, s>>>(u, gates, gate_bias, lam, (const bf16*)proj, ld, y_col, y_bias,
                                                            cu_seq, ctx_lens, state_slots, S, (bf16*)out, ldo, W, gate_c);
  return b200_check_launch("b200_gated_recurrence_scan");
}
