// Gated diagonal linear recurrence (a real-gated linear recurrent unit), state in fp32.
//
// Per channel c, with the convolved input u_t (fp32), the gate pre-activations r~_t, i~_t (block-diagonal
// projections of u_t, fp32) and their biases:
//     r = sigmoid(r~ + b_r),  i = sigmoid(i~ + b_i)
//     log a = -gate_c * r * softplus(lam_c),   a = exp(log a)
//     S_t = a S_(t-1) + sqrt(1 - a^2) * i * u_t          (S = 0 before a sequence's first token, also for that token)
//     out_t = S_t * gelu_tanh(y_t + b_y)                 (the second branch, read from the fused projection)
// Everything above is fp32; 1 - a^2 is formed as -expm1(2 log a), which keeps its digits when a is close to one.
// `scan`: one thread per (sequence, channel) walks the sequence's new rows in order (decode steps, short portions);
// `scan_chunked` (below) cuts prompt portions into chunks that run side by side.  The state of slot s is S [slots][W].
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

// ---- prompt portions: the same recurrence without the serial walk over a whole portion.  S_t = a_t S_(t-1) + x_t is
// linear in S, so a portion is cut into chunks of kGrChunk rows:
//   local   every (chunk, channel) forms P = prod a_t and the state L the chunk would reach from zero,
//   carry   every (sequence, channel) walks its chunks: start_c = S, S <- P_c S + L_c; the last S goes to the slot,
//   out     every (chunk, channel) runs its rows again from start_c and writes S_t * gelu(y_t).
// Chunk c of sequence s (rows from a = cu_seq[s] + c * kGrChunk) keeps P / L / start in workspace row a / kGrChunk + s,
// which no other chunk of the step maps to.  Only the grouping of the sums differs from the serial walk.
constexpr int kGrChunk = 64;

struct GrArgs {
  const float* u;
  const float* gates;
  const float* gate_bias;
  const float* lam;
  const void* proj;
  int64_t ld;
  int y_col;
  const float* y_bias;
  const int32_t* cu_seq;
  const int32_t* ctx_lens;
  const int32_t* state_slots;
  float* S_state;
  void* out;
  int64_t ldo;
  int W;
  float gate_c;
  float* ws_p;      // [rows of the workspace][W]
  float* ws_l;
};

__device__ __forceinline__ void gr_coeffs(const GrArgs& g, int t, int c, float sp, float br, float bi, float& a, float& x) {
  const float ut = g.u[(size_t)t * g.W + c];
  const float r = 1.0f / (1.0f + expf(-(g.gates[(size_t)t * 2 * g.W + c] + br)));
  const float i = 1.0f / (1.0f + expf(-(g.gates[(size_t)t * 2 * g.W + g.W + c] + bi)));
  const float la = -sp * r;
  a = expf(la);
  x = sqrtf(-expm1f(2.0f * la)) * i * ut;
}

// grid (n_seqs, chunks of the longest portion, ceil(W / 128)); PASS 0 local, 2 out
template <typename TA, int PASS>
__global__ void __launch_bounds__(128)
gated_recurrence_chunk_kernel(GrArgs g) {
  const int s = blockIdx.x, c = blockIdx.z * blockDim.x + threadIdx.x;
  if (c >= g.W || g.state_slots[s] < 0) return;
  const int t0 = g.cu_seq[s], t1 = g.cu_seq[s + 1];
  const int a0 = t0 + blockIdx.y * kGrChunk;
  if (a0 >= t1) return;
  const int a1 = min(a0 + kGrChunk, t1);
  const size_t wrow = (size_t)(a0 / kGrChunk + s) * g.W + c;
  const float l = g.lam[c];
  const float sp = g.gate_c * (l > 20.f ? l : log1pf(expf(l)));
  const float br = g.gate_bias[c], bi = g.gate_bias[g.W + c];
  if (PASS == 0) {
    float P = 1.f, L = 0.f;
    for (int t = a0; t < a1; ++t) {
      float a, x;
      gr_coeffs(g, t, c, sp, br, bi, a, x);
      P *= a;
      L = fmaf(a, L, x);
    }
    g.ws_p[wrow] = P;
    g.ws_l[wrow] = L;
  } else {
    float S = g.ws_l[wrow];                             // the carry pass left the chunk's start state here
    const float by = g.y_bias[c];
    const TA* proj = reinterpret_cast<const TA*>(g.proj);
    TA* out = reinterpret_cast<TA*>(g.out);
    for (int t = a0; t < a1; ++t) {
      float a, x;
      gr_coeffs(g, t, c, sp, br, bi, a, x);
      S = fmaf(a, S, x);
      gr_store(out + (size_t)t * g.ldo + c, S * gelu_tanh_f(gr_f32(proj[(size_t)t * g.ld + g.y_col + c]) + by));
    }
  }
}

// grid (n_seqs, ceil(W / 128))
__global__ void __launch_bounds__(128)
gated_recurrence_carry_kernel(GrArgs g) {
  const int s = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  const int slot = g.state_slots[s];
  if (c >= g.W || slot < 0) return;
  const int t0 = g.cu_seq[s], t1 = g.cu_seq[s + 1];
  if (t1 <= t0) return;
  float* Sp = g.S_state + (size_t)slot * g.W + c;
  float S = g.ctx_lens[s] == 0 ? 0.f : *Sp;
  for (int a0 = t0; a0 < t1; a0 += kGrChunk) {
    const size_t wrow = (size_t)(a0 / kGrChunk + s) * g.W + c;
    const float P = g.ws_p[wrow], L = g.ws_l[wrow];
    g.ws_l[wrow] = S;
    S = fmaf(P, S, L);
  }
  *Sp = S;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_gated_recurrence_chunk_rows(void) { return kGrChunk; }

// workspace: 2 * (T / chunk + n_seqs + 1) * W floats
extern "C" int b200_gated_recurrence_scan_chunked(const float* u, const float* gates, const float* gate_bias, const float* lam,
                                                  const void* proj, int f32, int64_t ld, int y_col, const float* y_bias,
                                                  const int32_t* cu_seq, const int32_t* ctx_lens, const int32_t* state_slots,
                                                  float* S, void* out, int64_t ldo, int n_seqs, int W, float gate_c, int T,
                                                  int max_len, float* workspace, int64_t workspace_floats, void* stream) {
  B200_REQUIRE(n_seqs >= 0 && W > 0 && T >= 0 && max_len >= 1, "gated_recurrence_scan_chunked: bad shape");
  if (n_seqs == 0 || T == 0) return B200_OK;
  const int64_t rows = (int64_t)T / kGrChunk + n_seqs + 1;
  B200_REQUIRE(workspace != nullptr && workspace_floats >= 2 * rows * W, "gated_recurrence_scan_chunked: workspace of %lld floats, %lld needed",
               (long long)workspace_floats, (long long)(2 * rows * W));
  cudaStream_t s = (cudaStream_t)stream;
  GrArgs g{u, gates, gate_bias, lam, proj, ld, y_col, y_bias, cu_seq, ctx_lens, state_slots, S, out, ldo, W, gate_c, workspace,
           workspace + rows * W};
  dim3 grid(n_seqs, (max_len + kGrChunk - 1) / kGrChunk, (W + 127) / 128);
  gated_recurrence_chunk_kernel<bf16, 0><<<grid, 128, 0, s>>>(g);
  gated_recurrence_carry_kernel<<<dim3(n_seqs, (W + 127) / 128), 128, 0, s>>>(g);
  if (f32) gated_recurrence_chunk_kernel<float, 2><<<grid, 128, 0, s>>>(g);
  else gated_recurrence_chunk_kernel<bf16, 2><<<grid, 128, 0, s>>>(g);
  return b200_check_launch("b200_gated_recurrence_scan_chunked");
}

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
