// Linear attention whose state decays at a data-dependent rate per key channel, state in fp32.
//
// Per head, with the decay alpha_t (one number per key channel and token):
//     S_t = diag(alpha_t) S_(t-1) + k_t v_t^T          (S: dk x dv, zero before a sequence's first token)
//     o_t = S_t^T q_t
//     alpha = sigmoid(z)^(1/tau) = exp(logsigmoid(z) / tau),   logsigmoid(z) = min(z, 0) - log1p(exp(-|z|))
// Queries, keys and values arrive as fp32 rows (rot_prep.cu: factors applied), z as fp32 rows [T][H * dk]; alpha is
// formed here, in fp32, when a token's rows are staged.  The state of slot s is S [slots][H][dv][dk] (key index
// fastest).  grid (sequences, heads, ceil(dv / 32)): a CTA owns 32 value columns of one head's state, each of its 8
// warps 4 of them; lane r holds the key rows r, r + 32, ... of those columns in registers; S^T q is a warp-shuffle
// reduction.  A sequence's new rows run in order, 16 staged at a time.
#include "common.cuh"
#include "runtime.h"
#include "../../include/b200.h"

namespace b200 {

constexpr int kGlWarps = 8, kGlColsPerWarp = 4, kGlCols = kGlWarps * kGlColsPerWarp, kGlTok = 16;

__device__ __forceinline__ float gl_alpha(float z, float inv_tau) {
  return expf((fminf(z, 0.f) - log1pf(expf(-fabsf(z)))) * inv_tau);
}

template <int EPT>
__global__ void __launch_bounds__(kGlWarps * 32)
gla_scan_kernel(const float* __restrict__ x, int64_t ld, int q_col, int k_col, int v_col, const float* __restrict__ z,
                int64_t ldz, float inv_tau, const int32_t* __restrict__ cu_seq, const int32_t* __restrict__ ctx_lens,
                const int32_t* __restrict__ state_slots, float* S_state, float* __restrict__ o_raw, int H, int dk, int dv) {
  extern __shared__ float smem[];
  float* qs = smem;                                   // [16][dk]
  float* ks = qs + kGlTok * dk;                       // [16][dk]
  float* as = ks + kGlTok * dk;                       // [16][dk]
  float* vs = as + kGlTok * dk;                       // [16][32]
  const int s = blockIdx.x, h = blockIdx.y, zc = blockIdx.z;
  const int slot = state_slots[s];
  if (slot < 0) return;
  const int t0 = cu_seq[s], t1 = cu_seq[s + 1];
  if (t1 <= t0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c0 = zc * kGlCols + warp * kGlColsPerWarp;
  float* Sp = S_state + ((size_t)slot * H + h) * dv * dk;
  const bool fresh = ctx_lens[s] == 0;
  float S[EPT][kGlColsPerWarp];
#pragma unroll
  for (int j = 0; j < EPT; ++j) {
    const int row = lane + 32 * j;
#pragma unroll
    for (int c = 0; c < kGlColsPerWarp; ++c)
      S[j][c] = (!fresh && row < dk && c0 + c < dv) ? Sp[(size_t)(c0 + c) * dk + row] : 0.f;
  }
  for (int ch = t0; ch < t1; ch += kGlTok) {
    const int nt = min(kGlTok, t1 - ch);
    __syncthreads();                                  // every warp is done with the previous chunk
    for (int i = threadIdx.x; i < nt * dk; i += blockDim.x) {
      const int tt = i / dk, dd = i - tt * dk;
      const float* row = x + (size_t)(ch + tt) * ld;
      qs[i] = row[q_col + h * dk + dd];
      ks[i] = row[k_col + h * dk + dd];
      as[i] = gl_alpha(z[(size_t)(ch + tt) * ldz + h * dk + dd], inv_tau);
    }
    for (int i = threadIdx.x; i < nt * kGlCols; i += blockDim.x) {
      const int tt = i / kGlCols, c = zc * kGlCols + (i % kGlCols);
      vs[i] = c < dv ? x[(size_t)(ch + tt) * ld + v_col + h * dv + c] : 0.f;
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      float v[kGlColsPerWarp], num[kGlColsPerWarp];
#pragma unroll
      for (int c = 0; c < kGlColsPerWarp; ++c) {
        v[c] = vs[tt * kGlCols + warp * kGlColsPerWarp + c];
        num[c] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < EPT; ++j) {
        const int row = lane + 32 * j;
        if (row < dk) {
          const float kk = ks[tt * dk + row], qq = qs[tt * dk + row], aa = as[tt * dk + row];
#pragma unroll
          for (int c = 0; c < kGlColsPerWarp; ++c) {
            S[j][c] = fmaf(aa, S[j][c], kk * v[c]);
            num[c] = fmaf(S[j][c], qq, num[c]);
          }
        }
      }
#pragma unroll
      for (int c = 0; c < kGlColsPerWarp; ++c) num[c] = warp_sum(num[c]);
      if (lane < kGlColsPerWarp && c0 + lane < dv) {
        float mine = num[0];
#pragma unroll
        for (int c = 1; c < kGlColsPerWarp; ++c) mine = lane == c ? num[c] : mine;
        o_raw[(size_t)(ch + tt) * H * dv + h * dv + c0 + lane] = mine;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < EPT; ++j) {
    const int row = lane + 32 * j;
#pragma unroll
    for (int c = 0; c < kGlColsPerWarp; ++c)
      if (row < dk && c0 + c < dv) Sp[(size_t)(c0 + c) * dk + row] = S[j][c];
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_gla_scan(const float* x, int64_t ld, int q_col, int k_col, int v_col, const float* z, int64_t ldz,
                             float inv_tau, const int32_t* cu_seq, const int32_t* ctx_lens, const int32_t* state_slots,
                             float* S, float* o_raw, int n_seqs, int H, int dk, int dv, void* stream) {
  B200_REQUIRE(n_seqs >= 0 && H > 0 && dk > 0 && dv > 0 && dk <= 256, "gla_scan: bad shape H=%d dk=%d dv=%d (dk <= 256)", H, dk,
               dv);
  if (n_seqs == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(n_seqs, H, (dv + kGlCols - 1) / kGlCols);
  const size_t smem = sizeof(float) * (3 * (size_t)kGlTok * dk + kGlTok * kGlCols);
#define B200_GL(E)                                                                                                     \
  gla_scan_kernel<E><<<grid, kGlWarps * 32, smem, s>>>(x, ld, q_col, k_col, v_col, z, ldz, inv_tau, cu_seq, ctx_lens, \
                                                       state_slots, S, o_raw, H, dk, dv)
  if (dk <= 32) B200_GL(1);
  else if (dk <= 64) B200_GL(2);
  else if (dk <= 128) B200_GL(4);
  else B200_GL(8);
#undef B200_GL
  return b200_check_launch("b200_gla_scan");
}
