// Linear attention whose state decays at a data-dependent rate per key channel, state in fp32.
//
// Per head, with the decay alpha_t (one number per key channel and token):
//     S_t = diag(alpha_t) S_(t-1) + k_t v_t^T          (S: dk x dv, zero before a sequence's first token)
//     o_t = S_t^T q_t
//     alpha = sigmoid(z)^(1/tau) = exp(logsigmoid(z) / tau),   logsigmoid(z) = min(z, 0) - log1p(exp(-|z|))
// Queries, keys and values arrive as fp32 rows (rot_prep.cu: factors applied), z as fp32 rows [T][H * dk]; alpha is
// formed here, in fp32, when a token's rows are staged.  The state of slot s is S [slots][H][dv][dk] (key index
// fastest).  grid (sequences, heads, ceil(dv / 32)): a CTA owns 32 value columns of one head's state; lane = column,
// each of its 8 warps holds RPW = ceil(dk / 8) neighbouring key rows of those columns in registers.  A token's update
// is then two FMAs per held element with the token's k, q and alpha broadcast from shared memory -- no shuffle; the
// warps' partial sums of S^T q meet in shared memory once per 16 staged tokens and are added in warp order (a fixed
// order, whatever the cut of the prompt).  A sequence's new rows run in order, 16 staged at a time.
#include "common.cuh"
#include "runtime.h"
#include "../../include/b200.h"

namespace b200 {

constexpr int kGlWarps = 8, kGlCols = 32, kGlTok = 16;

__device__ __forceinline__ float gl_alpha(float z, float inv_tau) {
  return expf((fminf(z, 0.f) - log1pf(expf(-fabsf(z)))) * inv_tau);
}

// RPW values from shared memory, the same address for every lane (16-byte loads when RPW allows)
template <int RPW>
__device__ __forceinline__ void gl_rows(const float* __restrict__ p, float (&r)[RPW]) {
  if constexpr (RPW % 4 == 0) {
#pragma unroll
    for (int j = 0; j < RPW; j += 4) {
      const float4 t = *reinterpret_cast<const float4*>(p + j);
      r[j] = t.x; r[j + 1] = t.y; r[j + 2] = t.z; r[j + 3] = t.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < RPW; ++j) r[j] = p[j];
  }
}

template <int RPW>
__global__ void __launch_bounds__(kGlWarps * 32)
gla_scan_kernel(const float* __restrict__ x, int64_t ld, int q_col, int k_col, int v_col, const float* __restrict__ z,
                int64_t ldz, float inv_tau, const int32_t* __restrict__ cu_seq, const int32_t* __restrict__ ctx_lens,
                const int32_t* __restrict__ state_slots, float* S_state, float* __restrict__ o_raw, int H, int dk, int dv) {
  extern __shared__ __align__(16) float smem[];
  constexpr int DKP = RPW * kGlWarps;                 // key rows, padded to the warps' shares
  float* qs = smem;                                   // [16][DKP]
  float* ks = qs + kGlTok * DKP;                      // [16][DKP]
  float* as = ks + kGlTok * DKP;                      // [16][DKP]
  float* vs = as + kGlTok * DKP;                      // [16][32]
  float* red = vs + kGlTok * kGlCols;                 // [8 warps][16][32] partial outputs
  const int s = blockIdx.x, h = blockIdx.y, zc = blockIdx.z;
  const int slot = state_slots[s];
  if (slot < 0) return;
  const int t0 = cu_seq[s], t1 = cu_seq[s + 1];
  if (t1 <= t0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = zc * kGlCols + lane, r0 = warp * RPW;
  float* Sp = S_state + ((size_t)slot * H + h) * dv * dk;
  const bool fresh = ctx_lens[s] == 0;
  float S[RPW];
#pragma unroll
  for (int j = 0; j < RPW; ++j) S[j] = (!fresh && r0 + j < dk && col < dv) ? Sp[(size_t)col * dk + r0 + j] : 0.f;
  // a chunk's rows travel global memory -> registers -> shared memory; the NEXT chunk's loads are issued before this
  // chunk's tokens are walked, so their latency hides behind the walk
  constexpr int PF = (kGlTok * DKP + kGlWarps * 32 - 1) / (kGlWarps * 32), PV = kGlTok * kGlCols / (kGlWarps * 32);
  float pq[PF], pk[PF], pz[PF], pv[PV];
  auto fetch = [&](int ch) {
    const int nt = min(kGlTok, t1 - ch);
#pragma unroll
    for (int e = 0; e < PF; ++e) {
      const int i = threadIdx.x + e * kGlWarps * 32, tt = i / DKP, dd = i - tt * DKP;
      pq[e] = pk[e] = pz[e] = 0.f;
      if (i < nt * DKP && dd < dk) {
        const float* row = x + (size_t)(ch + tt) * ld;
        pq[e] = row[q_col + h * dk + dd];
        pk[e] = row[k_col + h * dk + dd];
        pz[e] = z[(size_t)(ch + tt) * ldz + h * dk + dd];
      }
    }
#pragma unroll
    for (int e = 0; e < PV; ++e) {
      const int i = threadIdx.x + e * kGlWarps * 32, tt = i / kGlCols, cc = zc * kGlCols + (i % kGlCols);
      pv[e] = (i < nt * kGlCols && cc < dv) ? x[(size_t)(ch + tt) * ld + v_col + h * dv + cc] : 0.f;
    }
  };
  fetch(t0);
  for (int ch = t0; ch < t1; ch += kGlTok) {
    const int nt = min(kGlTok, t1 - ch);
    __syncthreads();                                  // every warp is done with the previous chunk
#pragma unroll
    for (int e = 0; e < PF; ++e) {
      const int i = threadIdx.x + e * kGlWarps * 32;
      if (i < kGlTok * DKP) {
        const int dd = i % DKP;
        qs[i] = pq[e]; ks[i] = pk[e];
        as[i] = dd < dk ? gl_alpha(pz[e], inv_tau) : 0.f;   // rows beyond dk: their state stays zero
      }
    }
#pragma unroll
    for (int e = 0; e < PV; ++e) vs[threadIdx.x + e * kGlWarps * 32] = pv[e];
    __syncthreads();
    if (ch + kGlTok < t1) fetch(ch + kGlTok);
    for (int tt = 0; tt < nt; ++tt) {
      const float v = vs[tt * kGlCols + lane];
      float kk[RPW], qq[RPW], aa[RPW];
      gl_rows<RPW>(ks + tt * DKP + r0, kk);
      gl_rows<RPW>(qs + tt * DKP + r0, qq);
      gl_rows<RPW>(as + tt * DKP + r0, aa);
      float num = 0.f;
#pragma unroll
      for (int j = 0; j < RPW; ++j) {
        S[j] = fmaf(aa[j], S[j], kk[j] * v);
        num = fmaf(S[j], qq[j], num);
      }
      red[(warp * kGlTok + tt) * kGlCols + lane] = num;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nt * kGlCols; i += blockDim.x) {
      const int tt = i / kGlCols, c = i % kGlCols;
      float o = 0.f;
#pragma unroll
      for (int w = 0; w < kGlWarps; ++w) o += red[(w * kGlTok + tt) * kGlCols + c];
      if (zc * kGlCols + c < dv) o_raw[(size_t)(ch + tt) * H * dv + h * dv + zc * kGlCols + c] = o;
    }
  }
#pragma unroll
  for (int j = 0; j < RPW; ++j)
    if (r0 + j < dk && col < dv) Sp[(size_t)col * dk + r0 + j] = S[j];
}

// Single rows (a decode step): lane r holds the key rows r, r + 32, ... of its warp's 4 value columns, so the state is read
// and written in whole lines; S^T q is a warp-shuffle reduction, which a step of one token can afford.
constexpr int kGlColsPerWarp = kGlCols / kGlWarps;

template <int EPT>
__global__ void __launch_bounds__(kGlWarps * 32)
gla_step_kernel(const float* __restrict__ x, int64_t ld, int q_col, int k_col, int v_col, const float* __restrict__ z,
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
  return b200_gla_scan_rows(x, ld, q_col, k_col, v_col, z, ldz, inv_tau, cu_seq, ctx_lens, state_slots, S, o_raw, n_seqs, H, dk, dv,
                            0, stream);
}

extern "C" int b200_gla_scan_rows(const float* x, int64_t ld, int q_col, int k_col, int v_col, const float* z, int64_t ldz,
                                  float inv_tau, const int32_t* cu_seq, const int32_t* ctx_lens, const int32_t* state_slots,
                                  float* S, float* o_raw, int n_seqs, int H, int dk, int dv, int max_len, void* stream) {
  B200_REQUIRE(n_seqs >= 0 && H > 0 && dk > 0 && dv > 0 && dk <= 256, "gla_scan: bad shape H=%d dk=%d dv=%d (dk <= 256)", H, dk,
               dv);
  if (n_seqs == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(n_seqs, H, (dv + kGlCols - 1) / kGlCols);
  const size_t smem1 = sizeof(float) * (3 * (size_t)kGlTok * dk + kGlTok * kGlCols);
  if (max_len == 1 && smem1 <= 48 * 1024) {       // no sequence brings more than one row
#define B200_GS(E)                                                                                                      \
  gla_step_kernel<E><<<grid, kGlWarps * 32, smem1, s>>>(x, ld, q_col, k_col, v_col, z, ldz, inv_tau, cu_seq, ctx_lens, \
                                                        state_slots, S, o_raw, H, dk, dv)
    if (dk <= 32) B200_GS(1);
    else if (dk <= 64) B200_GS(2);
    else if (dk <= 128) B200_GS(4);
    else B200_GS(8);
#undef B200_GS
    return b200_check_launch("b200_gla_scan");
  }
  const int rpw = dk <= 8 ? 1 : dk <= 16 ? 2 : dk <= 32 ? 4 : dk <= 64 ? 8 : dk <= 128 ? 16 : 32;   // key rows per warp
  const size_t smem = sizeof(float) * (3 * (size_t)kGlTok * rpw * kGlWarps + kGlTok * kGlCols + kGlWarps * kGlTok * kGlCols);
#define B200_GL(E)                                                                                                     \
  do {                                                                                                                 \
    if (smem > 48 * 1024) {                                                                                            \
      static bool attr = false;                                                                                        \
      if (!attr) {                                                                                                     \
        const cudaError_t e_ = cudaFuncSetAttribute(gla_scan_kernel<E>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                                    (int)smem);                                                        \
        if (e_ != cudaSuccess) {                                                                                       \
          b200_set_error("gla_scan: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e_));                    \
          return B200_ERR_CUDA;                                                                                        \
        }                                                                                                              \
        attr = true;                                                                                                   \
      }                                                                                                                \
    }                                                                                                                  \
    gla_scan_kernel<E><<<grid, kGlWarps * 32, smem, s>>>(x, ld, q_col, k_col, v_col, z, ldz, inv_tau, cu_seq, ctx_lens, \
                                                         state_slots, S, o_raw, H, dk, dv);                            \
  } while (0)
  switch (rpw) {
    case 1: B200_GL(1); break;
    case 2: B200_GL(2); break;
    case 4: B200_GL(4); break;
    case 8: B200_GL(8); break;
    case 16: B200_GL(16); break;
    default: B200_GL(32); break;
  }
#undef B200_GL
  return b200_check_launch("b200_gla_scan");
}
