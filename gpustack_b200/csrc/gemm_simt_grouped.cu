// Batched, grouped and gated linear layers on the CUDA cores: fp32 FMA accumulation in a fixed order over K,
// x bf16 or fp32, W bf16, y bf16 or fp32, no shape or alignment rule.  One kernel, four uses:
//   * batched:  grid.z problems with element strides between them (one small matrix per attention head:
//               the absorbed query  W_uk[h]^T q_h  and the value expansion  W_uv[h] o_h  of latent attention);
//   * grouped:  the rows are a permuted (token, expert) space in which every expert owns whole 64-row tiles
//               (tile_expert[], num_tiles[] from moe_align with block_x = 64); a tile multiplies by its expert's
//               matrix, tiles of experts >= n_real (identity experts) and unused tiles are skipped; the input
//               rows may be gathered through row_pair (row -> pair -> token = pair / top_k, -1 = padding) and
//               the output rows multiplied by row_scale (the routing weight) -- or, scale_in, the INPUT rows: the
//               accumulators are multiplied before the activation, which is the product of the scaled row;
//   * gated:    W holds interleaved rows (2n = gate_n, 2n + 1 = up_n), both products are accumulated and the
//               output is  act(g) * u'  computed in fp32 from the fp32 accumulators, rounded once:
//                 act 1  gelu_tanh(g) * u        gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
//                 act 2  g' sigmoid(1.702 g') (u' + 1),  g' = min(g, limit), u' = clamp(u, -limit, limit)
//                 act 3  silu(g) * u
//   * any combination (a routed gated expert layer is grouped + gated + gathered).
// A result element never depends on M, on the row's place in the batch or on the other rows of its tile.
#include "common.cuh"
#include "runtime.h"
#include "../../include/b200.h"

namespace b200 {

constexpr int kGsBM = 64, kGsBN = 64, kGsBK = 16;

__device__ __forceinline__ float gs_f32(float v) { return v; }
__device__ __forceinline__ float gs_f32(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void gs_out(float* p, float v) { *p = v; }
__device__ __forceinline__ void gs_out(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float gated_act(float g, float u, int act, float limit) {
  if (act == 1) {
    const float z = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    return 0.5f * g * (1.0f + tanhf(z)) * u;
  }
  if (act == 2) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
  }
  return g / (1.0f + expf(-g)) * u;
}

struct GsArgs {
  const void* X;
  const bf16* W;
  void* Y;
  int M, N, K;                       // N = output columns (gated: N gate/up pairs, W has 2N rows per matrix)
  int64_t ldx, ldw, ldy;
  int64_t bsx, bsw, bsy;             // element strides between the grid.z problems
  const int32_t* row_pair;           // NULL: row r reads input row r
  int top_k;
  const int32_t* tile_expert;        // NULL: one matrix
  const int32_t* num_tiles;
  int n_real;
  int64_t w_expert;                  // elements between the experts' matrices
  const float* row_scale;            // NULL: none
  int act;                           // 0 = plain linear
  float limit;
  int scale_in;                      // 1: row_scale multiplies the row's INPUT (the accumulators before the activation)
};

template <typename TX, typename TY, bool GATED>
__global__ void __launch_bounds__(256)
gemm_simt_grouped_kernel(GsArgs a) {
  __shared__ float Xs[kGsBK][kGsBM + 4];
  __shared__ float Ws[kGsBK][kGsBN + 4];
  __shared__ float Us[GATED ? kGsBK : 1][kGsBN + 4];
  __shared__ int src_row[kGsBM];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * kGsBM, n0 = blockIdx.x * kGsBN;
  const bf16* W = a.W + (size_t)blockIdx.z * a.bsw;
  if (a.tile_expert != nullptr) {
    if ((int)blockIdx.y >= a.num_tiles[0]) return;
    const int e = a.tile_expert[blockIdx.y];
    if (e >= a.n_real) return;
    W += (size_t)e * a.w_expert;
  }
  const TX* X = reinterpret_cast<const TX*>(a.X) + (size_t)blockIdx.z * a.bsx;
  TY* Y = reinterpret_cast<TY*>(a.Y) + (size_t)blockIdx.z * a.bsy;
  const int M = a.M, N = a.N, K = a.K;
  if (tid < kGsBM) {
    int r = m0 + tid;
    if (r >= M) r = -1;
    else if (a.row_pair != nullptr) {
      const int p = a.row_pair[r];
      r = p >= 0 ? p / a.top_k : -1;
    }
    src_row[tid] = r;
  }
  __syncthreads();
  float acc[4][4], accu[GATED ? 4 : 1][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc[i][j] = 0.f;
      if (GATED) accu[i][j] = 0.f;
    }
  const int lk = tid & 15, lr = tid >> 4;
  for (int k0 = 0; k0 < K; k0 += kGsBK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = lr + 16 * i;
      const int k = k0 + lk;
      float xv = 0.f, wv = 0.f, uv = 0.f;
      if (k < K) {
        const int sr = src_row[r];
        if (sr >= 0) xv = gs_f32(X[(int64_t)sr * a.ldx + k]);
        if (n0 + r < N) {
          if (GATED) {
            wv = __bfloat162float(W[(int64_t)(2 * (n0 + r)) * a.ldw + k]);
            uv = __bfloat162float(W[(int64_t)(2 * (n0 + r) + 1) * a.ldw + k]);
          } else {
            wv = __bfloat162float(W[(int64_t)(n0 + r) * a.ldw + k]);
          }
        }
      }
      Xs[lk][r] = xv;
      Ws[lk][r] = wv;
      if (GATED) Us[lk][r] = uv;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kGsBK; ++kk) {
      float x[4], w[4], u[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) x[i] = Xs[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        w[j] = Ws[kk][tx * 4 + j];
        if (GATED) u[j] = Us[kk][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(x[i], w[j], acc[i][j]);
          if (GATED) accu[i][j] = fmaf(x[i], u[j], accu[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
    const float rs = a.row_scale != nullptr ? a.row_scale[m] : 1.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (a.scale_in) {              // W (rs x) = rs (W x): the product is linear in the row
        v *= rs;
        if (GATED) v = gated_act(v, accu[i][j] * rs, a.act, a.limit);
      } else {
        if (GATED) v = gated_act(v, accu[i][j], a.act, a.limit);
        v *= rs;
      }
      gs_out(Y + (int64_t)m * a.ldy + n, v);
    }
  }
}

template <typename TX, typename TY>
static int launch_gs(const GsArgs& a, int batch, cudaStream_t s) {
  dim3 grid((a.N + kGsBN - 1) / kGsBN, (a.M + kGsBM - 1) / kGsBM, batch);
  if (a.act) gemm_simt_grouped_kernel<TX, TY, true><<<grid, 256, 0, s>>>(a);
  else gemm_simt_grouped_kernel<TX, TY, false><<<grid, 256, 0, s>>>(a);
  return b200_check_launch("b200_linear_simt_grouped");
}

}  // namespace b200

using namespace b200;

extern "C" int b200_linear_simt_grouped_ex(const void* X, int x_f32, const void* W, void* Y, int y_f32, int M, int N, int K,
                                           int64_t ldx, int64_t ldw, int64_t ldy, int batch, int64_t bsx, int64_t bsw,
                                           int64_t bsy, const int32_t* row_pair, int top_k, const int32_t* tile_expert,
                                           const int32_t* num_tiles, int n_real, int64_t w_expert, const float* row_scale,
                                           int act, float limit, int scale_in, void* stream) {
  B200_REQUIRE(M >= 0 && N > 0 && K > 0 && batch >= 1, "linear_simt_grouped: bad shape M=%d N=%d K=%d batch=%d", M, N, K, batch);
  B200_REQUIRE(ldx >= K && ldw >= K && ldy >= N, "linear_simt_grouped: leading dimensions too small");
  B200_REQUIRE(act >= 0 && act <= 3, "linear_simt_grouped: unknown activation %d", act);
  B200_REQUIRE(tile_expert == nullptr || (num_tiles != nullptr && M % kGsBM == 0), "linear_simt_grouped: grouped rows come in tiles of %d", kGsBM);
  B200_REQUIRE(row_pair == nullptr || top_k >= 1, "linear_simt_grouped: top_k");
  if (M == 0) return B200_OK;
  GsArgs a{X, (const bf16*)W, Y, M, N, K, ldx, ldw, ldy, bsx, bsw, bsy, row_pair, top_k, tile_expert, num_tiles, n_real,
           w_expert, row_scale, act, limit, (scale_in && row_scale != nullptr) ? 1 : 0};
  cudaStream_t s = (cudaStream_t)stream;
  if (x_f32 && y_f32) return launch_gs<float, float>(a, batch, s);
  if (x_f32) return launch_gs<float, bf16>(a, batch, s);
  if (y_f32) return launch_gs<bf16, float>(a, batch, s);
  return launch_gs<bf16, bf16>(a, batch, s);
}

extern "C" int b200_linear_simt_grouped(const void* X, int x_f32, const void* W, void* Y, int y_f32, int M, int N, int K,
                                        int64_t ldx, int64_t ldw, int64_t ldy, int batch, int64_t bsx, int64_t bsw,
                                        int64_t bsy, const int32_t* row_pair, int top_k, const int32_t* tile_expert,
                                        const int32_t* num_tiles, int n_real, int64_t w_expert, const float* row_scale,
                                        int act, float limit, void* stream) {
  return b200_linear_simt_grouped_ex(X, x_f32, W, Y, y_f32, M, N, K, ldx, ldw, ldy, batch, bsx, bsw, bsy, row_pair, top_k,
                                     tile_expert, num_tiles, n_real, w_expert, row_scale, act, limit, 0, stream);
}

extern "C" int b200_simt_group_rows(void) { return kGsBM; }
