// f32 matmul for the f32 parity path: C[M,N] = A[M,K] @ B[K,N] (+ bias[N]),
// the math of dotGeneral/matmul (src/rew/ops/linalg.nim:204-252) followed by
// Linear's bias add (src/rew/nn/linear.nim:43-49).  Plain FMA on CUDA cores,
// 64x64 tiles, f32 accumulation in k order within a thread.
#include "common.cuh"
#include "ptx.cuh"

namespace rewb {
namespace {

constexpr int TM = 64, TN = 64, TK = 16;

__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                        const float* __restrict__ bias, float* __restrict__ C,
                                                        int64_t M, int64_t K, int64_t N) {
  __shared__ float As[TK][TM + 1];
  __shared__ float Bs[TK][TN];
  pdl_launch_dependents();
  pdl_wait();
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int64_t m0 = (int64_t)blockIdx.y * TM, n0 = (int64_t)blockIdx.x * TN;
  float acc[4][4] = {};
  for (int64_t k0 = 0; k0 < K; k0 += TK) {
    for (int i = threadIdx.x; i < TM * TK; i += 256) {
      const int r = i / TK, c = i % TK;
      const int64_t gm = m0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? A[gm * K + gk] : 0.f;
    }
    for (int i = threadIdx.x; i < TK * TN; i += 256) {
      const int r = i / TN, c = i % TN;
      const int64_t gk = k0 + r, gn = n0 + c;
      Bs[r][c] = (gk < K && gn < N) ? B[gk * N + gn] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t gn = n0 + tx * 4 + j;
      if (gn < N) C[gm * N + gn] = acc[i][j] + (bias ? bias[gn] : 0.f);
    }
  }
}

}  // namespace

int gemm_f32_launch(Ctx* c, const float* A, const float* B, const float* bias, float* C, int64_t M, int64_t K,
                    int64_t N) {
  if (M == 0 || N == 0) return REWB200_OK;
  dim3 grid((unsigned)((N + TN - 1) / TN), (unsigned)((M + TM - 1) / TM));
  RB_CUDA(launch_k(gemm_f32_kernel, grid, dim3(256), 0, c->stream, c->use_pdl, A, B, bias, C, M, K, N));
  ++g_launch_total;
  return REWB200_OK;
}

}  // namespace rewb
