// f32 SIMT GEMM with arbitrary element strides and a batch dimension.  It serves the f32 parity
// path (the reference's default precision) where bit-level closeness to the CPU arms matters more
// than speed: matmul / matmul_trans_b and their gradients, and the batched Q K^T / P V products of
// the materialised attention chain with their four gradient products
// (kernels/ops_f32.cu:158-259, 342-511, 842-882).  bf16 work goes to the tcgen05 kernel instead.
//
//   C[b, m, n] (+)= sum_k A[b*a_bs + m*a_ms + k*a_ks] * B[b*b_bs + k*b_ks + n*b_ns]
#include "common.cuh"
#include "errors.h"
#include "../../include/eisen_b200.h"

namespace eisen {
namespace {

constexpr int TM = 64, TN = 64, TK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int M, int N,
                int K, long long a_bs, long long a_ms, long long a_ks, long long b_bs, long long b_ks,
                long long b_ns, long long c_bs, long long ldc, int accumulate) {
  __shared__ float As[TK][TM + 1];
  __shared__ float Bs[TK][TN + 1];
  const int bz = blockIdx.z;
  A += bz * a_bs;
  B += bz * b_bs;
  C += bz * c_bs;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < K; k0 += TK) {
    // 64x16 tiles, 1024 elements each, 4 per thread
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      const int e = threadIdx.x + l * 256;
      {
        // pick the index order that walks the contiguous dimension of A fastest
        int mm, kk;
        if (a_ks == 1) { kk = e % TK; mm = e / TK; } else { mm = e % TM; kk = e / TM; }
        const int gm = m0 + mm, gk = k0 + kk;
        As[kk][mm] = (gm < M && gk < K) ? A[gm * a_ms + gk * a_ks] : 0.0f;
      }
      {
        int nn, kk;
        if (b_ks == 1) { kk = e % TK; nn = e / TK; } else { nn = e % TN; kk = e / TN; }
        const int gn = n0 + nn, gk = k0 + kk;
        Bs[kk][nn] = (gn < N && gk < K) ? B[gk * b_ks + gn * b_ns] : 0.0f;
      }
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
        for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * b[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float* c = C + gm * ldc + gn;
      *c = accumulate ? *c + acc[i][j] : acc[i][j];
    }
  }
}

}  // namespace
}  // namespace eisen

using namespace eisen;

extern "C" int eisen_gemm_f32_strided(void* stream, const float* A, const float* B, float* C, long long batch,
                                      long long M, long long N, long long K, long long a_bs, long long a_ms,
                                      long long a_ks, long long b_bs, long long b_ks, long long b_ns,
                                      long long c_bs, long long ldc, int accumulate) {
  if (batch <= 0 || M <= 0 || N <= 0) return 0;
  if (batch > 65535) return fail(EISEN_ERR_LIMIT, "gemm_f32_strided: batch > 65535");
  dim3 grid((unsigned)((N + TN - 1) / TN), (unsigned)((M + TM - 1) / TM), (unsigned)batch);
  gemm_f32_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(A, B, C, (int)M, (int)N, (int)K, a_bs, a_ms, a_ks, b_bs,
                                                         b_ks, b_ns, c_bs, ldc, accumulate);
  return check_launch("gemm_f32_strided");
}
