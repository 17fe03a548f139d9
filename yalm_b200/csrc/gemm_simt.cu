// out[M,N] (+)= A[M,K] * W[N,K]^T with 32-bit FMA on CUDA cores.
//
// This is the matrix product of the true 32-bit path (no tensor cores, hence no
// reduced-precision matrix mode) and the cross-check of the tcgen05 kernel.  Each
// output element is one sequential fused-multiply-add chain over k, so a row's
// result does not depend on which other rows are in the batch.  The reference's
// counterparts are its GEMV kernels (matmul infer.cu:234-248 and the fused
// variants infer.cu:250-337), which also convert each weight to 32 bits and
// accumulate in 32 bits.
#include "api.h"
#include "common.cuh"

namespace yalm {

constexpr int SG_BM = 64, SG_BN = 64, SG_BK = 16;

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TO* __restrict__ out, int M,
                 int N, int K, int accumulate) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float As[SG_BK][SG_BM + 4];
  __shared__ float Ws[SG_BK][SG_BN + 4];
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int m0 = blockIdx.y * SG_BM, n0 = blockIdx.x * SG_BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += SG_BK) {
    // 64x16 elements per operand tile, 4 per thread; consecutive threads read along k
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = threadIdx.x + i * 256;
      const int r = idx / SG_BK, c = idx % SG_BK;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
      As[c][r] = (gm < M && gk < K) ? to_float(A[(size_t)gm * K + gk]) : 0.f;
      Ws[c][r] = (gn < N && gk < K) ? to_float(W[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < SG_BK; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
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
      const size_t o = (size_t)gm * N + gn;
      float v = acc[i][j];
      if (accumulate) v += to_float(out[o]);
      out[o] = from_float<TO>(v);
    }
  }
}

template <typename TA, typename TW>
static int launch_simt(const void* A, const void* W, void* out, int out_dtype, int M, int N, int K,
                       int accumulate, cudaStream_t stream) {
  const dim3 grid((N + SG_BN - 1) / SG_BN, (M + SG_BM - 1) / SG_BM);
  if (grid.y > 65535) return -4;
  if (out_dtype == DT_F32)
    launch_pdl(gemm_simt_kernel<TA, TW, float>, dim3(grid), dim3(256), 0, stream, (const TA*)A, (const TW*)W,
                                                              (float*)out, M, N, K, accumulate);
  else if (out_dtype == DT_BF16)
    launch_pdl(gemm_simt_kernel<TA, TW, __nv_bfloat16>, dim3(grid), dim3(256), 0, stream,
               (const TA*)A, (const TW*)W, (__nv_bfloat16*)out, M, N, K, accumulate);
  else if (out_dtype == DT_F16)
    launch_pdl(gemm_simt_kernel<TA, TW, __half>, dim3(grid), dim3(256), 0, stream, (const TA*)A,
               (const TW*)W, (__half*)out, M, N, K, accumulate);
  else
    return -3;
  YALM_LAUNCH_CHECK();
  return 0;
}

}  // namespace yalm

using namespace yalm;

extern "C" int yalm_gemm_simt(const void* A, int a_dtype, const void* W, int w_dtype, void* out,
                              int out_dtype, int M, int N, int K, int accumulate,
                              cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return -2;
  if (a_dtype == DT_F32 && w_dtype == DT_F32)
    return launch_simt<float, float>(A, W, out, out_dtype, M, N, K, accumulate, stream);
  if (a_dtype == DT_BF16 && w_dtype == DT_BF16)
    return launch_simt<__nv_bfloat16, __nv_bfloat16>(A, W, out, out_dtype, M, N, K, accumulate,
                                                     stream);
  if (a_dtype == DT_F32 && w_dtype == DT_BF16)
    return launch_simt<float, __nv_bfloat16>(A, W, out, out_dtype, M, N, K, accumulate, stream);
  if (a_dtype == DT_BF16 && w_dtype == DT_F32)
    return launch_simt<__nv_bfloat16, float>(A, W, out, out_dtype, M, N, K, accumulate, stream);
  if (a_dtype == DT_F16 && w_dtype == DT_F16)
    return launch_simt<__half, __half>(A, W, out, out_dtype, M, N, K, accumulate, stream);
  if (a_dtype == DT_F32 && w_dtype == DT_F16)
    return launch_simt<float, __half>(A, W, out, out_dtype, M, N, K, accumulate, stream);
  if (a_dtype == DT_F16 && w_dtype == DT_F32)
    return launch_simt<__half, float>(A, W, out, out_dtype, M, N, K, accumulate, stream);
  return -3;
}
