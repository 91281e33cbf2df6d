// A product per head: out[t, h, :N] = a[t, h, :K] . w[h]^T, with w [H, N, K] and the heads of a row lying
// `a_head_stride` / `out_head_stride` elements apart.  Used where every head has a matrix of its own
// between two small spaces (a query carried into a shared latent space, a latent result carried to the
// head's values).  32-bit accumulation in index order, a 32 x 32 tile of outputs per block.
#include "api.h"
#include "common.cuh"

namespace nib {

template <typename TA, typename TO>
__global__ void __launch_bounds__(256)
linear_heads_kernel(const TA* a, int lda, int a_hs, const TA* __restrict__ w, TO* out, int ldo, int o_hs, int M,
                    int N, int K) {
  pdl_trigger();
  __shared__ float As[32][33];
  __shared__ float Ws[32][33];
  const int tx = threadIdx.x, ty = threadIdx.y;      // 32 x 8
  const int n0 = blockIdx.x * 32, m0 = blockIdx.y * 32, h = blockIdx.z;
  const TA* wh = w + (size_t)h * N * K;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  pdl_wait();
  for (int k0 = 0; k0 < K; k0 += 32) {
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = ty + 8 * i, k = k0 + tx;
      const int m = m0 + r, n = n0 + r;
      As[r][tx] = (m < M && k < K) ? to_float(a[(size_t)m * lda + (size_t)h * a_hs + k]) : 0.0f;
      Ws[r][tx] = (n < N && k < K) ? to_float(wh[(size_t)n * K + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < 32; ++k) {
      const float wv = Ws[tx][k];
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] += As[ty + 8 * i][k] * wv;
    }
  }
  const int n = n0 + tx;
  if (n < N) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int m = m0 + ty + 8 * i;
      if (m < M) out[(size_t)m * ldo + (size_t)h * o_hs + n] = from_float<TO>(acc[i]);
    }
  }
}

}  // namespace nib

using namespace nib;

// a and w share a dtype; out is float32 or that dtype.
extern "C" int nib_linear_heads(int dtype, int out_dtype, const void* a, int lda, int a_head_stride, const void* w,
                                void* out, int ldo, int out_head_stride, int M, int n_head, int N, int K,
                                cudaStream_t stream) {
  if (M <= 0 || n_head <= 0 || N <= 0) return 0;
  if (K <= 0) return NIB_ERR_BAD_ARGUMENT;
  const dim3 grid((N + 31) / 32, (M + 31) / 32, n_head), block(32, 8);
  if (grid.y > 65535 || grid.z > 65535) return NIB_ERR_UNSUPPORTED_SIZE;
  if (dtype == DT_F32 && out_dtype == DT_F32)
    launch_pdl(linear_heads_kernel<float, float>, grid, block, 0, stream, (const float*)a, lda, a_head_stride,
               (const float*)w, (float*)out, ldo, out_head_stride, M, N, K);
  else if (dtype == DT_BF16 && out_dtype == DT_F32)
    launch_pdl(linear_heads_kernel<bf16, float>, grid, block, 0, stream, (const bf16*)a, lda, a_head_stride,
               (const bf16*)w, (float*)out, ldo, out_head_stride, M, N, K);
  else if (dtype == DT_BF16 && out_dtype == DT_BF16)
    launch_pdl(linear_heads_kernel<bf16, bf16>, grid, block, 0, stream, (const bf16*)a, lda, a_head_stride,
               (const bf16*)w, (bf16*)out, ldo, out_head_stride, M, N, K);
  else
    return NIB_ERR_BAD_ARGUMENT;
  NIB_LAUNCH_CHECK();
}
