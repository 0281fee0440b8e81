// out[M, N] = x[M, K] · w[N, K]^T with float32 FMA accumulation: the matrix product of the true
// 32-bit path, and the fallback of the bfloat16 path for shapes its tensor-core kernels refuse.
// (reference src/layers/ops/linear.py:101-122: y = x W^T, float32 accumulator.)
//
// No tensor cores and no reduced-precision mode: each output is a chain of fmaf over k = 0..K-1
// in that order, whatever M is and whichever rows share the tile, so a row's result does not depend
// on what else is in the batch.  Any M, N, K: edges are bounds-checked, loads are scalar.
#include "common.cuh"

#define GG_BM 64
#define GG_BN 64
#define GG_BK 16

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
gemm_generic_kernel(const TIn* __restrict__ x, const TIn* __restrict__ w, TOut* __restrict__ out,
                    int M, int N, int K) {
  __shared__ float xs[GG_BK][GG_BM + 4];
  __shared__ float ws[GG_BK][GG_BN + 4];
  pdl_launch_dependents();
  pdl_wait();
  const int m0 = blockIdx.y * GG_BM, n0 = blockIdx.x * GG_BN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // 16 x 16 threads, 4 x 4 outputs each
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += GG_BK) {
    // 64 rows x 16 k = 1024 elements per operand, 4 per thread; k fastest for coalescing
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = threadIdx.x + i * 256;
      const int r = e >> 4, kk = e & 15;
      const int gk = k0 + kk;
      const int gm = m0 + r, gn = n0 + r;
      xs[kk][r] = (gm < M && gk < K) ? to_f32(x[(size_t)gm * K + gk]) : 0.f;
      ws[kk][r] = (gn < N && gk < K) ? to_f32(w[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GG_BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
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
      if (gn < N) out[(size_t)gm * N + gn] = from_f32<TOut>(acc[i][j]);
    }
  }
}

extern "C" int qe_linear_generic(const void* x, const void* w, void* out, int M, int N, int K,
                                 int dtype, int out_f32, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) QE_REFUSE("linear: K must be positive");
  dim3 grid((N + GG_BN - 1) / GG_BN, (M + GG_BM - 1) / GG_BM);
  if (grid.y > 65535) QE_REFUSE("linear: M %d is too large for the generic kernel", M);
  if (dtype == QE_DTYPE_F32) {
    qe_launch(gemm_generic_kernel<float, float>, grid, dim3(256), 0, stream, (const float*)x, (const float*)w, (float*)out, M, N, K);
  } else if (dtype == QE_DTYPE_BF16) {
    if (out_f32)
      qe_launch(gemm_generic_kernel<__nv_bfloat16, float>, grid, dim3(256), 0, stream,
          (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (float*)out, M, N, K);
    else
      qe_launch(gemm_generic_kernel<__nv_bfloat16, __nv_bfloat16>, grid, dim3(256), 0, stream,
          (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, M, N, K);
  } else QE_REFUSE("linear: unknown dtype %d", dtype);
  QE_CHECK_LAUNCH("linear_generic");
  return 0;
}
