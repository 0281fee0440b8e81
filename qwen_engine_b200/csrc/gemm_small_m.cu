// out[M, N] = x[M, K] · w[N, K]^T for a few rows (M <= 64) in bfloat16: the matrix products of a
// decode step, where every weight is read once and nothing else matters.  (Same contract as the
// reference's linear, src/layers/ops/linear.py:101-122: float32 accumulation, result rounded once.)
//
// The weight rows ride the M dimension of mma.sync.m16n8k16 (16 weight rows per warp) and the
// tokens its N dimension (8 tokens per instruction, up to 8 instructions wide), so a 16-byte load
// of a weight row feeds the tensor core directly: lane (g, c) loads 8 consecutive k of row g and
// of row g + 8 and uses them as the k-slots {2c, 2c+1, 2c+8, 2c+9} of two instructions; the token
// operand is loaded with the same permutation of k, which a dot product does not see.
//
// One CTA owns 16 weight rows; its warps split K between them (so that enough loads are in
// flight to keep HBM busy even when N / 16 is small) and add their parts in shared memory in a
// fixed order.  Any N; K a multiple of 8 (16-byte rows); the launcher refuses the rest.
#include "common.cuh"

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream16(const void* p) {   // read once: do not keep in L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

template <int MT, typename TOut>
__global__ void __launch_bounds__(512)
gemm_small_m_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                    TOut* __restrict__ out, int M, int N, int K, int k_per_warp) {
  extern __shared__ float red[];                    // [warps][16][8 MT]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int n0 = blockIdx.x * 16;
  const int r0 = min(n0 + g, N - 1), r1 = min(n0 + g + 8, N - 1);     // clamped; discarded at the store
  const __nv_bfloat16* w0 = w + (size_t)r0 * K;
  const __nv_bfloat16* w1 = w + (size_t)r1 * K;
  const int kbeg = warp * k_per_warp, kend = min(K, kbeg + k_per_warp);

  float acc[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[t][i] = 0.f;

  const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll 2
  for (int k0 = kbeg; k0 < kend; k0 += 64) {
    const int ka = k0 + 8 * c, kb = k0 + 32 + 8 * c;
    const bool ina = ka < kend, inb = kb < kend;      // K and k_per_warp are multiples of 8
    const uint4 wa0 = ina ? ld_stream16(w0 + ka) : zero;
    const uint4 wb0 = ina ? ld_stream16(w1 + ka) : zero;
    const uint4 wa1 = inb ? ld_stream16(w0 + kb) : zero;
    const uint4 wb1 = inb ? ld_stream16(w1 + kb) : zero;
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      const int m = t * 8 + g;
      const __nv_bfloat16* xr = x + (size_t)m * K;
      const uint4 xa = (m < M && ina) ? __ldg(reinterpret_cast<const uint4*>(xr + ka)) : zero;
      const uint4 xb = (m < M && inb) ? __ldg(reinterpret_cast<const uint4*>(xr + kb)) : zero;
      mma_bf16_16816(acc[t], wa0.x, wb0.x, wa0.y, wb0.y, xa.x, xa.y);
      mma_bf16_16816(acc[t], wa0.z, wb0.z, wa0.w, wb0.w, xa.z, xa.w);
      mma_bf16_16816(acc[t], wa1.x, wb1.x, wa1.y, wb1.y, xb.x, xb.y);
      mma_bf16_16816(acc[t], wa1.z, wb1.z, wa1.w, wb1.w, xb.z, xb.w);
    }
  }
  // acc[t][0..1]: weight row g, tokens 8t + 2c + {0,1};  acc[t][2..3]: weight row g + 8
  constexpr int MW = 8 * MT;
  float* mine = red + (size_t)warp * 16 * MW;
#pragma unroll
  for (int t = 0; t < MT; ++t) {
    mine[g * MW + t * 8 + 2 * c] = acc[t][0];
    mine[g * MW + t * 8 + 2 * c + 1] = acc[t][1];
    mine[(g + 8) * MW + t * 8 + 2 * c] = acc[t][2];
    mine[(g + 8) * MW + t * 8 + 2 * c + 1] = acc[t][3];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < 16 * MW; e += blockDim.x) {
    const int m = e >> 4, i = e & 15;               // consecutive threads: consecutive weight rows
    const int n = n0 + i;
    if (m >= M || n >= N) continue;
    float s = 0.f;
    for (int wi = 0; wi < nwarps; ++wi) s += red[((size_t)wi * 16 + i) * MW + m];
    out[(size_t)m * N + n] = from_f32<TOut>(s);
  }
}

template <int MT>
static int launch_small_m(const void* x, const void* w, void* out, int M, int N, int K, int out_f32,
                          cudaStream_t stream) {
  // warps split K in slices that are multiples of 64; more warps when there are few CTAs
  const int ctas = (N + 15) / 16;
  int warps = ctas >= 2048 ? 4 : (ctas >= 256 ? 8 : 16);
  int k_per_warp = ((K + warps - 1) / warps + 63) / 64 * 64;
  warps = (K + k_per_warp - 1) / k_per_warp;
  const size_t smem = (size_t)warps * 16 * 8 * MT * sizeof(float);
  static bool configured = false;             // once, not per launch: launches may be under stream capture
  if (!configured) {
    const int max_smem = 16 * 16 * 8 * MT * (int)sizeof(float);
    cudaFuncSetAttribute(gemm_small_m_kernel<MT, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    cudaFuncSetAttribute(gemm_small_m_kernel<MT, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    configured = true;
  }
  if (out_f32) {
    gemm_small_m_kernel<MT, float><<<ctas, warps * 32, smem, stream>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (float*)out, M, N, K, k_per_warp);
  } else {
    gemm_small_m_kernel<MT, __nv_bfloat16><<<ctas, warps * 32, smem, stream>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, M, N, K, k_per_warp);
  }
  QE_CHECK_LAUNCH("linear_small_m");
  return 0;
}

// Returns 0 when run, 1 when refused (qe_last_error says why), 2 on a launch error.
extern "C" int qe_linear_small_m(const void* x, const void* w, void* out, int M, int N, int K,
                                 int out_f32, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64) QE_REFUSE("linear_small_m: M = %d is above 64", M);
  if (K <= 0 || K % 8) QE_REFUSE("linear_small_m: K = %d is not a positive multiple of 8", K);
  if (((uintptr_t)x | (uintptr_t)w) & 15) QE_REFUSE("linear_small_m: operands must be 16-byte aligned");
  if (M <= 8) return launch_small_m<1>(x, w, out, M, N, K, out_f32, stream);
  if (M <= 16) return launch_small_m<2>(x, w, out, M, N, K, out_f32, stream);
  if (M <= 32) return launch_small_m<4>(x, w, out, M, N, K, out_f32, stream);
  return launch_small_m<8>(x, w, out, M, N, K, out_f32, stream);
}
