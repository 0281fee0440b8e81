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

// silu(g) * u for a pair of bfloat16 values, in float32, rounded once (the reference's silumul,
// src/layers/fused_ops/silumul.py:50-53, without its intermediate rounding of silu).  The result has
// 8 bits of mantissa, so the fast exponential and division (errors of a few float32 ulps) are used:
// every CTA forms the whole activation again, and the exact routines would cost more than the product.
__device__ __forceinline__ float silu_fast(float g) { return __fdividef(g, 1.f + __expf(-g)); }
__device__ __forceinline__ uint32_t silu_mul_pair(uint32_t g, uint32_t u) {
  const float2 gf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&g));
  const float2 uf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u));
  __nv_bfloat162 r = __floats2bfloat162_rn(silu_fast(gf.x) * uf.x, silu_fast(gf.y) * uf.y);
  return *reinterpret_cast<uint32_t*>(&r);
}

// What the token operand is made of (formed while loading, so that no kernel and no buffer stands
// between the producer of the data and the product):
//   PLAIN  x[M, K] as it is;
//   SILU   x[m, k] = silu(gate_up[m, k]) * gate_up[m, K + k] from gate_up[M, 2K] (the feed-forward's
//          activation fused into its output projection);
//   NORM   x[m, k] = resid[m, k] * rstd[m] * norm_w[k] with rstd[m] = rsqrt(sum_k resid[m, k]^2 / K + eps):
//          the RMS norm of the float32 residual stream fused into the projection that follows it.  The
//          row's sum of squares comes in n_ssq partial sums that the kernel that last wrote the stream
//          left behind (see RESID), so no pass over the row is needed here.
// And what happens to the result:
//   RESID  the product is a branch's output: it is added into the float32 residual stream in place
//          (each element belongs to one thread), and the CTA leaves the sum of squares of its 16
//          columns of every row in ssq_out[m, blockIdx.x] for the norm that follows.
enum { X_PLAIN = 0, X_SILU = 1, X_NORM = 2 };

struct FuseArgs {
  const float* resid;               // NORM: [M, K] float32
  const float* ssq;                 // NORM: [M, ssq_ld] partial sums of squares of the rows
  const float* norm_w;              // NORM: [K]
  float* ssq_out;                   // RESID: [M, ssq_ld]
  int n_ssq, ssq_ld;
  float eps;
};

template <int MT, typename TOut, int XMODE, bool RESID>
__global__ void __launch_bounds__(512)
gemm_small_m_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                    TOut* __restrict__ out, int M, int N, int K, int k_per_warp, FuseArgs na) {
  constexpr bool SILU = XMODE == X_SILU;
  constexpr bool NORM = XMODE == X_NORM;
  extern __shared__ float red[];                    // [warps][16][8 MT]
  __shared__ float s_rstd[8 * MT];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int n0 = blockIdx.x * 16;
  const int r0 = min(n0 + g, N - 1), r1 = min(n0 + g + 8, N - 1);     // clamped; discarded at the store
  const __nv_bfloat16* w0 = w + (size_t)r0 * K;
  const __nv_bfloat16* w1 = w + (size_t)r1 * K;
  const int kbeg = warp * k_per_warp, kend = min(K, kbeg + k_per_warp);
  const int x_ld = SILU ? 2 * K : K;

  float acc[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[t][i] = 0.f;

  const uint4 zero = make_uint4(0, 0, 0, 0);
  // a chunk: 64 k of the 16 rows = four 16-byte loads per lane (K and k_per_warp are multiples of 8)
  struct Chunk { uint4 a0, b0, a1, b1; };
  auto load_chunk = [&](int k0) {
    Chunk ch;
    const int ka = k0 + 8 * c, kb = k0 + 32 + 8 * c;
    ch.a0 = ka < kend ? ld_stream16(w0 + ka) : zero;
    ch.b0 = ka < kend ? ld_stream16(w1 + ka) : zero;
    ch.a1 = kb < kend ? ld_stream16(w0 + kb) : zero;
    ch.b1 = kb < kend ? ld_stream16(w1 + kb) : zero;
    return ch;
  };
  auto load_x = [&](int m, int k) {
    if (m >= M || k >= kend) return zero;
    if (NORM) {
      const size_t o = (size_t)m * K + k;
      float f[8], wv[8];
      *reinterpret_cast<float4*>(f) = __ldcg(reinterpret_cast<const float4*>(na.resid + o));
      *reinterpret_cast<float4*>(f + 4) = __ldcg(reinterpret_cast<const float4*>(na.resid + o + 4));
      *reinterpret_cast<float4*>(wv) = __ldg(reinterpret_cast<const float4*>(na.norm_w + k));
      *reinterpret_cast<float4*>(wv + 4) = __ldg(reinterpret_cast<const float4*>(na.norm_w + k + 4));
      const float rs = s_rstd[m];
      uint4 v;
      __nv_bfloat162* vp = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) vp[i] = __floats2bfloat162_rn(f[2 * i] * rs * wv[2 * i], f[2 * i + 1] * rs * wv[2 * i + 1]);
      return v;
    }
    const __nv_bfloat16* p = x + (size_t)m * x_ld + k;
    uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
    if (SILU) {
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(p + K));
      v.x = silu_mul_pair(v.x, u.x); v.y = silu_mul_pair(v.y, u.y);
      v.z = silu_mul_pair(v.z, u.z); v.w = silu_mul_pair(v.w, u.w);
    }
    return v;
  };
  auto compute = [&](const Chunk& ch, int k0) {
    const int ka = k0 + 8 * c, kb = k0 + 32 + 8 * c;
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      const uint4 xa = load_x(t * 8 + g, ka);
      const uint4 xb = load_x(t * 8 + g, kb);
      mma_bf16_16816(acc[t], ch.a0.x, ch.b0.x, ch.a0.y, ch.b0.y, xa.x, xa.y);
      mma_bf16_16816(acc[t], ch.a0.z, ch.b0.z, ch.a0.w, ch.b0.w, xa.z, xa.w);
      mma_bf16_16816(acc[t], ch.a1.x, ch.b1.x, ch.a1.y, ch.b1.y, xb.x, xb.y);
      mma_bf16_16816(acc[t], ch.a1.z, ch.b1.z, ch.a1.w, ch.b1.w, xb.z, xb.w);
    }
  };
  // The weights are nobody's output: their first two chunks are on their way before this kernel
  // waits for the one before it, whose output x is.
  Chunk c0 = load_chunk(kbeg), c1 = load_chunk(kbeg + 64);
  pdl_launch_dependents();
  pdl_wait();
  float resid_old = 0.f;                            // RESID: this thread's element of the stream, fetched early
  if (RESID) {
    const int m = threadIdx.x >> 4, n = n0 + (threadIdx.x & 15);
    if (threadIdx.x < 16 * 8 * MT && m < M && n < N) resid_old = __ldcg(reinterpret_cast<const float*>(out) + (size_t)m * N + n);
  }
  if (NORM) {
    // the row norms from the partial sums of squares: a warp per row, all loads at once, summed in a
    // fixed order (lane l adds parts l, l + 32, ...; then the lanes are added in a tree)
    for (int m = warp; m < M; m += nwarps) {
      const float* p = na.ssq + (size_t)m * na.ssq_ld;
      float ss = 0.f;
      for (int i = lane; i < na.n_ssq; i += 32) ss += __ldcg(p + i);
      ss = warp_sum(ss);
      if (lane == 0) s_rstd[m] = rsqrtf(ss / (float)K + na.eps);
    }
    __syncthreads();
  }
  for (int k0 = kbeg; k0 < kend; k0 += 128) {
    const Chunk n0c = load_chunk(k0 + 128);
    compute(c0, k0);
    const Chunk n1c = load_chunk(k0 + 192);
    compute(c1, k0 + 64);
    c0 = n0c;
    c1 = n1c;
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
    if (!RESID) {
      if (m >= M || n >= N) continue;
      float s = 0.f;
      for (int wi = 0; wi < nwarps; ++wi) s += red[((size_t)wi * 16 + i) * MW + m];
      out[(size_t)m * N + n] = from_f32<TOut>(s);
    } else {
      // whole warps run this loop (16 MW is a multiple of 32); lanes outside the matrix add zero
      float v = 0.f;
      if (m < M && n < N) {
        float s = 0.f;
        for (int wi = 0; wi < nwarps; ++wi) s += red[((size_t)wi * 16 + i) * MW + m];
        float* dst = reinterpret_cast<float*>(out) + (size_t)m * N + n;
        v = (e == threadIdx.x ? resid_old : *dst) + s;
        *dst = v;
      }
      float sq = v * v;                              // over the 16 columns of the row: lanes i = 0..15
      sq += __shfl_xor_sync(0xffffffffu, sq, 8);
      sq += __shfl_xor_sync(0xffffffffu, sq, 4);
      sq += __shfl_xor_sync(0xffffffffu, sq, 2);
      sq += __shfl_xor_sync(0xffffffffu, sq, 1);
      if (i == 0 && m < M) na.ssq_out[(size_t)m * na.ssq_ld + blockIdx.x] = sq;
    }
  }
}

template <int MT, int XMODE, bool RESID>
static int launch_small_m(const void* x, const void* w, void* out, int M, int N, int K, int out_f32,
                          cudaStream_t stream, FuseArgs na) {
  // warps split K in slices that are multiples of 64; more warps when there are few CTAs
  const int ctas = (N + 15) / 16;
  int warps = ctas >= 2048 ? 4 : (ctas >= 256 ? 8 : 16);
  int k_per_warp = ((K + warps - 1) / warps + 63) / 64 * 64;
  warps = (K + k_per_warp - 1) / k_per_warp;
  const size_t smem = (size_t)warps * 16 * 8 * MT * sizeof(float);
  static bool configured = false;             // once, not per launch: launches may be under stream capture
  if (!configured) {
    const int max_smem = 16 * 16 * 8 * MT * (int)sizeof(float);
    cudaFuncSetAttribute(gemm_small_m_kernel<MT, float, XMODE, RESID>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (!RESID)
      cudaFuncSetAttribute(gemm_small_m_kernel<MT, __nv_bfloat16, XMODE, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    configured = true;
  }
  if (out_f32 || RESID) {
    qe_launch(gemm_small_m_kernel<MT, float, XMODE, RESID>, dim3(ctas), dim3(warps * 32), smem, stream,
              (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (float*)out, M, N, K, k_per_warp, na);
  } else {
    qe_launch(gemm_small_m_kernel<MT, __nv_bfloat16, XMODE, false>, dim3(ctas), dim3(warps * 32), smem, stream,
              (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, M, N, K, k_per_warp, na);
  }
  QE_CHECK_LAUNCH("linear_small_m");
  return 0;
}

template <int XMODE, bool RESID>
static int dispatch_small_m(const void* x, const void* w, void* out, int M, int N, int K, int out_f32,
                            cudaStream_t stream, FuseArgs na = FuseArgs{}) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64) QE_REFUSE("linear_small_m: M = %d is above 64", M);
  if (K <= 0 || K % 8) QE_REFUSE("linear_small_m: K = %d is not a positive multiple of 8", K);
  if (((uintptr_t)x | (uintptr_t)w) & 15) QE_REFUSE("linear_small_m: operands must be 16-byte aligned");
  if (M <= 8) return launch_small_m<1, XMODE, RESID>(x, w, out, M, N, K, out_f32, stream, na);
  if (M <= 16) return launch_small_m<2, XMODE, RESID>(x, w, out, M, N, K, out_f32, stream, na);
  if (M <= 32) return launch_small_m<4, XMODE, RESID>(x, w, out, M, N, K, out_f32, stream, na);
  return launch_small_m<8, XMODE, RESID>(x, w, out, M, N, K, out_f32, stream, na);
}

// Returns 0 when run, 1 when refused (qe_last_error says why), 2 on a launch error.
extern "C" int qe_linear_small_m(const void* x, const void* w, void* out, int M, int N, int K,
                                 int out_f32, cudaStream_t stream) {
  return dispatch_small_m<X_PLAIN, false>(x, w, out, M, N, K, out_f32, stream);
}

// out[M, N] = (silu(gate_up[:, :K]) * gate_up[:, K:]) · w[N, K]^T: the activation of the feed-forward
// formed while its output projection loads it.
extern "C" int qe_linear_small_m_silu(const void* gate_up, const void* w, void* out, int M, int N, int K,
                                      int out_f32, cudaStream_t stream) {
  return dispatch_small_m<X_SILU, false>(gate_up, w, out, M, N, K, out_f32, stream);
}

// resid[M, N] += x · w^T (silu: x formed from gate_up as above), float32 in place, and
// ssq_out[m, j] = sum of squares of resid[m, 16 j .. 16 j + 15] for j < ceil(N / 16).
extern "C" int qe_linear_small_m_resid(const void* x, const void* w, float* resid, float* ssq_out, int ssq_ld,
                                       int M, int N, int K, int silu, cudaStream_t stream) {
  if (!ssq_out || ssq_ld < (N + 15) / 16) QE_REFUSE("linear_small_m_resid: ssq_out must hold %d columns", (N + 15) / 16);
  FuseArgs na{};
  na.ssq_out = ssq_out;
  na.ssq_ld = ssq_ld;
  return silu ? dispatch_small_m<X_SILU, true>(x, w, resid, M, N, K, 1, stream, na)
              : dispatch_small_m<X_PLAIN, true>(x, w, resid, M, N, K, 1, stream, na);
}

// out[M, N] = rmsnorm(resid; norm_w, eps) · w[N, K]^T with the rows' sums of squares given as n_ssq
// partial sums per row in ssq[M, ssq_ld].
extern "C" int qe_linear_small_m_norm(const float* resid, const float* ssq, int n_ssq, int ssq_ld, const float* norm_w,
                                      float eps, const void* w, void* out, int M, int N, int K, int out_f32,
                                      cudaStream_t stream) {
  if (((uintptr_t)resid | (uintptr_t)norm_w) & 15) QE_REFUSE("linear_small_m_norm: operands must be 16-byte aligned");
  if (!ssq || n_ssq < 1 || n_ssq > ssq_ld) QE_REFUSE("linear_small_m_norm: bad partial sums (%d of %d)", n_ssq, ssq_ld);
  FuseArgs na{};
  na.resid = resid; na.ssq = ssq; na.norm_w = norm_w; na.n_ssq = n_ssq; na.ssq_ld = ssq_ld; na.eps = eps;
  return dispatch_small_m<X_NORM, false>(w, w, out, M, N, K, out_f32, stream, na);
}
