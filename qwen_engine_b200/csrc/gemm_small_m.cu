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
#include "gemm_small_m.cuh"

template <int MT, typename TOut, int XMODE, bool RESID, int ROWS = 16>
__global__ void __launch_bounds__(512)
gemm_small_m_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                    TOut* __restrict__ out, int M, int N, int K, int k_per_warp, FuseArgs na) {
  extern __shared__ float red[];                    // [warps][16][8 MT]
  __shared__ float s_rstd[8 * MT];
  // The weights are nobody's output: their first two chunks are on their way before this kernel
  // waits for the one before it, whose output the token operand is.
  GsmChunk c0, c1;
  gsm_prefetch<ROWS>(w, N, K, k_per_warp, blockIdx.x, c0, c1);
  if (gridDim.x <= 1024) {
    // (a grid that is resident all at once, waiting for the kernel before it: a layer's product, not
    // the vocabulary's) and L2 is asked for the rest of this CTA's rows (one contiguous block), in
    // pieces of 8 KB
    const int rows = min(ROWS, N - (int)blockIdx.x * ROWS);
    const unsigned bytes = (unsigned)rows * (unsigned)K * 2u;
    const unsigned off = threadIdx.x * 8192u;
    if (off < bytes) {
      const unsigned size = min(8192u, bytes - off);
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n"
                   :: "l"(reinterpret_cast<const unsigned char*>(w + (size_t)blockIdx.x * ROWS * K) + off), "r"(size) : "memory");
    }
  }
  if (na.next_bytes) {
    // pieces of 4 KB of the later kernel's weights, dealt to the CTAs and their threads in turn
    const unsigned long long pieces = (na.next_bytes + 4095) >> 12;
    const unsigned long long piece = (unsigned long long)threadIdx.x * gridDim.x + blockIdx.x;
    if (piece < pieces) {
      const unsigned long long off = piece << 12;
      const unsigned size = (unsigned)min(4096ull, na.next_bytes - off) & ~15u;
      if (size) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" :: "l"(na.next_w + off), "r"(size) : "memory");
    }
  }
  pdl_launch_dependents();
  pdl_wait();
  gsm_cta<MT, TOut, XMODE, RESID, false, false, ROWS>(x, w, out, M, N, K, k_per_warp, na, blockIdx.x, red, s_rstd, c0, c1);
}

// The same product by clusters of S CTAs that share 16 weight rows, a share of K each (see gsm_cta, CLUSTER): for weight
// matrices of so few rows that one CTA per 16 of them would leave most SMs without work.
template <int MT, typename TOut, int XMODE, bool RESID, bool PUSH>
__global__ void __launch_bounds__(512)
gemm_small_m_cluster_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                            TOut* __restrict__ out, int M, int N, int K, int k_per_warp, int k_per_cta, FuseArgs na) {
  extern __shared__ float red[];                    // [warps][16][8 MT], then this CTA's sums [16][8 MT] (pushed: and the other CTAs')
  __shared__ float s_rstd[8 * MT];
  __shared__ uint64_t push_bar;
  if (PUSH) {
    if (threadIdx.x == 0) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" :: "r"((uint32_t)__cvta_generic_to_shared(&push_bar)), "r"(1u));
      asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  }
  const int S = (int)cluster_num_ctas();
  const int vb = (int)blockIdx.x / S;
  const int k_off = (int)cluster_cta_rank() * k_per_cta;
  GsmChunk c0, c1;
  gsm_prefetch(w, N, K, k_per_warp, vb, c0, c1, k_off, k_per_cta);
  if (na.next_bytes) {
    const unsigned long long pieces = (na.next_bytes + 4095) >> 12;
    const unsigned long long piece = (unsigned long long)threadIdx.x * gridDim.x + blockIdx.x;
    if (piece < pieces) {
      const unsigned long long off = piece << 12;
      const unsigned size = (unsigned)min(4096ull, na.next_bytes - off) & ~15u;
      if (size) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" :: "l"(na.next_w + off), "r"(size) : "memory");
    }
  }
  pdl_launch_dependents();
  pdl_wait();
  gsm_cta<MT, TOut, XMODE, RESID, true, PUSH>(x, w, out, M, N, K, k_per_warp, na, vb, red, s_rstd, c0, c1, k_off, k_per_cta,
                                              PUSH ? &push_bar : nullptr);
}

// How many CTAs share 16 weight rows: 1 where the rows alone give (nearly) every SM a CTA, else 2 or 4 while every CTA
// still has 512 or more of K.  A function of the weight matrix alone, never of the number of rows of the step, so that
// the order of a row's sums does not depend on the batch.
static int g_small_m_max_cluster = 4;
// The most CTAs that may share 16 weight rows (1: never share; for measurements and tests).
extern "C" void qe_small_m_max_cluster(int ctas) { g_small_m_max_cluster = ctas < 1 ? 1 : (ctas > 4 ? 4 : ctas); }
// Whether the CTAs of a cluster push their sums to the first (1: where it was measured to gain; 2: always; 0: never:
// that one reads them).  The sums are added in the CTAs' order either way, so the result is the same to the bit.
// Measured on a B200 (0.6B sizes, a decode step, pushed against pulled): one row 0.725 against 0.746 ms, two rows 0.812
// against 0.800, four 0.842 against 0.836, eight 0.954 against 0.945: pushed for a single row only.
static int g_small_m_push = 1;
extern "C" void qe_small_m_push(int mode) { g_small_m_push = mode < 0 ? 0 : (mode > 2 ? 2 : mode); }
extern "C" int qe_small_m_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_gsm_status, sizeof(int));
  return v;
}
extern "C" void qe_small_m_clear_status() {
  int v = 0;
  cudaMemcpyToSymbol(g_gsm_status, &v, sizeof(int));
}
static int small_m_cluster_size(int N, int K) {
  const int ctas = (N + 15) / 16;
  if (g_small_m_max_cluster >= 4 && ctas * 4 <= 148 && K >= 4 * 512) return 4;
  if (g_small_m_max_cluster >= 2 && ctas * 2 <= 148 && K >= 2 * 512) return 2;
  return 1;
}

template <int MT, int XMODE, bool RESID>
static int launch_small_m_cluster(const void* x, const void* w, void* out, int M, int N, int K, int out_f32, int S,
                                  cudaStream_t stream, FuseArgs na) {
  const int ctas = (N + 15) / 16;
  const int k_per_cta = ((K + S - 1) / S + 63) / 64 * 64;
  int warps = 16;
  int k_per_warp = ((k_per_cta + warps - 1) / warps + 63) / 64 * 64;
  warps = (k_per_cta + k_per_warp - 1) / k_per_warp;
  const bool push = g_small_m_push == 2 || (g_small_m_push == 1 && M == 1);
  const size_t smem = (size_t)(warps + (push ? S : 1)) * 16 * 8 * MT * sizeof(float);
  static bool configured = false;
  if (!configured) {
    const int max_smem = 20 * 16 * 8 * MT * (int)sizeof(float);
    cudaFuncSetAttribute(gemm_small_m_cluster_kernel<MT, float, XMODE, RESID, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    cudaFuncSetAttribute(gemm_small_m_cluster_kernel<MT, float, XMODE, RESID, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (!RESID) {
      cudaFuncSetAttribute(gemm_small_m_cluster_kernel<MT, __nv_bfloat16, XMODE, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
      cudaFuncSetAttribute(gemm_small_m_cluster_kernel<MT, __nv_bfloat16, XMODE, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    }
    configured = true;
  }
  const dim3 grid(ctas * S), block(warps * 32);
  const __nv_bfloat16* xb = (const __nv_bfloat16*)x;
  const __nv_bfloat16* wb = (const __nv_bfloat16*)w;
  if (out_f32 || RESID) {
    if (push) qe_launch_cluster(gemm_small_m_cluster_kernel<MT, float, XMODE, RESID, true>, grid, block, smem, stream, (unsigned)S, xb, wb, (float*)out, M, N, K, k_per_warp, k_per_cta, na);
    else qe_launch_cluster(gemm_small_m_cluster_kernel<MT, float, XMODE, RESID, false>, grid, block, smem, stream, (unsigned)S, xb, wb, (float*)out, M, N, K, k_per_warp, k_per_cta, na);
  } else {
    if (push) qe_launch_cluster(gemm_small_m_cluster_kernel<MT, __nv_bfloat16, XMODE, false, true>, grid, block, smem, stream, (unsigned)S, xb, wb, (__nv_bfloat16*)out, M, N, K, k_per_warp, k_per_cta, na);
    else qe_launch_cluster(gemm_small_m_cluster_kernel<MT, __nv_bfloat16, XMODE, false, false>, grid, block, smem, stream, (unsigned)S, xb, wb, (__nv_bfloat16*)out, M, N, K, k_per_warp, k_per_cta, na);
  }
  QE_CHECK_LAUNCH("linear_small_m");
  return 0;
}

// Matrices of so few rows that 16 per CTA leave half of the SMs idle, and 8 per CTA fill them: 8 rows a CTA and the
// whole of K, instead of clusters of two that share 16 rows and meet (the meeting costs more than the loop over K).
static int g_small_m_rows8 = 0;                    // (off: see ops.SMALL_M_ROWS8)
extern "C" void qe_small_m_rows8(int on) { g_small_m_rows8 = on != 0; }
extern "C" int qe_small_m_tile_cols(int N, int K) {
  return g_small_m_rows8 && small_m_cluster_size(N, K) == 2 && (N + 7) / 8 <= 148 ? 8 : 16;
}

template <int MT, int XMODE, bool RESID>
static int launch_small_m_rows8(const void* x, const void* w, void* out, int M, int N, int K, int out_f32,
                                cudaStream_t stream, FuseArgs na) {
  const int ctas = (N + 7) / 8;
  int warps = 16;
  int k_per_warp = ((K + warps - 1) / warps + 127) / 128 * 128;
  warps = (K + k_per_warp - 1) / k_per_warp;
  const size_t smem = (size_t)warps * 16 * 8 * MT * sizeof(float);
  static bool configured = false;
  if (!configured) {
    const int max_smem = 16 * 16 * 8 * MT * (int)sizeof(float);
    cudaFuncSetAttribute(gemm_small_m_kernel<MT, float, XMODE, RESID, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (!RESID)
      cudaFuncSetAttribute(gemm_small_m_kernel<MT, __nv_bfloat16, XMODE, false, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    configured = true;
  }
  if (out_f32 || RESID) {
    qe_launch(gemm_small_m_kernel<MT, float, XMODE, RESID, 8>, dim3(ctas), dim3(warps * 32), smem, stream,
              (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (float*)out, M, N, K, k_per_warp, na);
  } else {
    qe_launch(gemm_small_m_kernel<MT, __nv_bfloat16, XMODE, false, 8>, dim3(ctas), dim3(warps * 32), smem, stream,
              (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, M, N, K, k_per_warp, na);
  }
  QE_CHECK_LAUNCH("linear_small_m");
  return 0;
}

template <int MT, int XMODE, bool RESID>
static int launch_small_m(const void* x, const void* w, void* out, int M, int N, int K, int out_f32,
                          cudaStream_t stream, FuseArgs na) {
  if (XMODE != X_NORM) {
    if (qe_small_m_tile_cols(N, K) == 8) return launch_small_m_rows8<MT, XMODE, RESID>(x, w, out, M, N, K, out_f32, stream, na);
    const int S = small_m_cluster_size(N, K);
    if (S > 1) return launch_small_m_cluster<MT, XMODE == X_NORM ? X_PLAIN : XMODE, RESID>(x, w, out, M, N, K, out_f32, S, stream, na);
  }
  // warps split K in slices that are multiples of 64; more warps when there are few CTAs
  const int ctas = (N + 15) / 16;
  int warps = ctas >= 2048 ? 4 : (ctas > 148 ? 8 : 16);     // (more CTAs than SMs: 8 warps, so that two CTAs fit an SM and all start at once)
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

// The weights that the next product launched from this thread asks L2 for (see FuseArgs::next_w); one launch
// takes them and clears them.  16-byte aligned; bytes 0 clears.
static thread_local const unsigned char* g_next_w = nullptr;
static thread_local unsigned long long g_next_bytes = 0;
extern "C" int qe_small_m_prefetch_next(const void* w, unsigned long long bytes) {
  if (((uintptr_t)w & 15) != 0) QE_REFUSE("small_m_prefetch_next: the weights must be 16-byte aligned");
  g_next_w = (const unsigned char*)w;
  g_next_bytes = w ? bytes : 0;
  return 0;
}

template <int XMODE, bool RESID>
static int dispatch_small_m(const void* x, const void* w, void* out, int M, int N, int K, int out_f32,
                            cudaStream_t stream, FuseArgs na = FuseArgs{}) {
  na.next_w = g_next_w;
  na.next_bytes = g_next_bytes;
  g_next_w = nullptr;
  g_next_bytes = 0;
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
  const int ssq_cols = (N + qe_small_m_tile_cols(N, K) - 1) / qe_small_m_tile_cols(N, K);
  if (!ssq_out || ssq_ld < ssq_cols) QE_REFUSE("linear_small_m_resid: ssq_out must hold %d columns", ssq_cols);
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

// ---- gate and up projections with the activation in their epilogue -----------------------------------------------
template <int MT>
__global__ void __launch_bounds__(512)
gemm_small_m_swiglu_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                           __nv_bfloat16* __restrict__ act, int M, int I, int K, int k_per_warp, FuseArgs na) {
  extern __shared__ float red[];                    // 2 x [warps][16][8 MT]
  if (na.next_bytes) {
    const unsigned long long pieces = (na.next_bytes + 4095) >> 12;
    const unsigned long long piece = (unsigned long long)threadIdx.x * gridDim.x + blockIdx.x;
    if (piece < pieces) {
      const unsigned long long off = piece << 12;
      const unsigned size = (unsigned)min(4096ull, na.next_bytes - off) & ~15u;
      if (size) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" :: "l"(na.next_w + off), "r"(size) : "memory");
    }
  }
  pdl_launch_dependents();
  gsm_cta_swiglu<MT>(x, w, act, M, I, K, k_per_warp, blockIdx.x, red);     // (waits for the kernel before it once its first weights are on their way)
}

// act[M, I] = silu(x · w[:I]^T) * (x · w[I:]^T) for the stacked weights w [2 I, K], M <= 16 rows, bfloat16: a CTA
// takes the gate rows and the up rows of the same 16 columns, so the activation never exists as gate and up in memory.
extern "C" int qe_linear_small_m_swiglu(const void* x, const void* w, void* act, int M, int I, int K, cudaStream_t stream) {
  FuseArgs na{};
  na.next_w = g_next_w;
  na.next_bytes = g_next_bytes;
  g_next_w = nullptr;
  g_next_bytes = 0;
  if (M <= 0 || I <= 0) return 0;
  if (M > 16) QE_REFUSE("linear_small_m_swiglu: M = %d is above 16", M);
  if (K <= 0 || K % 8) QE_REFUSE("linear_small_m_swiglu: K = %d is not a positive multiple of 8", K);
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)act) & 15) QE_REFUSE("linear_small_m_swiglu: operands must be 16-byte aligned");
  const int ctas = (I + 15) / 16;
  // As many warps a CTA as still let all CTAs start at once (two CTAs of 8 warps fit an SM, four of 4): 384 CTAs took
  // 13.8 us with 8 warps, in two rounds, and 12.1 with 4.  Beyond one round, 8 warps until the CTAs are many.
  int warps = ctas < 128 ? 16 : ctas <= 296 ? 8 : ctas <= 592 ? 4 : ctas < 1024 ? 8 : 4;
  int k_per_warp = ((K + warps - 1) / warps + 31) / 32 * 32;
  warps = (K + k_per_warp - 1) / k_per_warp;
  const int MT = M <= 8 ? 1 : 2;
  const size_t smem = (size_t)2 * warps * 16 * 8 * MT * sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(gemm_small_m_swiglu_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * 16 * 16 * 8 * 4);
    cudaFuncSetAttribute(gemm_small_m_swiglu_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * 16 * 16 * 16 * 4);
    configured = true;
  }
  if (MT == 1)
    qe_launch(gemm_small_m_swiglu_kernel<1>, dim3(ctas), dim3(warps * 32), smem, stream, (const __nv_bfloat16*)x,
              (const __nv_bfloat16*)w, (__nv_bfloat16*)act, M, I, K, k_per_warp, na);
  else
    qe_launch(gemm_small_m_swiglu_kernel<2>, dim3(ctas), dim3(warps * 32), smem, stream, (const __nv_bfloat16*)x,
              (const __nv_bfloat16*)w, (__nv_bfloat16*)act, M, I, K, k_per_warp, na);
  QE_CHECK_LAUNCH("linear_small_m_swiglu");
  return 0;
}


// ---- the QKV product with per-head norm, rotation and cache write in its epilogue (see gsm_cta_qkv_rope) ---------
template <int MT>
__global__ void __cluster_dims__(8, 1, 1) __launch_bounds__(512)
gemm_small_m_qkv_rope_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                             __nv_bfloat16* __restrict__ qkv, int M, int N, int K, int k_per_warp, GsmRope rp, FuseArgs na) {
  extern __shared__ float red[];                    // [warps][16][8 MT]
  __shared__ float s_val[16 * 8 * MT];              // this CTA's 16 columns of every row, read by the CTA four ranks away
  __shared__ float s_ssq[8 * MT];                   // their sums of squares, read by all CTAs of the head
  if (na.next_bytes) {
    const unsigned long long pieces = (na.next_bytes + 4095) >> 12;
    const unsigned long long piece = (unsigned long long)threadIdx.x * gridDim.x + blockIdx.x;
    if (piece < pieces) {
      const unsigned long long off = piece << 12;
      const unsigned size = (unsigned)min(4096ull, na.next_bytes - off) & ~15u;
      if (size) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" :: "l"(na.next_w + off), "r"(size) : "memory");
    }
  }
  pdl_launch_dependents();
  gsm_cta_qkv_rope<MT>(x, w, qkv, M, N, K, k_per_warp, rp, blockIdx.x, red, s_val, s_ssq);   // (waits for the kernel before it once its first weights are on their way)
}

// qkv[M, :Hq 128] = the q columns of x · w^T for the stacked q, k, v weights w [N = (Hq + 2 Hkv) 128, K], normed per
// head and rotated; the k (normed, rotated) and v columns go into the cache `pages` [pages, 2, Hkv, page_size, 128] at
// slot_mapping[row] (write_kv 0: they are dropped) and qkv's k and v columns are left as they were.  M <= 16 rows,
// bfloat16.  qw, kw: float32 [128] or null; the angles: cos_sin float32 [M, 64, 2] if given, else position *
// inv_freq[64] (both null: no rotation).  Returns 0 when run, 1 when refused, 2 on a launch error.
extern "C" int qe_linear_small_m_qkv_rope(const void* x, const void* w, void* qkv, int M, int N, int K,
                                          const float* qw, const float* kw, float eps, const int* positions,
                                          const float* inv_freq, const void* cos_sin, void* pages, const int* slot_mapping,
                                          int Hq, int Hkv, int page_size, int write_kv, cudaStream_t stream) {
  FuseArgs na{};
  na.next_w = g_next_w;
  na.next_bytes = g_next_bytes;
  g_next_w = nullptr;
  g_next_bytes = 0;
  if (M <= 0 || N <= 0) return 0;
  if (M > 16) QE_REFUSE("linear_small_m_qkv_rope: M = %d is above 16", M);
  if (K <= 0 || K % 8) QE_REFUSE("linear_small_m_qkv_rope: K = %d is not a positive multiple of 8", K);
  if (Hq < 1 || Hkv < 1 || N != (Hq + 2 * Hkv) * 128) QE_REFUSE("linear_small_m_qkv_rope: N = %d is not (%d + 2 x %d) heads of 128", N, Hq, Hkv);
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)qkv) & 15) QE_REFUSE("linear_small_m_qkv_rope: operands must be 16-byte aligned");
  if (inv_freq && !cos_sin && !positions) QE_REFUSE("linear_small_m_qkv_rope: angles need the positions");
  if (write_kv && (!pages || !slot_mapping || page_size < 1)) QE_REFUSE("linear_small_m_qkv_rope: cache write without a cache");
  const int ctas = N / 16;                           // 8 per head: the clusters
  int warps = ctas >= 1024 ? 4 : (ctas >= 256 ? 8 : 16);
  int k_per_warp = ((K + warps - 1) / warps + 63) / 64 * 64;
  warps = (K + k_per_warp - 1) / k_per_warp;
  const int MT = M <= 8 ? 1 : 2;
  if (warps < 4 * MT) warps = 4 * MT;                // a thread per element of the CTA's 16 columns (a short K leaves some warps without a slice)
  const size_t smem = (size_t)warps * 16 * 8 * MT * sizeof(float);
  GsmRope rp{qw, kw, eps, positions, inv_freq, (const float2*)cos_sin, (__nv_bfloat16*)pages, slot_mapping, Hq, Hkv, page_size, write_kv ? 1 : 0};
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(gemm_small_m_qkv_rope_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 16 * 16 * 8 * 4);
    cudaFuncSetAttribute(gemm_small_m_qkv_rope_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 16 * 16 * 16 * 4);
    configured = true;
  }
  if (MT == 1)
    qe_launch(gemm_small_m_qkv_rope_kernel<1>, dim3(ctas), dim3(warps * 32), smem, stream, (const __nv_bfloat16*)x,
              (const __nv_bfloat16*)w, (__nv_bfloat16*)qkv, M, N, K, k_per_warp, rp, na);
  else
    qe_launch(gemm_small_m_qkv_rope_kernel<2>, dim3(ctas), dim3(warps * 32), smem, stream, (const __nv_bfloat16*)x,
              (const __nv_bfloat16*)w, (__nv_bfloat16*)qkv, M, N, K, k_per_warp, rp, na);
  QE_CHECK_LAUNCH("linear_small_m_qkv_rope");
  return 0;
}
