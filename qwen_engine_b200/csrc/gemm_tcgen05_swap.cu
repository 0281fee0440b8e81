// out[M, N] = x[M, K] · w[N, K]^T in bfloat16 for a moderate number of rows (17..256: decode steps of
// many requests, short prompt portions) and many weight rows: the weights take the 128-row side of
// tcgen05.mma and the tokens its narrow side (N of the instruction = M rounded up to 16), so that a
// CTA streams 128 weight rows once through a deep TMA ring while the small token operand rides along.
// (Same contract as the reference's linear, src/layers/ops/linear.py:101-122.)  The kernel for a few
// rows (gemm_small_m.cu) re-reads the token operand for every 16 weight rows and is bound by that
// from some 16 rows on; the kernel for many rows (gemm_tcgen05.cu) pads the tokens to 128.
//
// One CTA per 128 weight rows, 6 warps: warp 0 feeds TMA, warp 1 owns tensor memory and issues the
// MMAs, warps 2-5 read the accumulator (lane = weight row, column = token) and store it transposed:
// for one token, a warp's 32 lanes write 32 consecutive outputs.  Every wait on an mbarrier is
// bounded, as in gemm_tcgen05.cu; qe_gemm_tc_swap_status() reads this kernel's flag.
//
// Needs K % 8 == 0 and 16-byte aligned bases (TMA strides); the launcher refuses the rest.
#include "tcgen05.cuh"

#define SW_BM 128               // weight rows per CTA
#define SW_BK 64
#define SW_THREADS 192

static __device__ int g_tc_status = 0;      // 0 = fine; else code of the first wait that ran out

template <int BT, int STAGES>    // BT: tokens at most (rows of the token operand's box)
struct __align__(1024) SwSmem {
  __nv_bfloat16 w[STAGES][SW_BM * SW_BK];       // 16 KB each
  __nv_bfloat16 x[STAGES][BT * SW_BK];
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

template <typename TOut, int BT, int STAGES>
__global__ void __launch_bounds__(SW_THREADS, 1)
gemm_tcgen05_swap_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                         TOut* __restrict__ out, int M, int N, int K) {
  extern __shared__ unsigned char smem_raw[];
  using Smem = SwSmem<BT, STAGES>;
  constexpr uint32_t TMEM_COLS = BT < 32 ? 32 : BT;
  pdl_launch_dependents();
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * SW_BM;
  const int num_kb = (K + SW_BK - 1) / SW_BK;
  const int mt = (M + 15) / 16 * 16;                  // tokens as the instruction sees them
  volatile int* abort_flag = &sm.abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
    mbar_init(&sm.acc_full, 1);
    sm.abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) tc_alloc(&sm.tmem_base, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;

  if (warp == 0) {
    // ---- producer: the weights are nobody's output, so the ring is filled before the wait for the
    // kernel that produces x; the token operand of those k-blocks follows after the wait ----------
    if (lane == 0) {
      const int ahead = min(num_kb, STAGES);
      for (int kb = 0; kb < ahead; ++kb) {
        mbar_expect_tx(&sm.full[kb], (SW_BM + BT) * SW_BK * sizeof(__nv_bfloat16));
        tma_load_2d(sm.w[kb], &map_w, &sm.full[kb], kb * SW_BK, n0);
      }
      pdl_wait();
      for (int kb = 0; kb < ahead; ++kb) tma_load_2d(sm.x[kb], &map_x, &sm.full[kb], kb * SW_BK, 0);
      int issued = ahead;
      for (int kb = ahead; kb < num_kb; ++kb) {
        const int s = kb % STAGES;
        if (!mbar_wait(&sm.empty[s], ((kb / STAGES) - 1) & 1, abort_flag, 11, &g_tc_status)) break;
        mbar_expect_tx(&sm.full[s], (SW_BM + BT) * SW_BK * sizeof(__nv_bfloat16));
        tma_load_2d(sm.w[s], &map_w, &sm.full[s], kb * SW_BK, n0);
        tma_load_2d(sm.x[s], &map_x, &sm.full[s], kb * SW_BK, 0);
        ++issued;
      }
      if (*abort_flag) {
        for (int i = max(0, issued - STAGES); i < issued; ++i)
          for (uint32_t spin = 0; spin < TC_WAIT_LIMIT; ++spin)
            if (mbar_try_wait(&sm.full[i % STAGES], (i / STAGES) & 1)) break;
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer -------------------------------------------------------------------------------
    if (lane == 0) {
      const uint32_t idesc = make_idesc(SW_BM, mt);
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % STAGES;
        ok = mbar_wait(&sm.full[s], (kb / STAGES) & 1, abort_flag, 12, &g_tc_status);
        if (!ok) break;
        tc_fence_after();
        const uint64_t da = make_smem_desc(smem_u32(sm.w[s]));
        const uint64_t db = make_smem_desc(smem_u32(sm.x[s]));
#pragma unroll
        for (int k = 0; k < SW_BK / 16; ++k) tc_mma_bf16(tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
        tc_commit(&sm.empty[s]);
      }
      if (ok) tc_commit(&sm.acc_full);
    }
  } else {
    // ---- epilogue: lane = weight row, columns = tokens ---------------------------------------------
    const int quarter = warp & 3;
    const bool ok = __all_sync(0xffffffffu, mbar_wait(&sm.acc_full, 0, abort_flag, 13, &g_tc_status));
    tc_fence_after();
    const int n = n0 + quarter * 32 + lane;
    if (ok) {
#pragma unroll 1
      for (int c0 = 0; c0 < mt; c0 += 16) {
        uint32_t r[16];
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(tmem + ((uint32_t)(quarter * 32) << 16) + c0) : "memory");
        tc_wait_ld();
        if (n < N) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (c0 + j < M) out[(size_t)(c0 + j) * N + n] = from_f32<TOut>(__uint_as_float(r[j]));
        }
      }
    }
  }
  // every thread waits for the previous kernel before the CTA ends (a kernel of this library never
  // completes before its predecessor)
  pdl_wait();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tc_dealloc(tmem, TMEM_COLS);
  }
}

template <int BT, int STAGES>
static int launch_swap(const void* x, const void* w, void* out, int M, int N, int K, int out_f32, cudaStream_t stream) {
  CUtensorMap map_w, map_x;
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    const uint64_t strides[1] = {(uint64_t)K * 2};
    const uint32_t box[2] = {SW_BK, SW_BM};
    if (!qe_tensor_map_bf16(w, 2, dims, strides, box, &map_w)) return 1;
  }
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    const uint64_t strides[1] = {(uint64_t)K * 2};
    const uint32_t box[2] = {SW_BK, (uint32_t)BT};
    if (!qe_tensor_map_bf16(x, 2, dims, strides, box, &map_x)) return 1;
  }
  const size_t smem = sizeof(SwSmem<BT, STAGES>) + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_swap_kernel<__nv_bfloat16, BT, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tcgen05_swap_kernel<float, BT, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) QE_REFUSE("linear_tcgen05_swap: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  const dim3 grid((unsigned)((N + SW_BM - 1) / SW_BM));
  if (out_f32)
    qe_launch(gemm_tcgen05_swap_kernel<float, BT, STAGES>, grid, dim3(SW_THREADS), smem, stream, map_w, map_x, (float*)out, M, N, K);
  else
    qe_launch(gemm_tcgen05_swap_kernel<__nv_bfloat16, BT, STAGES>, grid, dim3(SW_THREADS), smem, stream, map_w, map_x, (__nv_bfloat16*)out, M, N, K);
  QE_CHECK_LAUNCH("linear_tcgen05_swap");
  return 0;
}

extern "C" int qe_gemm_tc_swap_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int));
  return v;
}
extern "C" void qe_gemm_tc_swap_clear_status() {
  int v = 0;
  cudaMemcpyToSymbol(g_tc_status, &v, sizeof(int));
}

// 1 <= M <= 256.  Returns 0 when run, 1 when refused (qe_last_error says why), 2 on a launch error.
extern "C" int qe_linear_tcgen05_swap(const void* x, const void* w, void* out, int M, int N, int K, int out_f32,
                                      cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 256) QE_REFUSE("linear_tcgen05_swap: M = %d is above 256", M);
  if (K <= 0 || K % 8) QE_REFUSE("linear_tcgen05_swap: K = %d is not a positive multiple of 8", K);
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) QE_REFUSE("linear_tcgen05_swap: operands must be 16-byte aligned");
  if (M <= 64) return launch_swap<64, 8>(x, w, out, M, N, K, out_f32, stream);
  if (M <= 128) return launch_swap<128, 6>(x, w, out, M, N, K, out_f32, stream);
  return launch_swap<256, 4>(x, w, out, M, N, K, out_f32, stream);
}
