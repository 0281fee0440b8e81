// out[M, N] = x[M, K] · w[N, K]^T in bfloat16 on the fifth-generation tensor cores: the matrix
// products of prompt portions (many rows).  Operand tiles are brought into shared memory by TMA
// (128-byte swizzle), multiplied by tcgen05.mma issued by one thread, accumulated in float32 in
// tensor memory, read back with tcgen05.ld and rounded once.  (Contract of the reference's linear,
// src/layers/ops/linear.py:101-122; its Triton kernel leaves the instruction choice to the compiler.)
//
// One CTA per 128 x 128 output tile, 6 warps: warp 0 feeds TMA, warp 1 owns tensor memory and issues
// the MMAs, warps 2-5 are the epilogue (one quarter of the 128 accumulator lanes each).  A ring of
// STAGES shared-memory slots is handed back and forth through mbarriers: `full` (TMA bytes landed),
// `empty` (the MMAs that read the slot retired, signalled by tcgen05.commit), `acc_full` (all MMAs
// of the tile retired).  Two CTAs fit on an SM, so one tile's epilogue overlaps another's main loop.
// No cluster, no multicast: every CTA fetches its own tiles.
//
// Every wait on an mbarrier is bounded.  A wait that runs out records a code in a device flag, raises
// a CTA-wide abort that the other roles see in their own waits, and the CTA skips its stores, frees
// its tensor memory and returns; the host reads the flag with qe_gemm_tc_status().
//
// Edges: TMA fills what lies outside M, N or K with zeros, and the epilogue stores only rows < M and
// columns < N.  Needs K % 8 == 0 and 16-byte aligned bases (TMA strides); the launcher refuses the rest.
#include "tcgen05.cuh"

#define TC_BM 128
#define TC_BN 128
#define TC_BK 64
#define TC_STAGES 3
#define TC_THREADS 192
#define TC_TMEM_COLS 128

__device__ int g_tc_status = 0;      // 0 = fine; else code of the first wait that ran out

struct __align__(1024) TcSmem {
  __nv_bfloat16 a[TC_STAGES][TC_BM * TC_BK];       // 16 KB each
  __nv_bfloat16 b[TC_STAGES][TC_BN * TC_BK];       // 16 KB each
  uint64_t full[TC_STAGES];
  uint64_t empty[TC_STAGES];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

template <typename TOut>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    TOut* __restrict__ out, int M, int N, int K) {
  extern __shared__ unsigned char smem_raw[];
  pdl_launch_dependents();
  pdl_wait();
  TcSmem& sm = *reinterpret_cast<TcSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * TC_BM, n0 = blockIdx.x * TC_BN;
  const int num_kb = (K + TC_BK - 1) / TC_BK;
  volatile int* abort_flag = &sm.abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TC_STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
    mbar_init(&sm.acc_full, 1);
    sm.abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) {        // tensor memory: one warp allocates (and later frees) 128 columns
    tc_alloc(&sm.tmem_base, TC_TMEM_COLS);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;

  if (warp == 0) {
    // ---- producer: TMA loads of the k-blocks into the ring ----------------------------------
    if (lane == 0) {
      int issued = 0;
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % TC_STAGES;
        const uint32_t round = kb / TC_STAGES;
        if (round > 0 && !mbar_wait(&sm.empty[s], (round - 1) & 1, abort_flag, 1, &g_tc_status)) break;
        mbar_expect_tx(&sm.full[s], (TC_BM + TC_BN) * TC_BK * sizeof(__nv_bfloat16));
        tma_load_2d(sm.a[s], &map_x, &sm.full[s], kb * TC_BK, m0);
        tma_load_2d(sm.b[s], &map_w, &sm.full[s], kb * TC_BK, n0);
        ++issued;
      }
      if (*abort_flag) {
        // giving up: let the copies that are still in flight land before the CTA leaves (bounded)
        for (int i = max(0, issued - TC_STAGES); i < issued; ++i) {
          const int s = i % TC_STAGES;
          for (uint32_t spin = 0; spin < TC_WAIT_LIMIT; ++spin)
            if (mbar_try_wait(&sm.full[s], (i / TC_STAGES) & 1)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: one thread, 4 instructions of K = 16 per k-block -------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(TC_BM, TC_BN);
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % TC_STAGES;
        ok = mbar_wait(&sm.full[s], (kb / TC_STAGES) & 1, abort_flag, 2, &g_tc_status);
        if (!ok) break;
        tc_fence_after();
        const uint64_t da = make_smem_desc(smem_u32(sm.a[s]));
        const uint64_t db = make_smem_desc(smem_u32(sm.b[s]));
#pragma unroll
        for (int k = 0; k < TC_BK / 16; ++k) {
          // 16 bfloat16 = 32 bytes further along K inside the swizzled row: +2 in 16-byte units
          tc_mma_bf16(tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
        }
        tc_commit(&sm.empty[s]);          // arrives when the MMAs that read this slot have retired
      }
      if (ok) tc_commit(&sm.acc_full);
    }
  } else {
    // ---- epilogue: warps 2..5 read lanes 32 (warp % 4) .. +31, one output row per thread ------
    const int quarter = warp & 3;
    const bool ok = __all_sync(0xffffffffu, mbar_wait(&sm.acc_full, 0, abort_flag, 3, &g_tc_status));   // warp-uniform
    tc_fence_after();
    const int row = m0 + quarter * 32 + lane;
    if (ok) {
#pragma unroll 1
      for (int c0 = 0; c0 < TC_BN; c0 += 32) {
        uint32_t r[32];
        tc_ld_32x32b_x32(tmem + ((uint32_t)(quarter * 32) << 16) + c0, r);
        tc_wait_ld();
        if (row < M) {
          TOut* dst = out + (size_t)row * N + n0 + c0;
          if (n0 + c0 + 32 <= N && (N % 8) == 0) {
            if constexpr (sizeof(TOut) == 2) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 v;
                __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
                __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
                __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
                v.x = *reinterpret_cast<uint32_t*>(&p0); v.y = *reinterpret_cast<uint32_t*>(&p1);
                v.z = *reinterpret_cast<uint32_t*>(&p2); v.w = *reinterpret_cast<uint32_t*>(&p3);
                *reinterpret_cast<uint4*>(dst + j) = v;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                                  __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + c0 + j < N) dst[j] = from_f32<TOut>(__uint_as_float(r[j]));
          }
        }
      }
    }
  }
  // everyone meets here; the allocating warp frees the tensor memory
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tc_dealloc(tmem, TC_TMEM_COLS);
  }
}

// ---- host side ---------------------------------------------------------------------------------------------
// [rows, cols] bfloat16 row-major; box = box_rows x 64 columns; 128-byte swizzle; zero fill outside.
static bool get_map(const void* ptr, int rows, int cols, int box_rows, CUtensorMap* out) {
  const uint64_t dims[2] = {(uint64_t)cols, (uint64_t)rows};
  const uint64_t strides[1] = {(uint64_t)cols * sizeof(__nv_bfloat16)};
  const uint32_t box[2] = {TC_BK, (uint32_t)box_rows};
  return qe_tensor_map_bf16(ptr, 2, dims, strides, box, out);
}

extern "C" int qe_gemm_tc_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int));
  return v;
}
extern "C" void qe_gemm_tc_clear_status() {
  int v = 0;
  cudaMemcpyToSymbol(g_tc_status, &v, sizeof(int));
}

extern "C" int qe_linear_tcgen05(const void* x, const void* w, void* out, int M, int N, int K, int out_f32,
                                 cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8) QE_REFUSE("linear_tcgen05: K = %d is not a positive multiple of 8", K);
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) QE_REFUSE("linear_tcgen05: operands must be 16-byte aligned");
  dim3 grid((N + TC_BN - 1) / TC_BN, (M + TC_BM - 1) / TC_BM);
  if (grid.y > 65535) QE_REFUSE("linear_tcgen05: M = %d is too large", M);
  CUtensorMap map_x, map_w;
  if (!get_map(x, M, K, TC_BM, &map_x) || !get_map(w, N, K, TC_BN, &map_w)) return 1;
  const size_t smem = sizeof(TcSmem) + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tcgen05_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) QE_REFUSE("linear_tcgen05: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  if (out_f32)
    qe_launch(gemm_tcgen05_kernel<float>, grid, dim3(TC_THREADS), smem, stream, map_x, map_w, (float*)out, M, N, K);
  else
    qe_launch(gemm_tcgen05_kernel<__nv_bfloat16>, grid, dim3(TC_THREADS), smem, stream, map_x, map_w, (__nv_bfloat16*)out, M, N, K);
  QE_CHECK_LAUNCH("linear_tcgen05");
  return 0;
}
