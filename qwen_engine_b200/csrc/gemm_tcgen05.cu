// out[M, N] = x[M, K] · w[N, K]^T in bfloat16 on the fifth-generation tensor cores: the matrix
// products of prompt portions (many rows).  Operand tiles are brought into shared memory by TMA
// (128-byte swizzle), multiplied by tcgen05.mma issued by one thread, accumulated in float32 in
// tensor memory, read back with tcgen05.ld and rounded once.  (Contract of the reference's linear,
// src/layers/ops/linear.py:101-122; its Triton kernel leaves the instruction choice to the compiler.)
//
// A persistent kernel: one CTA per SM walks over the 128 x BN output tiles (BN = 256, or 128 when that
// gives too few tiles), 6 warps: warp 0 feeds TMA, warp 1 owns tensor memory and issues the MMAs,
// warps 2-5 are the epilogue (one quarter of the 128 accumulator lanes each).  A ring of STAGES
// shared-memory slots (all the shared memory an SM has: what is in flight bounds the rate at which an
// SM can pull operands from L2) is handed back and forth through mbarriers: `full` (TMA bytes landed),
// `empty` (the MMAs that read the slot retired, signalled by tcgen05.commit).  Two accumulators in
// tensor memory take turns (`acc_full`, `acc_empty`), so the epilogue of one tile runs under the main
// loop of the next.  No cluster, no multicast: every CTA fetches its own tiles.
//
// Every wait on an mbarrier is bounded.  A wait that runs out records a code in a device flag, raises
// a CTA-wide abort that the other roles see in their own waits, and the CTA skips its stores, frees
// its tensor memory and returns; the host reads the flag with qe_gemm_tc_status().
//
// Edges: TMA fills what lies outside M, N or K with zeros, and the epilogue stores only rows < M and
// columns < N.  Needs K % 8 == 0 and 16-byte aligned bases (TMA strides); the launcher refuses the rest.
#include "tcgen05.cuh"

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192

__device__ int g_tc_status = 0;      // 0 = fine; else code of the first wait that ran out

template <int BN, int STAGES>
struct __align__(1024) TcSmem {
  __nv_bfloat16 a[STAGES][TC_BM * TC_BK];       // 16 KB each
  __nv_bfloat16 b[STAGES][BN * TC_BK];          // 16 or 32 KB each
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// STARVED (the self-test of the give-up path, qe_gemm_tc_selftest_starved): the producer issues no load and arms
// no barrier, and the waits give up after `starved_limit` polls instead of TC_WAIT_LIMIT; everything else is
// the product kernel as it is.
template <typename TOut, int BN, int STAGES, bool STARVED = false>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    TOut* __restrict__ out, int M, int N, int K, int starved_limit) {
  extern __shared__ unsigned char smem_raw[];
  using Smem = TcSmem<BN, STAGES>;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  pdl_launch_dependents();
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (K + TC_BK - 1) / TC_BK;
  const int n_blocks = (N + BN - 1) / BN;
  const int n_tiles = n_blocks * ((M + TC_BM - 1) / TC_BM);
  volatile int* abort_flag = &sm.abort_flag;
  const uint32_t wait_limit = STARVED ? (uint32_t)starved_limit : TC_WAIT_LIMIT;

  // Everything up to the first load of x needs nothing from the kernel before this one (the weights
  // are nobody's output): it runs before the wait for that kernel.
  if (threadIdx.x == 0) {
    tma_prefetch_map(&map_x);
    tma_prefetch_map(&map_w);
    for (int s = 0; s < STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&sm.acc_full[s], 1); mbar_init(&sm.acc_empty[s], 4); }
    sm.abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) tc_alloc(&sm.tmem_base, TMEM_COLS);     // one warp allocates (and later frees) both accumulators
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;

  if (warp == 0) {
    // ---- producer: TMA loads of the k-blocks of this CTA's tiles into the ring -------------------
    if (lane == 0) {
      const int my_tiles = (int)blockIdx.x < n_tiles ? (n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
      const uint32_t total = (uint32_t)my_tiles * (uint32_t)num_kb;      // k-blocks of all this CTA's tiles
      const uint32_t ahead = total < (uint32_t)STAGES ? total : (uint32_t)STAGES;
      auto coords = [&](uint32_t kc, int& m0, int& n0, int& kb) {
        const int t = (int)(kc / (uint32_t)num_kb);
        kb = (int)(kc - (uint32_t)t * (uint32_t)num_kb);
        const int tile = (int)blockIdx.x + t * (int)gridDim.x;
        m0 = (tile / n_blocks) * TC_BM; n0 = (tile % n_blocks) * BN;
      };
      int m0, n0, kb;
      // the ring's first round: the weights' tiles at once, x's after the wait for the kernel before
      for (uint32_t kc = 0; kc < ahead; ++kc) {
        if (STARVED) break;
        coords(kc, m0, n0, kb);
        mbar_expect_tx(&sm.full[kc], (TC_BM + BN) * TC_BK * sizeof(__nv_bfloat16));
        tma_load_2d(sm.b[kc], &map_w, &sm.full[kc], kb * TC_BK, n0);
      }
      pdl_wait();
      for (uint32_t kc = 0; kc < ahead; ++kc) {
        if (STARVED) break;
        coords(kc, m0, n0, kb);
        tma_load_2d(sm.a[kc], &map_x, &sm.full[kc], kb * TC_BK, m0);
      }
      uint32_t kc = ahead;
      for (; kc < total; ++kc) {
        const uint32_t s = kc % STAGES, round = kc / STAGES;
        if (!mbar_wait(&sm.empty[s], (round - 1) & 1, abort_flag, 1, &g_tc_status, wait_limit)) break;
        coords(kc, m0, n0, kb);
        mbar_expect_tx(&sm.full[s], (TC_BM + BN) * TC_BK * sizeof(__nv_bfloat16));
        tma_load_2d(sm.a[s], &map_x, &sm.full[s], kb * TC_BK, m0);
        tma_load_2d(sm.b[s], &map_w, &sm.full[s], kb * TC_BK, n0);
      }
      if (*abort_flag && !STARVED) {
        // giving up: let the copies that are still in flight land before the CTA leaves (bounded)
        for (uint32_t i = kc > (uint32_t)STAGES ? kc - STAGES : 0; i < kc; ++i) {
          const uint32_t s = i % STAGES;
          for (uint32_t spin = 0; spin < wait_limit; ++spin)
            if (mbar_try_wait(&sm.full[s], (i / STAGES) & 1)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: one thread, 4 instructions of K = 16 per k-block -------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(TC_BM, BN);
      uint32_t kc = 0;
      bool ok = true;
      int it = 0;
      for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x, ++it) {
        const int buf = it & 1;
        // the epilogue has read this accumulator's previous tile out of tensor memory
        if (it >= 2 && !mbar_wait(&sm.acc_empty[buf], ((it >> 1) - 1) & 1, abort_flag, 4, &g_tc_status, wait_limit)) { ok = false; break; }
        tc_fence_after();
        const uint32_t acc = tmem + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++kc) {
          const uint32_t s = kc % STAGES;
          if (!mbar_wait(&sm.full[s], (kc / STAGES) & 1, abort_flag, 2, &g_tc_status, wait_limit)) { ok = false; break; }
          tc_fence_after();
          const uint64_t da = make_smem_desc(smem_u32(sm.a[s]));
          const uint64_t db = make_smem_desc(smem_u32(sm.b[s]));
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k) {
            // 16 bfloat16 = 32 bytes further along K inside the swizzled row: +2 in 16-byte units
            tc_mma_bf16(acc, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
          }
          tc_commit(&sm.empty[s]);          // arrives when the MMAs that read this slot have retired
        }
        if (ok) tc_commit(&sm.acc_full[buf]);
      }
    }
  } else {
    // ---- epilogue: warps 2..5 read lanes 32 (warp % 4) .. +31, one output row per thread ------
    const int quarter = warp & 3;
    int it = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
      const int buf = it & 1;
      const int m0 = (tile / n_blocks) * TC_BM, n0 = (tile % n_blocks) * BN;
      const bool ok = __all_sync(0xffffffffu, mbar_wait(&sm.acc_full[buf], (it >> 1) & 1, abort_flag, 3, &g_tc_status, wait_limit));
      if (!ok) break;                                     // warp-uniform
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tc_ld_32x32b_x32(tmem + ((uint32_t)(quarter * 32) << 16) + buf * BN + c0, r);
        tc_wait_ld();
        if (c0 + 32 == BN) {
          // the accumulator is in registers: the MMA warp may start the tile after the next in it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sm.acc_empty[buf]);
        }
        if (row < M && n0 + c0 < N) {
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
  // everyone meets here (no thread leaves before the kernel before this one has completed); the
  // allocating warp frees the tensor memory
  pdl_wait();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tc_dealloc(tmem, TMEM_COLS);
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

template <int BN, int STAGES>
static int launch_tc(const void* x, const void* w, void* out, int M, int N, int K, int out_f32, int sms, cudaStream_t stream) {
  CUtensorMap map_x, map_w;
  if (!get_map(x, M, K, TC_BM, &map_x) || !get_map(w, N, K, BN, &map_w)) return 1;
  const size_t smem = sizeof(TcSmem<BN, STAGES>) + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<__nv_bfloat16, BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tcgen05_kernel<float, BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) QE_REFUSE("linear_tcgen05: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  const long tiles = (long)((N + BN - 1) / BN) * ((M + TC_BM - 1) / TC_BM);
  const dim3 grid((unsigned)(tiles < sms ? tiles : sms));
  if (out_f32)
    qe_launch(gemm_tcgen05_kernel<float, BN, STAGES>, grid, dim3(TC_THREADS), smem, stream, map_x, map_w, (float*)out, M, N, K, 0);
  else
    qe_launch(gemm_tcgen05_kernel<__nv_bfloat16, BN, STAGES>, grid, dim3(TC_THREADS), smem, stream, map_x, map_w, (__nv_bfloat16*)out, M, N, K, 0);
  QE_CHECK_LAUNCH("linear_tcgen05");
  return 0;
}

// The give-up path on purpose, for a test: one CTA of the product kernel whose producer loads nothing, so that no
// barrier ever flips, with waits of `limit` polls (some thousands: milliseconds).  The CTA must leave without a
// store, free its tensor memory and record which wait ran out first (qe_gemm_tc_status: 1, 2 or 3).  Nothing
// traps, faults or hangs; a product launched afterwards finds the SM as any other kernel leaves it.
extern "C" int qe_gemm_tc_selftest_starved(const void* x, const void* w, void* out, int M, int N, int K, int limit,
                                           cudaStream_t stream) {
  if (M <= 0 || M > TC_BM || N <= 0 || N > 128 || K <= 0 || K % 8) QE_REFUSE("selftest: one tile of at most 128 x 128, K a multiple of 8");
  if (limit < 1 || limit > (1 << 20)) QE_REFUSE("selftest: a limit of 1 .. 2^20 polls");
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) QE_REFUSE("selftest: operands must be 16-byte aligned");
  CUtensorMap map_x, map_w;
  if (!get_map(x, M, K, TC_BM, &map_x) || !get_map(w, N, K, 128, &map_w)) return 1;
  const size_t smem = sizeof(TcSmem<128, 6>) + 1024;
  cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<__nv_bfloat16, 128, 6, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) QE_REFUSE("selftest: shared memory %zu: %s", smem, cudaGetErrorString(e));
  qe_launch(gemm_tcgen05_kernel<__nv_bfloat16, 128, 6, true>, dim3(1), dim3(TC_THREADS), smem, stream, map_x, map_w,
            (__nv_bfloat16*)out, M, N, K, limit);
  QE_CHECK_LAUNCH("selftest");
  return 0;
}

static int sm_count() {
  static int sms[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (sms[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    sms[dev] = v;
  }
  return sms[dev];
}

extern "C" int qe_linear_tcgen05(const void* x, const void* w, void* out, int M, int N, int K, int out_f32,
                                 cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8) QE_REFUSE("linear_tcgen05: K = %d is not a positive multiple of 8", K);
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) QE_REFUSE("linear_tcgen05: operands must be 16-byte aligned");
  const int sms = sm_count();
  // wide tiles reuse the fetched rows of x twice as often; narrow ones when wide ones would leave SMs idle
  const long wide_tiles = (long)((N + 255) / 256) * ((M + TC_BM - 1) / TC_BM);
  if (wide_tiles >= sms) return launch_tc<256, 4>(x, w, out, M, N, K, out_f32, sms, stream);
  return launch_tc<128, 6>(x, w, out, M, N, K, out_f32, sms, stream);
}
