// out[M, N] (+)= x[M, K] · w[N, K]^T in bfloat16 for up to 64 rows when the weight rows alone are too
// few to give every SM a CTA (the output and down projections of a decode step of many requests:
// N = hidden size): a cluster of S CTAs shares a tile of 128 weight rows, and each CTA of the cluster
// takes one share of K.  (Same contract as the reference's linear, src/layers/ops/linear.py:101-122.)
//
// As in gemm_tcgen05_swap.cu the weights take the 128-row side of tcgen05.mma and the tokens its narrow
// side, a CTA streams its weights once through a TMA ring, and the accumulator lies in tensor memory.
// The partial sums then meet on chip: every CTA puts its 128 x M partial tile into its own shared
// memory, the cluster meets at a barrier, and CTA r adds up, for the tokens r, r + S, ..., the S
// partial tiles through distributed shared memory, always in the order of the shares (so the result
// does not depend on timing), and writes those tokens' outputs.  A second barrier keeps every CTA's
// shared memory alive until its neighbours have read it.
//
// RESID: out is the float32 residual stream and the product is added to it (every element is read
// and written by exactly one thread).
//
// Six warps: warp 0 feeds TMA, warp 1 owns tensor memory and issues the MMAs, warps 2-5 read the
// accumulator (lane = weight row, column = token) and do the sum.  Every wait on an mbarrier is bounded,
// as in gemm_tcgen05.cu; a CTA whose wait ran out still takes part in both cluster barriers, so that
// its neighbours return; qe_gemm_tc_splitk_status() reads this kernel's flag.
//
// Needs K % 8 == 0, N % 4 == 0 and 16-byte aligned bases; the launcher refuses the rest.
#include "tcgen05.cuh"

#define SK_BM 128               // weight rows per cluster
#define SK_BK 64
#define SK_BT 64                // tokens at most
#define SK_THREADS 192

static __device__ int g_tc_status = 0;      // 0 = fine; else code of the first wait that ran out

template <int STAGES>
struct __align__(1024) SkSmem {
  __nv_bfloat16 w[STAGES][SK_BM * SK_BK];       // 16 KB each
  __nv_bfloat16 x[STAGES][SK_BT * SK_BK];       // 8 KB each
  float part[SK_BT][SK_BM];                     // this CTA's partial sums, [token][weight row]: 32 KB
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

template <typename TOut, int S, int STAGES, bool RESID>
__global__ void __launch_bounds__(SK_THREADS, 1)
gemm_tcgen05_splitk_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                           TOut* __restrict__ out, int M, int N, int K) {
  extern __shared__ unsigned char smem_raw[];
  using Smem = SkSmem<STAGES>;
  constexpr uint32_t TMEM_COLS = SK_BT;
  pdl_launch_dependents();
  // the same offset in every CTA of the cluster: the dynamic shared memory starts at the same address
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)cluster_cta_rank();           // this CTA's share of K
  const int n0 = (blockIdx.x / S) * SK_BM;
  const int num_kb = (K + SK_BK - 1) / SK_BK;
  const int per = (num_kb + S - 1) / S;
  const int kb0 = min(num_kb, rank * per), kb1 = min(num_kb, kb0 + per);
  const int n_kb = kb1 - kb0;
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
      const int ahead = min(n_kb, STAGES);
      for (int i = 0; i < ahead; ++i) {
        mbar_expect_tx(&sm.full[i], (SK_BM + SK_BT) * SK_BK * sizeof(__nv_bfloat16));
        tma_load_2d(sm.w[i], &map_w, &sm.full[i], (kb0 + i) * SK_BK, n0);
      }
      pdl_wait();
      for (int i = 0; i < ahead; ++i) tma_load_2d(sm.x[i], &map_x, &sm.full[i], (kb0 + i) * SK_BK, 0);
      int issued = ahead;
      for (int i = ahead; i < n_kb; ++i) {
        const int s = i % STAGES;
        if (!mbar_wait(&sm.empty[s], ((i / STAGES) - 1) & 1, abort_flag, 21, &g_tc_status)) break;
        mbar_expect_tx(&sm.full[s], (SK_BM + SK_BT) * SK_BK * sizeof(__nv_bfloat16));
        tma_load_2d(sm.w[s], &map_w, &sm.full[s], (kb0 + i) * SK_BK, n0);
        tma_load_2d(sm.x[s], &map_x, &sm.full[s], (kb0 + i) * SK_BK, 0);
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
    if (lane == 0 && n_kb > 0) {
      const uint32_t idesc = make_idesc(SK_BM, mt);
      bool ok = true;
      for (int i = 0; i < n_kb && ok; ++i) {
        const int s = i % STAGES;
        ok = mbar_wait(&sm.full[s], (i / STAGES) & 1, abort_flag, 22, &g_tc_status);
        if (!ok) break;
        tc_fence_after();
        const uint64_t da = make_smem_desc(smem_u32(sm.w[s]));
        const uint64_t db = make_smem_desc(smem_u32(sm.x[s]));
#pragma unroll
        for (int k = 0; k < SK_BK / 16; ++k) tc_mma_bf16(tmem, da + 2 * k, db + 2 * k, idesc, (i | k) != 0);
        tc_commit(&sm.empty[s]);
      }
      if (ok) tc_commit(&sm.acc_full);
    }
  } else {
    // ---- this CTA's partial sums into its shared memory: lane = weight row, columns = tokens -----------
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    bool ok = true;
    if (n_kb > 0) ok = __all_sync(0xffffffffu, mbar_wait(&sm.acc_full, 0, abort_flag, 23, &g_tc_status));
    tc_fence_after();
#pragma unroll 1
    for (int c0 = 0; c0 < mt; c0 += 16) {
      uint32_t r[16];
      if (n_kb > 0 && ok) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(tmem + ((uint32_t)(quarter * 32) << 16) + c0) : "memory");
        tc_wait_ld();
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) r[j] = 0u;      // a share without k-blocks adds nothing
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) sm.part[c0 + j][row] = __uint_as_float(r[j]);
    }
    if (RESID) pdl_wait();                            // the stream is an earlier kernel's output
  }

  cluster_sync_all();                                 // every CTA's partial sums are in place

  if (warp >= 2) {
    // ---- CTA r: tokens r, r + S, ...; a warp per token, a lane per 4 weight rows -----------------------
    const int w4 = warp - 2;
    uint32_t base[S];
#pragma unroll
    for (int s = 0; s < S; ++s) base[s] = cluster_map_shared(&sm.part[0][0], (uint32_t)s);
    const int n = n0 + 4 * lane;
#pragma unroll 2
    for (int c = rank + S * w4; c < M; c += 4 * S) {
      float4 v[S];
#pragma unroll
      for (int s = 0; s < S; ++s) v[s] = cluster_ld_f32x4(base[s] + (uint32_t)(c * SK_BM + 4 * lane) * 4u);
      float4 acc = v[0];
#pragma unroll
      for (int s = 1; s < S; ++s) { acc.x += v[s].x; acc.y += v[s].y; acc.z += v[s].z; acc.w += v[s].w; }
      if (n < N) {                                    // N % 4 == 0: the four lie inside together
        TOut* dst = out + (size_t)c * N + n;
        if constexpr (sizeof(TOut) == 4) {
          float4* d4 = reinterpret_cast<float4*>(dst);
          if (RESID) { const float4 o = *d4; acc.x += o.x; acc.y += o.y; acc.z += o.z; acc.w += o.w; }
          *d4 = acc;
        } else {
          __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
          uint2 u;
          u.x = *reinterpret_cast<uint32_t*>(&lo);
          u.y = *reinterpret_cast<uint32_t*>(&hi);
          *reinterpret_cast<uint2*>(dst) = u;
        }
      }
    }
  }

  cluster_sync_all();                                 // nobody reads this CTA's shared memory any more
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

template <typename TOut, int S, int STAGES, bool RESID>
static int launch_splitk_as(const CUtensorMap& map_w, const CUtensorMap& map_x, void* out, int M, int N, int K, cudaStream_t stream) {
  const size_t smem = sizeof(SkSmem<STAGES>) + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_splitk_kernel<TOut, S, STAGES, RESID>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) QE_REFUSE("linear_tcgen05_splitk: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  const dim3 grid((unsigned)((N + SK_BM - 1) / SK_BM) * S);
  qe_launch_cluster(gemm_tcgen05_splitk_kernel<TOut, S, STAGES, RESID>, grid, dim3(SK_THREADS), smem, stream, (unsigned)S,
                    map_w, map_x, (TOut*)out, M, N, K);
  QE_CHECK_LAUNCH("linear_tcgen05_splitk");
  return 0;
}

template <int S>
static int launch_splitk(const void* x, const void* w, void* out, int M, int N, int K, int mode, cudaStream_t stream) {
  CUtensorMap map_w, map_x;
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    const uint64_t strides[1] = {(uint64_t)K * 2};
    const uint32_t box[2] = {SK_BK, SK_BM};
    if (!qe_tensor_map_bf16(w, 2, dims, strides, box, &map_w)) return 1;
  }
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    const uint64_t strides[1] = {(uint64_t)K * 2};
    const uint32_t box[2] = {SK_BK, SK_BT};
    if (!qe_tensor_map_bf16(x, 2, dims, strides, box, &map_x)) return 1;
  }
  if (mode == 2) return launch_splitk_as<float, S, 6, true>(map_w, map_x, out, M, N, K, stream);
  if (mode == 1) return launch_splitk_as<float, S, 6, false>(map_w, map_x, out, M, N, K, stream);
  return launch_splitk_as<__nv_bfloat16, S, 6, false>(map_w, map_x, out, M, N, K, stream);
}

extern "C" int qe_gemm_tc_splitk_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int));
  return v;
}
extern "C" void qe_gemm_tc_splitk_clear_status() {
  int v = 0;
  cudaMemcpyToSymbol(g_tc_status, &v, sizeof(int));
}

// 1 <= M <= 64; splits: 2, 4 or 8 CTAs per 128 weight rows (each gets ceil(K / 64 / splits) blocks of
// K; shares beyond K's end add nothing).  mode 0: out bfloat16; 1: out float32; 2: out float32 += the
// product.  Returns 0 when run, 1 when refused (qe_last_error says why), 2 on a launch error.
extern "C" int qe_linear_tcgen05_splitk(const void* x, const void* w, void* out, int M, int N, int K, int splits, int mode,
                                        cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > SK_BT) QE_REFUSE("linear_tcgen05_splitk: M = %d is above %d", M, SK_BT);
  if (K <= 0 || K % 8) QE_REFUSE("linear_tcgen05_splitk: K = %d is not a positive multiple of 8", K);
  if (N % 4) QE_REFUSE("linear_tcgen05_splitk: N = %d is not a multiple of 4", N);
  if (mode < 0 || mode > 2) QE_REFUSE("linear_tcgen05_splitk: mode %d", mode);
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) QE_REFUSE("linear_tcgen05_splitk: operands must be 16-byte aligned");
  if (splits == 2) return launch_splitk<2>(x, w, out, M, N, K, mode, stream);
  if (splits == 4) return launch_splitk<4>(x, w, out, M, N, K, mode, stream);
  if (splits == 8) return launch_splitk<8>(x, w, out, M, N, K, mode, stream);
  QE_REFUSE("linear_tcgen05_splitk: %d splits (2, 4 or 8)", splits);
}
