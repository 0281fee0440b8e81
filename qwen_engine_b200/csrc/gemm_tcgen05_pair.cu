// out[M, N] = x[M, K] · w[N, K]^T in bfloat16 for many rows, by pairs of CTAs (tcgen05 cta_group::2):
// two CTAs on neighbouring SMs share one 256 x BN output tile.  Each brings its own 128 rows of x and
// only its half of the BN rows of w; one thread of the leading CTA issues MMAs that read both CTAs'
// shared memory and write both CTAs' tensor memory.  An SM so fetches a quarter less (BN = 128) or a
// third less (BN = 256) from L2 per multiply-add than alone with a 128 x BN tile, and what an SM can
// pull from L2 is what bounds these products.  (Contract of the reference's linear,
// src/layers/ops/linear.py:101-122.)
//
// Persistent: a cluster of two CTAs per pair of SMs walks over the tiles.  Per CTA 10 warps: warp 0
// feeds TMA (its loads count their bytes on the leading CTA's `full` barrier), warp 1 owns tensor
// memory (and, in the leading CTA, issues the MMAs), warps 2-9 read this CTA's 128 rows of the
// accumulator and store them: a warp reaches the 32 rows of tensor memory that its number modulo 4
// names, so warps 2-5 take the first half of the tile's columns and warps 6-9 the second (with a
// short K the epilogue of a tile takes as long as its products: eight warps keep it off the critical path).  `empty` and `acc_full` are signalled to both CTAs by tcgen05.commit
// with a CTA mask; `acc_empty` lives in the leading CTA and collects the epilogue warps of both.  No
// TMA multicast.  Every wait on an mbarrier is bounded, as in gemm_tcgen05.cu.
//
//
// SWIGLU: w is the feed-forward's stacked gate and up weights [2 I, K].  A tile's 256 columns are 128
// columns of gate and the same 128 columns of up (the leading CTA loads the gate rows, the other CTA
// the up rows: only the TMA coordinate differs), and the epilogue writes silu(gate) * up, computed on
// the float32 accumulators, as 128 columns of out [M, I]: the activation never exists as gate_up in
// memory (reference: src/layers/fused_ops/silumul.py:50-53 applies it to the rounded products).
//
// ROPE: w is an attention layer's stacked q, k, v weights with head size 128, so a tile's 256 columns are
// two whole heads and an epilogue thread holds a token's whole head.  The epilogue does what the rotary
// kernel would do to the product afterwards (elementwise.cu, rope_d128.cuh: the product rounded to
// bfloat16, per-head RMS norm of q and k in float32, rotation of the pairs (d, d + 64) by the step's table
// of angles, rounded once): q goes to out, k and v go straight into the cache pages at the tokens' slots
// and are not written to out at all.  The rotary kernel's launch and its pass over the product disappear.
//
// Needs K % 8 == 0 and 16-byte aligned bases (TMA strides); the launcher refuses the rest.
#include "tcgen05.cuh"

struct PrRope {
  const float* qw; const float* kw; float eps;      // norm weights [128] (null: no norm)
  const float2* cos_sin;                            // [M, 64] (cos, sin) of every token's angles (null: no rotation)
  __nv_bfloat16* pages; const int* slot_mapping;    // the cache [pages, 2, Hkv, page, 128] and the tokens' slots
  int Hq, Hkv, page_size, write_kv;
};

#define PR_BM 128               // rows of x per CTA (256 per pair)
#define PR_BK 64
#define PR_THREADS 320
#define PR_EPI_WARPS 8          // two per quarter of the accumulator's rows, each with half of the tile's columns

static __device__ int g_tc_status = 0;      // 0 = fine; else code of the first wait that ran out

// the epilogue warps of a CTA among themselves
__device__ __forceinline__ void pr_epilogue_sync() { asm volatile("bar.sync 1, %0;\n" :: "n"(PR_EPI_WARPS * 32) : "memory"); }
// the same, and whether `ok` holds in all of their threads: after a wait that may have run out in some warps only,
// so that all of them go on or none does
__device__ __forceinline__ bool pr_epilogue_all(bool ok) {
  uint32_t all;
  asm volatile("{\n.reg .pred p, q;\nsetp.ne.u32 q, %1, 0;\nbar.red.and.pred p, 1, %2, q;\nselp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(all) : "r"((uint32_t)ok), "n"(PR_EPI_WARPS * 32) : "memory");
  return all != 0;
}

template <int BN, int STAGES, bool ROPE = false>
struct __align__(1024) PrSmem {
  __nv_bfloat16 a[STAGES][PR_BM * PR_BK];            // 16 KB each
  __nv_bfloat16 b[STAGES][(BN / 2) * PR_BK];         // this CTA's half of the tile's rows of w
  __nv_bfloat16 stage[PR_BM * 128];                  // 32 KB between the accumulator and memory: ROPE: one head of this CTA's 128 rows; else 4 KB per epilogue warp
  float stage_ssq[ROPE ? 2 * PR_BM : 2];             // ... and the sums of squares of the two halves of every row
  uint64_t full[STAGES];                             // used in the leading CTA
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];                             // used in the leading CTA
  uint32_t tmem_base;
  int abort_flag;
};

// 32 rows x COLS bfloat16 columns of the output, from the warp whose lane l holds row l (as the accumulator leaves
// tensor memory: packed[i] = columns 2 i, 2 i + 1 of the lane's row), to memory with lanes along the columns: through
// 4 KB of shared memory of the warp's own (16-byte chunks XORed with the row's low bits), then 128 or 64 bytes of a
// row per 8 or 4 lanes.  Stored with lanes along the rows, every instruction touched 32 rows with 16 bytes each, and a
// tile's epilogue took 3.5-5.8 us (measured with the timeline build), as long as its products.
// dst: row 0, column 0 of the 32 x COLS block; ld: elements per row of the output; rows, cols: how many of them exist.
template <int COLS>
__device__ __forceinline__ void pr_store_block(unsigned char* wst, const uint32_t (&packed)[COLS / 2], __nv_bfloat16* dst, size_t ld,
                                               int rows, int cols, int lane) {
  constexpr int CH = COLS / 8, RB = COLS * 2, RPI = 32 / CH;     // chunks per row, bytes per row, rows per instruction
#pragma unroll
  for (int j = 0; j < CH; ++j)
    *reinterpret_cast<uint4*>(wst + lane * RB + ((j ^ (lane & (CH - 1))) << 4)) =
        make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
  __syncwarp();
  const int cj = lane % CH;
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    const int rr = i * RPI + lane / CH;
    const uint4 v = *reinterpret_cast<const uint4*>(wst + rr * RB + ((cj ^ (rr & (CH - 1))) << 4));
    if (rr < rows) {
      __nv_bfloat16* d = dst + (size_t)rr * ld + cj * 8;
      if (cj * 8 + 8 <= cols) {
        *reinterpret_cast<uint4*>(d) = v;
      } else {
        const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&v);
        for (int k = 0; k < 8; ++k)
          if (cj * 8 + k < cols) d[k] = e[k];
      }
    }
  }
  __syncwarp();
}

// K split over S pairs of a cluster: CTA (pair `cpair`, parity `rank`) finishes 1 / S of the columns of its 128 rows.
// `stg`: this CTA's sums in shared memory, row r at r x BN x 4 bytes, 16-byte chunks XORed with the row's low bits;
// the other shares lie at the same place in the CTAs of the same parity.  The loads of four chunks' shares are all
// in flight before the first is used (a load from another CTA's shared memory takes some hundreds of cycles).
template <typename TOut, int BN, int S>
__device__ __forceinline__ void pr_meet_shares(const unsigned char* stg, TOut* __restrict__ out, int M, int N, int m0, int n0,
                                               uint32_t rank, uint32_t cpair) {
  constexpr int CPR = (BN / 4) / S;                  // 16-byte chunks of a row that this CTA finishes
  constexpr int BATCH = 4;
  static_assert((PR_BM * CPR) % (PR_EPI_WARPS * 32 * BATCH) == 0, "whole batches per thread");
  const int t = (int)threadIdx.x - 64;
  uint32_t base[S];
#pragma unroll
  for (int sp = 0; sp < S; ++sp) base[sp] = cluster_map_shared(stg, (uint32_t)(2 * sp) + rank);
#pragma unroll 1
  for (int item0 = t; item0 < PR_BM * CPR; item0 += PR_EPI_WARPS * 32 * BATCH) {
    float4 v[BATCH][S];
#pragma unroll
    for (int b = 0; b < BATCH; ++b) {
      const int item = item0 + b * PR_EPI_WARPS * 32;
      const int rr = item / CPR, chunk = (int)cpair * CPR + item % CPR;
      const uint32_t off = (uint32_t)rr * (BN * 4) + (uint32_t)((chunk ^ (rr & 7)) << 4);
#pragma unroll
      for (int sp = 0; sp < S; ++sp) v[b][sp] = cluster_ld_f32x4(base[sp] + off);
    }
#pragma unroll
    for (int b = 0; b < BATCH; ++b) {
      const int item = item0 + b * PR_EPI_WARPS * 32;
      const int rr = item / CPR, chunk = (int)cpair * CPR + item % CPR;
      float4 acc = v[b][0];                          // in the order of the shares
#pragma unroll
      for (int sp = 1; sp < S; ++sp) { acc.x += v[b][sp].x; acc.y += v[b][sp].y; acc.z += v[b][sp].z; acc.w += v[b][sp].w; }
      const int row = m0 + rr, col = n0 + chunk * 4;
      if (row < M && col < N) {                      // N is a multiple of 8 here (the launcher's rule)
        if constexpr (sizeof(TOut) == 2) {
          __nv_bfloat162 p0 = __floats2bfloat162_rn(acc.x, acc.y), p1 = __floats2bfloat162_rn(acc.z, acc.w);
          *reinterpret_cast<uint2*>(out + (size_t)row * N + col) = make_uint2(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1));
        } else {
          *reinterpret_cast<float4*>(out + (size_t)row * N + col) = acc;
        }
      }
    }
  }
}

// N: columns of the product (SWIGLU: 2 I); n_up: SWIGLU: the first row of up in w (= I), else 0
template <typename TOut, int BN, int STAGES, bool SWIGLU, bool ROPE = false>
__global__ void __launch_bounds__(PR_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                         TOut* __restrict__ out, int M, int N, int K, int n_up, PrRope rp, int splits) {
  static_assert(!SWIGLU || BN == 256, "the fused activation pairs 128 columns of gate with 128 of up");
  static_assert(!ROPE || (BN == 256 && !SWIGLU && sizeof(TOut) == 2), "the fused rotation takes two heads of 128 per tile, in bfloat16");
  extern __shared__ unsigned char smem_raw[];
  using Smem = PrSmem<BN, STAGES, ROPE>;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  constexpr uint32_t STAGE_BYTES = (PR_BM + BN / 2) * PR_BK * sizeof(__nv_bfloat16);
  pdl_launch_dependents();
  QE_TL_STAMPS(32);
  QE_TL_STAMP(threadIdx.x == 0 ? 0 : -1);           // (timeline build: the CTA's start)
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // The cluster is one pair, or (plain products with few tiles) `splits` pairs that work on the same tile with
  // a share of K each; ranks 2p and 2p + 1 are pair p.
  const uint32_t crank = cluster_cta_rank();
  const uint32_t rank = crank & 1u;                  // 0: the leading CTA of the pair
  const uint32_t cpair = crank >> 1;                 // which share of K
  const uint16_t pair_mask = (uint16_t)(3u << (2 * cpair));
  const int all_kb = (K + PR_BK - 1) / PR_BK;
  const int kb_per = (all_kb + splits - 1) / splits;
  const int kb_first = (int)cpair * kb_per;
  const int num_kb = max(0, min(all_kb, kb_first + kb_per) - kb_first);     // this pair's k-blocks (the launcher leaves none empty)
  const int n_blocks = SWIGLU ? (n_up + BN / 2 - 1) / (BN / 2) : (N + BN - 1) / BN;
  const int n_tiles = n_blocks * ((M + 2 * PR_BM - 1) / (2 * PR_BM));
  const int pair = (int)blockIdx.x / (2 * splits), n_pairs = (int)gridDim.x / (2 * splits);   // (with splits: which cluster, how many)
  volatile int* abort_flag = &sm.abort_flag;

  // Everything up to the first load of x needs nothing from the kernel before this one (the weights
  // are nobody's output): it runs before the wait for that kernel.
  if (threadIdx.x == 0) {
    tma_prefetch_map(&map_x);
    tma_prefetch_map(&map_w);
    for (int s = 0; s < STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&sm.acc_full[s], 1); mbar_init(&sm.acc_empty[s], 2 * PR_EPI_WARPS); }
    sm.abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) tc_alloc_pair(&sm.tmem_base, TMEM_COLS);   // the same warp in both CTAs
  tc_fence_before();
  cluster_sync_all();                                // barriers and tensor memory of both CTAs are ready
  QE_TL_STAMP(threadIdx.x == 0 ? 1 : -1);           // (... set-up done in both CTAs)
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  bool split_staged = false;                         // K split over pairs: this thread has put its sums into shared memory

  if (warp == 0) {
    // ---- producer: this CTA's rows of x and its half of the rows of w; bytes counted in the leading CTA
    if (lane == 0) {
      const int my_tiles = pair < n_tiles ? (n_tiles - pair + n_pairs - 1) / n_pairs : 0;
      const uint32_t total = (uint32_t)my_tiles * (uint32_t)num_kb;      // k-blocks of all this pair's tiles
      const uint32_t ahead = total < (uint32_t)STAGES ? total : (uint32_t)STAGES;
      auto coords = [&](uint32_t kc, int& m0, int& n0, int& kb) {
        const int t = (int)(kc / (uint32_t)num_kb);
        kb = kb_first + (int)(kc - (uint32_t)t * (uint32_t)num_kb);
        const int tile = pair + t * n_pairs;
        m0 = (tile / n_blocks) * 2 * PR_BM + (int)rank * PR_BM;
        n0 = SWIGLU ? (tile % n_blocks) * (BN / 2) + (int)rank * n_up      // gate rows, or the same rows of up
                    : (tile % n_blocks) * BN + (int)rank * (BN / 2);
      };
      int m0, n0, kb;
      // the ring's first round: the weights' tiles at once, x's after the wait for the kernel before
      for (uint32_t kc = 0; kc < ahead; ++kc) {
        coords(kc, m0, n0, kb);
        if (rank == 0) mbar_expect_tx(&sm.full[kc], 2 * STAGE_BYTES);    // both CTAs' bytes
        tma_load_2d_pair(sm.b[kc], &map_w, smem_u32(&sm.full[kc]) & TC_PEER_BIT_MASK, kb * PR_BK, n0);
      }
      pdl_wait();
      QE_TL_STAMP(2);                                // (... the kernel before has completed)
      for (uint32_t kc = 0; kc < ahead; ++kc) {
        coords(kc, m0, n0, kb);
        tma_load_2d_pair(sm.a[kc], &map_x, smem_u32(&sm.full[kc]) & TC_PEER_BIT_MASK, kb * PR_BK, m0);
      }
      for (uint32_t kc = ahead; kc < total; ++kc) {
        const uint32_t s = kc % STAGES, round = kc / STAGES;
        if (!mbar_wait(&sm.empty[s], (round - 1) & 1, abort_flag, 21, &g_tc_status)) break;
        coords(kc, m0, n0, kb);
        if (rank == 0) mbar_expect_tx(&sm.full[s], 2 * STAGE_BYTES);
        const uint32_t full_addr = smem_u32(&sm.full[s]) & TC_PEER_BIT_MASK;
        tma_load_2d_pair(sm.a[s], &map_x, full_addr, kb * PR_BK, m0);
        tma_load_2d_pair(sm.b[s], &map_w, full_addr, kb * PR_BK, n0);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: one thread of the leading CTA ----------------------------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc(2 * PR_BM, BN);
      uint32_t kc = 0;
      bool ok = true;
      int it = 0;
      for (int tile = pair; ok && tile < n_tiles; tile += n_pairs, ++it) {
        const int buf = it & 1;
        if (it >= 2 && !mbar_wait(&sm.acc_empty[buf], ((it >> 1) - 1) & 1, abort_flag, 24, &g_tc_status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t acc = tmem + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++kc) {
          const uint32_t s = kc % STAGES;
          if (!mbar_wait(&sm.full[s], (kc / STAGES) & 1, abort_flag, 22, &g_tc_status)) { ok = false; break; }
          tc_fence_after();
          const uint64_t da = make_smem_desc(smem_u32(sm.a[s]));
          const uint64_t db = make_smem_desc(smem_u32(sm.b[s]));
#pragma unroll
          for (int k = 0; k < PR_BK / 16; ++k) tc_mma_bf16_pair(acc, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
          tc_commit_pair(&sm.empty[s], pair_mask);     // both CTAs' producers may refill the slot
        }
        if (ok) tc_commit_pair(&sm.acc_full[buf], pair_mask);
      }
    }
  } else {
    // ---- epilogue: this CTA's 128 rows of the accumulator ----------------------------------------
    const int quarter = warp & 3;
    const int ch = (warp - 2) >> 2;                  // which half of the tile's columns
    // ROPE: this lane's elements (2l, 2l + 1, 64 + 2l, 64 + 2l + 1) of the norm weights of q and of k
    [[maybe_unused]] float4 nw_q = make_float4(1.f, 1.f, 1.f, 1.f), nw_k = nw_q;
    if constexpr (ROPE) {
      if (rp.qw) {
        const float2 a = __ldg(reinterpret_cast<const float2*>(rp.qw) + lane), b = __ldg(reinterpret_cast<const float2*>(rp.qw + 64) + lane);
        nw_q = make_float4(a.x, a.y, b.x, b.y);
      }
      if (rp.kw) {
        const float2 a = __ldg(reinterpret_cast<const float2*>(rp.kw) + lane), b = __ldg(reinterpret_cast<const float2*>(rp.kw + 64) + lane);
        nw_k = make_float4(a.x, a.y, b.x, b.y);
      }
    }
    int it = 0;
    for (int tile = pair; tile < n_tiles; tile += n_pairs, ++it) {
      const int buf = it & 1;
      const int m0 = (tile / n_blocks) * 2 * PR_BM + (int)rank * PR_BM, n0 = (tile % n_blocks) * BN;
      // ROPE: what this warp's 16 rows need from memory besides the accumulator (their angles, their slots in the
      // cache) is the same for both heads of the tile and is asked for before the wait for the tile's products
      [[maybe_unused]] float4 rope_t[ROPE ? PR_BM / PR_EPI_WARPS : 1];
      [[maybe_unused]] int rope_slot = 0;
      if constexpr (ROPE) {
        const int e = warp - 2;
        if (rp.cos_sin != nullptr) {
#pragma unroll
          for (int i = 0; i < PR_BM / PR_EPI_WARPS; ++i) {
            const int r = min(m0 + e + i * PR_EPI_WARPS, M - 1);
            rope_t[i] = __ldg(reinterpret_cast<const float4*>(rp.cos_sin + (size_t)r * 64) + lane);   // (cos, sin) of elements 2l, 2l + 1
          }
        }
        if (rp.write_kv && lane < PR_BM / PR_EPI_WARPS) {
          const int r = m0 + e + lane * PR_EPI_WARPS;
          rope_slot = r < M ? __ldg(rp.slot_mapping + r) : 0;
        }
      }
      bool ok = __all_sync(0xffffffffu, mbar_wait(&sm.acc_full[buf], (it >> 1) & 1, abort_flag, 23, &g_tc_status));
      QE_TL_STAMP(warp == 2 && lane == 0 ? 16 + 2 * (it > 0) : -1);   // (... a tile's sums are ready: the first, the last)
      if constexpr (ROPE) ok = pr_epilogue_all(ok);    // its warps meet at barriers below: all go on or none
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      if constexpr (SWIGLU) {
        // this warp's 64 columns of gate and of up -> 64 columns of the activation
        const int I = n_up, i0 = (tile % n_blocks) * (BN / 2);
        constexpr int WC = BN / 4;                   // activation columns per warp
        if (sizeof(TOut) == 2 && (I % 8) == 0) {
          // bfloat16 rows whose pieces of 8 are 16-byte aligned: all loads from tensor memory in flight together, then
          // the accumulator is free; stored with lanes along the columns
          uint32_t g[WC / 32][32], u[WC / 32][32];
#pragma unroll
          for (int q = 0; q < WC / 32; ++q) {
            tc_ld_32x32b_x32(tmem + ((uint32_t)(quarter * 32) << 16) + buf * BN + ch * WC + 32 * q, g[q]);
            tc_ld_32x32b_x32(tmem + ((uint32_t)(quarter * 32) << 16) + buf * BN + BN / 2 + ch * WC + 32 * q, u[q]);
          }
          tc_wait_ld();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(smem_u32(&sm.acc_empty[buf]) & TC_PEER_BIT_MASK);
          uint32_t pk[WC / 2];
#pragma unroll
          for (int q = 0; q < WC / 32; ++q)
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const float g0 = __uint_as_float(g[q][j]), g1 = __uint_as_float(g[q][j + 1]);
              __nv_bfloat162 pj = __floats2bfloat162_rn(__fdividef(g0, 1.f + __expf(-g0)) * __uint_as_float(u[q][j]),
                                                        __fdividef(g1, 1.f + __expf(-g1)) * __uint_as_float(u[q][j + 1]));
              pk[16 * q + (j >> 1)] = *reinterpret_cast<uint32_t*>(&pj);
            }
          const int r_first = m0 + quarter * 32, c0 = ch * WC;
          pr_store_block<WC>(reinterpret_cast<unsigned char*>(sm.stage) + (warp - 2) * 4096, pk,
                             reinterpret_cast<__nv_bfloat16*>(out) + (size_t)r_first * I + i0 + c0, (size_t)I,
                             M - r_first, I - (i0 + c0), lane);
        } else {
#pragma unroll 1
        for (int c0 = ch * WC; c0 < (ch + 1) * WC; c0 += 32) {
          uint32_t g[32], u[32];
          tc_ld_32x32b_x32(tmem + ((uint32_t)(quarter * 32) << 16) + buf * BN + c0, g);
          tc_ld_32x32b_x32(tmem + ((uint32_t)(quarter * 32) << 16) + buf * BN + BN / 2 + c0, u);
          tc_wait_ld();
          if (c0 + 32 == (ch + 1) * WC) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(smem_u32(&sm.acc_empty[buf]) & TC_PEER_BIT_MASK);
          }
          if (row < M && i0 + c0 < I) {
            TOut* dst = out + (size_t)row * I + i0 + c0;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float gv = __uint_as_float(g[j]);
              if (i0 + c0 + j < I) dst[j] = from_f32<TOut>(__fdividef(gv, 1.f + __expf(-gv)) * __uint_as_float(u[j]));
            }
          }
        }
        }
      } else if constexpr (ROPE) {
        // Two heads of 128 columns, one after the other, each in two halves.  First every thread takes 64 columns
        // of its own row of the accumulator (a thread of warp w reaches row 32 (w mod 4) + lane of tensor memory),
        // rounds them to bfloat16 as the plain product's output is rounded, and puts them into shared memory
        // (16-byte chunks, their index XORed with the row's low bits: no bank conflicts either way).  Then the eight
        // warps walk over the 128 rows, a row per warp at a time, lanes along the head: lane l holds elements 2l,
        // 2l + 1 and their partners 64 further, the sum of squares is a warp reduction, the row's angles are one
        // 512-byte load and its outputs two 128-byte stores.  (With lanes along the rows, as the accumulator comes
        // out of tensor memory, every load of angles and every store touched 32 rows at once: the epilogue then
        // took longer than the tile's products.)
        unsigned char* stg = reinterpret_cast<unsigned char*>(sm.stage);
        const uint32_t tm_row = tmem + ((uint32_t)(quarter * 32) << 16) + buf * BN;
        const int r_mine = quarter * 32 + lane;          // this thread's row of the CTA's 128
        const int e = warp - 2;                          // 0..7
#pragma unroll 1
        for (int hh = 0; hh < 2; ++hh) {
          const int col0 = n0 + hh * 128, head = col0 >> 7;
          const bool is_q = head < rp.Hq, is_v = head >= rp.Hq + rp.Hkv;
          const bool wanted = col0 < N && (is_q || rp.write_kv);   // (keys and values of a layer that reads another's cache are dropped)
          {
            uint32_t a[32], b[32];
            tc_ld_32x32b_x32(tm_row + hh * 128 + ch * 64, a);
            tc_ld_32x32b_x32(tm_row + hh * 128 + ch * 64 + 32, b);
            tc_wait_ld();
            if (hh == 1) {
              // the accumulator is in registers: tell the leading CTA's MMA thread
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive_cluster(smem_u32(&sm.acc_empty[buf]) & TC_PEER_BIT_MASK);
            }
            unsigned char* mine = stg + r_mine * 256;
            float s4[4] = {0.f, 0.f, 0.f, 0.f};      // of the rounded values, as the norm of the plain product sees them
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              const uint32_t* src = c < 4 ? a + 8 * c : b + 8 * (c - 4);
              uint32_t v[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 pj = __floats2bfloat162_rn(__uint_as_float(src[2 * j]), __uint_as_float(src[2 * j + 1]));
                v[j] = *reinterpret_cast<uint32_t*>(&pj);
                const float x0 = __uint_as_float(v[j] << 16), x1 = __uint_as_float(v[j] & 0xffff0000u);
                s4[j] = fmaf(x0, x0, fmaf(x1, x1, s4[j]));
              }
              *reinterpret_cast<uint4*>(mine + (((ch * 8 + c) ^ (r_mine & 7)) << 4)) = make_uint4(v[0], v[1], v[2], v[3]);
            }
            sm.stage_ssq[ch * PR_BM + r_mine] = (s4[0] + s4[1]) + (s4[2] + s4[3]);
          }
          QE_TL_STAMP(warp == 2 && lane == 0 && it == 0 ? 8 + 4 * hh : -1);      // (timeline build: first tile, head hh staged by this warp)
          pr_epilogue_sync();                        // the head is in shared memory
          QE_TL_STAMP(warp == 2 && lane == 0 && it == 0 ? 9 + 4 * hh : -1);      // (... by all warps)
          if (wanted) {
            const float* w = is_v ? nullptr : (is_q ? rp.qw : rp.kw);
            const float w0 = is_q ? nw_q.x : nw_k.x, w1 = is_q ? nw_q.y : nw_k.y, w2 = is_q ? nw_q.z : nw_k.z, w3 = is_q ? nw_q.w : nw_k.w;
            const bool rotate = !is_v && rp.cos_sin != nullptr;
            const int kv_h = is_v ? head - rp.Hq - rp.Hkv : head - rp.Hq;
            const int page_shift = (rp.page_size & (rp.page_size - 1)) == 0 ? __ffs(rp.page_size) - 1 : -1;
            // 16 rows per warp, in two rounds of 8 whose loads are all issued before the first is used and whose
            // arithmetic the compiler interleaves (a row alone is one chain of dependent shuffles and loads)
            constexpr int ROUND = 8;
#pragma unroll 1
            for (int r0 = e; r0 < PR_BM; r0 += ROUND * PR_EPI_WARPS) {
              const int i0 = (r0 - e) / PR_EPI_WARPS;        // 0 or ROUND: where this round's rows are among the warp's 16
              uint32_t ul[ROUND], uh[ROUND];
#pragma unroll
              for (int i = 0; i < ROUND; ++i) {
                const int rr = r0 + i * PR_EPI_WARPS;
                const unsigned char* src = stg + rr * 256 + ((lane & 3) << 2);
                ul[i] = *reinterpret_cast<const uint32_t*>(src + (((lane >> 2) ^ (rr & 7)) << 4));
                uh[i] = *reinterpret_cast<const uint32_t*>(src + (((8 + (lane >> 2)) ^ (rr & 7)) << 4));
              }
              float rstd[ROUND];
              if (w) {
#pragma unroll
                for (int i = 0; i < ROUND; ++i) {
                  const int rr = r0 + i * PR_EPI_WARPS;
                  rstd[i] = rsqrtf((sm.stage_ssq[rr] + sm.stage_ssq[PR_BM + rr]) / 128.f + rp.eps);
                }
              }
#pragma unroll
              for (int i = 0; i < ROUND; ++i) {
                const int r = m0 + r0 + i * PR_EPI_WARPS;
                float l0 = __uint_as_float(ul[i] << 16), l1 = __uint_as_float(ul[i] & 0xffff0000u);
                float h0 = __uint_as_float(uh[i] << 16), h1 = __uint_as_float(uh[i] & 0xffff0000u);
                if (w) { l0 = l0 * rstd[i] * w0; l1 = l1 * rstd[i] * w1; h0 = h0 * rstd[i] * w2; h1 = h1 * rstd[i] * w3; }
                if (rotate) {
                  const float a0 = l0, b0 = h0, a1 = l1, b1 = h1;
                  const float4 t = i0 == 0 ? rope_t[i] : rope_t[ROUND + i];
                  l0 = t.x * a0 - t.y * b0;  h0 = t.y * a0 + t.x * b0;
                  l1 = t.z * a1 - t.w * b1;  h1 = t.w * a1 + t.z * b1;
                }
                const int slot = __shfl_sync(0xffffffffu, rope_slot, i0 + i);
                __nv_bfloat16* dst;
                if (is_q) {
                  dst = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)r * N + col0;
                } else {
                  // slot = page * page_size + off: the row of (page, K or V, h, off) in the cache
                  const int page = page_shift >= 0 ? slot >> page_shift : slot / rp.page_size;
                  dst = rp.pages + ((size_t)slot + ((size_t)page * (2 * rp.Hkv - 1) + (is_v ? rp.Hkv : 0) + kv_h) * rp.page_size) * 128;
                }
                if (r < M) {
                  __nv_bfloat162 pl = __floats2bfloat162_rn(l0, l1), ph = __floats2bfloat162_rn(h0, h1);
                  reinterpret_cast<uint32_t*>(dst)[lane] = *reinterpret_cast<uint32_t*>(&pl);
                  reinterpret_cast<uint32_t*>(dst + 64)[lane] = *reinterpret_cast<uint32_t*>(&ph);
                }
              }
            }
          }
          QE_TL_STAMP(warp == 2 && lane == 0 && it == 0 ? 10 + 4 * hh : -1);     // (... this warp's rows of the head are written)
          pr_epilogue_sync();                        // the buffer is free for the next head
        }
      } else if (splits > 1) {
        // K split over the cluster's pairs: this pair's sums go to shared memory (the ring is idle: every load
        // has been used and every product has retired), row r at r x BN x 4 bytes, 16-byte chunks XORed with the
        // row's low bits; they meet after the cluster's barrier below
        unsigned char* stg = reinterpret_cast<unsigned char*>(sm.a);
        const int r_mine = quarter * 32 + lane;
#pragma unroll 1
        for (int c0 = ch * (BN / 2); c0 < (ch + 1) * (BN / 2); c0 += 32) {
          uint32_t r[32];
          tc_ld_32x32b_x32(tmem + ((uint32_t)(quarter * 32) << 16) + buf * BN + c0, r);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(stg + (size_t)r_mine * (BN * 4) + ((((c0 >> 2) + j) ^ (r_mine & 7)) << 4)) =
                make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        }
        split_staged = true;
      } else if (sizeof(TOut) == 2 && (N % 8) == 0) {
        // bfloat16 rows whose pieces of 8 are 16-byte aligned: this warp's half of the columns in one go (all
        // loads from tensor memory in flight together, then the accumulator is free), stored 64 columns at a time
        // with lanes along the columns
        constexpr int NLD = BN / 64;                 // loads of 32 columns
        uint32_t r[NLD][32];
#pragma unroll
        for (int q = 0; q < NLD; ++q)
          tc_ld_32x32b_x32(tmem + ((uint32_t)(quarter * 32) << 16) + buf * BN + ch * (BN / 2) + 32 * q, r[q]);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(smem_u32(&sm.acc_empty[buf]) & TC_PEER_BIT_MASK);
        const int r_first = m0 + quarter * 32;
#pragma unroll
        for (int h = 0; h < NLD / 2; ++h) {
          uint32_t pk[32];
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            __nv_bfloat162 pa = __floats2bfloat162_rn(__uint_as_float(r[2 * h][j]), __uint_as_float(r[2 * h][j + 1]));
            __nv_bfloat162 pb = __floats2bfloat162_rn(__uint_as_float(r[2 * h + 1][j]), __uint_as_float(r[2 * h + 1][j + 1]));
            pk[j >> 1] = *reinterpret_cast<uint32_t*>(&pa);
            pk[16 + (j >> 1)] = *reinterpret_cast<uint32_t*>(&pb);
          }
          const int c0 = ch * (BN / 2) + 64 * h;
          pr_store_block<64>(reinterpret_cast<unsigned char*>(sm.stage) + (warp - 2) * 4096, pk,
                             reinterpret_cast<__nv_bfloat16*>(out) + (size_t)r_first * N + n0 + c0, (size_t)N,
                             M - r_first, N - (n0 + c0), lane);
        }
      } else {
#pragma unroll 1
      for (int c0 = ch * (BN / 2); c0 < (ch + 1) * (BN / 2); c0 += 32) {
        uint32_t r[32];
        tc_ld_32x32b_x32(tmem + ((uint32_t)(quarter * 32) << 16) + buf * BN + c0, r);
        tc_wait_ld();
        if (c0 + 32 == (ch + 1) * (BN / 2)) {
          // the accumulator is in registers: tell the leading CTA's MMA thread
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(smem_u32(&sm.acc_empty[buf]) & TC_PEER_BIT_MASK);
        }
        if (row < M && n0 + c0 < N) {
          TOut* dst = out + (size_t)row * N + n0 + c0;
          if (n0 + c0 + 32 <= N && (N % 8) == 0) {
            if constexpr (sizeof(TOut) == 2) {
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
      }   // plain epilogue
      QE_TL_STAMP(warp == 2 && lane == 0 ? 17 + 2 * (it > 0) : -1);   // (... an epilogue warp is done with a tile: the first, the last)
    }
  }
  if (splits > 1) {
    // ---- K split over the cluster's pairs: the shares meet ------------------------------------------------
    // Every CTA finishes 1 / splits of the columns of its 128 rows: it adds up, in the order of the shares, what
    // the CTAs with its rows (the same parity in every pair) hold for those columns, and stores them, lanes along
    // the columns.  Reached by every thread of the cluster, whatever happened before.
    cluster_sync_all();
    if (warp >= 2 && split_staged) {
      const int tile = pair;
      const int m0 = (tile / n_blocks) * 2 * PR_BM + (int)rank * PR_BM, n0 = (tile % n_blocks) * BN;
      if (splits == 2) pr_meet_shares<TOut, BN, 2>(reinterpret_cast<const unsigned char*>(sm.a), out, M, N, m0, n0, rank, cpair);
      else pr_meet_shares<TOut, BN, 4>(reinterpret_cast<const unsigned char*>(sm.a), out, M, N, m0, n0, rank, cpair);
    }
  }
  // both CTAs meet here: neither leaves while the other may still signal its barriers, read its
  // shared memory or write its tensor memory; then the allocating warps free the tensor memory
  QE_TL_STAMP(threadIdx.x == 0 ? 24 : -1);          // (... all roles done in this CTA's first thread)
  pdl_wait();                                        // no thread leaves before the kernel before this one has completed
  tc_fence_before();
  cluster_sync_all();
  QE_TL_STAMP(threadIdx.x == 0 ? 25 : -1);          // (timeline build: the tail's barrier passed)
  if (warp == 1) {
    tc_fence_after();
    tc_dealloc_pair(tmem, TMEM_COLS);
  }
  QE_TL_FLUSH_STAMPS();
}

template <int BN, int STAGES, bool SWIGLU = false, bool ROPE = false>
static int launch_pair(const void* x, const void* w, void* out, int M, int N, int K, int out_f32, int sms, cudaStream_t stream,
                       PrRope rp = PrRope{}, int splits = 1) {
  const int n_up = SWIGLU ? N / 2 : 0;
  CUtensorMap map_x, map_w;
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    const uint64_t strides[1] = {(uint64_t)K * 2};
    const uint32_t box[2] = {PR_BK, PR_BM};
    if (!qe_tensor_map_bf16(x, 2, dims, strides, box, &map_x)) return 1;
  }
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    const uint64_t strides[1] = {(uint64_t)K * 2};
    const uint32_t box[2] = {PR_BK, BN / 2};
    if (!qe_tensor_map_bf16(w, 2, dims, strides, box, &map_w)) return 1;
  }
#ifdef QE_TIMELINE
  // (the timeline build's stamps are 256 bytes of static shared memory, which precede the dynamic part and count as
  // part of the slack for its alignment: the variant with the staged head uses every byte an SM has)
  const size_t smem = sizeof(PrSmem<BN, STAGES, ROPE>) + 1024 - 256;
#else
  const size_t smem = sizeof(PrSmem<BN, STAGES, ROPE>) + 1024;
#endif
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<__nv_bfloat16, BN, STAGES, SWIGLU, ROPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if constexpr (!ROPE)
      if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<float, BN, STAGES, SWIGLU, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) QE_REFUSE("linear_tcgen05_pair: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  const long n_blocks = SWIGLU ? (n_up + BN / 2 - 1) / (BN / 2) : (N + BN - 1) / BN;
  const long tiles = n_blocks * ((M + 2 * PR_BM - 1) / (2 * PR_BM));
  // one cluster per pair of SMs walks over the tiles; with K split, a cluster of `splits` pairs per tile
  const long pairs = splits > 1 ? tiles * splits : (tiles < sms / 2 ? tiles : sms / 2);
  const dim3 grid((unsigned)(2 * pairs));
  const unsigned cluster = 2u * (unsigned)splits;
  if constexpr (ROPE) {
    qe_launch_cluster(gemm_tcgen05_pair_kernel<__nv_bfloat16, BN, STAGES, false, true>, grid, dim3(PR_THREADS), smem, stream, cluster, map_x, map_w, (__nv_bfloat16*)out, M, N, K, n_up, rp, 1);
  } else {
    if (out_f32)
      qe_launch_cluster(gemm_tcgen05_pair_kernel<float, BN, STAGES, SWIGLU, false>, grid, dim3(PR_THREADS), smem, stream, cluster, map_x, map_w, (float*)out, M, N, K, n_up, rp, splits);
    else
      qe_launch_cluster(gemm_tcgen05_pair_kernel<__nv_bfloat16, BN, STAGES, SWIGLU, false>, grid, dim3(PR_THREADS), smem, stream, cluster, map_x, map_w, (__nv_bfloat16*)out, M, N, K, n_up, rp, splits);
  }
  QE_CHECK_LAUNCH("linear_tcgen05_pair");
  return 0;
}

// How many clusters of `cluster_ctas` CTAs of the plain 256-column kernel the device holds at once (their shared
// memory leaves room for one CTA per SM, and a cluster has to lie in one GPC); 0 if the driver cannot say.
extern "C" int qe_pair_max_active_clusters(int cluster_ctas) {
  static int cached[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
  if (cluster_ctas < 2 || cluster_ctas > 8) return 0;
  if (cached[cluster_ctas] == 0) {
    const size_t smem = sizeof(PrSmem<256, 6, false>) + 1024;
    auto kernel = gemm_tcgen05_pair_kernel<__nv_bfloat16, 256, 6, false, false>;
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)cluster_ctas * 64);
    cfg.blockDim = dim3(PR_THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster_ctas;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) { cudaGetLastError(); n = -1; }
    cached[cluster_ctas] = n > 0 ? n : -1;
  }
  return cached[cluster_ctas] > 0 ? cached[cluster_ctas] : 0;
}

// Which tcgen05 product kernel serves a plain bfloat16 product, by a model of their times fitted to measurements on
// a B200 (microseconds; kb: k-blocks of 64; rounds: tiles per CTA or cluster):
//   one CTA per 128 x 128 tile (gemm_tcgen05.cu)        2.1 + rounds x kb x 0.36
//   a pair per 256 x 128 tile                           5.4 + rounds x kb x 0.31
//   a pair per 256 x 256 tile                           3.1 + rounds x (0.4 + kb x 0.42)
//   2 or 4 pairs per 256 x 256 tile, a share of K each  8.0 + kb / pairs x 0.33   (one tile per cluster; the device
//                                                       holds 33 clusters of 4 CTAs and 15 of 8 at once)
// (2048 rows: 1024 x 2048 13.7 / 15.3 / - / 12.7 us, 1024 x 3072 19.4 / 20.3 / - / 15.3, 2048 x 2048 24.4 / - / 16.9 / -,
// 4096 x 1024 17.7 / - / 17.3 / -; 528 rows: 1024 x 3072 19.9 / 21.3 / - / 13.2, 4096 x 1024 13.3 / - / 11.3 / -.)
// Returns 0: the single-CTA kernel, 1: pairs with narrow tiles, 2: pairs with wide tiles, 3 / 4: wide tiles with K
// split over 2 / 4 pairs.  `pairs_only`: the best of 1..4.
static int g_pair_split_max = 4;
extern "C" void qe_pair_k_splits_max(int splits) { g_pair_split_max = splits < 1 ? 1 : (splits > 4 ? 4 : splits); }
extern "C" int qe_tc_product_plan(int M, int N, int K, int pairs_only) {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0, v = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    sms = v > 1 ? v : 148;
  }
  if (M <= 0 || N <= 0 || K <= 0) return pairs_only ? 1 : 0;
  const double kb = (double)((K + PR_BK - 1) / PR_BK);
  auto rounds = [](long tiles, long slots) { return (double)((tiles + slots - 1) / slots); };
  const long m128 = (M + 127) / 128, m256 = (M + 255) / 256, n128 = (N + 127) / 128, n256 = (N + 255) / 256;
  double best = pairs_only ? 1e30 : 2.1 + rounds(m128 * n128, sms) * kb * 0.36;
  int plan = 0;
  const double narrow = 5.4 + rounds(m256 * n128, sms / 2) * kb * 0.31;
  if (narrow < best) { best = narrow; plan = 1; }
  const double wide = 3.1 + rounds(m256 * n256, sms / 2) * (0.4 + kb * 0.42);
  if (wide < best) { best = wide; plan = 2; }
  for (int s = 2; s <= g_pair_split_max; s <<= 1) {
    const int cap = qe_pair_max_active_clusters(2 * s);
    if (N % 8 || m256 * n256 > cap || kb < 4 * s) continue;
    const double split = 8.0 + (double)(((long)kb + s - 1) / s) * 0.33;
    if (split < best) { best = split; plan = s == 2 ? 3 : 4; }
  }
  return plan;
}
// Into how many pairs per tile the CTA-pair product splits K for this shape (1: it does not).
extern "C" int qe_pair_k_splits(int M, int N, int K, int sms) {
  (void)sms;
  const int plan = qe_tc_product_plan(M, N, K, 1);
  return plan == 3 ? 2 : (plan == 4 ? 4 : 1);
}

extern "C" int qe_gemm_tc_pair_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int));
  return v;
}
extern "C" void qe_gemm_tc_pair_clear_status() {
  int v = 0;
  cudaMemcpyToSymbol(g_tc_status, &v, sizeof(int));
}

// Returns 0 when run, 1 when refused (qe_last_error says why), 2 on a launch error.
extern "C" int qe_linear_tcgen05_pair(const void* x, const void* w, void* out, int M, int N, int K, int out_f32,
                                      cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8) QE_REFUSE("linear_tcgen05_pair: K = %d is not a positive multiple of 8", K);
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) QE_REFUSE("linear_tcgen05_pair: operands must be 16-byte aligned");
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms < 2) QE_REFUSE("linear_tcgen05_pair: needs at least two SMs");
  // wide tiles, wide tiles with K split over 2 or 4 pairs, or narrow tiles: see qe_tc_product_plan
  const int plan = qe_tc_product_plan(M, N, K, 1);
  if (plan == 2) return launch_pair<256, 6>(x, w, out, M, N, K, out_f32, sms, stream);
  if (plan >= 3) return launch_pair<256, 6>(x, w, out, M, N, K, out_f32, sms, stream, PrRope{}, plan == 3 ? 2 : 4);
  return launch_pair<128, 8>(x, w, out, M, N, K, out_f32, sms, stream);
}

// out[M, I] = silu(x · w[:I]^T) * (x · w[I:]^T) for the stacked gate and up weights w [2 I, K] (see SWIGLU
// above).  Returns 0 when run, 1 when refused, 2 on a launch error.
extern "C" int qe_linear_swiglu_tcgen05_pair(const void* x, const void* w, void* out, int M, int I, int K, int out_f32,
                                             cudaStream_t stream) {
  if (M <= 0 || I <= 0) return 0;
  if (K <= 0 || K % 8) QE_REFUSE("linear_swiglu: K = %d is not a positive multiple of 8", K);
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) QE_REFUSE("linear_swiglu: operands must be 16-byte aligned");
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms < 2) QE_REFUSE("linear_swiglu: needs at least two SMs");
  return launch_pair<256, 6, true>(x, w, out, M, 2 * I, K, out_f32, sms, stream);
}

// out[M, N] = the q columns of x · w^T for the stacked q, k, v weights w [N = (Hq + 2 Hkv) 128, K], normed per head
// and rotated; the k and v columns go into the cache `pages` [pages, 2, Hkv, page_size, 128] at slot_mapping[row]
// (write_kv 0: they are dropped: a layer that reads another layer's cache) and out's k and v columns are left as
// they were (see ROPE above).  qw, kw: float32 [128] or null; cos_sin: float32 [M, 64, 2] or null.
// Returns 0 when run, 1 when refused, 2 on a launch error.
extern "C" int qe_linear_qkv_rope_tcgen05_pair(const void* x, const void* w, void* out, int M, int N, int K,
                                               const float* qw, const float* kw, float eps, const void* cos_sin,
                                               void* pages, const int* slot_mapping, int Hq, int Hkv, int page_size,
                                               int write_kv, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8) QE_REFUSE("linear_qkv_rope: K = %d is not a positive multiple of 8", K);
  if (Hq < 1 || Hkv < 1 || N != (Hq + 2 * Hkv) * 128) QE_REFUSE("linear_qkv_rope: N = %d is not (%d + 2 x %d) heads of 128", N, Hq, Hkv);
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out | (uintptr_t)qw | (uintptr_t)kw | (uintptr_t)cos_sin | (uintptr_t)pages) & 15)
    QE_REFUSE("linear_qkv_rope: operands must be 16-byte aligned");
  if (write_kv && (!pages || !slot_mapping || page_size < 1)) QE_REFUSE("linear_qkv_rope: cache write without a cache");
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms < 2) QE_REFUSE("linear_qkv_rope: needs at least two SMs");
  PrRope rp{qw, kw, eps, (const float2*)cos_sin, (__nv_bfloat16*)pages, slot_mapping, Hq, Hkv, page_size, write_kv ? 1 : 0};
  return launch_pair<256, 6, false, true>(x, w, out, M, N, K, 0, sms, stream, rp);
}
