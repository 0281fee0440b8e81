// out[M, N] = x[M, K] · w[N, K]^T in bfloat16 for many rows, by pairs of CTAs (tcgen05 cta_group::2):
// two CTAs on neighbouring SMs share one 256 x BN output tile.  Each brings its own 128 rows of x and
// only its half of the BN rows of w; one thread of the leading CTA issues MMAs that read both CTAs'
// shared memory and write both CTAs' tensor memory.  An SM so fetches a quarter less (BN = 128) or a
// third less (BN = 256) from L2 per multiply-add than alone with a 128 x BN tile, and what an SM can
// pull from L2 is what bounds these products.  (Contract of the reference's linear,
// src/layers/ops/linear.py:101-122.)
//
// Persistent: a cluster of two CTAs per pair of SMs walks over the tiles.  Per CTA 6 warps: warp 0
// feeds TMA (its loads count their bytes on the leading CTA's `full` barrier), warp 1 owns tensor
// memory (and, in the leading CTA, issues the MMAs), warps 2-5 read this CTA's 128 rows of the
// accumulator and store them.  `empty` and `acc_full` are signalled to both CTAs by tcgen05.commit
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
#define PR_THREADS 192

static __device__ int g_tc_status = 0;      // 0 = fine; else code of the first wait that ran out

template <int BN, int STAGES>
struct __align__(1024) PrSmem {
  __nv_bfloat16 a[STAGES][PR_BM * PR_BK];            // 16 KB each
  __nv_bfloat16 b[STAGES][(BN / 2) * PR_BK];         // this CTA's half of the tile's rows of w
  uint64_t full[STAGES];                             // used in the leading CTA
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];                             // used in the leading CTA
  uint32_t tmem_base;
  int abort_flag;
};

// N: columns of the product (SWIGLU: 2 I); n_up: SWIGLU: the first row of up in w (= I), else 0
template <typename TOut, int BN, int STAGES, bool SWIGLU, bool ROPE = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PR_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                         TOut* __restrict__ out, int M, int N, int K, int n_up, PrRope rp) {
  static_assert(!SWIGLU || BN == 256, "the fused activation pairs 128 columns of gate with 128 of up");
  static_assert(!ROPE || (BN == 256 && !SWIGLU && sizeof(TOut) == 2), "the fused rotation takes two heads of 128 per tile, in bfloat16");
  extern __shared__ unsigned char smem_raw[];
  using Smem = PrSmem<BN, STAGES>;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  constexpr uint32_t STAGE_BYTES = (PR_BM + BN / 2) * PR_BK * sizeof(__nv_bfloat16);
  pdl_launch_dependents();
  Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();          // 0: the leading CTA of the pair
  const int num_kb = (K + PR_BK - 1) / PR_BK;
  const int n_blocks = SWIGLU ? (n_up + BN / 2 - 1) / (BN / 2) : (N + BN - 1) / BN;
  const int n_tiles = n_blocks * ((M + 2 * PR_BM - 1) / (2 * PR_BM));
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  volatile int* abort_flag = &sm.abort_flag;

  // Everything up to the first load of x needs nothing from the kernel before this one (the weights
  // are nobody's output): it runs before the wait for that kernel.
  if (threadIdx.x == 0) {
    tma_prefetch_map(&map_x);
    tma_prefetch_map(&map_w);
    for (int s = 0; s < STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&sm.acc_full[s], 1); mbar_init(&sm.acc_empty[s], 8); }
    sm.abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) tc_alloc_pair(&sm.tmem_base, TMEM_COLS);   // the same warp in both CTAs
  tc_fence_before();
  cluster_sync_all();                                // barriers and tensor memory of both CTAs are ready
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;

  if (warp == 0) {
    // ---- producer: this CTA's rows of x and its half of the rows of w; bytes counted in the leading CTA
    if (lane == 0) {
      const int my_tiles = pair < n_tiles ? (n_tiles - pair + n_pairs - 1) / n_pairs : 0;
      const uint32_t total = (uint32_t)my_tiles * (uint32_t)num_kb;      // k-blocks of all this pair's tiles
      const uint32_t ahead = total < (uint32_t)STAGES ? total : (uint32_t)STAGES;
      auto coords = [&](uint32_t kc, int& m0, int& n0, int& kb) {
        const int t = (int)(kc / (uint32_t)num_kb);
        kb = (int)(kc - (uint32_t)t * (uint32_t)num_kb);
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
          tc_commit_pair(&sm.empty[s], 3);             // both CTAs' producers may refill the slot
        }
        if (ok) tc_commit_pair(&sm.acc_full[buf], 3);
      }
    }
  } else {
    // ---- epilogue: this CTA's 128 rows of the accumulator ----------------------------------------
    const int quarter = warp & 3;
    int it = 0;
    for (int tile = pair; tile < n_tiles; tile += n_pairs, ++it) {
      const int buf = it & 1;
      const int m0 = (tile / n_blocks) * 2 * PR_BM + (int)rank * PR_BM, n0 = (tile % n_blocks) * BN;
      const bool ok = __all_sync(0xffffffffu, mbar_wait(&sm.acc_full[buf], (it >> 1) & 1, abort_flag, 23, &g_tc_status));
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      if constexpr (SWIGLU) {
        // columns c0.. of gate and of up -> 32 columns of the activation
        const int I = n_up, i0 = (tile % n_blocks) * (BN / 2);
#pragma unroll 1
        for (int c0 = 0; c0 < BN / 2; c0 += 32) {
          uint32_t g[32], u[32];
          tc_ld_32x32b_x32(tmem + ((uint32_t)(quarter * 32) << 16) + buf * BN + c0, g);
          tc_ld_32x32b_x32(tmem + ((uint32_t)(quarter * 32) << 16) + buf * BN + BN / 2 + c0, u);
          tc_wait_ld();
          if (c0 + 32 == BN / 2) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(smem_u32(&sm.acc_empty[buf]) & TC_PEER_BIT_MASK);
          }
          if (row < M && i0 + c0 < I) {
            float a[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float gv = __uint_as_float(g[j]);
              a[j] = __fdividef(gv, 1.f + __expf(-gv)) * __uint_as_float(u[j]);
            }
            TOut* dst = out + (size_t)row * I + i0 + c0;
            if (i0 + c0 + 32 <= I && (I % 8) == 0 && sizeof(TOut) == 2) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 v;
                __nv_bfloat162 p0 = __floats2bfloat162_rn(a[j], a[j + 1]), p1 = __floats2bfloat162_rn(a[j + 2], a[j + 3]);
                __nv_bfloat162 p2 = __floats2bfloat162_rn(a[j + 4], a[j + 5]), p3 = __floats2bfloat162_rn(a[j + 6], a[j + 7]);
                v.x = *reinterpret_cast<uint32_t*>(&p0); v.y = *reinterpret_cast<uint32_t*>(&p1);
                v.z = *reinterpret_cast<uint32_t*>(&p2); v.w = *reinterpret_cast<uint32_t*>(&p3);
                *reinterpret_cast<uint4*>(dst + j) = v;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (i0 + c0 + j < I) dst[j] = from_f32<TOut>(a[j]);
            }
          }
        }
      } else if constexpr (ROPE) {
        // two heads of 128 columns; this thread holds its token's whole head.  Per head two passes over the
        // accumulator (tensor memory is cheap to read again): the sum of squares, then, for the columns
        // (0-31, 64-95) and (32-63, 96-127), norm, rotation and store, with the angles' loads in flight
        // beside the accumulator's.
        const bool row_ok = row < M;
        int slot = 0;
        if (row_ok && rp.write_kv) slot = __ldg(rp.slot_mapping + row);
        const float4* tp = reinterpret_cast<const float4*>(rp.cos_sin + (size_t)(row_ok ? row : 0) * 64);
        const uint32_t tm_row = tmem + ((uint32_t)(quarter * 32) << 16) + buf * BN;
        auto rnd = [](uint32_t u) { return __bfloat162float(__float2bfloat16_rn(__uint_as_float(u))); };   // as the plain product's output is rounded
#pragma unroll 1
        for (int hh = 0; hh < 2; ++hh) {
          const int col0 = n0 + hh * 128, head = col0 >> 7;
          const bool is_q = head < rp.Hq, is_v = head >= rp.Hq + rp.Hkv;
          const bool wanted = row_ok && col0 < N && (is_q || rp.write_kv);   // (keys and values of a layer that reads another's cache are dropped)
          const float* w = is_v ? nullptr : (is_q ? rp.qw : rp.kw);
          float rstd = 1.f;
          if (w) {                                   // warp-uniform
            float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < 4; c += 2) {
              uint32_t a[32], b[32];
              tc_ld_32x32b_x32(tm_row + hh * 128 + c * 32, a);
              tc_ld_32x32b_x32(tm_row + hh * 128 + c * 32 + 32, b);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; i += 2) {
                const float a0 = rnd(a[i]), a1 = rnd(a[i + 1]), b0 = rnd(b[i]), b1 = rnd(b[i + 1]);
                s4[0] = fmaf(a0, a0, s4[0]); s4[1] = fmaf(a1, a1, s4[1]); s4[2] = fmaf(b0, b0, s4[2]); s4[3] = fmaf(b1, b1, s4[3]);
              }
            }
            rstd = rsqrtf(((s4[0] + s4[1]) + (s4[2] + s4[3])) / 128.f + rp.eps);
          }
          __nv_bfloat16* dst = nullptr;
          if (wanted) {
            if (is_q) {
              dst = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)row * N + col0;
            } else {
              // slot = page * page_size + off: the row of (page, K or V, h, off) in the cache
              const int h = is_v ? head - rp.Hq - rp.Hkv : head - rp.Hq;
              const int page = (rp.page_size & (rp.page_size - 1)) == 0 ? slot >> (__ffs(rp.page_size) - 1) : slot / rp.page_size;
              dst = rp.pages + ((size_t)slot + ((size_t)page * (2 * rp.Hkv - 1) + (is_v ? rp.Hkv : 0) + h) * rp.page_size) * 128;
            }
          }
#pragma unroll
          for (int half = 0; half < 2; ++half) {     // columns 32 half .. + 31 and their partners 64 further
            uint32_t lo[32], hi[32];
            tc_ld_32x32b_x32(tm_row + hh * 128 + half * 32, lo);
            tc_ld_32x32b_x32(tm_row + hh * 128 + 64 + half * 32, hi);
            float4 t[16];
            const bool rotate = !is_v && rp.cos_sin != nullptr;
            if (rotate && wanted) {
#pragma unroll
              for (int j = 0; j < 16; ++j) t[j] = __ldg(tp + half * 16 + j);     // (cos, sin) of elements 32 half + 2j, + 2j + 1
            }
            tc_wait_ld();
            if (hh == 1 && half == 1) {
              // the accumulator is in registers: tell the leading CTA's MMA thread
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive_cluster(smem_u32(&sm.acc_empty[buf]) & TC_PEER_BIT_MASK);
            }
            if (!wanted) continue;
            float xl[32], xh[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) { xl[i] = rnd(lo[i]); xh[i] = rnd(hi[i]); }
            if (w) {
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                const float4 wl = __ldg(reinterpret_cast<const float4*>(w + half * 32 + i));
                const float4 wh = __ldg(reinterpret_cast<const float4*>(w + 64 + half * 32 + i));
                xl[i] = xl[i] * rstd * wl.x; xl[i + 1] = xl[i + 1] * rstd * wl.y; xl[i + 2] = xl[i + 2] * rstd * wl.z; xl[i + 3] = xl[i + 3] * rstd * wl.w;
                xh[i] = xh[i] * rstd * wh.x; xh[i + 1] = xh[i + 1] * rstd * wh.y; xh[i + 2] = xh[i + 2] * rstd * wh.z; xh[i + 3] = xh[i + 3] * rstd * wh.w;
              }
            }
            if (rotate) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float l0 = xl[2 * j], h0 = xh[2 * j], l1 = xl[2 * j + 1], h1 = xh[2 * j + 1];
                xl[2 * j] = t[j].x * l0 - t[j].y * h0;      xh[2 * j] = t[j].y * l0 + t[j].x * h0;
                xl[2 * j + 1] = t[j].z * l1 - t[j].w * h1;  xh[2 * j + 1] = t[j].w * l1 + t[j].z * h1;
              }
            }
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 v, u;
              __nv_bfloat162 p0 = __floats2bfloat162_rn(xl[j], xl[j + 1]), p1 = __floats2bfloat162_rn(xl[j + 2], xl[j + 3]);
              __nv_bfloat162 p2 = __floats2bfloat162_rn(xl[j + 4], xl[j + 5]), p3 = __floats2bfloat162_rn(xl[j + 6], xl[j + 7]);
              v.x = *reinterpret_cast<uint32_t*>(&p0); v.y = *reinterpret_cast<uint32_t*>(&p1);
              v.z = *reinterpret_cast<uint32_t*>(&p2); v.w = *reinterpret_cast<uint32_t*>(&p3);
              __nv_bfloat162 q0 = __floats2bfloat162_rn(xh[j], xh[j + 1]), q1 = __floats2bfloat162_rn(xh[j + 2], xh[j + 3]);
              __nv_bfloat162 q2 = __floats2bfloat162_rn(xh[j + 4], xh[j + 5]), q3 = __floats2bfloat162_rn(xh[j + 6], xh[j + 7]);
              u.x = *reinterpret_cast<uint32_t*>(&q0); u.y = *reinterpret_cast<uint32_t*>(&q1);
              u.z = *reinterpret_cast<uint32_t*>(&q2); u.w = *reinterpret_cast<uint32_t*>(&q3);
              *reinterpret_cast<uint4*>(dst + half * 32 + j) = v;
              *reinterpret_cast<uint4*>(dst + 64 + half * 32 + j) = u;
            }
          }
        }
      } else {
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tc_ld_32x32b_x32(tmem + ((uint32_t)(quarter * 32) << 16) + buf * BN + c0, r);
        tc_wait_ld();
        if (c0 + 32 == BN) {
          // the accumulator is in registers: tell the leading CTA's MMA thread
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(smem_u32(&sm.acc_empty[buf]) & TC_PEER_BIT_MASK);
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
      }   // plain epilogue
    }
  }
  // both CTAs meet here: neither leaves while the other may still signal its barriers, read its
  // shared memory or write its tensor memory; then the allocating warps free the tensor memory
  pdl_wait();                                        // no thread leaves before the kernel before this one has completed
  tc_fence_before();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tc_dealloc_pair(tmem, TMEM_COLS);
  }
}

template <int BN, int STAGES, bool SWIGLU = false, bool ROPE = false>
static int launch_pair(const void* x, const void* w, void* out, int M, int N, int K, int out_f32, int sms, cudaStream_t stream,
                       PrRope rp = PrRope{}) {
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
  const size_t smem = sizeof(PrSmem<BN, STAGES>) + 1024;
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
  const long pairs = tiles < sms / 2 ? tiles : sms / 2;
  const dim3 grid((unsigned)(2 * pairs));
  if constexpr (ROPE) {
    qe_launch(gemm_tcgen05_pair_kernel<__nv_bfloat16, BN, STAGES, false, true>, grid, dim3(PR_THREADS), smem, stream, map_x, map_w, (__nv_bfloat16*)out, M, N, K, n_up, rp);
  } else {
    if (out_f32)
      qe_launch(gemm_tcgen05_pair_kernel<float, BN, STAGES, SWIGLU, false>, grid, dim3(PR_THREADS), smem, stream, map_x, map_w, (float*)out, M, N, K, n_up, rp);
    else
      qe_launch(gemm_tcgen05_pair_kernel<__nv_bfloat16, BN, STAGES, SWIGLU, false>, grid, dim3(PR_THREADS), smem, stream, map_x, map_w, (__nv_bfloat16*)out, M, N, K, n_up, rp);
  }
  QE_CHECK_LAUNCH("linear_tcgen05_pair");
  return 0;
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
  // wide tiles when they give every pair of SMs a tile; else narrow ones
  const long wide_tiles = (long)((N + 255) / 256) * ((M + 2 * PR_BM - 1) / (2 * PR_BM));
  if (wide_tiles >= sms / 2) return launch_pair<256, 6>(x, w, out, M, N, K, out_f32, sms, stream);
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
