// Flash attention over the paged cache in bfloat16 with tensor cores (mma.sync.m16n8k16), for
// prompt portions and for decoded tokens alike.
//
// One CTA serves one kv head and a tile of 64 "rows": a row is (query token, query head of the kv
// head's group), so the keys and values of a kv head are read once for all its query heads (the
// reference reads them once per query head, src/layers/fused_ops/attn.py:181-182, 405-406).  Keys come
// in tiles of 64 through a two-stage cp.async pipeline, gathered page by page from the block table.
// Scores, running max, running sum and the output accumulator are float32; P is rounded to
// bfloat16 before P·V (attn.py:263); the mask is key <= position (and > position - window)
// (attn.py:195, 239).  Tiles above the causal frontier are never visited.
//
// A work item may cover only a range of keys (a split of a long context for a decoded token:
// flash decoding, attn.py:374-594 with split_size 256); then it writes its unnormalised
// accumulator with max and sum in float32 to scratch memory and a merge kernel combines the parts.
//
// Work items (int32 x 12): req, q0 (first token of the tile within the request's new tokens),
// kv_lo, kv_hi (key range; kv_hi is further capped by causality), part (-1: write the output;
// else index of the partial), n_splits, split (when n_splits > 0 the key range is computed here
// from the request's length: the keys from the window's start on, cut into n_splits equal runs
// of whole key tiles, of which this item takes run `split`), then the request's first row in the
// flat batch, its number of new tokens and its tokens already in the cache (copies of cu_q and
// ctx_lens, so that a CTA needs one load to know its work), 2 unused.
// Merge items (int32 x 4): req, q0, first part, number of parts.
#pragma once
#include "common.cuh"
#include <math.h>

#define FA_BM 64
#define FA_BN 64
#define FA_WARPS 4
#define FA_THREADS (FA_WARPS * 32)
#define FA_ITEM_INTS 12

__device__ __forceinline__ void fa_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"(a), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" :: "n"(N)); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// One warp's share of a key tile: rows [row_base, row_base + 16) of the query tile against NB blocks
// of 16 keys starting at block kb0 of the tile.  Updates the rows' running max, sum and output.
// `all_allowed`: every key of the tile is allowed for every row of the warp (a tile below the causal
// diagonal, inside the key range and the window): the mask is skipped (uniform over the warp).
template <int D, int NB>
__device__ __forceinline__ void fa_tile(const __nv_bfloat16* sq, const __nv_bfloat16* tk, const __nv_bfloat16* tv,
                                        int row_base, int kb0, int kt, int kv_begin, int kv_end, int pos_lo, int pos_hi,
                                        int window, float scale_log2, int lane, float& m_lo, float& m_hi, float& l_lo,
                                        float& l_hi, float (&o)[D / 8][4], bool all_allowed) {
  constexpr int LD = D + 8, KS = D / 16;
  const int c = lane & 3;
  // ---- S = Q K^T ---------------------------------------------------------------------------
  float s[2 * NB][4];
#pragma unroll
  for (int i = 0; i < 2 * NB; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    uint32_t a[4];
    // A fragment of Q: matrices (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15)
    ldsm_x4(a, sq + (row_base + (lane & 15)) * LD + ks * 16 + (lane >> 4) * 8);
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      uint32_t b[4];
      // B fragments of two groups of 8 keys: (keys 0-7, k 0-7), (keys 0-7, k 8-15), (keys 8-15, k 0-7), (keys 8-15, k 8-15)
      ldsm_x4(b, tk + ((kb0 + nb) * 16 + (lane >> 4) * 8 + (lane & 7)) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
      fa_mma(s[2 * nb], a, b[0], b[1]);
      fa_mma(s[2 * nb + 1], a, b[2], b[3]);
    }
  }
  // ---- mask, online softmax --------------------------------------------------------------------
  float mx_lo = -INFINITY, mx_hi = -INFINITY;
  if (all_allowed) {
#pragma unroll
    for (int i = 0; i < 2 * NB; ++i) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        s[i][e] *= scale_log2;
        s[i][2 + e] *= scale_log2;
        mx_lo = fmaxf(mx_lo, s[i][e]);
        mx_hi = fmaxf(mx_hi, s[i][2 + e]);
      }
    }
  } else
#pragma unroll
  for (int i = 0; i < 2 * NB; ++i) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int key = kt + kb0 * 16 + i * 8 + 2 * c + e;
      const bool in_range = key >= kv_begin && key < kv_end;
      const bool ok_lo = in_range && key <= pos_lo && (window <= 0 || key > pos_lo - window);
      const bool ok_hi = in_range && key <= pos_hi && (window <= 0 || key > pos_hi - window);
      s[i][e] = ok_lo ? s[i][e] * scale_log2 : -INFINITY;
      s[i][2 + e] = ok_hi ? s[i][2 + e] * scale_log2 : -INFINITY;
      mx_lo = fmaxf(mx_lo, s[i][e]);
      mx_hi = fmaxf(mx_hi, s[i][2 + e]);
    }
  }
  mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
  mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
  mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
  mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
  const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
  const float base_lo = mn_lo == -INFINITY ? 0.f : mn_lo;      // a row with nothing allowed so far
  const float base_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
  const float al_lo = exp2f(m_lo - base_lo), al_hi = exp2f(m_hi - base_hi);
  m_lo = mn_lo; m_hi = mn_hi;
  float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
  for (int i = 0; i < 2 * NB; ++i) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      s[i][e] = exp2f(s[i][e] - base_lo);
      s[i][2 + e] = exp2f(s[i][2 + e] - base_hi);
      sum_lo += s[i][e];
      sum_hi += s[i][2 + e];
    }
  }
  sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
  sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
  sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
  sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
  l_lo = l_lo * al_lo + sum_lo;
  l_hi = l_hi * al_hi + sum_hi;
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { o[i][0] *= al_lo; o[i][1] *= al_lo; o[i][2] *= al_hi; o[i][3] *= al_hi; }
  // ---- O += P V --------------------------------------------------------------------------------
#pragma unroll
  for (int kk = 0; kk < NB; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int dp = 0; dp < D / 16; ++dp) {
      uint32_t b[4];
      // transposed loads of V: (keys 0-7, d 0-7), (keys 8-15, d 0-7), (keys 0-7, d 8-15), (keys 8-15, d 8-15)
      ldsm_x4_t(b, tv + ((kb0 + kk) * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LD + dp * 16 + (lane >> 4) * 8);
      fa_mma(o[2 * dp], a, b[0], b[1]);
      fa_mma(o[2 * dp + 1], a, b[2], b[3]);
    }
  }
}

// Combine the parts of one (request, kv head): out = sum_s 2^(m_s - m) acc_s / sum_s 2^(m_s - m) l_s
// (reference attn.py:520-594), in float32, in the order of the parts.  Run by a whole CTA.
template <int D>
__device__ __forceinline__ void fa_merge_parts(const float* part_acc, const float* part_ml, int part_rows, int first,
                                               int n, int hkv, int Hkv, int nrows, int G, int Hq,
                                               __nv_bfloat16* out_row0 /* row of the tile's first token */) {
  for (int e = threadIdx.x; e < nrows * D; e += FA_THREADS) {       // the computing threads only
    const int r = e / D, d = e - r * D;
    float m = -INFINITY;
    for (int sp = 0; sp < n; ++sp) m = fmaxf(m, __ldcg(part_ml + 2 * ((((size_t)first + sp) * Hkv + hkv) * part_rows + r)));
    if (m == -INFINITY) m = 0.f;          // every part of the row empty: weights 0, not exp2(-inf + inf)
    float l = 0.f, acc = 0.f;
    for (int sp = 0; sp < n; ++sp) {
      const size_t slot = (((size_t)first + sp) * Hkv + hkv) * part_rows + r;
      const float wgt = exp2f(__ldcg(part_ml + 2 * slot) - m);
      l += wgt * __ldcg(part_ml + 2 * slot + 1);
      acc += wgt * __ldcg(part_acc + slot * D + d);
    }
    const int ti = r / G, hg = r - ti * G;
    out_row0[(size_t)ti * ((size_t)Hq * D) + (size_t)(hkv * G + hg) * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
  }
}

// D: head size, a multiple of 16 up to 256.  Rows of the shared-memory tiles are padded by 16 bytes
// so that the 8 row addresses of an ldmatrix fall into different banks for every D.
//
// Two ways of sharing a key tile between the 4 warps.  A tile of many rows (a prompt portion): each
// warp owns 16 rows and visits all 64 keys.  A tile of at most 16 rows (decoded tokens: the query
// heads of one group): every warp takes the same rows and 16 of the 64 keys, with a running max, sum
// and output of its own; the four are combined in shared memory at the end.
//
// `counters` (may be null): one int per (first part, kv head), zero before the launch.  The CTA that
// finishes a request's last part combines the parts itself and sets the counter back to zero, so no
// merge kernel is needed; with a null pointer the parts are left for flash_merge_kernel.
// ---- mbarrier helpers of the tile pipeline; every wait is bounded ------------------------------------
#define FA_WAIT_LIMIT (1u << 22)
static __device__ int g_fa_status = 0;          // 0 = fine; else code of the first wait that ran out

__device__ __forceinline__ uint32_t fa_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void fa_bar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" :: "r"(fa_smem(bar)), "r"(count));
}
__device__ __forceinline__ void fa_bar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" :: "r"(fa_smem(bar)) : "memory");
}
// arrives (without adding to the expected count) once this thread's earlier cp.async have landed
__device__ __forceinline__ void fa_bar_arrive_on_copies(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" :: "r"(fa_smem(bar)) : "memory");
}
__device__ __forceinline__ bool fa_bar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code) {
  for (uint32_t i = 0; i < FA_WAIT_LIMIT; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok) : "r"(fa_smem(bar)), "r"(parity) : "memory");
    if (ok) return true;
    if ((i & 63) == 63 && *abort_flag) return false;
  }
  *abort_flag = 1;
  atomicCAS(&g_fa_status, 0, code);
  return false;
}
__device__ __forceinline__ void fa_consumer_sync() { asm volatile("bar.sync 1, %0;\n" :: "n"(FA_THREADS) : "memory"); }

// STAGES: depth of the key-tile pipeline; QROWS: rows of the query tile that are staged (64, or 16 in
// launches whose items all have at most 16 rows: decode steps, which then afford a third stage).
//
// 8 warps: warps 0-3 compute, warps 4-7 only fetch.  The fetching warps run ahead of the computing
// ones by up to STAGES tiles: they gather a tile's keys and values page by page with cp.async into a
// free slot and arrive on the slot's `full` barrier when their copies have landed; a computing warp
// waits for `full`, works on the tile, and arrives on the slot's `empty` barrier, which the fetching
// warps wait for before they reuse the slot.  So no address arithmetic and no CTA-wide barrier sits
// between two tiles of the computing warps.
//
// Two ways of sharing a key tile between the 4 computing warps.  A tile of many rows (a prompt
// portion): each warp owns 16 rows and visits all 64 keys.  A tile of at most 16 rows (decoded
// tokens: the query heads of one group): every warp takes the same rows and 16 of the 64 keys, with
// a running max, sum and output of its own; the four are combined in shared memory at the end.
//
// `counters` (may be null): one int per (first part, kv head), zero before the launch.  The CTA that
// finishes a request's last part combines the parts itself and sets the counter back to zero, so no
// merge kernel is needed; with a null pointer the parts are left for flash_merge_kernel.
struct FaArgs {
  const __nv_bfloat16* q; long q_stride;
  const __nv_bfloat16* pages; const int* block_tables; int max_blocks;
  const int* items; __nv_bfloat16* out;
  float* part_acc; float* part_ml; int part_rows;
  int* counters; float scale_log2; int window, Hq, Hkv, page_size;
};

// The work of one CTA (work item `item_idx`, kv head `hkv`) by 256 threads; `smem_raw`: the dynamic
// shared memory (16-byte aligned).  PERSIST: the caller is a kernel that goes on after this call
// (the decode program): no thread leaves early, and all threads meet at the end so that the next
// call may reuse the shared memory and the barriers.
template <int D, int STAGES, int QROWS, bool PERSIST>
__device__ __forceinline__ void flash_attention_cta(const FaArgs& A, int item_idx, int hkv, unsigned char* smem_raw) {
  const __nv_bfloat16* __restrict__ q = A.q; const long q_stride = A.q_stride;
  const __nv_bfloat16* __restrict__ pages = A.pages; const int* __restrict__ block_tables = A.block_tables;
  const int max_blocks = A.max_blocks; const int* __restrict__ items = A.items; __nv_bfloat16* __restrict__ out = A.out;
  float* __restrict__ part_acc = A.part_acc; float* __restrict__ part_ml = A.part_ml; const int part_rows = A.part_rows;
  int* __restrict__ counters = A.counters; const float scale_log2 = A.scale_log2;
  const int window = A.window, Hq = A.Hq, Hkv = A.Hkv, page_size = A.page_size;
  constexpr int LD = D + 8;                         // padded row, in elements
  constexpr int CH = D / 8;                         // 16-byte chunks in a row
  __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(smem_raw);          // [QROWS][LD]
  __nv_bfloat16* sk = sq + QROWS * LD;                                     // [STAGES][64][LD]
  __nv_bfloat16* sv = sk + STAGES * FA_BN * LD;                            // [STAGES][64][LD]
  __shared__ uint64_t bar_full[STAGES], bar_empty[STAGES], bar_q;
  __shared__ int s_last, s_abort;

  // the work lists come from the host's copy, not from a kernel
  if (!PERSIST) pdl_launch_dependents();
  const int* it = items + (size_t)item_idx * FA_ITEM_INTS;
  const int req = it[0], q0 = it[1], part = it[4], n_splits = it[5], split = it[6];
  int kv_lo = it[2], kv_hi_item = it[3];
  const int G = Hq / Hkv;
  const int tpt = FA_BM / G;                        // tokens in a tile
  const int row0 = it[7], q_len = it[8], ctx = it[9];
  const int ntok = min(tpt, q_len - q0);
  const int nrows = ntok * G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;

  const int first_pos = ctx + q0;
  if (n_splits > 0) {
    const int total = ctx + q_len;
    const int lo = window > 0 ? max(0, ctx - window + 1) / FA_BN * FA_BN : 0;
    const int per = ((total - lo + n_splits - 1) / n_splits + FA_BN - 1) / FA_BN * FA_BN;
    kv_lo = lo + split * per;
    kv_hi_item = min(total, kv_lo + per);
  }
  const int kv_end = min(kv_hi_item, first_pos + ntok);                    // causal frontier of the tile
  int kv_begin = kv_lo;
  if (window > 0) kv_begin = max(kv_begin, first_pos - window + 1);
  kv_begin = max(kv_begin, 0);
  const int kt_first = (kv_begin / FA_BN) * FA_BN;
  const int n_tiles = kv_end > kt_first ? (kv_end - kt_first + FA_BN - 1) / FA_BN : 0;

  if (threadIdx.x == 0) {
    for (int st = 0; st < STAGES; ++st) {
      fa_bar_init(&bar_full[st], 2 * FA_THREADS);   // each fetching thread: once for its copies, once for its stores
      fa_bar_init(&bar_empty[st], FA_WARPS);        // one arrival per computing warp
    }
    fa_bar_init(&bar_q, 2 * FA_THREADS);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  const bool skip = QROWS < FA_BM && nrows > QROWS; // the launcher promised small tiles (never true)
  volatile int* abort_flag = &s_abort;
  // The previous kernel of the step wrote q and the keys and values of the new tokens (positions
  // from ctx on).  Key tiles that end before ctx hold only what earlier steps wrote: the fetching
  // warps start on them at once and wait for the previous kernel only before they touch the rest.

  if (skip) {
  } else if (warp >= FA_WARPS) {
    // ================= fetching warps ==================================================================
    const int ptid = threadIdx.x - FA_THREADS;
    const int* table = block_tables + (size_t)req * max_blocks;
    // address arithmetic of the gather, hoisted: a page's stride, this head's offset in a page, K -> V
    const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;
    const size_t page_stride = (size_t)2 * Hkv * page_size * D;
    const size_t v_off = (size_t)Hkv * page_size * D;
    const __nv_bfloat16* head_base = pages + (size_t)hkv * page_size * D;
    bool waited = false;
    auto wait_and_fetch_q = [&]() {
      if (!PERSIST) pdl_wait();
      waited = true;
      if (n_tiles > 0) {
        for (int e = ptid; e < QROWS * CH; e += FA_THREADS) {
          const int r = e / CH, ch = e - r * CH;
          __nv_bfloat16* dst = sq + r * LD + ch * 8;
          if (r < nrows) {
            const int ti = r / G, hg = r - ti * G;
            cp_async16(dst, q + (size_t)(row0 + q0 + ti) * q_stride + (size_t)(hkv * G + hg) * D + ch * 8);
          } else {
            *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
          }
        }
        fa_bar_arrive_on_copies(&bar_q);
        fa_bar_arrive(&bar_q);
      }
    };
    for (int t = 0; t < n_tiles; ++t) {
      const int stage = t % STAGES;
      const int kt = kt_first + t * FA_BN;
      // the query rows are fetched as soon as the head of the pipeline is on its way, or before the
      // first tile that may hold a new token's keys
      if (!waited && (t >= STAGES - 1 || kt + FA_BN > ctx)) wait_and_fetch_q();
      if (t >= STAGES && !fa_bar_wait(&bar_empty[stage], ((t / STAGES) - 1) & 1, abort_flag, 1)) break;
      __nv_bfloat16* dk = sk + stage * FA_BN * LD;
      __nv_bfloat16* dv = sv + stage * FA_BN * LD;
#pragma unroll 4
      for (int e = ptid; e < FA_BN * CH; e += FA_THREADS) {
        const int j = e / CH, ch = e - j * CH;
        const int kj = kt + j;
        const int so = j * LD + ch * 8;
        if (kj >= kv_begin && kj < kv_end) {
          int blk, off;
          if (page_shift >= 0) { blk = kj >> page_shift; off = kj & (page_size - 1); }
          else { blk = kj / page_size; off = kj - blk * page_size; }
          const __nv_bfloat16* src = head_base + (size_t)table[blk] * page_stride + off * D + ch * 8;
          cp_async16(dk + so, src);
          cp_async16(dv + so, src + v_off);
        } else {
          *reinterpret_cast<uint4*>(dk + so) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(dv + so) = make_uint4(0, 0, 0, 0);
        }
      }
      fa_bar_arrive_on_copies(&bar_full[stage]);    // when this thread's copies have landed
      fa_bar_arrive(&bar_full[stage]);              // and its zero stores are released
    }
    if (!waited) wait_and_fetch_q();
    cp_async_commit();
    cp_async_wait<0>();                             // nothing of this thread's is in flight when it leaves
  } else {
  // ================= computing warps =====================================================================
  const bool keysplit = nrows <= 16 || QROWS < FA_BM;   // few rows: the warps share the keys, not the rows
  const int row_base = keysplit ? 0 : warp * 16;
  // rows of this thread: r_lo = row_base + g and r_lo + 8
  const int r_lo = row_base + g, r_hi = r_lo + 8;
  const int pos_lo = r_lo < nrows ? first_pos + r_lo / G : -1;             // -1: the row is padding
  const int pos_hi = r_hi < nrows ? first_pos + r_hi / G : -1;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

  const bool warp_active = keysplit || warp * 16 < nrows;       // a warp without rows only hands slots back
  if (!PERSIST) pdl_wait();
  bool ok = n_tiles == 0 || __all_sync(0xffffffffu, fa_bar_wait(&bar_q, 0, abort_flag, 3));
  for (int t = 0; ok && t < n_tiles; ++t) {
    const int stage = t % STAGES;
    ok = __all_sync(0xffffffffu, fa_bar_wait(&bar_full[stage], (t / STAGES) & 1, abort_flag, 2));
    if (!ok) break;
    if (warp_active) {
      const int kt = kt_first + t * FA_BN;
      const __nv_bfloat16* tk = sk + stage * FA_BN * LD;
      const __nv_bfloat16* tv = sv + stage * FA_BN * LD;
      // whether the whole tile is allowed for all 16 rows of this warp (then no mask is needed)
      const int row_first = row_base, row_last = min(row_base + 15, nrows - 1);
      const int pos_first = first_pos + row_first / G, pos_last = first_pos + row_last / G;
      const bool all_allowed = row_base + 16 <= nrows && kt >= kv_begin && kt + FA_BN <= kv_end &&
                               kt + FA_BN - 1 <= pos_first && (window <= 0 || kt > pos_last - window);
      if (keysplit)
        fa_tile<D, 1>(sq, tk, tv, 0, warp, kt, kv_begin, kv_end, pos_lo, pos_hi, window, scale_log2, lane,
                      m_lo, m_hi, l_lo, l_hi, o, false);
      else
        fa_tile<D, FA_BN / 16>(sq, tk, tv, row_base, 0, kt, kv_begin, kv_end, pos_lo, pos_hi, window, scale_log2,
                               lane, m_lo, m_hi, l_lo, l_hi, o, all_allowed);
    }
    __syncwarp();
    if (lane == 0) fa_bar_arrive(&bar_empty[stage]);      // this warp is done with the slot
  }
  if (ok) {                                         // else a wait ran out: the status flag says so; nothing is written
  __nv_bfloat16* out_row0 = out + (size_t)(row0 + q0) * ((size_t)Hq * D);
  if (keysplit) {
    // ---- combine the four warps' shares of the keys in shared memory (the tiles are done) ------
    fa_consumer_sync();
    float* xo = reinterpret_cast<float*>(sk);                  // [4 warps][16 rows][D]
    float* xml = xo + FA_WARPS * 16 * D;                        // [4 warps][16 rows][2]
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      *reinterpret_cast<float2*>(xo + ((size_t)warp * 16 + g) * D + i * 8 + 2 * c) = make_float2(o[i][0], o[i][1]);
      *reinterpret_cast<float2*>(xo + ((size_t)warp * 16 + g + 8) * D + i * 8 + 2 * c) = make_float2(o[i][2], o[i][3]);
    }
    if (c == 0) {
      xml[(warp * 16 + g) * 2] = m_lo; xml[(warp * 16 + g) * 2 + 1] = l_lo;
      xml[(warp * 16 + g + 8) * 2] = m_hi; xml[(warp * 16 + g + 8) * 2 + 1] = l_hi;
    }
    fa_consumer_sync();
    for (int e = threadIdx.x; e < nrows * D; e += FA_THREADS) {
      const int r = e / D, d = e - r * D;
      float m = -INFINITY;
#pragma unroll
      for (int w = 0; w < FA_WARPS; ++w) m = fmaxf(m, xml[(w * 16 + r) * 2]);
      const float base = m == -INFINITY ? 0.f : m;
      float l = 0.f, acc = 0.f;
#pragma unroll
      for (int w = 0; w < FA_WARPS; ++w) {
        const float wgt = exp2f(xml[(w * 16 + r) * 2] - base);
        l += wgt * xml[(w * 16 + r) * 2 + 1];
        acc += wgt * xo[((size_t)w * 16 + r) * D + d];
      }
      if (part < 0) {
        const int ti = r / G, hg = r - ti * G;
        out_row0[(size_t)ti * ((size_t)Hq * D) + (size_t)(hkv * G + hg) * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
      } else {
        const size_t slot = ((size_t)part * Hkv + hkv) * part_rows + r;
        part_acc[slot * D + d] = acc;
        if (d == 0) { part_ml[2 * slot] = m; part_ml[2 * slot + 1] = l; }
      }
    }
  } else if (warp_active) {
    // ---- write: the output, or this part's accumulator with max and sum ------------------------
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = half ? r_hi : r_lo;
      if (r >= nrows) continue;
      const int ti = r / G, hg = r - ti * G;
      const float l = half ? l_hi : l_lo, m = half ? m_hi : m_lo;
      if (part < 0) {
        const float inv = 1.f / l;
        __nv_bfloat16* dst = out_row0 + (size_t)ti * ((size_t)Hq * D) + (size_t)(hkv * G + hg) * D;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
          const float v0 = o[i][2 * half] * inv, v1 = o[i][2 * half + 1] * inv;
          *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * c) = pack_bf16(v0, v1);
        }
      } else {
        const size_t slot = ((size_t)part * Hkv + hkv) * part_rows + r;
        float* dst = part_acc + slot * D;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
          *reinterpret_cast<float2*>(dst + i * 8 + 2 * c) = make_float2(o[i][2 * half], o[i][2 * half + 1]);
        }
        if (c == 0) { part_ml[2 * slot] = m; part_ml[2 * slot + 1] = l; }
      }
    }
  }
  // ---- the CTA that finishes a request's last part combines the parts ---------------------------------
  if (part >= 0 && counters != nullptr && n_splits > 0) {
    const int first = part - split;
    __threadfence();                                // this CTA's part is visible before it is counted
    fa_consumer_sync();
    if (threadIdx.x == 0) {
      const int done = atomicAdd(&counters[first * Hkv + hkv], 1);
      s_last = (done == n_splits - 1);
      if (s_last) counters[first * Hkv + hkv] = 0;  // ready for the next launch
    }
    fa_consumer_sync();
    if (s_last) {
      __threadfence();
      fa_merge_parts<D>(part_acc, part_ml, part_rows, first, n_splits, hkv, Hkv, nrows, G, Hq, out_row0);
    }
  }
  }   // ok
  }   // computing warps
  if (PERSIST) __syncthreads();                      // shared memory and barriers are free for the next call
}

