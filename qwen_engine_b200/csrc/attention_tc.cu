// Flash attention over the paged cache on the fifth-generation tensor cores, for prompt portions:
// head size 128 in bfloat16.  (What it computes is the reference's prefill attention,
// src/layers/fused_ops/attn.py:130-290: scores and softmax statistics in float32, P rounded to
// bfloat16 before P·V, the mask key <= position and > position - window.  The reference's Triton
// kernel leaves the instructions to the compiler; here S = Q·K^T and O += P·V are tcgen05.mma with
// the accumulators, and P itself, in tensor memory.)
//
// A work unit is one kv head and a tile of 256 "rows" (a row is a query token x a query head of the kv
// head's group, so the keys and values are read once for the whole group), as two halves of 128 rows,
// one per softmax group.  The kernel runs one CTA per SM at most; each walks the units that the host's
// schedule gives it (qe_flash_attention_tc_schedule), one after the other through the same pipelines.
// Twelve warps:
//   warps 0-3, 4-7  the two softmax groups: one thread per row (= tensor-memory lane), 208 registers a
//                   thread (setmaxnreg).  Per key step a thread reads its row of S from tensor memory,
//                   masks, takes the running max, exponentiates, writes P (bfloat16) back over S, and
//                   rescales O when the max grew; at a unit's end it writes the rows out;
//   warp 8          fetches a unit's Q and the key and value tiles of every step (128 keys) with TMA, page
//                   by page from the block table, through a two-stage ring that runs on across units;
//   warp 9          owns tensor memory and issues all MMAs from one thread;
//   warps 10, 11    idle (they make the third group of four warps whole, for setmaxnreg).
// While one group works on its softmax, the tensor core runs the other group's products.
// Tensor memory (512 columns): S of group 0 | S of group 1 | O of group 0 | O of group 1; P lies over
// the first 64 columns of its S.
//
// The running max is allowed to lag: O and the running sum are rescaled only when the max grew by more
// than 2^8 since the last rescale, which leaves the quotient O / sum unchanged but for rounding.
//
// A work item may cover only a range of keys (a part of a long tile).  Of a tile's parts, those that are
// not the last to get to their end write their unnormalised accumulator with max and sum in float32 to
// scratch memory; the last one adds them to its own, which never leaves tensor memory, in the order of
// the parts, and writes the tile's rows (two counters a tile and kv head: parts arrived, parts written).
//
// Keys of a tile that lie in no page (block table entry -1, or past the table) are read as zeros; keys
// of a held page past the request's length are read as they are and masked, so pages must hold finite
// values (the cache starts as zeros and only kernels write to it).
//
// Every wait on an mbarrier, and the last part's wait for the others' to be written, is bounded: a wait that
// runs out records a code in a device flag, raises a CTA-wide abort that the other roles see in their own waits, and the CTA skips its stores, frees its
// tensor memory and returns; the host reads the flag with qe_flash_attention_tc_status().
#include "tcgen05.cuh"
#include <math.h>
#include <type_traits>

#define AT_ROWS 128             // rows of a softmax group
#define AT_BN 128               // keys per step
#define AT_D 128                // head size
#define AT_THREADS 384             // 8 softmax warps, the fetching warp, the issuing warp, and two idle warps that fill the third group of four
#define AT_UNITS_SMEM 48           // work units of a CTA whose descriptions are kept in shared memory
#define AT_SOFTMAX_THREADS 256
#define AT_ITEM_INTS 12
#define AT_TMEM_COLS 512
#define AT_RESCALE_STEP 8.0f    // log2 of the growth of the max that forces a rescale
#define AT_MAX_PARTS 8          // parts of one tile at most

static __device__ int g_at_status = 0;          // 0 = fine; else code of the first wait that ran out

// A work unit (a work item for one kv head) as every role of the CTA sees it.
struct AtUnit {
  int req, q0, part, n_parts, split, row0, hkv;
  int nrows, first_pos, kv_begin, kv_end, kt_first, n_steps;
  bool two;                                         // the second softmax group has rows
};
struct __align__(1024) AtSmem {
  __nv_bfloat16 q[2][2][AT_ROWS * 64];          // [group][half of D][row][64]: 128-byte swizzled rows
  __nv_bfloat16 k[2][2][AT_BN * 64];            // [stage][half of D][key][64]
  __nv_bfloat16 v[2][2][AT_BN * 64];
  uint64_t q_full[2], q_empty[2], k_full[2], k_empty[2], v_full[2], v_empty[2], s_ready[2], p_ready[2], o_ready[2];
  uint32_t tmem_base;
  int abort_flag, last;
  AtUnit units[AT_UNITS_SMEM];
  uint4 stage[8][128];                          // 2 KB per softmax warp: rows on their way to global memory
};

struct AtArgs {
  const int* block_tables; int max_blocks; int num_pages;
  const int* items; const int* sched; __nv_bfloat16* out;
  float* part_acc; float* part_ml; int part_rows; int* counters;
  float scale_log2; int window, Hq, Hkv, page_shift;
};

__device__ __forceinline__ uint32_t at_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// 2^x by the special-function unit alone (no range fix-up: denormal results are flushed to zero)
__device__ __forceinline__ float at_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float at_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// two float32 operations in one instruction (packed pairs in 64-bit registers)
__device__ __forceinline__ float2 at_fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}\n"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 at_add2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "add.rn.f32x2 rd, ra, rb;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}\n"
      : "=f"(d.x), "=f"(d.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
// A warp's 32 rows of 64 bytes, a row per lane in registers, to global memory through the warp's 2 KB of shared memory, so
// that four lanes write a row's 64 bytes side by side (a row per lane would touch 32 lines per instruction).  dst[k]: where
// this lane's 16 bytes of the warp's row 8 k + lane / 4 go (nullptr: nowhere); the caller works them out once for all
// passes.  Chunk c of row r lies at 4 r + (c ^ (r / 2 & 3)): neither the writes nor the reads meet in a bank.
__device__ __forceinline__ void at_store_rows(uint4* stage, const uint32_t* v, int lane, char* const (&dst)[4], int offset) {
#pragma unroll
  for (int c = 0; c < 4; ++c)
    stage[lane * 4 + (c ^ ((lane >> 1) & 3))] = make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
  __syncwarp();
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int row = 8 * k + (lane >> 2);
    const uint4 x = stage[row * 4 + ((lane & 3) ^ ((row >> 1) & 3))];
    if (dst[k] != nullptr) *reinterpret_cast<uint4*>(dst[k] + offset) = x;
  }
  __syncwarp();
}
__device__ __forceinline__ void at_softmax_sync() { asm volatile("bar.sync 1, %0;\n" :: "n"(AT_SOFTMAX_THREADS) : "memory"); }

__device__ __forceinline__ AtUnit at_unit(const AtArgs& A, int unit) {
  AtUnit U;
  const int item_idx = unit / A.Hkv;
  U.hkv = unit - item_idx * A.Hkv;
  const int* it = A.items + (size_t)item_idx * AT_ITEM_INTS;      // (the work lists come from the host's copy, not from a kernel)
  U.req = it[0]; U.q0 = it[1]; U.part = it[4]; U.n_parts = it[5]; U.split = it[6]; U.row0 = it[7];
  const int q_len = it[8], ctx = it[9];
  const int G = A.Hq / A.Hkv;
  const int ntok = min(2 * (AT_ROWS / G), q_len - U.q0);
  U.nrows = ntok * G;
  U.two = U.nrows > AT_ROWS;
  U.first_pos = ctx + U.q0;
  U.kv_end = min(it[3], U.first_pos + ntok);        // causal frontier of the tile
  U.kv_begin = max(it[2], 0);
  if (A.window > 0) U.kv_begin = max(U.kv_begin, U.first_pos - A.window + 1);
  U.kt_first = U.kv_begin / AT_BN * AT_BN;
  U.n_steps = U.kv_end > U.kt_first ? (U.kv_end - U.kt_first + AT_BN - 1) / AT_BN : 0;
  return U;
}

// A CTA runs the work units that the host's schedule gives it (sched[b] .. sched[b + 1] index the unit numbers behind
// the CTAs' offsets), one after the other through the same pipelines: the key and value ring, the tensor-memory
// columns and the barriers' phases run on across units, so a unit's first scores are formed while the softmax groups
// still write the output of the unit before, and a unit costs its key steps plus about one step instead of a launch.
__global__ void __launch_bounds__(AT_THREADS, 1)
flash_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, AtArgs A) {
  extern __shared__ unsigned char smem_raw[];
  pdl_launch_dependents();
  QE_TL_STAMPS(128);                                // (timeline build: the CTA's n-th unit, n < 8, leaves stamps 16 n + 8 g + .. for softmax group g)
  AtSmem& sm = *reinterpret_cast<AtSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int Hq = A.Hq, Hkv = A.Hkv, window = A.window;
  const int G = Hq / Hkv;
  const int tpw = AT_ROWS / G;                      // tokens of one softmax group
  const int u_begin = A.sched[blockIdx.x], u_end = A.sched[blockIdx.x + 1];
  volatile int* abort_flag = &sm.abort_flag;
  // the CTA's units, worked out once (every role walks them, and a description is two dependent reads away)
  if (threadIdx.x >= 32 && threadIdx.x - 32 < min(u_end - u_begin, AT_UNITS_SMEM))
    sm.units[threadIdx.x - 32] = at_unit(A, A.sched[u_begin + threadIdx.x - 32]);
  auto unit_at = [&](int ui) { return ui - u_begin < AT_UNITS_SMEM ? sm.units[ui - u_begin] : at_unit(A, A.sched[ui]); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sm.q_full[s], 1); mbar_init(&sm.q_empty[s], 1);
      mbar_init(&sm.k_full[s], 1); mbar_init(&sm.k_empty[s], 1);
      mbar_init(&sm.v_full[s], 1); mbar_init(&sm.v_empty[s], 1);
      mbar_init(&sm.s_ready[s], 1); mbar_init(&sm.p_ready[s], AT_ROWS); mbar_init(&sm.o_ready[s], 1);
    }
    sm.abort_flag = 0;
    sm.last = 0;
    mbar_init_fence();
  }
  if (warp == 9) tc_alloc(&sm.tmem_base, AT_TMEM_COLS);
  if (warp == 8 && u_begin < u_end) {
    // what the first copies will need and no kernel writes: the tensor maps, and the block-table entries of the first
    // unit's first keys (the step's index data come from the host's copy)
    if (lane == 0) { tma_prefetch_map(&map_q); tma_prefetch_map(&map_kv); }
    const AtUnit U0 = at_unit(A, A.sched[u_begin]);
    const int blk = (U0.kt_first >> A.page_shift) + lane;
    if (blk < A.max_blocks) asm volatile("prefetch.global.L1 [%0];\n" :: "l"(A.block_tables + (size_t)U0.req * A.max_blocks + blk));
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  pdl_wait();                                       // q, the new keys and values: the previous kernels' outputs

  // registers: the softmax threads hold a row of scores and of P each; the other warps need few
  if (warp >= 8) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 88;\n");
  if (warp == 8) {
    // ================= producer ==========================================================================
    const int page_shift = A.page_shift, page_size = 1 << page_shift;
    const int box_rows = min(page_size, AT_BN);
    const int nb = AT_BN / box_rows;                // boxes per half tile
    // Keys and values of a step are asked for separately, each as soon as its slot is free: the keys' slot when
    // the scores of the step two before have been formed, the values' slot a whole step later, when that step's
    // P V has retired.  (Asked for together, the keys of step j + 1 waited for the values' slot and arrived
    // after the tensor cores wanted them.)  A unit's queries are asked for behind its first keys, a group's as
    // soon as the last Q K^T of the unit before has read that group's.
    int gk = 0;                                     // key steps so far, over all units
    int issued_k = 0, issued_v = 0, issued_q[2] = {0, 0};
    bool ok = true;
    for (int ui = u_begin; ok && ui < u_end; ++ui) {
      const AtUnit U = unit_at(ui);
      const int* table = A.block_tables + (size_t)U.req * A.max_blocks;
      for (int j = 0; ok && j < U.n_steps; ++j, ++gk) {
        const int st = gk & 1;
        const uint32_t par = ((gk >> 1) - 1) & 1;
        const int kt = U.kt_first + j * AT_BN;
        for (int kind = 0; ok && kind < 2; ++kind) {
          if (gk >= 2) ok = mbar_wait(kind ? &sm.v_empty[st] : &sm.k_empty[st], par, abort_flag, 1 + kind, &g_at_status);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          if (lane == 0) mbar_expect_tx(kind ? &sm.v_full[st] : &sm.k_full[st], AT_BN * AT_D * (uint32_t)sizeof(__nv_bfloat16));
          __syncwarp();
          for (int idx = lane; idx < 2 * nb; idx += 32) {
            const int box = idx >> 1, half = idx & 1;
            const int key0 = kt + box * box_rows;
            const int blk = key0 >> page_shift, y = key0 & (page_size - 1);
            int page = blk < A.max_blocks ? table[blk] : -1;
            if (page < 0) page = A.num_pages;       // outside the tensor: the box is filled with zeros
            __nv_bfloat16* dst = (kind ? sm.v[st][half] : sm.k[st][half]) + (size_t)box * box_rows * 64;
            tma_load_5d(dst, &map_kv, kind ? &sm.v_full[st] : &sm.k_full[st], half * 64, y, U.hkv, kind, page);
          }
          if (kind) ++issued_v; else ++issued_k;
          if (kind == 0 && j == 0) {
            for (int w = 0; ok && w < (U.two ? 2 : 1); ++w) {
              if (issued_q[w] > 0) ok = mbar_wait(&sm.q_empty[w], (issued_q[w] - 1) & 1, abort_flag, 10, &g_at_status);
              ok = __all_sync(0xffffffffu, ok);
              if (!ok) break;
              if (lane == 0) {
                mbar_expect_tx(&sm.q_full[w], AT_ROWS * AT_D * (uint32_t)sizeof(__nv_bfloat16));
                for (int half = 0; half < 2; ++half)
                  tma_load_3d(sm.q[w][half], &map_q, &sm.q_full[w], half * 64, U.hkv * G, U.row0 + U.q0 + w * tpw);
              }
              ++issued_q[w];
            }
          }
        }
      }
    }
    if (*abort_flag && lane == 0) {
      // giving up: let the copies that are still in flight land before the CTA leaves (bounded)
      for (int w = 0; w < 2; ++w)
        if (issued_q[w] > 0)
          for (uint32_t spin = 0; spin < TC_WAIT_LIMIT; ++spin) if (mbar_try_wait(&sm.q_full[w], (issued_q[w] - 1) & 1)) break;
      for (int i = max(0, issued_k - 2); i < issued_k; ++i)
        for (uint32_t spin = 0; spin < TC_WAIT_LIMIT; ++spin) if (mbar_try_wait(&sm.k_full[i & 1], (i >> 1) & 1)) break;
      for (int i = max(0, issued_v - 2); i < issued_v; ++i)
        for (uint32_t spin = 0; spin < TC_WAIT_LIMIT; ++spin) if (mbar_try_wait(&sm.v_full[i & 1], (i >> 1) & 1)) break;
    }
  } else if (warp == 9) {
    // ================= MMA issuer: one thread ===========================================================
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(AT_ROWS, AT_BN);
      constexpr uint32_t idesc_pv = make_idesc(AT_ROWS, AT_D, true);
      // The operands' descriptors are worked out once: the issuing thread's own instructions, not the tensor cores, set
      // the pace of the products otherwise (a descriptor built per instruction costs a dozen dependent operations, and a
      // 128 x 128 x 16 product is over in 64 cycles).
      const uint64_t dq00 = make_smem_desc(smem_u32(sm.q[0][0])), dq01 = make_smem_desc(smem_u32(sm.q[0][1]));
      const uint64_t dq10 = make_smem_desc(smem_u32(sm.q[1][0])), dq11 = make_smem_desc(smem_u32(sm.q[1][1]));
      const uint64_t dk00 = make_smem_desc(smem_u32(sm.k[0][0])), dk01 = make_smem_desc(smem_u32(sm.k[0][1]));
      const uint64_t dk10 = make_smem_desc(smem_u32(sm.k[1][0])), dk11 = make_smem_desc(smem_u32(sm.k[1][1]));
      const uint64_t dv0 = make_smem_desc_mn(smem_u32(sm.v[0][0]), AT_BN * 128, 1024);
      const uint64_t dv1 = make_smem_desc_mn(smem_u32(sm.v[1][0]), AT_BN * 128, 1024);
      auto issue_qk = [&](int w, int st) {          // S_w = Q_w · K^T: 8 instructions of k = 16 over the head size
        const uint64_t qa = w ? dq10 : dq00, qb = w ? dq11 : dq01;
        const uint64_t ka = st ? dk10 : dk00, kb = st ? dk11 : dk01;
        const uint32_t d = tmem + w * AT_BN;
#pragma unroll
        for (int ks = 0; ks < AT_D / 16; ++ks)
          tc_mma_bf16(d, (ks < 4 ? qa : qb) + 2 * (ks & 3), (ks < 4 ? ka : kb) + 2 * (ks & 3), idesc_qk, ks != 0);
      };
      auto issue_pv = [&](int w, int st, bool acc) {  // O_w (+)= P_w · V: 8 instructions of k = 16 over the keys
        const uint64_t dv = st ? dv1 : dv0;
        const uint32_t d = tmem + 2 * AT_BN + w * AT_D, a = tmem + w * AT_BN;
#pragma unroll
        for (int ks = 0; ks < AT_BN / 16; ++ks)
          tc_mma_bf16_ts(d, a + ks * 8, dv + ks * (2048 >> 4), idesc_pv, acc || ks != 0);
      };
      int ui = u_begin;
      auto next_unit = [&](AtUnit& U) {             // the next unit that has keys to visit
        while (ui < u_end) {
          U = unit_at(ui++);
          if (U.n_steps > 0) return true;
        }
        return false;
      };
      uint32_t began = 0, taken = 0;                // bit w: the phase of group w's queries' barrier, of its P's barrier
      // the scores of a step for group w; `first`: the step opens a unit (its queries must have landed), `last`: it
      // closes one (nothing reads the group's queries after it)
      auto scores = [&](int w, int st, bool first, bool last) {
        if (first) {
          if (!mbar_wait(&sm.q_full[w], (began >> w) & 1, abort_flag, 3, &g_at_status)) return false;
          began ^= 1u << w;
          tc_fence_after();
        }
        issue_qk(w, st);
        tc_commit(&sm.s_ready[w]);
        if (last) tc_commit(&sm.q_empty[w]);
        return true;
      };
      AtUnit cur, nxt;
      bool have = next_unit(cur);
      bool ok = true;
      int gj = 0;                                   // key steps so far, over all units
      if (have) {
        ok = mbar_wait(&sm.k_full[0], 0, abort_flag, 4, &g_at_status);
        if (ok) {
          tc_fence_after();
#pragma unroll
          for (int w = 0; w < 2; ++w)
            if (ok && (w == 0 || cur.two)) ok = scores(w, 0, true, cur.n_steps == 1);
          if (ok) tc_commit(&sm.k_empty[0]);
        }
      }
      while (ok && have) {
        const int groups = cur.two ? 2 : 1;
        // ---- all steps but the unit's last: the step after is the same unit's --------------------------------
        for (int j = 0; ok && j + 1 < cur.n_steps; ++j, ++gj) {
          const int st = gj & 1, nst = st ^ 1;
          const bool closes = j + 2 == cur.n_steps;           // the scores formed here are the unit's last
          ok = mbar_wait(&sm.v_full[st], (gj >> 1) & 1, abort_flag, 5, &g_at_status);
#pragma unroll
          for (int w = 0; w < 2; ++w) {
            if (!ok || w >= groups) continue;
            ok = mbar_wait(&sm.p_ready[w], (taken >> w) & 1, abort_flag, 6, &g_at_status);
            if (!ok) continue;
            taken ^= 1u << w;
            tc_fence_after();
            issue_pv(w, st, j > 0);
            if (w == groups - 1) tc_commit(&sm.v_empty[st]);        // the values' slot, as soon as the last P V that reads it retires
            if (w == 0) {
              ok = mbar_wait(&sm.k_full[nst], ((gj + 1) >> 1) & 1, abort_flag, 7, &g_at_status);
              if (!ok) continue;
              tc_fence_after();
            }
            issue_qk(w, nst);
            tc_commit(&sm.s_ready[w]);
            if (closes) tc_commit(&sm.q_empty[w]);
          }
          if (ok) tc_commit(&sm.k_empty[nst]);
        }
        // ---- the unit's last step: the step after, if any, opens the next unit -------------------------------
        bool have_next = false;
        if (ok) {
          const int st = gj & 1, nst = st ^ 1;
          const bool acc = cur.n_steps > 1;
          have_next = next_unit(nxt);
          const int n_groups = have_next ? (nxt.two ? 2 : 1) : 0;
          const bool n_last = have_next && nxt.n_steps == 1;
          const uint32_t k_par = ((gj + 1) >> 1) & 1;
          ok = mbar_wait(&sm.v_full[st], (gj >> 1) & 1, abort_flag, 5, &g_at_status);
          bool keys_here = false;
          uint32_t scored = 0;
#pragma unroll
          for (int w = 0; w < 2; ++w) {
            if (ok && w < groups) {
              ok = mbar_wait(&sm.p_ready[w], (taken >> w) & 1, abort_flag, 6, &g_at_status);
              if (ok) {
                taken ^= 1u << w;
                tc_fence_after();
                issue_pv(w, st, acc);
                if (w == groups - 1) tc_commit(&sm.v_empty[st]);
                tc_commit(&sm.o_ready[w]);
              }
            }
            // The next unit's first scores wait for its queries, which may still be on their way: the other group's
            // P V must not wait behind them, so they are formed here only if everything has landed, else below.
            if (ok && w < n_groups && mbar_try_wait(&sm.q_full[w], (began >> w) & 1) &&
                (keys_here || mbar_try_wait(&sm.k_full[nst], k_par))) {
              if (!keys_here) { tc_fence_after(); keys_here = true; }
              ok = scores(w, nst, true, n_last);
              scored |= 1u << w;
            }
          }
#pragma unroll
          for (int w = 0; w < 2; ++w) {
            if (!ok || w >= n_groups || ((scored >> w) & 1)) continue;
            if (!keys_here) {
              ok = mbar_wait(&sm.k_full[nst], k_par, abort_flag, 7, &g_at_status);
              tc_fence_after();
              keys_here = true;
            }
            if (ok) ok = scores(w, nst, true, n_last);
          }
          if (ok && n_groups > 0) tc_commit(&sm.k_empty[nst]);
          ++gj;
        }
        cur = nxt;
        have = have_next;
      }
    }
  }
  // (warps 10 and 11 are idle: they only make the third group of four warps whole)
  } else {
    // ================= softmax groups ====================================================================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;\n");
    const int w = warp >> 2, quarter = warp & 3;
    const int r = w * AT_ROWS + quarter * 32 + lane;        // row of the tile
    const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
    const uint32_t s_col = w * AT_BN, o_col = 2 * AT_BN + w * AT_D;
    const float scale_log2 = A.scale_log2;
    int seen_s = 0, seen_o = 0;                             // phases of this group's score and output barriers
    bool ok = true;
    for (int ui = u_begin; ui < u_end; ++ui) {
      const AtUnit U = unit_at(ui);
      const int n_steps = U.n_steps, hkv = U.hkv, part = U.part;
      const bool active = w == 0 || U.two;
      const bool valid = r < U.nrows;
      const int pos = valid ? U.first_pos + r / G : -1;
      const int hi = valid ? min(U.kv_end, pos + 1) : 0;      // keys [lo, hi) are allowed for this row
      const int lo = window > 0 ? max(U.kv_begin, pos - window + 1) : U.kv_begin;
      float m_run = -INFINITY, l_run = 0.f;
      // (timeline build: 0 the unit's first scores are ready, 1 its first P is handed over, 2 its last P, 3 its last P V has
      // retired, 4 its output is written, 5 the parts are merged, if that fell to this CTA)
#define AT_STAMP(k) QE_TL_STAMP(quarter == 0 && lane == 0 && ui - u_begin < 8 ? 16 * (ui - u_begin) + 8 * w + (k) : -1)
      if (active && ok) {
        for (int j = 0; j < n_steps; ++j) {
          ok = __all_sync(0xffffffffu, mbar_wait(&sm.s_ready[w], seen_s & 1, abort_flag, 8, &g_at_status));
          if (!ok) break;
          ++seen_s;
          tc_fence_after();
          if (j == 0) AT_STAMP(0);
          uint32_t s[4][32];
#pragma unroll
          for (int c = 0; c < 4; ++c) tc_ld_32x32b_x32(lane_base + s_col + c * 32, s[c]);
          tc_wait_ld();
          const int kt = U.kt_first + j * AT_BN;
          float mx = -INFINITY;
          // A step's 128 keys as four runs of 32: where a run is allowed for all of the warp's rows (every run of a step
          // before the diagonal) the maxima are chains of three-input instructions; where it is forbidden for all of
          // them (behind the diagonal of the warp's first rows, before a window) nothing is computed for it at all; only
          // the runs that the mask's edge crosses are masked key by key.  The decisions are the warp's, so no lane idles.
          uint32_t live = 0;                              // bit c: run c has a key that some row of the warp may see
          if (__all_sync(0xffffffffu, kt >= lo && kt + AT_BN <= hi)) {
            float mc[4];                                  // four chains of three-input maxima
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              mc[c] = fmaxf(__uint_as_float(s[c][0]), __uint_as_float(s[c][1]));
#pragma unroll
              for (int i = 2; i < 32; i += 2) mc[c] = at_max3(mc[c], __uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1]));
            }
            mx = fmaxf(fmaxf(mc[0], mc[1]), fmaxf(mc[2], mc[3]));
            live = 15u;
          } else
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int k0 = kt + 32 * c;
            const bool all_in = __all_sync(0xffffffffu, k0 >= lo && k0 + 32 <= hi);
            const bool all_out = !all_in && __all_sync(0xffffffffu, k0 >= hi || k0 + 32 <= lo);
            if (all_in) {
              float mc = at_max3(__uint_as_float(s[c][0]), __uint_as_float(s[c][1]), __uint_as_float(s[c][2]));
              float md = at_max3(__uint_as_float(s[c][3]), __uint_as_float(s[c][4]), __uint_as_float(s[c][5]));
#pragma unroll
              for (int i = 6; i < 30; i += 4) {
                mc = at_max3(mc, __uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1]));
                md = at_max3(md, __uint_as_float(s[c][i + 2]), __uint_as_float(s[c][i + 3]));
              }
              mx = at_max3(mx, fmaxf(mc, __uint_as_float(s[c][30])), fmaxf(md, __uint_as_float(s[c][31])));
              live |= 1u << c;
            } else if (!all_out) {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const int key = k0 + i;
                const float v = (key >= lo && key < hi) ? __uint_as_float(s[c][i]) : -INFINITY;
                s[c][i] = __float_as_uint(v);
                mx = fmaxf(mx, v);
              }
              live |= 1u << c;
            }
          }
          mx *= scale_log2;                               // the scale is positive
          // the reference max moves only when the row's max has grown by more than the step
          const bool grow = mx > m_run + AT_RESCALE_STEP;
          const float alpha = grow ? exp2f(m_run - mx) : 1.f;
          if (grow) m_run = mx;
          const float base = m_run == -INFINITY ? 0.f : m_run;   // a row with nothing allowed so far
          if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
              uint32_t o[32];
              tc_ld_32x32b_x32(lane_base + o_col + c * 32, o);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tc_st_32x32b_x32(lane_base + o_col + c * 32, o);
            }
          }
          uint32_t pk[2][32];
          float2 sums[4];
          const float2 sc2 = make_float2(scale_log2, scale_log2), nb2 = make_float2(-base, -base);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            sums[c] = make_float2(0.f, 0.f);
            if (!((live >> c) & 1)) {                     // nothing of this run is allowed: its P is zero
#pragma unroll
              for (int i = 0; i < 16; ++i) pk[c >> 1][(c & 1) * 16 + i] = 0u;
              continue;
            }
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float2 x = at_fma2(make_float2(__uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1])), sc2, nb2);
              const float2 p = make_float2(at_ex2(x.x), at_ex2(x.y));
              sums[c] = at_add2(sums[c], p);
              pk[c >> 1][(c & 1) * 16 + (i >> 1)] = at_pack(p.x, p.y);
            }
          }
          const float2 s01 = at_add2(sums[0], sums[1]), s23 = at_add2(sums[2], sums[3]);
          l_run = l_run * alpha + ((s01.x + s01.y) + (s23.x + s23.y));
          tc_st_32x32b_x32(lane_base + s_col, pk[0]);
          tc_st_32x32b_x32(lane_base + s_col + 32, pk[1]);
          tc_wait_st();
          tc_fence_before();
          mbar_arrive(&sm.p_ready[w]);
          if (j == 0) AT_STAMP(1);
          if (j == n_steps - 1) AT_STAMP(2);
        }
        if (ok && n_steps > 0) {
          ok = __all_sync(0xffffffffu, mbar_wait(&sm.o_ready[w], seen_o & 1, abort_flag, 9, &g_at_status));
          ++seen_o;
        }
        AT_STAMP(3);
      }
      // ---- a part of a tile: is this the last of the tile's parts to get here? ---------------------------------
      // 0: a whole tile; 1: a part, and others are still at work: its accumulator goes to scratch memory with max and
      // sum; 2: the last part to get here: it takes the others' from scratch memory and writes the tile's output, its
      // own accumulator never leaving tensor memory; 3: the CTA is giving up.
      int role = 0;
      const bool is_part = part >= 0 && A.counters != nullptr && U.n_parts > 0;
      int* const arrived = is_part ? A.counters + 2 * ((part - U.split) * Hkv + hkv) : nullptr;     // [1]: parts written
      if (is_part) {
        if (!ok) sm.abort_flag = 1;
        at_softmax_sync();
        if (threadIdx.x == 0) {
          int r2 = 3;
          if (!sm.abort_flag) r2 = atomicAdd(arrived, 1) == U.n_parts - 1 ? 2 : 1;
          if (r2 == 2) {
            // the others have their tickets, so they are running and will get there; wait until they have written
            bool there = false;
            for (uint32_t spin = 0; spin < TC_WAIT_LIMIT && !there; ++spin) {
              there = *reinterpret_cast<volatile int*>(arrived + 1) == U.n_parts - 1;
              if (!there) __nanosleep(64);
            }
            if (there) { arrived[0] = 0; arrived[1] = 0; }     // ready for the next launch
            else { sm.abort_flag = 1; atomicCAS(&g_at_status, 0, 11); r2 = 3; }
          }
          sm.last = r2;
        }
        at_softmax_sync();
        role = sm.last;                               // (read before the next meeting, behind which it may change)
        AT_STAMP(7);
        if (role == 2) __threadfence();
      }
      // ---- the tile's output, or this part's accumulator with max and sum ----------------------------
      if (active && ok && role < 2) {
        {
          tc_fence_after();
          const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
          const size_t slot = part >= 0 ? ((size_t)part * Hkv + hkv) * A.part_rows + r : 0;
          const int wrow0 = w * AT_ROWS + quarter * 32;       // the warp's first row of the tile
          uint4* stage = sm.stage[warp];
          const int nrows = U.nrows;
          // where this lane's 16 bytes of the warp's rows 8 k + lane / 4 go: the output's row (token, head) or the part's
          char* dst[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int row = 8 * k + (lane >> 2), rr = wrow0 + row;
            if (rr >= nrows) { dst[k] = nullptr; continue; }
            if (part < 0) {
              const int t2 = rr / G, h2 = rr - t2 * G;
              dst[k] = reinterpret_cast<char*>(A.out + (size_t)(U.row0 + U.q0 + t2) * ((size_t)Hq * AT_D) + (size_t)(hkv * G + h2) * AT_D) + 16 * (lane & 3);
            } else {
              dst[k] = reinterpret_cast<char*>(A.part_acc + (((size_t)part * Hkv + hkv) * A.part_rows + rr) * AT_D) + 16 * (lane & 3);
            }
          }
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            if (n_steps > 0) {
              tc_ld_32x32b_x32(lane_base + o_col + c * 32, o);
              tc_wait_ld();
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = 0u;
            }
            if (part < 0) {
              uint32_t pk[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) pk[i] = at_pack(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv);
              at_store_rows(stage, pk, lane, dst, c * 64);
            } else {
              at_store_rows(stage, o, lane, dst, c * 128);
              at_store_rows(stage, o + 16, lane, dst, c * 128 + 64);
            }
          }
          if (valid && part >= 0) { A.part_ml[2 * slot] = m_run; A.part_ml[2 * slot + 1] = l_run; }
        }
        AT_STAMP(4);
      }
      if (role == 1) {
        __threadfence();                              // this CTA's part is visible before it is counted as written
        at_softmax_sync();
        if (threadIdx.x == 0) atomicAdd(arrived + 1, 1);
      }
      // ---- the last part: out = sum_s 2^(m_s - m) acc_s / sum_s 2^(m_s - m) l_s, in float32, in the order of the
      // parts whichever of them this is (reference attn.py:520-594) ---------------------------------------------
      if (role == 2 && active) {
        tc_fence_after();
        const int first = part - U.split, me = U.split, n_parts_of_tile = U.n_parts, nrows = U.nrows;
        const int wrow0 = w * AT_ROWS + quarter * 32;
        uint4* stage = sm.stage[warp];
        const size_t part_stride = (size_t)Hkv * A.part_rows;        // rows between a part and the next
        auto merged_out = [&](auto p2_tag, auto ch_tag) {
          // P2: the parts, rounded up; CH: columns of the others' accumulators asked for at a time (all loads in flight)
          constexpr int P2 = decltype(p2_tag)::value, CH = decltype(ch_tag)::value, PASSES = CH / 16;
          // this lane works on 16 bytes of the warp's rows 8 k + lane / 4: the parts' weights for those rows
          float fw[4][P2];
          const float* src[4];
          char* outp[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int row = 8 * k + (lane >> 2), rr = wrow0 + row;
            const float m_own = __shfl_sync(0xffffffffu, m_run, row), l_own = __shfl_sync(0xffffffffu, l_run, row);
            const bool in = rr < nrows;
            const size_t sl0 = ((size_t)first * Hkv + hkv) * A.part_rows + rr;
            float mm[P2], ll[P2];
#pragma unroll
            for (int sp = 0; sp < P2; ++sp) {
              mm[sp] = -INFINITY; ll[sp] = 0.f;
              if (sp == me) { mm[sp] = m_own; ll[sp] = l_own; }
              else if (sp < n_parts_of_tile && in) {
                mm[sp] = __ldcg(A.part_ml + 2 * (sl0 + sp * part_stride));
                ll[sp] = __ldcg(A.part_ml + 2 * (sl0 + sp * part_stride) + 1);
              }
            }
            float m = -INFINITY;
#pragma unroll
            for (int sp = 0; sp < P2; ++sp) m = fmaxf(m, mm[sp]);
            const float mb = m == -INFINITY ? 0.f : m;
            float l = 0.f;
#pragma unroll
            for (int sp = 0; sp < P2; ++sp) { fw[k][sp] = exp2f(mm[sp] - mb); l += fw[k][sp] * ll[sp]; }
            const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
            for (int sp = 0; sp < P2; ++sp) fw[k][sp] *= inv;
            src[k] = in ? A.part_acc + sl0 * AT_D + 4 * (lane & 3) : nullptr;
            const int t2 = rr / G, h2 = rr - t2 * G;
            outp[k] = in ? reinterpret_cast<char*>(A.out + (size_t)(U.row0 + U.q0 + t2) * ((size_t)Hq * AT_D) + (size_t)(hkv * G + h2) * AT_D) + 8 * (lane & 3)
                         : nullptr;
          }
          uint32_t o[32];
#pragma unroll
          for (int c0 = 0; c0 < AT_D; c0 += CH) {
            // (with many parts the loads of a row are asked for only when the row's turn comes: registers)
            constexpr bool AHEAD = P2 <= 4;
            float4 oth[AHEAD ? PASSES : 1][AHEAD ? 4 : 1][P2];
            auto ask = [&](int ps, int k, float4 (&into)[P2]) {
#pragma unroll
              for (int sp = 0; sp < P2; ++sp)
                into[sp] = sp != me && sp < n_parts_of_tile && src[k] != nullptr
                               ? __ldcg(reinterpret_cast<const float4*>(src[k] + sp * part_stride * AT_D + c0 + ps * 16))
                               : make_float4(0.f, 0.f, 0.f, 0.f);
            };
            if (AHEAD) {
#pragma unroll
              for (int ps = 0; ps < PASSES; ++ps)
#pragma unroll
                for (int k = 0; k < 4; ++k) ask(ps, k, oth[AHEAD ? ps : 0][AHEAD ? k : 0]);
            }
#pragma unroll
            for (int ps = 0; ps < PASSES; ++ps) {
              const int col = c0 + ps * 16;
              if (col % 32 == 0) {
                if (n_steps > 0) {
                  tc_ld_32x32b_x32(lane_base + o_col + col, o);
                  tc_wait_ld();
                } else {
#pragma unroll
                  for (int i = 0; i < 32; ++i) o[i] = 0u;
                }
              }
              // this warp's own 32 rows x 16 columns, from a row per lane to 16 bytes of four rows per lane
              const uint32_t* v = o + (col % 32);
#pragma unroll
              for (int c = 0; c < 4; ++c)
                stage[lane * 4 + (c ^ ((lane >> 1) & 3))] = make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
              __syncwarp();
              uint4 own[4];
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const int row = 8 * k + (lane >> 2);
                own[k] = stage[row * 4 + ((lane & 3) ^ ((row >> 1) & 3))];
              }
              __syncwarp();
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                float4 (&theirs)[P2] = oth[AHEAD ? ps : 0][AHEAD ? k : 0];
                if (!AHEAD) ask(ps, k, theirs);
#pragma unroll
                for (int sp = 0; sp < P2; ++sp) {
                  const bool mine = sp == me;
                  const float4 x = make_float4(mine ? __uint_as_float(own[k].x) : theirs[sp].x, mine ? __uint_as_float(own[k].y) : theirs[sp].y,
                                               mine ? __uint_as_float(own[k].z) : theirs[sp].z, mine ? __uint_as_float(own[k].w) : theirs[sp].w);
                  const float wgt = fw[k][sp];
                  acc.x += wgt * x.x; acc.y += wgt * x.y; acc.z += wgt * x.z; acc.w += wgt * x.w;
                }
                if (outp[k] != nullptr) {
                  uint2 v2;
                  v2.x = at_pack(acc.x, acc.y);
                  v2.y = at_pack(acc.z, acc.w);
                  *reinterpret_cast<uint2*>(outp[k] + 2 * col) = v2;
                }
              }
            }
          }
        };
        if (n_parts_of_tile <= 2) merged_out(std::integral_constant<int, 2>(), std::integral_constant<int, 64>());
        else if (n_parts_of_tile <= 4) merged_out(std::integral_constant<int, 4>(), std::integral_constant<int, 16>());
        else merged_out(std::integral_constant<int, AT_MAX_PARTS>(), std::integral_constant<int, 16>());
      }
      AT_STAMP(5);
#undef AT_STAMP
      // (a group whose wait ran out walks the remaining units without work: the other group may be waiting for it
      // at a meeting above)
    }
  }
  // everyone meets here; the allocating warp frees the tensor memory
  tc_fence_before();
  __syncthreads();
  QE_TL_FLUSH_STAMPS();
  if (warp == 9) {
    tc_fence_after();
    tc_dealloc(tmem, AT_TMEM_COLS);
  }
}

extern "C" int qe_flash_attention_tc_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_at_status, sizeof(int));
  return v;
}
extern "C" void qe_flash_attention_tc_clear_status() {
  int v = 0;
  cudaMemcpyToSymbol(g_at_status, &v, sizeof(int));
}

// Host side: how to cut a step's tiles so that the CTAs keep all SMs busy to the end.  A tile of a
// prompt visits as many key steps as its place in the prompt asks for, so the tiles of one prompt
// are as unequal as 1 : 2 : ... : n, and with fewer tiles than a few per SM the longest tile alone sets
// the kernel's time.  Given the tiles' key steps, this tries a few caps (the most steps a work item may
// have; longer tiles are cut into parts of equal length, at most max_parts), lays each candidate's
// items out as the GPU will run them (longest first, each to the SM that is free first, every item
// once per kv head) and returns the cap with the shortest schedule, 0 for "cut nothing".  Costs are in
// key steps: item_cost for a CTA's start and end, part_cost on top for a part's scratch and merge.
extern "C" int qe_flash_attention_tc_balance(const int* steps, int n_tiles, int Hkv, int sms, int min_part_steps,
                                             int max_parts, float item_cost, float part_cost) {
  if (n_tiles <= 0 || Hkv <= 0 || sms <= 0 || max_parts < 2) return 0;
  int longest = 0;
  for (int i = 0; i < n_tiles; ++i) longest = steps[i] > longest ? steps[i] : longest;
  if (longest < 2 * min_part_steps) return 0;
  auto schedule = [&](int cap) {
    float* items = new float[(size_t)n_tiles * max_parts];
    int n = 0;
    for (int i = 0; i < n_tiles; ++i) {
      int parts = cap > 0 ? (steps[i] + cap - 1) / cap : 1;
      if (parts > max_parts) parts = max_parts;
      if (parts <= 1) { items[n++] = (float)steps[i] + item_cost; continue; }
      const int per = (steps[i] + parts - 1) / parts;
      for (int done = 0; done < steps[i]; done += per) {
        const int len = steps[i] - done < per ? steps[i] - done : per;
        items[n++] = (float)len + item_cost + part_cost;
      }
    }
    // longest first (insertion sort would do for these sizes; a simple heap sort keeps it n log n)
    for (int i = 1; i < n; ++i) {
      const float v = items[i];
      int j = i - 1;
      while (j >= 0 && items[j] < v) { items[j + 1] = items[j]; --j; }
      items[j + 1] = v;
    }
    float* free_at = new float[sms];                // a binary min-heap of the SMs' free times
    for (int i = 0; i < sms; ++i) free_at[i] = 0.f;
    float end = 0.f;
    for (int i = 0; i < n; ++i)
      for (int h = 0; h < Hkv; ++h) {
        float t = free_at[0] + items[i];
        end = t > end ? t : end;
        int k = 0;                                  // replace the root and sift down
        for (;;) {
          const int l = 2 * k + 1, r = l + 1;
          int m = k;
          float best = t;
          if (l < sms && free_at[l] < best) { m = l; best = free_at[l]; }
          if (r < sms && free_at[r] < best) { m = r; best = free_at[r]; }
          if (m == k) break;
          free_at[k] = free_at[m];
          k = m;
        }
        free_at[k] = t;
      }
    delete[] items;
    delete[] free_at;
    return end;
  };
  const float whole = schedule(0);
  float best = whole * 0.95f;                       // cutting has to gain something
  int best_cap = 0, last = 0;
  for (int f = 7; f >= 1; --f) {
    int cap = (longest * f + 7) / 8;
    if (cap < min_part_steps) cap = min_part_steps;
    if (cap == last || cap >= longest) continue;
    last = cap;
    const float t = schedule(cap);
    if (t < best) { best = t; best_cap = cap; }
  }
  return best_cap;
}

// Whether the kernel takes this geometry: head size 128; a group size (query heads per kv head) that
// divides 128; pages of a power of two of at least 8 tokens.
extern "C" int qe_flash_attention_tc_supported(int Hq, int Hkv, int D, int page_size) {
  if (D != AT_D || Hkv < 1 || Hq % Hkv) return 0;
  const int G = Hq / Hkv;
  if (G > AT_ROWS || (G & (G - 1))) return 0;
  if (page_size < 8 || (page_size & (page_size - 1))) return 0;
  return 1;
}

// Which CTA runs which work units: the units (item i for kv head h is unit i Hkv + h) in the order of the item list,
// which the caller has sorted by key steps, longest first, each to the CTA with the least work so far; item_cost[i] is
// what a unit of item i costs (its key steps plus what its start, its end and, for a part, its scratch and merge
// cost, in key steps).  out: n_ctas + 1 offsets into out itself, then the CTAs' unit numbers; it must hold
// n_ctas + 1 + n_items Hkv ints.  Returns the number of ints written, 0 if the arguments make no sense.
extern "C" int qe_flash_attention_tc_schedule(const float* item_cost, int n_items, int Hkv, int n_ctas, int* out) {
  if (n_items <= 0 || Hkv <= 0 || n_ctas <= 0) return 0;
  const long n_units = (long)n_items * Hkv;
  if (n_units > 0x3fffffffL) return 0;
  struct Slot { float load; int cta; };
  Slot* heap = new Slot[n_ctas];                    // a binary min-heap by (load, cta)
  int* owner = new int[n_units];
  int* count = new int[n_ctas];
  for (int i = 0; i < n_ctas; ++i) { heap[i] = Slot{0.f, i}; count[i] = 0; }
  auto less = [](const Slot& a, const Slot& b) { return a.load < b.load || (a.load == b.load && a.cta < b.cta); };
  for (long u = 0; u < n_units; ++u) {
    Slot top = heap[0];
    owner[u] = top.cta;
    ++count[top.cta];
    top.load += item_cost[u / Hkv];
    int k = 0;                                      // replace the root and sift down
    for (;;) {
      const int l = 2 * k + 1, r = l + 1;
      int m = k;
      Slot best = top;
      if (l < n_ctas && less(heap[l], best)) { m = l; best = heap[l]; }
      if (r < n_ctas && less(heap[r], best)) { m = r; best = heap[r]; }
      if (m == k) break;
      heap[k] = heap[m];
      k = m;
    }
    heap[k] = top;
  }
  int at = n_ctas + 1;
  for (int c = 0; c < n_ctas; ++c) { out[c] = at; at += count[c]; count[c] = out[c]; }
  out[n_ctas] = at;
  for (long u = 0; u < n_units; ++u) out[count[owner[u]]++] = (int)u;
  delete[] heap;
  delete[] owner;
  delete[] count;
  return at;
}

// q: the step's queries [T, Hq, 128] with q_stride elements between tokens; pages [num_pages, 2, Hkv,
// page_size, 128]; items: 12 ints each (see attention_flash.cuh; a tile here is 256 / G tokens, and
// n_splits is the number of parts of the tile when part >= 0); sched: what qe_flash_attention_tc_schedule
// wrote for these items and n_ctas CTAs, on the device; counters: two ints per (first part, kv
// head), zero before the first launch (the kernel leaves them zero), needed when any item has part >= 0.
extern "C" int qe_flash_attention_tc(const void* q, long q_stride, int T, const void* pages, int num_pages,
                                     const int* block_tables, int max_blocks, const int* items, int n_items,
                                     const int* sched, int n_ctas,
                                     void* out, float* part_acc, float* part_ml, int part_rows, int* counters,
                                     float scale, int window, int Hq, int Hkv, int D, int page_size,
                                     cudaStream_t stream) {
  if (n_items <= 0) return 0;
  if (sched == nullptr || n_ctas <= 0 || (long)n_ctas > (long)n_items * Hkv)
    QE_REFUSE("flash_attention_tc: a schedule for 1 to %ld CTAs is needed, not one for %d", (long)n_items * Hkv, n_ctas);
  if (part_acc && part_rows != 2 * AT_ROWS) QE_REFUSE("flash_attention_tc: parts have %d rows, not %d", part_rows, 2 * AT_ROWS);
  if (!qe_flash_attention_tc_supported(Hq, Hkv, D, page_size))
    QE_REFUSE("flash_attention_tc: heads %d/%d, head_dim %d, page size %d are not supported", Hq, Hkv, D, page_size);
  if ((((uintptr_t)q | (uintptr_t)pages | (uintptr_t)out) & 15) || (q_stride % 8))
    QE_REFUSE("flash_attention_tc: operands must be 16-byte aligned");
  if (scale <= 0.f) QE_REFUSE("flash_attention_tc: the scale must be positive");
  if ((long)n_items * Hkv > 0x7fffffffL) QE_REFUSE("flash_attention_tc: too many work items");
  const int G = Hq / Hkv;
  CUtensorMap map_q, map_kv;
  {
    const uint64_t dims[3] = {(uint64_t)AT_D, (uint64_t)Hq, (uint64_t)T};
    const uint64_t strides[2] = {(uint64_t)AT_D * 2, (uint64_t)q_stride * 2};
    const uint32_t box[3] = {64, (uint32_t)G, (uint32_t)(AT_ROWS / G)};
    if (!qe_tensor_map_bf16(q, 3, dims, strides, box, &map_q)) return 1;
  }
  {
    const uint64_t P = (uint64_t)page_size;
    const uint64_t dims[5] = {(uint64_t)AT_D, P, (uint64_t)Hkv, 2, (uint64_t)num_pages};
    const uint64_t strides[4] = {(uint64_t)AT_D * 2, P * AT_D * 2, (uint64_t)Hkv * P * AT_D * 2, 2ull * Hkv * P * AT_D * 2};
    const uint32_t box[5] = {64, (uint32_t)(page_size < AT_BN ? page_size : AT_BN), 1, 1, 1};
    if (!qe_tensor_map_bf16(pages, 5, dims, strides, box, &map_kv)) return 1;
  }
  int page_shift = 0;
  while ((1 << page_shift) < page_size) ++page_shift;
  AtArgs args{block_tables, max_blocks, num_pages, items, sched, (__nv_bfloat16*)out, part_acc, part_ml, part_rows, counters,
              scale * 1.4426950408889634f, window, Hq, Hkv, page_shift};
  const size_t smem = sizeof(AtSmem) + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(flash_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) QE_REFUSE("flash_attention_tc: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  qe_launch(flash_attention_tc_kernel, dim3((unsigned)n_ctas), dim3(AT_THREADS), smem, stream, map_q, map_kv, args);
  QE_CHECK_LAUNCH("flash_attention_tc");
  return 0;
}
