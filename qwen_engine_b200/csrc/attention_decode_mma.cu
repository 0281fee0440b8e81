// Attention of decoded tokens over the paged cache in bfloat16, head size 128, up to 16 query rows
// per kv head (token x query head of the group), with the arithmetic on the tensor cores
// (mma.sync.m16n8k16; the 16 rows of the instruction are the item's rows, padded with zeros) and the
// loads organised for bandwidth: flash decoding as the reference's (src/layers/fused_ops/attn.py:374-594),
// every key and value read once for all query heads of its kv head.
//
// One CTA (4 warps, or 8) serves one work item (a request's rows, a range of its keys) and one kv head.  The
// keys are dealt to the warps in groups of 16: group i belongs to warp i mod 4 (8), which copies the
// group's keys and values into shared memory of its own (cp.async, 16 bytes a lane, rows padded so
// that ldmatrix meets no bank conflict), three groups ahead, and works on them alone: scores, masked
// online softmax in float32 with a running max and sum of its own, P rounded to bfloat16 (attn.py:263),
// P V.  No barrier of the CTA stands in the loop; the warps' results are combined in shared
// memory once at the end, by the formula that combines the parts of a split context.  Two CTAs of 4
// warps fit an SM, or one of 8, so up to 24 groups (192 KB) are in flight per SM.  Groups that hold only
// keys of earlier steps are requested before the kernel waits for its predecessor (the rotary kernel wrote
// the new keys).  The wide form is for steps with no more CTAs than SMs: all of them start at once, beside
// the CTAs of the kernel before, where two CTAs per SM would leave some waiting for room.
//
// A decode step is a chain of short kernels, each of which waits for the latency of its first loads.  The
// keys and values do not depend on the step's activations, so this kernel can ask L2 for the NEXT
// layer's keys and values (`prefetch_delta`: the distance in bytes from this layer's cache to the next
// layer's, which has the same pages at the same places; 0: nothing is asked) while it works on its own:
// they arrive during the kernels between the two attentions, and the next layer's attention finds them
// on the chip.  The caller asks for that only when a layer's keys and values are a fraction of L2.
//
// Work items, parts, scratch and counters are those of the flash kernel for few rows (attention_flash.cuh: 12 ints an
// item; a part writes its accumulator, max and sum to scratch memory and the last CTA to finish combines them), or the
// parts of a request form a thread-block cluster and meet in its first CTA's shared memory.
#include "attention_flash.cuh"

#define DM_MAX_WARPS 8            // warps of a CTA: 4 (two CTAs per SM) or 8 (one CTA per SM), a template parameter
#define DM_D 128
#define DM_LD (DM_D + 8)          // padded row of a tile in shared memory, in elements
#define DM_GK 16                  // keys per group
#define DM_MAX_STAGES 3           // groups in flight per warp at most (a template parameter chooses 2 or 3)
#define DM_ROWS 16                // rows of an item at most
#define DM_PART_ALIGN 16          // a request's parts are multiples of this many keys (the host's plan cuts them so)

#define DM_TILE_BYTES (DM_GK * DM_LD * 2)                       // keys or values of a group: 4352
#define DM_WARP_BYTES_OF(stages) ((stages) * 2 * DM_TILE_BYTES)     // a warp's stages: 17408 or 26112
#define DM_Q_BYTES (DM_ROWS * DM_LD * 2)                        // the item's queries: 4352
#define DM_SMEM_BYTES_OF(stages, warps) (DM_Q_BYTES + (warps) * DM_WARP_BYTES_OF(stages) + (warps) * 128)
static_assert(DM_WARP_BYTES_OF(2) >= 2 * DM_ROWS * DM_D * 4, "a warp's stages hold its float32 result and the CTA's at the end");

__device__ __forceinline__ void dm_cp_async16_zfill(void* smem, const void* gmem, bool valid) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;                 // 0: nothing is read, the 16 bytes are zeroed
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" :: "r"(a), "l"(gmem), "r"(bytes));
}

template <bool CL, int DM_STAGES, int DM_WARPS>
__global__ void __launch_bounds__(DM_WARPS * 32, DM_WARPS == 4 ? 2 : 1)
decode_attention_mma_kernel(FaArgs A, long long prefetch_delta, int early_issue, int push_rows) {
  constexpr int DM_THREADS = DM_WARPS * 32;
  constexpr int DM_WARP_BYTES = DM_WARP_BYTES_OF(DM_STAGES);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int D = DM_D, LD = DM_LD;
  __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  unsigned char* stages = smem_raw + DM_Q_BYTES;
  float* s_m = reinterpret_cast<float*>(smem_raw + DM_Q_BYTES + DM_WARPS * DM_WARP_BYTES);   // [warps][16] warps' maxima
  float* s_l = s_m + DM_WARPS * DM_ROWS;                                                     // [warps][16] warps' sums
  __shared__ float m_run[DM_ROWS], l_run[DM_ROWS];  // the CTA's max and sum (read by the cluster's first CTA)
  __shared__ int s_last;
  __shared__ uint64_t merge_bar;                    // CL, push_rows > 0: in the cluster's first CTA, counts the other parts' bytes
  __shared__ int s_abort;
  pdl_launch_dependents();
  if constexpr (CL) {
    // Parts that meet by being pushed (push_rows > 0: the rows an item may have, for which the launcher has added an
    // in-box per part behind the warps' memory): the first CTA's barrier is set up, and every CTA says so to the
    // cluster now and looks for the others' word only when its own part is done.
    if (push_rows > 0) {
      if (threadIdx.x == 0) {
        fa_bar_init(&merge_bar, 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
      }
      asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    }
  }
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hkv = blockIdx.y;
  const int Hq = A.Hq, Hkv = A.Hkv, window = A.window, page_size = A.page_size;
  const int G = Hq / Hkv;

  // the work lists come from the host's copy, not from a kernel
  const int* it = A.items + (size_t)blockIdx.x * FA_ITEM_INTS;
  const int req = it[0], q0 = it[1], part = it[4], n_splits = it[5], split = it[6];
  int kv_lo = it[2], kv_hi_item = it[3];
  const int row0 = it[7], q_len = it[8], ctx = it[9];
  const int ntok = min(DM_ROWS / G, min(FA_BM / G, q_len - q0));
  const int nrows = ntok * G;                       // the launcher promised that the item's rows fit
  const int first_pos = ctx + q0;
  if (n_splits > 0) {
    const int total = ctx + q_len;
    const int lo = window > 0 ? max(0, ctx - window + 1) / FA_BN * FA_BN : 0;
    const int per = ((total - lo + n_splits - 1) / n_splits + DM_PART_ALIGN - 1) / DM_PART_ALIGN * DM_PART_ALIGN;
    kv_lo = lo + split * per;
    kv_hi_item = min(total, kv_lo + per);
  }
  const int kv_end = min(kv_hi_item, first_pos + ntok);
  int kv_begin = max(kv_lo, 0);
  if (window > 0) kv_begin = max(kv_begin, first_pos - window + 1);
  const int n_groups = kv_end > kv_begin ? (kv_end - kv_begin + DM_GK - 1) / DM_GK : 0;

  const int* __restrict__ table = A.block_tables + (size_t)req * A.max_blocks;
  const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;
  const size_t page_stride = (size_t)2 * Hkv * page_size * D;
  const size_t v_off = (size_t)Hkv * page_size * D;
  const __nv_bfloat16* head_base = A.pages + (size_t)hkv * page_size * D;
  // a group that starts at a multiple of 16 keys lies in one page when pages are multiples of 16 keys
  const bool one_page = page_shift >= 4 && (kv_begin & 15) == 0;

  unsigned char* my_stages = stages + (size_t)warp * DM_WARP_BYTES;
  const int ch = lane & 15, rsub = lane >> 4;       // this lane's 16-byte piece of a row; rows rsub, rsub + 2, ...
  // keys and values of group `gidx` into stage `st` of this warp
  auto issue = [&](int gidx, int st) {
    const int j0 = kv_begin + gidx * DM_GK;
    unsigned char* kdst = my_stages + (size_t)st * 2 * DM_TILE_BYTES;
    unsigned char* vdst = kdst + DM_TILE_BYTES;
    if (one_page) {
      const __nv_bfloat16* base = head_base + (size_t)__ldg(table + (j0 >> page_shift)) * page_stride +
                                  (size_t)(j0 & (page_size - 1)) * D + ch * 8;
#pragma unroll
      for (int i = 0; i < DM_GK / 2; ++i) {
        const int row = rsub + 2 * i;
        const bool ok = j0 + row < kv_end;
        const __nv_bfloat16* src = ok ? base + (size_t)row * D : A.pages;
        dm_cp_async16_zfill(kdst + row * (LD * 2) + ch * 16, src, ok);
        dm_cp_async16_zfill(vdst + row * (LD * 2) + ch * 16, ok ? src + v_off : A.pages, ok);
      }
    } else {
#pragma unroll
      for (int i = 0; i < DM_GK / 2; ++i) {
        const int row = rsub + 2 * i, j = j0 + row;
        const bool ok = j < kv_end;
        const __nv_bfloat16* src = A.pages;
        if (ok) {
          int blk, off;
          if (page_shift >= 0) { blk = j >> page_shift; off = j & (page_size - 1); }
          else { blk = j / page_size; off = j - blk * page_size; }
          src = head_base + (size_t)__ldg(table + blk) * page_stride + (size_t)off * D + ch * 8;
        }
        dm_cp_async16_zfill(kdst + row * (LD * 2) + ch * 16, src, ok);
        dm_cp_async16_zfill(vdst + row * (LD * 2) + ch * 16, ok ? src + v_off : A.pages, ok);
      }
    }
  };

  // ---- the first groups: those of earlier steps' keys at once, the rest after the wait -----------------
  // (this warp's groups are warp, warp + 4, ...; its i-th group uses stage i mod DM_STAGES)
  bool early[DM_STAGES];
#pragma unroll
  for (int s = 0; s < DM_STAGES; ++s) {
    const int gidx = warp + s * DM_WARPS;
    early[s] = early_issue && gidx < n_groups && kv_begin + (gidx + 1) * DM_GK <= ctx;
    if (early[s]) issue(gidx, s);
  }
  if (prefetch_delta != 0) {
    // (before the wait for the kernel before this one: nothing here depends on it, and the CTA has microseconds to
    // spare until that kernel is done)
    // the same keys and values of the next layer, into L2: whole runs of a page where a group lies in one
    // (two lanes: keys, values), else row by row (a lane each)
    for (int gidx = warp; gidx < n_groups; gidx += DM_WARPS) {
      const int j0 = kv_begin + gidx * DM_GK;
      const int row = one_page ? 0 : (lane & 15), is_v = one_page ? lane : (lane >> 4);
      const int j = j0 + row;
      if (j < kv_end && is_v < 2) {
        int blk, off;
        if (page_shift >= 0) { blk = j >> page_shift; off = j & (page_size - 1); }
        else { blk = j / page_size; off = j - blk * page_size; }
        const __nv_bfloat16* src = head_base + (size_t)__ldg(table + blk) * page_stride + (size_t)off * D + (is_v ? v_off : 0);
        const unsigned bytes = (unsigned)(one_page ? min(DM_GK, kv_end - j0) : 1) * (unsigned)(D * 2);
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n"
                     :: "l"(reinterpret_cast<const unsigned char*>(src) + prefetch_delta), "r"(bytes) : "memory");
      }
    }
  }
  pdl_wait();                                       // q and the new tokens' keys and values: the previous kernels' outputs
#pragma unroll
  for (int s = 0; s < DM_STAGES; ++s) {
    const int gidx = warp + s * DM_WARPS;
    if (!early[s] && gidx < n_groups) issue(gidx, s);
    cp_async_commit();                              // one commit per stage, issued or not: the waits below count them
  }
  // the item's queries: row r = (token r / G, head r mod G of the group); rows beyond the item's are zero
  for (int e = tid; e < DM_ROWS * (D / 8); e += DM_THREADS) {
    const int r = e / (D / 8), c8 = e - r * (D / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < nrows) {
      const int ti = r / G, hg = r - ti * G;
      v = __ldcg(reinterpret_cast<const uint4*>(A.q + (size_t)(row0 + q0 + ti) * A.q_stride + (size_t)(hkv * G + hg) * D) + c8);
    }
    *reinterpret_cast<uint4*>(sq + r * LD + c8 * 8) = v;
  }
  if (tid == 0) s_last = 0;
  __syncthreads();

  // ---- this warp's groups ---------------------------------------------------------------------------------
  const int g = lane >> 2;
  const int pos_lo = first_pos + g / G, pos_hi = first_pos + (g + 8) / G;
  const int last_pos = first_pos + ntok - 1;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  int st = 0;
  QE_TL_MARK(2);
  for (int gidx = warp; gidx < n_groups; gidx += DM_WARPS) {
    cp_async_wait<DM_STAGES - 1>();                 // all but the latest commits of the other stages have landed: this group has
    __syncwarp();
    const int j0 = kv_begin + gidx * DM_GK;
    const __nv_bfloat16* tk = reinterpret_cast<const __nv_bfloat16*>(my_stages + (size_t)st * 2 * DM_TILE_BYTES);
    const __nv_bfloat16* tv = tk + DM_GK * LD;
    const bool all_allowed = j0 + DM_GK <= kv_end && j0 + DM_GK - 1 <= first_pos && (window <= 0 || j0 > last_pos - window);
    fa_tile<D, 1>(sq, tk, tv, 0, 0, j0, kv_begin, kv_end, pos_lo, pos_hi, window, A.scale_log2, lane,
                  m_lo, m_hi, l_lo, l_hi, o, all_allowed);
    __syncwarp();                                   // every lane is done with the stage before it is filled again
    const int nxt = gidx + DM_STAGES * DM_WARPS;
    if (nxt < n_groups) issue(nxt, st);
    cp_async_commit();
    st = st + 1 == DM_STAGES ? 0 : st + 1;
  }
  cp_async_wait<0>();
  __syncwarp();
  QE_TL_MARK(3);

  // ---- the four warps' results meet (each in its own stages' memory first) ------------------------------
  float* mine = reinterpret_cast<float*>(my_stages);                  // [16][128]
  {
    const int c = lane & 3;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {               // (only the item's rows are read below)
      if (g < nrows) *reinterpret_cast<float2*>(mine + g * D + i * 8 + 2 * c) = make_float2(o[i][0], o[i][1]);
      if (g + 8 < nrows) *reinterpret_cast<float2*>(mine + (g + 8) * D + i * 8 + 2 * c) = make_float2(o[i][2], o[i][3]);
    }
    if (c == 0) {
      s_m[warp * DM_ROWS + g] = m_lo; s_m[warp * DM_ROWS + g + 8] = m_hi;
      s_l[warp * DM_ROWS + g] = l_lo; s_l[warp * DM_ROWS + g + 8] = l_hi;
    }
  }
  __syncthreads();
  float* fin = reinterpret_cast<float*>(stages) + DM_ROWS * D;        // CL: [16][128] after warp 0's result
  __nv_bfloat16* out_row0 = A.out + (size_t)(row0 + q0) * ((size_t)Hq * D);
  for (int e = tid; e < nrows * D; e += DM_THREADS) {
    const int r = e / D, d = e - r * D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < DM_WARPS; ++w) m = fmaxf(m, s_m[w * DM_ROWS + r]);
    const float mb = m == -INFINITY ? 0.f : m;
    float l = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < DM_WARPS; ++w) {
      const float wgt = exp2f(s_m[w * DM_ROWS + r] - mb);
      l += wgt * s_l[w * DM_ROWS + r];
      acc += wgt * reinterpret_cast<const float*>(stages + (size_t)w * DM_WARP_BYTES)[r * D + d];
    }
    if (d == 0) { m_run[r] = m; l_run[r] = l; }
    if constexpr (CL) {
      fin[r * D + d] = acc;
    } else if (part < 0) {
      const int ti = r / G, hg = r - ti * G;
      out_row0[(size_t)ti * ((size_t)Hq * D) + (size_t)(hkv * G + hg) * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    } else {
      const size_t slot = ((size_t)part * Hkv + hkv) * A.part_rows + r;
      A.part_acc[slot * D + d] = acc;
      if (d == 0) { A.part_ml[2 * slot] = m; A.part_ml[2 * slot + 1] = l; }
    }
  }
  if constexpr (CL) {
    if (push_rows > 0) {
      // ---- the parts meet in the cluster's first CTA, pushed there ---------------------------------------
      // Every other CTA stores its accumulator, max and sum into its in-box in the first CTA's shared memory with
      // st.async, which counts the bytes on that CTA's barrier, and is done: no CTA waits for another except the first
      // for the bytes.  (Pulled, the parts cost two barriers of the whole cluster on the step's critical path.)
      asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");     // (arrived at the top: the barrier exists)
      const uint32_t crank = cluster_cta_rank();
      const int S = (int)cluster_num_ctas();        // = n_splits, at most 8
      float* inbox = s_l + DM_WARPS * DM_ROWS;      // [S - 1][push_rows (D + 2)]: accumulators, then (max, sum) per row
      const int per = push_rows * (D + 2);
      if (crank != 0) {
        const uint32_t dst = cluster_map_shared(inbox + (size_t)(crank - 1) * per, 0);
        const uint32_t bar = cluster_map_shared(&merge_bar, 0);
        for (int e = tid; e < nrows * D; e += DM_THREADS) {
          asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];\n"
                       :: "r"(dst + 4u * (uint32_t)e), "r"(__float_as_uint(fin[e])), "r"(bar) : "memory");
          const int r = e / D;
          if (e - r * D == 0) {
            asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];\n"
                         :: "r"(dst + 4u * (uint32_t)(push_rows * D + 2 * r)), "r"(__float_as_uint(m_run[r])), "r"(bar) : "memory");
            asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];\n"
                         :: "r"(dst + 4u * (uint32_t)(push_rows * D + 2 * r + 1)), "r"(__float_as_uint(l_run[r])), "r"(bar) : "memory");
          }
        }
        return;
      }
      __syncthreads();                              // this CTA's own max and sum of every row are in place
      if (tid == 0) {
        const uint32_t bytes = (uint32_t)(S - 1) * (uint32_t)(nrows * D + 2 * nrows) * 4u;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" :: "r"(fa_smem(&merge_bar)), "r"(bytes) : "memory");
      }
      if (!fa_bar_wait(&merge_bar, 0, &s_abort, 5)) return;          // bounded: the word says so, nothing is written
      for (int e = tid; e < nrows * D; e += DM_THREADS) {
        const int r = e / D, d = e - r * D;
        float mm[8], ll[8], aa[8];
        mm[0] = m_run[r]; ll[0] = l_run[r]; aa[0] = fin[e];
#pragma unroll
        for (int sp = 1; sp < 8; ++sp) {
          mm[sp] = -INFINITY; ll[sp] = 0.f; aa[sp] = 0.f;
          if (sp < S) {
            const float* box = inbox + (size_t)(sp - 1) * per;
            mm[sp] = box[push_rows * D + 2 * r];
            ll[sp] = box[push_rows * D + 2 * r + 1];
            aa[sp] = box[e];
          }
        }
        // out = sum_s 2^(m_s - m) acc_s / sum_s 2^(m_s - m) l_s, in float32, in the order of the parts
        float m = -INFINITY;
#pragma unroll
        for (int sp = 0; sp < 8; ++sp) m = fmaxf(m, mm[sp]);
        const float mb = m == -INFINITY ? 0.f : m;
        float l = 0.f, acc = 0.f;
#pragma unroll
        for (int sp = 0; sp < 8; ++sp) {
          if (sp < S) {
            const float wgt = exp2f(mm[sp] - mb);
            l += wgt * ll[sp];
            acc += wgt * aa[sp];
          }
        }
        const int ti = r / G, hg = r - ti * G;
        out_row0[(size_t)ti * ((size_t)Hq * D) + (size_t)(hkv * G + hg) * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
      }
      return;
    }
    // ---- the parts meet in the cluster's first CTA -------------------------------------------------------
    cluster_sync_all();                             // every part's accumulator, max and sum are in place
    if (cluster_cta_rank() == 0) {
      const int S = (int)cluster_num_ctas();        // = n_splits, at most 8
      for (int e = tid; e < nrows * D; e += DM_THREADS) {
        const int r = e / D, d = e - r * D;
        float mm[8], ll[8], aa[8];
#pragma unroll
        for (int sp = 0; sp < 8; ++sp) {
          mm[sp] = -INFINITY; ll[sp] = 0.f; aa[sp] = 0.f;
          if (sp < S) {
            mm[sp] = cluster_ld_f32(cluster_map_shared(&m_run[r], (uint32_t)sp));
            ll[sp] = cluster_ld_f32(cluster_map_shared(&l_run[r], (uint32_t)sp));
            aa[sp] = cluster_ld_f32(cluster_map_shared(&fin[r * D + d], (uint32_t)sp));
          }
        }
        // out = sum_s 2^(m_s - m) acc_s / sum_s 2^(m_s - m) l_s, in float32, in the order of the parts
        float m = -INFINITY;
#pragma unroll
        for (int sp = 0; sp < 8; ++sp) m = fmaxf(m, mm[sp]);
        const float mb = m == -INFINITY ? 0.f : m;
        float l = 0.f, acc = 0.f;
#pragma unroll
        for (int sp = 0; sp < 8; ++sp) {
          if (sp < S) {
            const float wgt = exp2f(mm[sp] - mb);
            l += wgt * ll[sp];
            acc += wgt * aa[sp];
          }
        }
        const int ti = r / G, hg = r - ti * G;
        out_row0[(size_t)ti * ((size_t)Hq * D) + (size_t)(hkv * G + hg) * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
      }
    }
    cluster_sync_all();                             // nobody reads this CTA's shared memory any more
    return;
  }
  // ---- the CTA that finishes a request's last part combines the parts ---------------------------------
  if (part >= 0 && A.counters != nullptr && n_splits > 0) {
    const int first = part - split;
    __threadfence();                                // this CTA's part is visible before it is counted
    __syncthreads();
    if (tid == 0) {
      const int done = atomicAdd(&A.counters[first * Hkv + hkv], 1);
      s_last = (done == n_splits - 1);
      if (s_last) A.counters[first * Hkv + hkv] = 0;         // ready for the next launch
    }
    __syncthreads();
    if (s_last) {
      __threadfence();
      for (int e = tid; e < nrows * D; e += DM_THREADS) {
        const int r = e / D, d = e - r * D;
        float m = -INFINITY;
        for (int sp = 0; sp < n_splits; ++sp)
          m = fmaxf(m, __ldcg(A.part_ml + 2 * ((((size_t)first + sp) * Hkv + hkv) * A.part_rows + r)));
        const float mb = m == -INFINITY ? 0.f : m;
        float l = 0.f, acc = 0.f;
        for (int sp = 0; sp < n_splits; ++sp) {
          const size_t slot = (((size_t)first + sp) * Hkv + hkv) * A.part_rows + r;
          const float wgt = exp2f(__ldcg(A.part_ml + 2 * slot) - mb);
          l += wgt * __ldcg(A.part_ml + 2 * slot + 1);
          acc += wgt * __ldcg(A.part_acc + slot * D + d);
        }
        const int ti = r / G, hg = r - ti * G;
        out_row0[(size_t)ti * ((size_t)Hq * D) + (size_t)(hkv * G + hg) * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
      }
    }
  }
}

static int g_dm_stages = 3;
static int g_dm_early = 1;
// Whether groups of earlier steps' keys are requested before the kernel waits for its predecessor (they then
// compete for memory with the kernels that are still running, which are on the step's critical path).
extern "C" void qe_decode_attention_mma_early(int early) { g_dm_early = early ? 1 : 0; }
// How many groups of keys a warp keeps in flight: 2 (two CTAs of the kernel leave room on an SM for the CTAs of
// the kernels around it) or 3.
extern "C" void qe_decode_attention_mma_stages(int stages) { g_dm_stages = stages >= 3 ? 3 : 2; }

// Whether the parts of a cluster are pushed to its first CTA (1; else that CTA reads them from the others).
static int g_dm_push = 1;
extern "C" void qe_decode_attention_mma_push(int on) { g_dm_push = on ? 1 : 0; }

template <bool CL, int STAGES, int WARPS>
static int launch_decode_mma_as(const FaArgs& fa, long long prefetch_delta, int n_items, int Hkv, int cluster, int max_rows, cudaStream_t stream) {
  constexpr int base_smem = DM_SMEM_BYTES_OF(STAGES, WARPS);
  constexpr int limit = 226 * 1024;                 // (an SM has 227 KB; the kernel's static variables take some)
  // the in-boxes of the other parts behind the warps' memory, if they fit
  const int inbox = CL ? (cluster - 1) * max_rows * (DM_D + 2) * 4 : 0;
  const int push_rows = (CL && g_dm_push && base_smem + inbox <= limit) ? max_rows : 0;
  const int smem = base_smem + (push_rows ? inbox : 0);
  static int configured = 0;
  if (configured < smem) {
    cudaError_t e = cudaFuncSetAttribute(decode_attention_mma_kernel<CL, STAGES, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, CL ? limit : base_smem);
    if (e != cudaSuccess) QE_REFUSE("decode_attention_mma: shared memory %d: %s", smem, cudaGetErrorString(e));
    configured = CL ? limit : base_smem;
  }
  if (CL)
    qe_launch_cluster(decode_attention_mma_kernel<CL, STAGES, WARPS>, dim3(n_items, Hkv), dim3(WARPS * 32), smem, stream, (unsigned)cluster, fa, prefetch_delta, g_dm_early, push_rows);
  else
    qe_launch(decode_attention_mma_kernel<CL, STAGES, WARPS>, dim3(n_items, Hkv), dim3(WARPS * 32), smem, stream, fa, prefetch_delta, g_dm_early, 0);
  QE_CHECK_LAUNCH("decode_attention_mma");
  return 0;
}
// wide: CTAs of 8 warps, one per SM (for steps whose items are at most as many as SMs), else 4 warps, two per SM
template <bool CL>
static int launch_decode_mma(const FaArgs& fa, long long prefetch_delta, int n_items, int Hkv, int cluster, int wide, int max_rows, cudaStream_t stream) {
  if (wide) return launch_decode_mma_as<CL, 3, 8>(fa, prefetch_delta, n_items, Hkv, cluster, max_rows, stream);
  return g_dm_stages == 3 ? launch_decode_mma_as<CL, 3, 4>(fa, prefetch_delta, n_items, Hkv, cluster, max_rows, stream)
                          : launch_decode_mma_as<CL, 2, 4>(fa, prefetch_delta, n_items, Hkv, cluster, max_rows, stream);
}

// Whether the kernel takes this geometry with at most max_rows rows (token x head of the group) per item:
// head size 128 and a group of query heads that fits the instruction's 16 rows.
extern "C" int qe_decode_attention_mma_supported(int Hq, int Hkv, int D, int max_rows) {
  return (D == DM_D && Hkv >= 1 && Hkv <= 65535 && Hq % Hkv == 0 && Hq / Hkv <= DM_ROWS && max_rows >= 1 && max_rows <= DM_ROWS) ? 1 : 0;
}

// q, pages, block tables, items, out and scratch as for the flash kernel; every item has at most max_rows rows, all of
// whole tokens; parts are combined by the CTA that finishes last (counters), or inside clusters (`cluster`:
// the number of parts of every request, 2, 4 or 8, when the items are exactly those parts in order).
// prefetch_pages: null, or another layer's cache of the same shape whose keys and values for the same requests
// L2 is asked for (see the top of this file).
// wide: CTAs of 8 warps, one per SM, instead of 4 warps, two per SM (for steps with at most as many CTAs as SMs).
// Returns 0 when run, 1 when refused, 2 on a launch error.
extern "C" int qe_decode_attention_mma(const void* q, long q_stride, const void* pages, const void* prefetch_pages, const int* block_tables,
                                       int max_blocks, const int* items, int n_items, void* out, float* part_acc,
                                       float* part_ml, int part_rows, int* counters, int max_rows, int cluster, int wide, float scale,
                                       int window, int Hq, int Hkv, int D, int page_size, cudaStream_t stream) {
  if (n_items <= 0) return 0;
  if (!qe_decode_attention_mma_supported(Hq, Hkv, D, max_rows))
    QE_REFUSE("decode_attention_mma: heads %d/%d, head_dim %d, %d rows are not supported", Hq, Hkv, D, max_rows);
  if ((((uintptr_t)q | (uintptr_t)pages | (uintptr_t)prefetch_pages) & 15) || (q_stride % 8))
    QE_REFUSE("decode_attention_mma: operands must be 16-byte aligned");
  const long long delta = prefetch_pages ? (long long)((intptr_t)prefetch_pages - (intptr_t)pages) : 0;
  if (part_acc && counters == nullptr && !cluster) QE_REFUSE("decode_attention_mma: parts need the counters");
  FaArgs fa{(const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)pages, block_tables, max_blocks, items,
            (__nv_bfloat16*)out, part_acc, part_ml, part_rows, counters, scale * 1.4426950408889634f, window, Hq, Hkv,
            page_size};
  if (cluster == 0) return launch_decode_mma<false>(fa, delta, n_items, Hkv, 0, wide, max_rows, stream);
  if ((cluster != 2 && cluster != 4 && cluster != 8) || n_items % cluster)
    QE_REFUSE("decode_attention_mma: %d items cannot form clusters of %d", n_items, cluster);
  return launch_decode_mma<true>(fa, delta, n_items, Hkv, cluster, wide, max_rows, stream);
}

// The status word of the bounded wait for the pushed parts (0 = fine).
extern "C" int qe_decode_attention_mma_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_fa_status, sizeof(int));
  return v;
}
extern "C" void qe_decode_attention_mma_clear_status() {
  int v = 0;
  cudaMemcpyToSymbol(g_fa_status, &v, sizeof(int));
}
