// Attention of decoded tokens over the paged cache in bfloat16, head size 128, for a few query rows
// per kv head (one token x the query heads of the group): the latency-bound case of the reference's
// flash decoding (src/layers/fused_ops/attn.py:374-594).  With so few rows the tensor cores have
// nothing to do; what matters is that a CTA's keys and values are all on their way at once and that
// nothing stands between them and the arithmetic.  So: no matrix instructions, no tile pipeline.
//
// One CTA (256 threads) serves one work item (a request's rows, a range of its keys) and one kv head;
// it walks its keys in chunks of 160.  Per chunk:
//   keys    8 lanes share a key (16 elements each, two 16-byte loads into registers), 32 keys per
//           pass, 5 passes; dot products with the rows' queries in float32, summed over the 8 lanes
//           by shuffles; scores (scaled to base 2, masked) go to shared memory;
//   values  the chunk's values are copied to shared memory with cp.async (one buffer ahead), issued
//           together with the keys' loads;
//   softmax a warp per row: running max and sum, P in shared memory (float32: P is not rounded to
//           bfloat16 here, which is closer to the exact result than attn.py:263);
//   P·V     a warp takes every 8th key, a lane 4 elements of the head; float32 accumulators, rescaled
//           when the max moves; the 8 warps' sums meet in shared memory at the end.
// The loads of chunk c + 1 are issued before the softmax of chunk c.
//
// Work items, parts and the merge by the CTA that finishes a request's last part are those of the
// mma.sync kernel (attention_flash.cuh): same item layout, same scratch layout, same counters.
//
// CL: every request is cut into the same number of parts (2, 4 or 8) and the parts of a request are
// the CTAs of one thread-block cluster.  Then the parts never leave the chip: each CTA keeps its
// accumulator, max and sum in its shared memory, the cluster meets at a barrier, and its first CTA
// combines the parts through distributed shared memory (same formula, same order) and writes the
// output; no scratch memory, no counters, no round trips to L2 at the end of the kernel.
//
// FUSE: the kernel takes q, k and v as the QKV product left them and does what the rotary kernel
// would have done in between (elementwise.cu, rope_d128.cuh: per-head RMS norm of q and k, rotation
// of both by position x inverse frequency, the new keys and values into the cache), with the same
// arithmetic and the same rounding of q and k to bfloat16: a launch less per layer in a decode step.
// Every CTA norms and rotates its rows' queries; the CTA whose keys include a new token's position
// norms and rotates that token's key, writes it and the value into the cache, and uses its own copy.
#include "attention_flash.cuh"
#include <stddef.h>

#define AD_THREADS 256
#define AD_CH 160               // keys per chunk: 5 passes of 32
#define AD_PASSES (AD_CH / 32)
#define AD_D 128
#define AD_PART_ALIGN 16        // a request's parts are multiples of this many keys

struct AdFuse {
  const __nv_bfloat16* k; const __nv_bfloat16* v;   // the step's keys and values [T, Hkv, 128], strides as q's
  const float* qw; const float* kw; float eps;      // norm weights (null: no norm)
  const float* inv_freq;                            // [64]
  __nv_bfloat16* pages_out;                         // the cache, to be written (null: this layer reads another's)
};

template <int R>
struct AdSmem {
  // (members that are read or written 8 or 16 bytes at a time are aligned for it whatever R is)
  alignas(16) __nv_bfloat16 v[2][AD_CH * AD_D];     // 40 KB each
  float sc[R][AD_CH];                   // scores, then P
  alignas(16) float red[8][R][AD_D];    // the warps' accumulators at the end
  float m_run[R], l_run[R], alpha[R];
  int tab[2][AD_CH + 2];                // pages of a chunk's keys (one entry per page the chunk touches)
  int last;
  float fin[R][AD_D];                   // CL: this part's accumulator, for the cluster's first CTA
  alignas(16) float2 cs[R][64];         // FUSE: (cos, sin) of the rows' tokens' angles
  alignas(16) __nv_bfloat16 knew[R][AD_D];   // FUSE: the new tokens' keys after norm and rotation
};

__device__ __forceinline__ float2 ad_bf2(uint32_t u) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u));
}

// R: rows (query token x head of the group) a CTA holds at most: 1, 2 or 4
// x: 16 consecutive elements (from 16 sub on) of a head's 128, held by 8 lanes; norm over the head,
// rotation of the pairs (d, d + 64) by the angles in cs, the result rounded to bfloat16 as the
// rotary kernel rounds it
__device__ __forceinline__ void ad_norm_rotate(float (&x)[16], const float* w, float eps, const float2* cs, int sub) {
  if (w) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) ss += x[i] * x[i];
    ss += __shfl_xor_sync(0xffffffffu, ss, 4);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    const float rstd = rsqrtf(ss / (float)AD_D + eps);
#pragma unroll
    for (int i = 0; i < 16; ++i) x[i] = x[i] * rstd * w[sub * 16 + i];
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float partner = __shfl_xor_sync(0xffffffffu, x[i], 4);      // element d +- 64
    const float2 c = cs[(sub & 3) * 16 + i];
    x[i] = sub < 4 ? c.x * x[i] - c.y * partner : c.y * partner + c.x * x[i];
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) x[i] = __bfloat162float(__float2bfloat16_rn(x[i]));
}

template <int R, bool FUSE, bool CL>
__global__ void __launch_bounds__(AD_THREADS, 2)
decode_attention_kernel(FaArgs A, AdFuse F) {
  static_assert(offsetof(AdSmem<R>, knew) % 16 == 0 && offsetof(AdSmem<R>, red) % 16 == 0 && offsetof(AdSmem<R>, cs) % 8 == 0,
                "vector accesses to shared memory need their alignment");
  extern __shared__ __align__(16) unsigned char smem_raw[];
  AdSmem<R>& sm = *reinterpret_cast<AdSmem<R>*>(smem_raw);
  constexpr int D = AD_D;
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hkv = blockIdx.y;
  const int Hq = A.Hq, Hkv = A.Hkv, window = A.window, page_size = A.page_size;
  const int G = Hq / Hkv;

  // the work lists come from the host's copy, not from a kernel
  const int* it = A.items + (size_t)blockIdx.x * FA_ITEM_INTS;
  const int req = it[0], q0 = it[1], part = it[4], n_splits = it[5], split = it[6];
  int kv_lo = it[2], kv_hi_item = it[3];
  const int row0 = it[7], q_len = it[8], ctx = it[9];
  const int ntok = min(FA_BM / G, q_len - q0);
  const int nrows = min(ntok * G, R);               // the launcher promised nrows <= R
  const int first_pos = ctx + q0;
  if (n_splits > 0) {
    const int total = ctx + q_len;
    const int lo = window > 0 ? max(0, ctx - window + 1) / FA_BN * FA_BN : 0;
    // (parts of equal length up to 16 keys: this kernel has no key tiles that a part should be a multiple of)
    const int per = ((total - lo + n_splits - 1) / n_splits + AD_PART_ALIGN - 1) / AD_PART_ALIGN * AD_PART_ALIGN;
    kv_lo = lo + split * per;
    kv_hi_item = min(total, kv_lo + per);
  }
  const int kv_end = min(kv_hi_item, first_pos + ntok);
  int kv_begin = max(kv_lo, 0);
  if (window > 0) kv_begin = max(kv_begin, first_pos - window + 1);
  const int n_chunks = kv_end > kv_begin ? (kv_end - kv_begin + AD_CH - 1) / AD_CH : 0;
  // FUSE: this CTA's keys include the new tokens' positions (they lie together at the end of the
  // request; a tile whose tokens straddle two parts is not launched with FUSE: every item holds one token)
  const bool own_new = FUSE && F.pages_out != nullptr && kv_begin <= first_pos && kv_end >= first_pos + ntok;

  const int* table = A.block_tables + (size_t)req * A.max_blocks;
  const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;
  const size_t page_stride = (size_t)2 * Hkv * page_size * D;
  const size_t v_off = (size_t)Hkv * page_size * D;
  const __nv_bfloat16* head_base = A.pages + (size_t)hkv * page_size * D;

  // pages of chunk c's keys into tab[c & 1]: entry e is the page of block (first block of the chunk) + e
  auto load_table = [&](int c) {
    const int k0 = kv_begin + c * AD_CH;
    const int b0 = page_shift >= 0 ? k0 >> page_shift : k0 / page_size;
    const int k1 = min(k0 + AD_CH, kv_end) - 1;
    const int b1 = page_shift >= 0 ? k1 >> page_shift : k1 / page_size;
    for (int e = tid; e <= b1 - b0; e += AD_THREADS) sm.tab[c & 1][e] = table[b0 + e];
  };
  // address of key j's row of this head in the cache (K; + v_off for V)
  auto row_of = [&](int c, int j) -> const __nv_bfloat16* {
    const int k0 = kv_begin + c * AD_CH;
    int blk, off, b0;
    if (page_shift >= 0) { blk = j >> page_shift; off = j & (page_size - 1); b0 = k0 >> page_shift; }
    else { blk = j / page_size; off = j - blk * page_size; b0 = k0 / page_size; }
    return head_base + (size_t)sm.tab[c & 1][blk - b0] * page_stride + (size_t)off * D;
  };

  // ---- per-thread roles --------------------------------------------------------------------------
  const int gi = tid >> 3, sub = tid & 7;           // keys: 8 lanes per key, 16 elements each
  uint4 kreg[AD_PASSES][2];
  auto issue_keys = [&](int c) {
    const int k0 = kv_begin + c * AD_CH;
#pragma unroll
    for (int p = 0; p < AD_PASSES; ++p) {
      const int j = k0 + p * 32 + gi;
      if (j < kv_end) {
        const uint4* src = reinterpret_cast<const uint4*>(row_of(c, j) + sub * 16);
        kreg[p][0] = __ldcg(src);
        kreg[p][1] = __ldcg(src + 1);
      } else {
        kreg[p][0] = kreg[p][1] = make_uint4(0, 0, 0, 0);
      }
    }
  };
  auto issue_values = [&](int c) {
    const int k0 = kv_begin + c * AD_CH;
    __nv_bfloat16* dst = sm.v[c & 1];
    const int ch = tid & (D / 8 - 1);                // this thread's 16-byte piece of a row; 16 rows per turn
#pragma unroll
    for (int kc = tid / (D / 8); kc < AD_CH; kc += AD_THREADS / (D / 8)) {
      const int j = k0 + kc;
      if (FUSE && own_new && j >= first_pos && j < kv_end)
        cp_async16(dst + kc * D + ch * 8, F.v + (size_t)(row0 + q0 + (j - first_pos)) * A.q_stride + (size_t)hkv * D + ch * 8);
      else if (j < kv_end) cp_async16(dst + kc * D + ch * 8, row_of(c, j) + v_off + ch * 8);
      else *reinterpret_cast<uint4*>(dst + kc * D + ch * 8) = make_uint4(0, 0, 0, 0);
    }
    cp_async_commit();
  };

  if (n_chunks > 0) load_table(0);
  if (tid < R) { sm.m_run[tid] = -INFINITY; sm.l_run[tid] = 0.f; sm.alpha[tid] = 1.f; }
  if (tid == 0) sm.last = 0;
  pdl_wait();                                       // q and the new token's key and value: the previous kernels' outputs
  __syncthreads();
  // the first chunk's keys and values are on their way before anything else is done
  if (n_chunks > 0) { issue_values(0); issue_keys(0); }

  if constexpr (FUSE) {
    // the angles of the tile's tokens, one (cos, sin) per thread
    for (int e = tid; e < ntok * 64; e += AD_THREADS) {
      const int t = e >> 6, jf = e & 63;
      float sn, cs;
      sincosf((float)(first_pos + t) * F.inv_freq[jf], &sn, &cs);
      sm.cs[t][jf] = make_float2(cs, sn);
    }
    __syncthreads();
    // the new tokens' keys and values: group t of 8 lanes takes token t (whole warps take part in the
    // shuffles: a group without a token works on the last token and writes nothing)
    if (own_new && warp * 4 < ntok) {
      const bool mine = gi < ntok;
      const int tk = mine ? gi : ntok - 1;
      const size_t tok = (size_t)(row0 + q0 + tk) * A.q_stride + (size_t)hkv * D + sub * 16;
      const uint4 ka = __ldcg(reinterpret_cast<const uint4*>(F.k + tok)), kb = __ldcg(reinterpret_cast<const uint4*>(F.k + tok) + 1);
      const uint32_t kraw[8] = {ka.x, ka.y, ka.z, ka.w, kb.x, kb.y, kb.z, kb.w};
      float x[16];
#pragma unroll
      for (int i = 0; i < 8; ++i) { const float2 f2 = ad_bf2(kraw[i]); x[2 * i] = f2.x; x[2 * i + 1] = f2.y; }
      ad_norm_rotate(x, F.kw, F.eps, sm.cs[tk], sub);
      if (mine) {
        uint32_t kout[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) kout[i] = pack_bf16(x[2 * i], x[2 * i + 1]);
        const uint4 o0 = make_uint4(kout[0], kout[1], kout[2], kout[3]), o1 = make_uint4(kout[4], kout[5], kout[6], kout[7]);
        *reinterpret_cast<uint4*>(&sm.knew[tk][sub * 16]) = o0;
        *(reinterpret_cast<uint4*>(&sm.knew[tk][sub * 16]) + 1) = o1;
        // into the cache, for the steps to come: page of the position from the block table
        const int pos = first_pos + tk;
        const int blk = page_shift >= 0 ? pos >> page_shift : pos / page_size;
        const int off = pos - blk * page_size;
        __nv_bfloat16* row = F.pages_out + (size_t)table[blk] * page_stride + (size_t)hkv * page_size * D + (size_t)off * D + sub * 16;
        *reinterpret_cast<uint4*>(row) = o0;
        *(reinterpret_cast<uint4*>(row) + 1) = o1;
        const uint4* vsrc = reinterpret_cast<const uint4*>(F.v + tok);
        *reinterpret_cast<uint4*>(row + v_off) = __ldcg(vsrc);
        *(reinterpret_cast<uint4*>(row + v_off) + 1) = __ldcg(vsrc + 1);
      }
    }
    __syncthreads();
  }
  // this thread's 16 elements of every row's query: in float32 for up to 2 rows (converted once),
  // else as packed bfloat16 (converted at every use: registers are the tighter resource then)
  constexpr bool QF32 = R <= 2;
  float2 qf[QF32 ? R : 1][8];
  uint32_t qreg[QF32 ? 1 : R][8];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    uint32_t w8[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
    if (r < nrows) {
      const int ti = r / G, hg = r - ti * G;
      const uint4* src = reinterpret_cast<const uint4*>(A.q + (size_t)(row0 + q0 + ti) * A.q_stride +
                                                        (size_t)(hkv * G + hg) * D + sub * 16);
      const uint4 a = __ldcg(src), b = __ldcg(src + 1);
      w8[0] = a.x; w8[1] = a.y; w8[2] = a.z; w8[3] = a.w; w8[4] = b.x; w8[5] = b.y; w8[6] = b.z; w8[7] = b.w;
      if constexpr (FUSE) {
        float x[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) { const float2 f2 = ad_bf2(w8[i]); x[2 * i] = f2.x; x[2 * i + 1] = f2.y; }
        ad_norm_rotate(x, F.qw, F.eps, sm.cs[ti], sub);
#pragma unroll
        for (int i = 0; i < 8; ++i) w8[i] = pack_bf16(x[2 * i], x[2 * i + 1]);
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if constexpr (QF32) qf[r][i] = ad_bf2(w8[i]); else qreg[r][i] = w8[i];
    }
  }

  float o[R][4];                                    // P·V: this warp's keys, this lane's 4 elements
#pragma unroll
  for (int r = 0; r < R; ++r) { o[r][0] = o[r][1] = o[r][2] = o[r][3] = 0.f; }

  for (int c = 0; c < n_chunks; ++c) {
    const int k0 = kv_begin + c * AD_CH;
    const int clen = min(AD_CH, kv_end - k0);
    if (c + 1 < n_chunks) load_table(c + 1);        // needed after the next barrier
    // ---- scores of the chunk ---------------------------------------------------------------------
#pragma unroll
    for (int p = 0; p < AD_PASSES; ++p) {
      uint32_t kw[8] = {kreg[p][0].x, kreg[p][0].y, kreg[p][0].z, kreg[p][0].w,
                        kreg[p][1].x, kreg[p][1].y, kreg[p][1].z, kreg[p][1].w};
      if constexpr (FUSE) {
        // a new token's key: this CTA's own copy (its write to the cache may not be visible yet)
        const int j = k0 + p * 32 + gi;
        if (own_new && j >= first_pos && j < kv_end) {
          const uint4* src = reinterpret_cast<const uint4*>(&sm.knew[j - first_pos][sub * 16]);
          const uint4 a = src[0], b = src[1];
          kw[0] = a.x; kw[1] = a.y; kw[2] = a.z; kw[3] = a.w; kw[4] = b.x; kw[5] = b.y; kw[6] = b.z; kw[7] = b.w;
        }
      }
      float dot[R];
#pragma unroll
      for (int r = 0; r < R; ++r) dot[r] = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 kf = ad_bf2(kw[i]);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          float2 q2;
          if constexpr (QF32) q2 = qf[r][i]; else q2 = ad_bf2(qreg[r][i]);
          dot[r] = fmaf(q2.x, kf.x, dot[r]);
          dot[r] = fmaf(q2.y, kf.y, dot[r]);
        }
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        dot[r] += __shfl_xor_sync(0xffffffffu, dot[r], 4);
        dot[r] += __shfl_xor_sync(0xffffffffu, dot[r], 2);
        dot[r] += __shfl_xor_sync(0xffffffffu, dot[r], 1);
      }
      if (sub == 0) {
        const int kc = p * 32 + gi, j = k0 + kc;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int pos = first_pos + r / G;
          const bool ok = r < nrows && j < kv_end && j <= pos && (window <= 0 || j > pos - window);
          sm.sc[r][kc] = ok ? dot[r] * A.scale_log2 : -INFINITY;
        }
      }
    }
    __syncthreads();                                // scores written; the next chunk's pages known
    if (c + 1 < n_chunks) { issue_values(c + 1); issue_keys(c + 1); }
    // ---- softmax: a warp per row --------------------------------------------------------------------
    for (int r = warp; r < R; r += AD_THREADS / 32) {
      float s[AD_PASSES];
      float mx = -INFINITY;
#pragma unroll
      for (int p = 0; p < AD_PASSES; ++p) { s[p] = sm.sc[r][p * 32 + lane]; mx = fmaxf(mx, s[p]); }
      mx = warp_max(mx);
      const float m_old = sm.m_run[r];
      const float m_new = fmaxf(m_old, mx);
      const float base = m_new == -INFINITY ? 0.f : m_new;
      float sum = 0.f;
#pragma unroll
      for (int p = 0; p < AD_PASSES; ++p) {
        const float pv = exp2f(s[p] - base);
        sm.sc[r][p * 32 + lane] = pv;
        sum += pv;
      }
      sum = warp_sum(sum);
      if (lane == 0) {
        const float al = exp2f(m_old - base);       // 0 when nothing was allowed before
        sm.alpha[r] = al;
        sm.l_run[r] = sm.l_run[r] * al + sum;
        sm.m_run[r] = m_new;
      }
    }
    if (c + 1 < n_chunks) cp_async_wait<1>(); else cp_async_wait<0>();   // this chunk's values have landed
    __syncthreads();                                // P, alpha and everybody's copies are visible
    // ---- P·V ----------------------------------------------------------------------------------------------
    {
      float al[R];
#pragma unroll
      for (int r = 0; r < R; ++r) { al[r] = sm.alpha[r]; o[r][0] *= al[r]; o[r][1] *= al[r]; o[r][2] *= al[r]; o[r][3] *= al[r]; }
      const __nv_bfloat16* vb = sm.v[c & 1];
      for (int kc = warp; kc < clen; kc += AD_THREADS / 32) {
        const uint2 raw = *reinterpret_cast<const uint2*>(vb + kc * D + 4 * lane);
        const float2 v01 = ad_bf2(raw.x), v23 = ad_bf2(raw.y);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const float pv = sm.sc[r][kc];
          o[r][0] = fmaf(pv, v01.x, o[r][0]); o[r][1] = fmaf(pv, v01.y, o[r][1]);
          o[r][2] = fmaf(pv, v23.x, o[r][2]); o[r][3] = fmaf(pv, v23.y, o[r][3]);
        }
      }
    }
    __syncthreads();                                // the scores' and this value buffer's readers are done
  }

  // ---- the 8 warps' sums meet --------------------------------------------------------------------------
#pragma unroll
  for (int r = 0; r < R; ++r)
    *reinterpret_cast<float4*>(&sm.red[warp][r][4 * lane]) = make_float4(o[r][0], o[r][1], o[r][2], o[r][3]);
  __syncthreads();
  __nv_bfloat16* out_row0 = A.out + (size_t)(row0 + q0) * ((size_t)Hq * D);
  for (int e = tid; e < nrows * D; e += AD_THREADS) {
    const int r = e / D, d = e - r * D;
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < AD_THREADS / 32; ++w) acc += sm.red[w][r][d];
    const float l = sm.l_run[r];
    if constexpr (CL) {
      sm.fin[r][d] = acc;
    } else if (part < 0) {
      const int ti = r / G, hg = r - ti * G;
      out_row0[(size_t)ti * ((size_t)Hq * D) + (size_t)(hkv * G + hg) * D + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    } else {
      const size_t slot = ((size_t)part * Hkv + hkv) * A.part_rows + r;
      A.part_acc[slot * D + d] = acc;
      if (d == 0) { A.part_ml[2 * slot] = sm.m_run[r]; A.part_ml[2 * slot + 1] = l; }
    }
  }
  if constexpr (CL) {
    // ---- the parts meet in the cluster's first CTA -------------------------------------------------------
    cluster_sync_all();                             // every part's accumulator, max and sum are in place
    if (cluster_cta_rank() == 0) {
      const int S = (int)cluster_num_ctas();        // = n_splits, at most 8
      for (int e = tid; e < nrows * D; e += AD_THREADS) {
        const int r = e / D, d = e - r * D;
        float mm[8], ll[8], aa[8];
#pragma unroll
        for (int sp = 0; sp < 8; ++sp) {
          mm[sp] = -INFINITY; ll[sp] = 0.f; aa[sp] = 0.f;
          if (sp < S) {
            mm[sp] = cluster_ld_f32(cluster_map_shared(&sm.m_run[r], (uint32_t)sp));
            ll[sp] = cluster_ld_f32(cluster_map_shared(&sm.l_run[r], (uint32_t)sp));
            aa[sp] = cluster_ld_f32(cluster_map_shared(&sm.fin[r][d], (uint32_t)sp));
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
      sm.last = (done == n_splits - 1);
      if (sm.last) A.counters[first * Hkv + hkv] = 0;        // ready for the next launch
    }
    __syncthreads();
    if (sm.last) {
      __threadfence();
      // out = sum_s 2^(m_s - m) acc_s / sum_s 2^(m_s - m) l_s, in float32, in the order of the parts
      for (int e = tid; e < nrows * D; e += AD_THREADS) {
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

template <int R, bool FUSE, bool CL>
static int launch_decode_as(const FaArgs& fa, const AdFuse& fu, int n_items, int Hkv, int cluster, cudaStream_t stream) {
  const size_t smem = sizeof(AdSmem<R>);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(decode_attention_kernel<R, FUSE, CL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) QE_REFUSE("decode_attention: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  if (CL)
    qe_launch_cluster(decode_attention_kernel<R, FUSE, CL>, dim3(n_items, Hkv), dim3(AD_THREADS), smem, stream, (unsigned)cluster, fa, fu);
  else
    qe_launch(decode_attention_kernel<R, FUSE, CL>, dim3(n_items, Hkv), dim3(AD_THREADS), smem, stream, fa, fu);
  QE_CHECK_LAUNCH("decode_attention");
  return 0;
}

// cluster: 0, or the number of parts of every request (2, 4 or 8) when the items are exactly those
// parts, request by request in the order of the parts: then the parts of a request form a cluster
template <int R, bool FUSE>
static int launch_decode(const FaArgs& fa, const AdFuse& fu, int n_items, int Hkv, int cluster, cudaStream_t stream) {
  if (cluster == 0) return launch_decode_as<R, FUSE, false>(fa, fu, n_items, Hkv, 0, stream);
  if ((cluster != 2 && cluster != 4 && cluster != 8) || n_items % cluster)
    QE_REFUSE("decode_attention: %d items cannot form clusters of %d", n_items, cluster);
  return launch_decode_as<R, FUSE, true>(fa, fu, n_items, Hkv, cluster, stream);
}

// Whether the kernel takes this geometry with at most max_rows rows (token x head of the group) per item.
extern "C" int qe_decode_attention_supported(int Hq, int Hkv, int D, int max_rows) {
  return (D == AD_D && Hkv >= 1 && Hkv <= 65535 && Hq % Hkv == 0 && max_rows >= 1 && max_rows <= 4) ? 1 : 0;
}

// Same arguments as qe_flash_attention_fused_merge's (attention_flash.cu) where they share a name;
// every item has at most max_rows rows; parts are combined by the CTA that finishes last (counters
// as there), or inside clusters (`cluster`, see launch_decode; scratch and counters are then unused).
// Returns 0 when run, 1 when refused, 2 on a launch error.
extern "C" int qe_decode_attention(const void* q, long q_stride, const void* pages, const int* block_tables,
                                   int max_blocks, const int* items, int n_items, void* out, float* part_acc,
                                   float* part_ml, int part_rows, int* counters, int max_rows, int cluster, float scale,
                                   int window, int Hq, int Hkv, int D, int page_size, cudaStream_t stream) {
  if (n_items <= 0) return 0;
  if (!qe_decode_attention_supported(Hq, Hkv, D, max_rows))
    QE_REFUSE("decode_attention: heads %d/%d, head_dim %d, %d rows are not supported", Hq, Hkv, D, max_rows);
  if ((((uintptr_t)q | (uintptr_t)pages) & 15) || (q_stride % 8)) QE_REFUSE("decode_attention: operands must be 16-byte aligned");
  if (part_acc && counters == nullptr && !cluster) QE_REFUSE("decode_attention: parts need the counters");
  FaArgs fa{(const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)pages, block_tables, max_blocks, items,
            (__nv_bfloat16*)out, part_acc, part_ml, part_rows, counters, scale * 1.4426950408889634f, window, Hq, Hkv,
            page_size};
  const AdFuse none{};
  if (max_rows <= 1) return launch_decode<1, false>(fa, none, n_items, Hkv, cluster, stream);
  if (max_rows <= 2) return launch_decode<2, false>(fa, none, n_items, Hkv, cluster, stream);
  return launch_decode<4, false>(fa, none, n_items, Hkv, cluster, stream);
}

// The same with the per-head norm, the rotation and the cache write of the step's q, k, v done here
// (see FUSE above).  qkv: the QKV product's output [T, (Hq + 2 Hkv) 128] as it left the product; qw, kw:
// norm weights [128] or null; inv_freq [64]; write_kv 0: a layer that reads another layer's cache (its
// keys are there already; only the queries are normed and rotated).  Every item must hold one token.
extern "C" int qe_decode_attention_fused(const void* qkv, long q_stride, void* pages, const int* block_tables,
                                         int max_blocks, const int* items, int n_items, void* out, float* part_acc,
                                         float* part_ml, int part_rows, int* counters, int max_rows, int cluster, float scale,
                                         int window, const float* qw, const float* kw, float eps, const float* inv_freq,
                                         int write_kv, int Hq, int Hkv, int D, int page_size, cudaStream_t stream) {
  if (n_items <= 0) return 0;
  if (!qe_decode_attention_supported(Hq, Hkv, D, max_rows) || max_rows > Hq / Hkv)
    QE_REFUSE("decode_attention_fused: heads %d/%d, head_dim %d, %d rows are not supported", Hq, Hkv, D, max_rows);
  if ((((uintptr_t)qkv | (uintptr_t)pages | (uintptr_t)qw | (uintptr_t)kw) & 15) || (q_stride % 8))
    QE_REFUSE("decode_attention_fused: operands must be 16-byte aligned");
  if (part_acc && counters == nullptr && !cluster) QE_REFUSE("decode_attention_fused: parts need the counters");
  if (!inv_freq) QE_REFUSE("decode_attention_fused: needs the inverse frequencies");
  const __nv_bfloat16* q = (const __nv_bfloat16*)qkv;
  FaArgs fa{q, q_stride, (const __nv_bfloat16*)pages, block_tables, max_blocks, items,
            (__nv_bfloat16*)out, part_acc, part_ml, part_rows, counters, scale * 1.4426950408889634f, window, Hq, Hkv,
            page_size};
  AdFuse fu{q + (size_t)Hq * D, q + (size_t)(Hq + Hkv) * D, qw, kw, eps, inv_freq, write_kv ? (__nv_bfloat16*)pages : nullptr};
  if (max_rows <= 1) return launch_decode<1, true>(fa, fu, n_items, Hkv, cluster, stream);
  if (max_rows <= 2) return launch_decode<2, true>(fa, fu, n_items, Hkv, cluster, stream);
  return launch_decode<4, true>(fa, fu, n_items, Hkv, cluster, stream);
}
