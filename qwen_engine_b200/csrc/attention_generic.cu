// Attention of a step's new queries over the paged cache, for any mixture of prompt portions
// and single decoded tokens, any head size up to 512, any page size, any number of heads and
// groups, float32 or bfloat16 storage; all arithmetic in float32 with expf.
//
// For the query at position i of a request, key j is allowed iff j <= i and (window == 0 or
// j > i - window) (reference src/layers/fused_ops/attn.py:195, 239); scores are scale * q·k,
// softmax runs online over key tiles of 32 that start at multiples of 32 of the absolute key
// position, so the order of a query's reduction does not depend on how the request was cut into
// steps (attn.py:236-267 has the same algebra per BLOCK_N).  Query head h reads kv head
// h / (Hq / Hkv) (attn.py:181-182).
//
// One CTA per (tile of 16 queries of one request, query head); 4 warps, 4 queries each.  Within a
// warp lane j owns key j of the tile for the scores and dims d = lane + 32 i of the output.
#include "common.cuh"
#include <math.h>

#define AG_BM 16
#define AG_BN 32
#define AG_WARPS 4
#define AG_MAX_D 512

template <typename T>
__global__ void __launch_bounds__(AG_WARPS * 32)
attention_generic_kernel(const T* __restrict__ q, long q_stride, const T* __restrict__ pages,
                         const int* __restrict__ block_tables, int max_blocks,
                         const int* __restrict__ cu_q, const int* __restrict__ ctx_lens,
                         const int* __restrict__ tiles, T* __restrict__ out, float scale, int window,
                         int Hq, int Hkv, int D, int page_size) {
  extern __shared__ float smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int Dp = D + 1;
  float* qs = smem;                           // [AG_BM][D]
  float* ks = qs + AG_BM * D;                 // [AG_BN][D + 1]
  float* vs = ks + AG_BN * Dp;                // [AG_BN][D]
  const int tile = blockIdx.x, hq = blockIdx.y;
  const int hkv = hq / (Hq / Hkv);
  const int req = tiles[2 * tile], q0 = tiles[2 * tile + 1];
  const int row0 = cu_q[req];
  const int q_len = cu_q[req + 1] - row0;
  const int ctx = ctx_lens[req];
  const int nq = min(AG_BM, q_len - q0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int* table = block_tables + (size_t)req * max_blocks;

  for (int e = threadIdx.x; e < AG_BM * D; e += blockDim.x) {
    const int r = e / D, d = e - r * D;
    qs[e] = r < nq ? to_f32(q[(size_t)(row0 + q0 + r) * q_stride + (size_t)hq * D + d]) : 0.f;
  }

  constexpr int QPW = AG_BM / AG_WARPS;       // queries per warp
  constexpr int DREG = AG_MAX_D / 32;
  float m[QPW], l[QPW];
  float acc[QPW][DREG];
#pragma unroll
  for (int i = 0; i < QPW; ++i) {
    m[i] = -INFINITY; l[i] = 0.f;
#pragma unroll
    for (int c = 0; c < DREG; ++c) acc[i][c] = 0.f;
  }
  const int dregs = (D + 31) / 32;

  const int first_pos = ctx + q0;                       // position of the tile's first query
  const int kv_end = ctx + q0 + nq;                     // one past the last allowed key
  const int kv_begin = window > 0 ? max(0, first_pos - window + 1) : 0;
  for (int kt = (kv_begin / AG_BN) * AG_BN; kt < kv_end; kt += AG_BN) {
    __syncthreads();
    for (int e = threadIdx.x; e < AG_BN * D; e += blockDim.x) {
      const int j = e / D, d = e - j * D;
      const int kj = kt + j;
      float kvl = 0.f, vvl = 0.f;
      if (kj >= kv_begin && kj < kv_end) {
        const int page = table[kj / page_size];
        const size_t base = ((((size_t)page * 2) * Hkv + hkv) * page_size + (kj % page_size)) * D + d;
        kvl = to_f32(pages[base]);
        vvl = to_f32(pages[base + (size_t)Hkv * page_size * D]);
      }
      ks[j * Dp + d] = kvl;
      vs[j * D + d] = vvl;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < QPW; ++i) {
      const int r = warp * QPW + i;
      if (r >= nq) continue;                            // uniform within the warp
      const int pos = first_pos + r;
      const int kj = kt + lane;
      const bool ok = kj <= pos && (window <= 0 || kj > pos - window);
      float s = 0.f;
      const float* qr = qs + r * D;
      const float* kr = ks + lane * Dp;
      for (int d = 0; d < D; ++d) s = fmaf(qr[d], kr[d], s);
      s = ok ? s * scale : -INFINITY;
      const float tile_max = warp_max(s);
      if (tile_max == -INFINITY) continue;              // nothing allowed in this tile
      const float m_new = fmaxf(m[i], tile_max);
      const float alpha = expf(m[i] - m_new);           // exp(-inf) = 0 on the first tile
      const float p = ok ? expf(s - m_new) : 0.f;
      l[i] = l[i] * alpha + warp_sum(p);
      m[i] = m_new;
#pragma unroll
      for (int c = 0; c < DREG; ++c) if (c < dregs) acc[i][c] *= alpha;
      for (int j = 0; j < AG_BN; ++j) {
        const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
        for (int c = 0; c < DREG; ++c) {
          const int d = lane + 32 * c;
          if (c < dregs && d < D) acc[i][c] = fmaf(pj, vs[j * D + d], acc[i][c]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < QPW; ++i) {
    const int r = warp * QPW + i;
    if (r >= nq) continue;
    const float inv = 1.f / l[i];
    T* o = out + (size_t)(row0 + q0 + r) * ((size_t)Hq * D) + (size_t)hq * D;
#pragma unroll
    for (int c = 0; c < DREG; ++c) {
      const int d = lane + 32 * c;
      if (c < dregs && d < D) o[d] = from_f32<T>(acc[i][c] * inv);
    }
  }
}

extern "C" int qe_paged_attention_generic(const void* q, long q_stride, const void* pages,
                                          const int* block_tables, int max_blocks, const int* cu_q,
                                          const int* ctx_lens, const int* tiles, int n_tiles, void* out,
                                          float scale, int window, int Hq, int Hkv, int D, int page_size,
                                          int dtype, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (D > AG_MAX_D || D < 1) QE_REFUSE("paged_attention: head_dim %d is outside 1..%d", D, AG_MAX_D);
  if (Hkv < 1 || Hq % Hkv) QE_REFUSE("paged_attention: %d query heads do not group over %d kv heads", Hq, Hkv);
  if (Hq > 65535) QE_REFUSE("paged_attention: too many heads (%d)", Hq);
  const size_t smem = ((size_t)AG_BM * D + (size_t)AG_BN * (D + 1) + (size_t)AG_BN * D) * sizeof(float);
  dim3 grid(n_tiles, Hq);
  // the largest head size sets the limit once (not per launch: launches may be under stream capture)
  static bool configured = false;
  if (!configured) {
    const int max_smem = (int)(((size_t)AG_BM * AG_MAX_D + (size_t)AG_BN * (AG_MAX_D + 1) + (size_t)AG_BN * AG_MAX_D) * sizeof(float));
    cudaError_t e = cudaFuncSetAttribute(attention_generic_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attention_generic_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
    if (e != cudaSuccess) QE_REFUSE("paged_attention: shared memory %d: %s", max_smem, cudaGetErrorString(e));
    configured = true;
  }
  if (dtype == QE_DTYPE_F32) {
    qe_launch(attention_generic_kernel<float>, grid, dim3(AG_WARPS * 32), smem, stream,
        (const float*)q, q_stride, (const float*)pages, block_tables, max_blocks, cu_q, ctx_lens, tiles,
        (float*)out, scale, window, Hq, Hkv, D, page_size);
  } else if (dtype == QE_DTYPE_BF16) {
    qe_launch(attention_generic_kernel<__nv_bfloat16>, grid, dim3(AG_WARPS * 32), smem, stream,
        (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)pages, block_tables, max_blocks, cu_q, ctx_lens,
        tiles, (__nv_bfloat16*)out, scale, window, Hq, Hkv, D, page_size);
  } else QE_REFUSE("paged_attention: unknown dtype %d", dtype);
  QE_CHECK_LAUNCH("paged_attention_generic");
  return 0;
}
