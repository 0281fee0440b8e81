// Device functions of the product for a few rows (see gemm_small_m.cu), as a header so that the kernels of that
// file (a CTA per 16 weight rows, clusters that share K, the fused epilogues) are built from the same pieces.
#pragma once
#include "common.cuh"

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream16(const void* p) {   // read once: do not keep in L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// silu(g) * u for a pair of bfloat16 values, in float32, rounded once (the reference's silumul,
// src/layers/fused_ops/silumul.py:50-53, without its intermediate rounding of silu).  The result has
// 8 bits of mantissa, so the fast exponential and division (errors of a few float32 ulps) are used:
// every CTA forms the whole activation again, and the exact routines would cost more than the product.
__device__ __forceinline__ float silu_fast(float g) { return __fdividef(g, 1.f + __expf(-g)); }
__device__ __forceinline__ uint32_t silu_mul_pair(uint32_t g, uint32_t u) {
  const float2 gf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&g));
  const float2 uf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u));
  __nv_bfloat162 r = __floats2bfloat162_rn(silu_fast(gf.x) * uf.x, silu_fast(gf.y) * uf.y);
  return *reinterpret_cast<uint32_t*>(&r);
}

// What the token operand is made of (formed while loading, so that no kernel and no buffer stands
// between the producer of the data and the product):
//   PLAIN  x[M, K] as it is;
//   SILU   x[m, k] = silu(gate_up[m, k]) * gate_up[m, K + k] from gate_up[M, 2K] (the feed-forward's
//          activation fused into its output projection);
//   NORM   x[m, k] = resid[m, k] * rstd[m] * norm_w[k] with rstd[m] = rsqrt(sum_k resid[m, k]^2 / K + eps):
//          the RMS norm of the float32 residual stream fused into the projection that follows it.  The
//          row's sum of squares comes in n_ssq partial sums that the kernel that last wrote the stream
//          left behind (see RESID), so no pass over the row is needed here.
// And what happens to the result:
//   RESID  the product is a branch's output: it is added into the float32 residual stream in place
//          (each element belongs to one thread), and the CTA leaves the sum of squares of its 16
//          columns of every row in ssq_out[m, blockIdx.x] for the norm that follows.
enum { X_PLAIN = 0, X_SILU = 1, X_NORM = 2 };

struct FuseArgs {
  const float* resid;               // NORM: [M, K] float32
  const float* ssq;                 // NORM: [M, ssq_ld] partial sums of squares of the rows
  const float* norm_w;              // NORM: [K]
  float* ssq_out;                   // RESID: [M, ssq_ld]
  int n_ssq, ssq_ld;
  float eps;
  // Weights that a later kernel of the step will read (nobody writes them): the CTAs ask L2 for them,
  // a slice each, once their own weights are on their way.  A decode step is a chain of short kernels,
  // and a kernel that starts on weights that are already on the chip is done sooner.
  const unsigned char* next_w;
  unsigned long long next_bytes;
};

// a chunk of weights: 64 k of 16 rows = four 16-byte loads per lane (a: row g, b: row g + 8); where a CTA has 8
// rows (ROWS = 8), 128 k of 8 rows (a: k .. k + 63, b: k + 64 .. k + 127 of row g)
struct GsmChunk { uint4 a0, b0, a1, b1; };

// The first two chunks of the weights of CTA `vb` (16 rows from 16 vb on), for the calling warp's
// slice of K.  They depend on nothing a kernel writes, so a caller issues them before it waits for
// whatever produces the token operand (the previous kernel).
template <int ROWS = 16>
__device__ __forceinline__ void gsm_prefetch(const __nv_bfloat16* __restrict__ w, int N, int K, int k_per_warp, int vb,
                                             GsmChunk& c0, GsmChunk& c1, int k_off = 0, int k_len = 1 << 30) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int n0 = vb * ROWS;
  const __nv_bfloat16* w0 = w + (size_t)min(n0 + g, N - 1) * K;
  const __nv_bfloat16* w1 = ROWS == 16 ? w + (size_t)min(n0 + g + 8, N - 1) * K : w0 + 64;     // (8 rows: the same row, 64 k on)
  const int kbeg = k_off + warp * k_per_warp, kend = min(min(K, k_off + k_len), kbeg + k_per_warp);
  const uint4 zero = make_uint4(0, 0, 0, 0);
  auto load_chunk = [&](int k0, GsmChunk& ch) {
    const int ka = k0 + 8 * c, kb = k0 + 32 + 8 * c;
    const int far = ROWS == 16 ? 0 : 64;
    ch.a0 = ka < kend ? ld_stream16(w0 + ka) : zero;
    ch.b0 = ka + far < kend ? ld_stream16(w1 + ka) : zero;
    ch.a1 = kb < kend ? ld_stream16(w0 + kb) : zero;
    ch.b1 = kb + far < kend ? ld_stream16(w1 + kb) : zero;
  };
  load_chunk(kbeg, c0);
  load_chunk(kbeg + (ROWS == 16 ? 64 : 128), c1);
}

// The work of CTA `vb` of the product, by all threads of the calling CTA (blockDim.x / 32 warps split
// K in slices of k_per_warp).  `red`: shared memory for (warps x 16 x 8 MT) floats; `s_rstd`: 8 MT
// floats; c0, c1: what gsm_prefetch fetched for this vb.  Loads of everything a kernel may have
// written bypass L1 (ld.global.cg), so the function may also run in a kernel that outlives the
// producer of its operands.
//
// CLUSTER: the CTAs of a thread-block cluster share the 16 weight rows and take a share of K each (k_off, k_len:
// this CTA's); their sums meet in the cluster's first CTA through distributed shared memory, in the order of the
// CTAs, and that CTA alone writes the result.  For products whose weight rows are too few to give every SM a CTA.
//
// `push_bar` (CLUSTER only; null: the first CTA reads the others' sums from their shared memory between two barriers of
// the cluster): an mbarrier of count 1, initialised in every CTA, after which every thread of the cluster has arrived at
// the cluster's barrier (arrive only).  The other CTAs then push their sums into in-boxes behind the first CTA's own
// sums with st.async, which counts the bytes on that CTA's barrier, and leave; the first CTA waits for the bytes
// (bounded: on giving up it records code 1 in g_gsm_status and writes nothing).  The order of the sum stays the CTAs'.
static __device__ int g_gsm_status = 0;
//
// ROWS = 8: the CTA owns 8 weight rows instead of 16 (the instructions' rows 8 to 15 stay empty) and a chunk is 128 k of
// them: twice the CTAs without a cluster's meeting, for matrices of so few rows that 16 per CTA leave half of the SMs idle
// (not with CLUSTER).  k_per_warp is then a multiple of 128.
template <int MT, typename TOut, int XMODE, bool RESID, bool CLUSTER = false, bool PUSH = false, int ROWS = 16>
__device__ __forceinline__ void gsm_cta(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                        TOut* __restrict__ out, int M, int N, int K, int k_per_warp, const FuseArgs& na,
                                        int vb, float* red, float* s_rstd, GsmChunk c0, GsmChunk c1, int k_off = 0,
                                        int k_len = 1 << 30, uint64_t* push_bar = nullptr) {
  constexpr bool SILU = XMODE == X_SILU;
  constexpr bool NORM = XMODE == X_NORM;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, c = lane & 3;
  static_assert(ROWS == 16 || (ROWS == 8 && !CLUSTER), "8 rows a CTA: without clusters");
  const int n0 = vb * ROWS;
  const int r0 = min(n0 + g, N - 1), r1 = min(n0 + g + 8, N - 1);     // clamped; discarded at the store
  const __nv_bfloat16* w0 = w + (size_t)r0 * K;
  const __nv_bfloat16* w1 = ROWS == 16 ? w + (size_t)r1 * K : w0 + 64;
  const int kbeg = k_off + warp * k_per_warp, kend = min(min(K, k_off + k_len), kbeg + k_per_warp);
  const int x_ld = SILU ? 2 * K : K;
  const bool writer = !CLUSTER || cluster_cta_rank() == 0;

  float acc[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[t][i] = 0.f;

  const uint4 zero = make_uint4(0, 0, 0, 0);
  auto load_chunk = [&](int k0) {
    GsmChunk ch;
    const int ka = k0 + 8 * c, kb = k0 + 32 + 8 * c;
    const int far = ROWS == 16 ? 0 : 64;
    ch.a0 = ka < kend ? ld_stream16(w0 + ka) : zero;
    ch.b0 = ka + far < kend ? ld_stream16(w1 + ka) : zero;
    ch.a1 = kb < kend ? ld_stream16(w0 + kb) : zero;
    ch.b1 = kb + far < kend ? ld_stream16(w1 + kb) : zero;
    return ch;
  };
  auto load_x = [&](int m, int k) {
    if (m >= M || k >= kend) return zero;
    if (NORM) {
      const size_t o = (size_t)m * K + k;
      float f[8], wv[8];
      *reinterpret_cast<float4*>(f) = __ldcg(reinterpret_cast<const float4*>(na.resid + o));
      *reinterpret_cast<float4*>(f + 4) = __ldcg(reinterpret_cast<const float4*>(na.resid + o + 4));
      *reinterpret_cast<float4*>(wv) = __ldg(reinterpret_cast<const float4*>(na.norm_w + k));
      *reinterpret_cast<float4*>(wv + 4) = __ldg(reinterpret_cast<const float4*>(na.norm_w + k + 4));
      const float rs = s_rstd[m];
      uint4 v;
      __nv_bfloat162* vp = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) vp[i] = __floats2bfloat162_rn(f[2 * i] * rs * wv[2 * i], f[2 * i + 1] * rs * wv[2 * i + 1]);
      return v;
    }
    const __nv_bfloat16* p = x + (size_t)m * x_ld + k;
    uint4 v = __ldcg(reinterpret_cast<const uint4*>(p));
    if (SILU) {
      const uint4 u = __ldcg(reinterpret_cast<const uint4*>(p + K));
      v.x = silu_mul_pair(v.x, u.x); v.y = silu_mul_pair(v.y, u.y);
      v.z = silu_mul_pair(v.z, u.z); v.w = silu_mul_pair(v.w, u.w);
    }
    return v;
  };
  auto compute = [&](const GsmChunk& ch, int k0) {
    const int ka = k0 + 8 * c, kb = k0 + 32 + 8 * c;
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      const uint4 xa = load_x(t * 8 + g, ka);
      const uint4 xb = load_x(t * 8 + g, kb);
      if (ROWS == 16) {
        mma_bf16_16816(acc[t], ch.a0.x, ch.b0.x, ch.a0.y, ch.b0.y, xa.x, xa.y);
        mma_bf16_16816(acc[t], ch.a0.z, ch.b0.z, ch.a0.w, ch.b0.w, xa.z, xa.w);
        mma_bf16_16816(acc[t], ch.a1.x, ch.b1.x, ch.a1.y, ch.b1.y, xb.x, xb.y);
        mma_bf16_16816(acc[t], ch.a1.z, ch.b1.z, ch.a1.w, ch.b1.w, xb.z, xb.w);
      } else {
        const uint4 xc = load_x(t * 8 + g, ka + 64);
        const uint4 xd = load_x(t * 8 + g, kb + 64);
        mma_bf16_16816(acc[t], ch.a0.x, 0u, ch.a0.y, 0u, xa.x, xa.y);
        mma_bf16_16816(acc[t], ch.a0.z, 0u, ch.a0.w, 0u, xa.z, xa.w);
        mma_bf16_16816(acc[t], ch.a1.x, 0u, ch.a1.y, 0u, xb.x, xb.y);
        mma_bf16_16816(acc[t], ch.a1.z, 0u, ch.a1.w, 0u, xb.z, xb.w);
        mma_bf16_16816(acc[t], ch.b0.x, 0u, ch.b0.y, 0u, xc.x, xc.y);
        mma_bf16_16816(acc[t], ch.b0.z, 0u, ch.b0.w, 0u, xc.z, xc.w);
        mma_bf16_16816(acc[t], ch.b1.x, 0u, ch.b1.y, 0u, xd.x, xd.y);
        mma_bf16_16816(acc[t], ch.b1.z, 0u, ch.b1.w, 0u, xd.z, xd.w);
      }
    }
  };
  float resid_old = 0.f;                            // RESID: this thread's element of the stream, fetched early
  if (RESID && writer) {
    const int m = threadIdx.x / ROWS, n = n0 + (threadIdx.x & (ROWS - 1));
    if (threadIdx.x < ROWS * 8 * MT && m < M && n < N) resid_old = __ldcg(reinterpret_cast<const float*>(out) + (size_t)m * N + n);
  }
  if (NORM) {
    // the row norms from the partial sums of squares: a warp per row, all loads at once, summed in a
    // fixed order (lane l adds parts l, l + 32, ...; then the lanes are added in a tree)
    for (int m = warp; m < M; m += nwarps) {
      const float* p = na.ssq + (size_t)m * na.ssq_ld;
      float ss = 0.f;
      for (int i = lane; i < na.n_ssq; i += 32) ss += __ldcg(p + i);
      ss = warp_sum(ss);
      if (lane == 0) s_rstd[m] = rsqrtf(ss / (float)K + na.eps);
    }
    __syncthreads();
  }
  constexpr int CK = ROWS == 16 ? 64 : 128;         // k of a chunk
  for (int k0 = kbeg; k0 < kend; k0 += 2 * CK) {
    const GsmChunk n0c = load_chunk(k0 + 2 * CK);
    compute(c0, k0);
    const GsmChunk n1c = load_chunk(k0 + 3 * CK);
    compute(c1, k0 + CK);
    c0 = n0c;
    c1 = n1c;
  }
  QE_TL_MARK(2);
  // acc[t][0..1]: weight row g, tokens 8t + 2c + {0,1};  acc[t][2..3]: weight row g + 8
  constexpr int MW = 8 * MT;
  float* mine = red + (size_t)warp * 16 * MW;
#pragma unroll
  for (int t = 0; t < MT; ++t) {
    mine[g * MW + t * 8 + 2 * c] = acc[t][0];
    mine[g * MW + t * 8 + 2 * c + 1] = acc[t][1];
    mine[(g + 8) * MW + t * 8 + 2 * c] = acc[t][2];
    mine[(g + 8) * MW + t * 8 + 2 * c + 1] = acc[t][3];
  }
  __syncthreads();
  float* part = red + (size_t)nwarps * 16 * MW;     // CLUSTER: this CTA's sums [16 MW] (pulled: read by the cluster's first CTA; pushed: the others' follow)
  constexpr bool pushed = CLUSTER && PUSH;          // (a template parameter: the pulled form stays as lean as it was)
  if (CLUSTER) {
    uint32_t dst = 0, bar = 0;
    if (pushed) {
      asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");     // (arrived at the kernel's top: the first CTA's barrier exists)
      if (!writer) {
        dst = cluster_map_shared(part + (size_t)16 * MW * cluster_cta_rank(), 0);
        bar = cluster_map_shared(push_bar, 0);
      }
    }
    for (int e = threadIdx.x; e < 16 * MW; e += blockDim.x) {
      const int m = e >> 4, i = e & 15;
      float s = 0.f;
      for (int wi = 0; wi < nwarps; ++wi) s += red[((size_t)wi * 16 + i) * MW + m];
      part[e] = s;
    }
    if (pushed && !writer) {
      // 16 bytes a thread: a quarter of the stores and of the barrier's updates
      __syncthreads();
      for (int e4 = threadIdx.x; e4 < 4 * MW; e4 += blockDim.x) {
        const float4 v = *reinterpret_cast<const float4*>(part + 4 * e4);
        asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];\n"
                     :: "r"(dst + 16u * (uint32_t)e4), "r"(__float_as_uint(v.x)), "r"(__float_as_uint(v.y)),
                        "r"(__float_as_uint(v.z)), "r"(__float_as_uint(v.w)), "r"(bar) : "memory");
      }
    }
    if (pushed) {
      if (!writer) return;
      if (threadIdx.x == 0) {
        const uint32_t bytes = (cluster_num_ctas() - 1u) * (uint32_t)(16 * MW) * 4u;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n"
                     :: "r"((uint32_t)__cvta_generic_to_shared(push_bar)), "r"(bytes) : "memory");
      }
      bool landed = false;
      for (uint32_t spin = 0; spin < (1u << 22) && !landed; ++spin) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}\n"
                     : "=r"(ok) : "r"((uint32_t)__cvta_generic_to_shared(push_bar)), "r"(0u) : "memory");
        landed = ok != 0;
      }
      if (!landed) { atomicCAS(&g_gsm_status, 0, 1); return; }
    } else {
      cluster_sync_all();                           // every CTA's sums are in place
    }
  }
  if (writer)
  for (int e = threadIdx.x; e < ROWS * MW; e += blockDim.x) {
    const int m = e / ROWS, i = e & (ROWS - 1);     // consecutive threads: consecutive weight rows
    const int n = n0 + i;
    // the sum over K: the warps' parts in order, or (CLUSTER) the CTAs' sums in order
    auto total = [&]() {
      float s = 0.f;
      if (CLUSTER) {
        const uint32_t S = cluster_num_ctas();
        if (pushed) for (uint32_t r = 0; r < S; ++r) s += part[(size_t)16 * MW * r + e];
        else for (uint32_t r = 0; r < S; ++r) s += cluster_ld_f32(cluster_map_shared(&part[e], r));
      } else {
        for (int wi = 0; wi < nwarps; ++wi) s += red[((size_t)wi * 16 + i) * MW + m];
      }
      return s;
    };
    if (!RESID) {
      if (m >= M || n >= N) continue;
      out[(size_t)m * N + n] = from_f32<TOut>(total());
    } else {
      // whole warps run this loop (ROWS MW is a multiple of 32); lanes outside the matrix add zero
      float v = 0.f;
      if (m < M && n < N) {
        const float s = total();
        float* dst = reinterpret_cast<float*>(out) + (size_t)m * N + n;
        v = (e == threadIdx.x ? resid_old : __ldcg(dst)) + s;
        *dst = v;
      }
      float sq = v * v;                              // over the CTA's columns of the row: lanes i = 0 .. ROWS - 1
      if (ROWS == 16) sq += __shfl_xor_sync(0xffffffffu, sq, 8);
      sq += __shfl_xor_sync(0xffffffffu, sq, 4);
      sq += __shfl_xor_sync(0xffffffffu, sq, 2);
      sq += __shfl_xor_sync(0xffffffffu, sq, 1);
      if (i == 0 && m < M) na.ssq_out[(size_t)m * na.ssq_ld + vb] = sq;
    }
  }
  if (CLUSTER && !pushed) cluster_sync_all();       // nobody reads this CTA's shared memory any more
  QE_TL_MARK(3);
}

// The gate and up projections of a feed-forward and its activation in one: CTA `vb` takes the 16 gate rows from
// 16 vb on AND the 16 up rows of the same columns (rows I + 16 vb ... of the stacked weights w [2 I, K]), and writes
// act[m, n] = silu(g) * u for its 16 columns: g and u rounded to bfloat16 as if stored, silu in float32, rounded once
// (reference src/models/qwen3/model.py:233-236, src/layers/fused_ops/silumul.py:50-53).  The token operand is loaded
// once for both.  `red`: shared memory for 2 x (warps x 16 x 8 MT) floats.
template <int MT>
__device__ __forceinline__ void gsm_cta_swiglu(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                               __nv_bfloat16* __restrict__ act, int M, int I, int K, int k_per_warp,
                                               int vb, float* red) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int n0 = vb * 16;
  const int r0 = min(n0 + g, I - 1), r1 = min(n0 + g + 8, I - 1);     // clamped; discarded at the store
  const __nv_bfloat16* wg0 = w + (size_t)r0 * K;
  const __nv_bfloat16* wg1 = w + (size_t)r1 * K;
  const __nv_bfloat16* wu0 = w + ((size_t)I + r0) * K;
  const __nv_bfloat16* wu1 = w + ((size_t)I + r1) * K;
  const int kbeg = warp * k_per_warp, kend = min(K, kbeg + k_per_warp);
  float ag[MT][4], au[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) { ag[t][i] = 0.f; au[t][i] = 0.f; }
  const uint4 zero = make_uint4(0, 0, 0, 0);
  struct Pair { uint4 ga, gb, ua, ub; };            // 32 k of the four rows
  auto load_w = [&](int k) {
    Pair p;
    const int ka = k + 8 * c;
    const bool ok = ka < kend;
    p.ga = ok ? ld_stream16(wg0 + ka) : zero;
    p.gb = ok ? ld_stream16(wg1 + ka) : zero;
    p.ua = ok ? ld_stream16(wu0 + ka) : zero;
    p.ub = ok ? ld_stream16(wu1 + ka) : zero;
    return p;
  };
  // the weights are nobody's output: the first loads go out before the wait for the kernel before this one
  Pair p0 = load_w(kbeg), p1 = load_w(kbeg + 32), p2 = load_w(kbeg + 64), p3 = load_w(kbeg + 96);
  pdl_wait();
  auto compute = [&](const Pair& p, int k) {
    const int ka = k + 8 * c;
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      const int m = t * 8 + g;
      const uint4 xa = (m < M && ka < kend) ? __ldcg(reinterpret_cast<const uint4*>(x + (size_t)m * K + ka)) : zero;
      mma_bf16_16816(ag[t], p.ga.x, p.gb.x, p.ga.y, p.gb.y, xa.x, xa.y);
      mma_bf16_16816(ag[t], p.ga.z, p.gb.z, p.ga.w, p.gb.w, xa.z, xa.w);
      mma_bf16_16816(au[t], p.ua.x, p.ub.x, p.ua.y, p.ub.y, xa.x, xa.y);
      mma_bf16_16816(au[t], p.ua.z, p.ub.z, p.ua.w, p.ub.w, xa.z, xa.w);
    }
  };
  for (int k0 = kbeg; k0 < kend; k0 += 128) {
    const Pair n0p = load_w(k0 + 128);
    compute(p0, k0);
    const Pair n1p = load_w(k0 + 160);
    compute(p1, k0 + 32);
    const Pair n2p = load_w(k0 + 192);
    compute(p2, k0 + 64);
    const Pair n3p = load_w(k0 + 224);
    compute(p3, k0 + 96);
    p0 = n0p; p1 = n1p; p2 = n2p; p3 = n3p;
  }
  QE_TL_MARK(2);
  constexpr int MW = 8 * MT;
  float* mine_g = red + (size_t)warp * 16 * MW;
  float* mine_u = red + ((size_t)nwarps + warp) * 16 * MW;
#pragma unroll
  for (int t = 0; t < MT; ++t) {
    mine_g[g * MW + t * 8 + 2 * c] = ag[t][0];
    mine_g[g * MW + t * 8 + 2 * c + 1] = ag[t][1];
    mine_g[(g + 8) * MW + t * 8 + 2 * c] = ag[t][2];
    mine_g[(g + 8) * MW + t * 8 + 2 * c + 1] = ag[t][3];
    mine_u[g * MW + t * 8 + 2 * c] = au[t][0];
    mine_u[g * MW + t * 8 + 2 * c + 1] = au[t][1];
    mine_u[(g + 8) * MW + t * 8 + 2 * c] = au[t][2];
    mine_u[(g + 8) * MW + t * 8 + 2 * c + 1] = au[t][3];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < 16 * MW; e += blockDim.x) {
    const int m = e >> 4, i = e & 15;
    const int n = n0 + i;
    if (m >= M || n >= I) continue;
    float sg = 0.f, su = 0.f;
    for (int wi = 0; wi < nwarps; ++wi) {
      sg += red[((size_t)wi * 16 + i) * MW + m];
      su += red[((size_t)(nwarps + wi) * 16 + i) * MW + m];
    }
    const float gb = __bfloat162float(__float2bfloat16_rn(sg)), ub = __bfloat162float(__float2bfloat16_rn(su));
    act[(size_t)m * I + n] = __float2bfloat16_rn(silu_fast(gb) * ub);
  }
  QE_TL_MARK(3);
}


// ---- the QKV product of a decode step with what follows it in its epilogue ---------------------------------------
// A head of 128 columns is the work of a cluster of 8 CTAs (16 columns each).  After the product, the CTAs of a q or
// k head exchange two things through distributed shared memory: the sums of squares of their 16 columns of every row
// (the per-head RMS norm needs the head's), and the normed values, because the rotation pairs element d with d + 64,
// which lies in the CTA four ranks away.  Then every CTA writes its 16 columns: q into the qkv buffer, k and v
// straight into the cache page of the token's slot (the k and v columns of the qkv buffer are not written).  The
// arithmetic is the rotary kernel's (rope_d128.cuh): the product rounded to bfloat16 first (as if stored), norm and
// rotation in float32 with sincosf of position * inv_freq (or the step's table), rounded once.
struct GsmRope {
  const float* qw; const float* kw; float eps;       // norm weights [128] (null: no norm)
  const int* positions; const float* inv_freq;       // angles = position * inv_freq[d mod 64] (inv_freq null: no rotation) ...
  const float2* cos_sin;                             // ... or, if given, the step's table [M, 64] of (cos, sin)
  __nv_bfloat16* pages; const int* slot_mapping;     // the cache [pages, 2, Hkv, page, 128] and the tokens' slots
  int Hq, Hkv, page_size, write_kv;
};

template <int MT>
__device__ __forceinline__ void gsm_cta_qkv_rope(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                 __nv_bfloat16* __restrict__ qkv, int M, int N, int K, int k_per_warp,
                                                 const GsmRope& rp, int vb, float* red, float* s_val, float* s_ssq) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int n0 = vb * 16;
  const __nv_bfloat16* w0 = w + (size_t)(n0 + g) * K;
  const __nv_bfloat16* w1 = w + (size_t)(n0 + g + 8) * K;
  const int kbeg = warp * k_per_warp, kend = min(K, kbeg + k_per_warp);
  constexpr int MW = 8 * MT;
  const uint4 zero = make_uint4(0, 0, 0, 0);
  auto load_chunk = [&](int k0) {
    GsmChunk ch;
    const int ka = k0 + 8 * c, kb = k0 + 32 + 8 * c;
    ch.a0 = ka < kend ? ld_stream16(w0 + ka) : zero;
    ch.b0 = ka < kend ? ld_stream16(w1 + ka) : zero;
    ch.a1 = kb < kend ? ld_stream16(w0 + kb) : zero;
    ch.b1 = kb < kend ? ld_stream16(w1 + kb) : zero;
    return ch;
  };
  // the weights are nobody's output, and the angles come from the step's positions, which the host wrote: both are
  // on their way before the wait for the kernel before this one
  GsmChunk c0 = load_chunk(kbeg), c1 = load_chunk(kbeg + 64);
  const uint32_t rank = cluster_cta_rank();            // which 16 columns of the head
  const int head = n0 >> 7;
  const bool is_q = head < rp.Hq, is_v = head >= rp.Hq + rp.Hkv;
  const int e = threadIdx.x;                           // the epilogue's element of this thread: row e / 16, column e mod 16
  const int em = e >> 4, ei = e & 15;
  const int d = (int)rank * 16 + ei;                   // the element's place in its head
  const bool mine = e < 16 * MW && em < M;
  const bool rotate = !is_v && (rp.inv_freq != nullptr || rp.cos_sin != nullptr);
  float cs = 1.f, sn = 0.f, nw_self = 1.f, nw_pair = 1.f;
  int slot = 0;
  if (mine) {
    if (rotate) {
      if (rp.cos_sin) { const float2 t = __ldg(rp.cos_sin + (size_t)em * 64 + (d & 63)); cs = t.x; sn = t.y; }
      else sincosf((float)__ldg(rp.positions + em) * __ldg(rp.inv_freq + (d & 63)), &sn, &cs);
    }
    const float* nw = is_v ? nullptr : (is_q ? rp.qw : rp.kw);
    if (nw) { nw_self = __ldg(nw + d); nw_pair = __ldg(nw + (d ^ 64)); }
    if (!is_q && rp.write_kv) slot = __ldg(rp.slot_mapping + em);
  }
  pdl_wait();
  float acc[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[t][i] = 0.f;
  auto compute = [&](const GsmChunk& ch, int k0) {
    const int ka = k0 + 8 * c, kb = k0 + 32 + 8 * c;
#pragma unroll
    for (int t = 0; t < MT; ++t) {
      const int m = t * 8 + g;
      const uint4 xa = (m < M && ka < kend) ? __ldcg(reinterpret_cast<const uint4*>(x + (size_t)m * K + ka)) : zero;
      const uint4 xb = (m < M && kb < kend) ? __ldcg(reinterpret_cast<const uint4*>(x + (size_t)m * K + kb)) : zero;
      mma_bf16_16816(acc[t], ch.a0.x, ch.b0.x, ch.a0.y, ch.b0.y, xa.x, xa.y);
      mma_bf16_16816(acc[t], ch.a0.z, ch.b0.z, ch.a0.w, ch.b0.w, xa.z, xa.w);
      mma_bf16_16816(acc[t], ch.a1.x, ch.b1.x, ch.a1.y, ch.b1.y, xb.x, xb.y);
      mma_bf16_16816(acc[t], ch.a1.z, ch.b1.z, ch.a1.w, ch.b1.w, xb.z, xb.w);
    }
  };
  for (int k0 = kbeg; k0 < kend; k0 += 128) {
    const GsmChunk n0c = load_chunk(k0 + 128);
    compute(c0, k0);
    const GsmChunk n1c = load_chunk(k0 + 192);
    compute(c1, k0 + 64);
    c0 = n0c;
    c1 = n1c;
  }
  QE_TL_MARK(2);
  float* part = red + (size_t)warp * 16 * MW;
#pragma unroll
  for (int t = 0; t < MT; ++t) {
    part[g * MW + t * 8 + 2 * c] = acc[t][0];
    part[g * MW + t * 8 + 2 * c + 1] = acc[t][1];
    part[(g + 8) * MW + t * 8 + 2 * c] = acc[t][2];
    part[(g + 8) * MW + t * 8 + 2 * c + 1] = acc[t][3];
  }
  __syncthreads();
  // the product's element (em, n0 + ei), the warps' parts in order, rounded as the plain product's output is
  float y = 0.f;
  if (e < 16 * MW) {
    for (int wi = 0; wi < nwarps; ++wi) y += red[((size_t)wi * 16 + ei) * MW + em];
    y = __bfloat162float(__float2bfloat16_rn(y));
  }
  const bool exchange = !is_v && (rotate || rp.qw != nullptr || rp.kw != nullptr);      // the same in all CTAs of the head
  float outv = y;
  if (exchange) {
    if (e < 16 * MW) {                                 // whole warps (16 MW is a multiple of 32)
      float sq = y * y;                                // over the 16 columns of the row: lanes ei = 0..15
      sq += __shfl_xor_sync(0xffffffffu, sq, 8);
      sq += __shfl_xor_sync(0xffffffffu, sq, 4);
      sq += __shfl_xor_sync(0xffffffffu, sq, 2);
      sq += __shfl_xor_sync(0xffffffffu, sq, 1);
      if (ei == 0) s_ssq[em] = sq;
      s_val[e] = y;
    }
    cluster_sync_all();                                // every CTA's values and sums of squares are in place
    if (mine) {
      float rstd = 1.f;
      if ((is_q ? rp.qw : rp.kw) != nullptr) {
        float ss = 0.f;
#pragma unroll
        for (uint32_t r = 0; r < 8; ++r) ss += cluster_ld_f32(cluster_map_shared(&s_ssq[em], r));
        rstd = rsqrtf(ss / 128.f + rp.eps);
      }
      const float self = y * rstd * nw_self;
      if (rotate) {
        const float pair = cluster_ld_f32(cluster_map_shared(&s_val[e], rank ^ 4u)) * rstd * nw_pair;
        outv = d < 64 ? cs * self - sn * pair : sn * pair + cs * self;      // (lo, hi) -> (cos lo - sin hi, sin lo + cos hi)
      } else {
        outv = self;
      }
    }
  }
  if (mine) {
    if (is_q) {
      qkv[(size_t)em * N + n0 + ei] = __float2bfloat16_rn(outv);
    } else if (rp.write_kv) {
      // slot = page * page_size + off: the row of (page, K or V, h, off) in the cache
      const int h = is_v ? head - rp.Hq - rp.Hkv : head - rp.Hq;
      const int page = slot / rp.page_size;
      rp.pages[((size_t)slot + ((size_t)page * (2 * rp.Hkv - 1) + (is_v ? rp.Hkv : 0) + h) * rp.page_size) * 128 + d] = __float2bfloat16_rn(outv);
    }
  }
  if (exchange) cluster_sync_all();                    // nobody reads this CTA's shared memory any more
  QE_TL_MARK(3);
}
