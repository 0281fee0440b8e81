// Embedding gather, residual add + RMS norm, SiLU-multiply, and the fused
// per-head norm + rotary encoding + cache write.  Every kernel is a template
// over the element type (float: the true 32-bit path; bfloat16: serving) and
// does its arithmetic in float32.
#include "common.cuh"
#include "rope_d128.cuh"

// ---------------------------------------------------------------------------------------
// out[t, :] = float(table[ids[t], :])      (reference src/layers/ops/embedding.py:28-44)
// The residual stream is float32 in both paths.  An id outside the table gives NaN rows.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ out, int H, int V, float* __restrict__ ssq_out, int ssq_ld) {
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  // after the wait: the ids of a step launched ahead are put in place by a kernel (place_tokens) from the tokens
  // that the step before it sampled; read earlier, an id could still be the place holder
  const int id = ids[t];
  float* dst = out + (size_t)t * H;
  if (id < 0 || id >= V) {
    for (int h = threadIdx.x; h < H; h += blockDim.x) dst[h] = __int_as_float(0x7fc00000);
    return;
  }
  const T* src = table + (size_t)id * H;
  float ss = 0.f;
  for (int h = threadIdx.x; h < H; h += blockDim.x) { const float v = to_f32(src[h]); dst[h] = v; ss += v * v; }
  if (ssq_out) {                                   // the row's sum of squares, for a norm fused downstream
    ss = block_sum(ss, scratch);
    if (threadIdx.x == 0) ssq_out[(size_t)t * ssq_ld] = ss;
  }
}

extern "C" int qe_embedding(const int* ids, const void* table, float* out, int T, int H, int V,
                            int dtype, float* ssq_out, int ssq_ld, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dtype == QE_DTYPE_F32)
    qe_launch(embedding_kernel<float>, dim3(T), dim3(256), 0, stream, ids, (const float*)table, out, H, V, ssq_out, ssq_ld);
  else if (dtype == QE_DTYPE_BF16)
    qe_launch(embedding_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, ids, (const __nv_bfloat16*)table, out, H, V, ssq_out, ssq_ld);
  else QE_REFUSE("embedding: unknown dtype %d", dtype);
  QE_CHECK_LAUNCH("embedding");
  return 0;
}

// ---------------------------------------------------------------------------------------
// x = resid[row] (+ delta[row]);  out = x * rsqrt(mean(x^2) + eps) * w
// (reference src/layers/ops/layernorm.py:50-88).  Without `rows` the sum is written back
// to the float32 stream; with `rows` (the rows whose logits are wanted) row n of the output
// comes from row rows[n] and the stream is left alone.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                   const int* __restrict__ rows, const float* __restrict__ w,
                                   float eps, T* __restrict__ out, int H) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x;
  const int src_row = rows ? rows[n] : n;
  float* r = resid + (size_t)src_row * H;
  const T* d = delta ? delta + (size_t)src_row * H : nullptr;
  T* o = out + (size_t)n * H;
  float ss = 0.f;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    float x = r[h];
    if (d) x += to_f32(d[h]);
    if (d && !rows) r[h] = x;
    ss += x * x;
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)H + eps);
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    float x = r[h];
    if (d && rows) x += to_f32(d[h]);
    o[h] = from_f32<T>(x * rstd * w[h]);
  }
}

// The same for bfloat16 with H % 8 == 0: 8 elements per thread and step (16- and 32-byte accesses).
__device__ __forceinline__ void bf16x8_to_f32(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(p[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ uint4 f32_to_bf16x8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

__global__ void add_rmsnorm_bf16x8_kernel(float* __restrict__ resid, const __nv_bfloat16* __restrict__ delta,
                                          const int* __restrict__ rows, const float* __restrict__ w,
                                          float eps, __nv_bfloat16* __restrict__ out, int H) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x;
  const int src_row = rows ? rows[n] : n;
  float* r = resid + (size_t)src_row * H;
  const __nv_bfloat16* d = delta ? delta + (size_t)src_row * H : nullptr;
  __nv_bfloat16* o = out + (size_t)n * H;
  float ss = 0.f;
  for (int h = threadIdx.x * 8; h < H; h += blockDim.x * 8) {
    float x[8];
    *reinterpret_cast<float4*>(x) = *reinterpret_cast<const float4*>(r + h);
    *reinterpret_cast<float4*>(x + 4) = *reinterpret_cast<const float4*>(r + h + 4);
    if (d) {
      float dv[8];
      bf16x8_to_f32(*reinterpret_cast<const uint4*>(d + h), dv);
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] += dv[i];
      if (!rows) {
        *reinterpret_cast<float4*>(r + h) = *reinterpret_cast<const float4*>(x);
        *reinterpret_cast<float4*>(r + h + 4) = *reinterpret_cast<const float4*>(x + 4);
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
  }
  ss = block_sum(ss, scratch);
  const float rstd = rsqrtf(ss / (float)H + eps);
  for (int h = threadIdx.x * 8; h < H; h += blockDim.x * 8) {
    float x[8], wv[8];
    *reinterpret_cast<float4*>(x) = *reinterpret_cast<const float4*>(r + h);
    *reinterpret_cast<float4*>(x + 4) = *reinterpret_cast<const float4*>(r + h + 4);
    if (d && rows) {
      float dv[8];
      bf16x8_to_f32(*reinterpret_cast<const uint4*>(d + h), dv);
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] += dv[i];
    }
    *reinterpret_cast<float4*>(wv) = *reinterpret_cast<const float4*>(w + h);
    *reinterpret_cast<float4*>(wv + 4) = *reinterpret_cast<const float4*>(w + h + 4);
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = x[i] * rstd * wv[i];
    *reinterpret_cast<uint4*>(o + h) = f32_to_bf16x8(x);
  }
}

// The same with one warp per row, for widths that are multiples of 256 up to 2048: a lane keeps its
// NC pieces of 8 elements in registers between the sum of squares and the scaling, all its loads are
// in flight together, and no block-wide barrier is needed.
template <int NC>
__global__ void add_rmsnorm_bf16_warp_kernel(float* __restrict__ resid, const __nv_bfloat16* __restrict__ delta,
                                             const int* __restrict__ rows, const float* __restrict__ w,
                                             float eps, __nv_bfloat16* __restrict__ out, int n_rows) {
  constexpr int H = NC * 256;
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  // the scale vector is a weight and the row list comes with the step's host copy: both are fetched
  // while the kernel before this one is still running
  float wv[NC][8];
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int h = (c * 32 + lane) * 8;
    *reinterpret_cast<float4*>(wv[c]) = __ldg(reinterpret_cast<const float4*>(w + h));
    *reinterpret_cast<float4*>(wv[c] + 4) = __ldg(reinterpret_cast<const float4*>(w + h + 4));
  }
  const int src_row = n < n_rows ? (rows ? __ldg(rows + n) : n) : 0;
  pdl_wait();
  if (n >= n_rows) return;
  float* r = resid + (size_t)src_row * H;
  const __nv_bfloat16* d = delta ? delta + (size_t)src_row * H : nullptr;
  float x[NC][8];
  uint4 dv[NC];
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int h = (c * 32 + lane) * 8;
    *reinterpret_cast<float4*>(x[c]) = __ldcg(reinterpret_cast<const float4*>(r + h));
    *reinterpret_cast<float4*>(x[c] + 4) = __ldcg(reinterpret_cast<const float4*>(r + h + 4));
    if (d) dv[c] = __ldcg(reinterpret_cast<const uint4*>(d + h));
  }
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int h = (c * 32 + lane) * 8;
    if (d) {
      float f[8];
      bf16x8_to_f32(dv[c], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) x[c][i] += f[i];
      if (!rows) {
        *reinterpret_cast<float4*>(r + h) = *reinterpret_cast<const float4*>(x[c]);
        *reinterpret_cast<float4*>(r + h + 4) = *reinterpret_cast<const float4*>(x[c] + 4);
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += x[c][i] * x[c][i];
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / (float)H + eps);
  __nv_bfloat16* o = out + (size_t)n * H;
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int h = (c * 32 + lane) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) x[c][i] = x[c][i] * rstd * wv[c][i];
    *reinterpret_cast<uint4*>(o + h) = f32_to_bf16x8(x[c]);
  }
}

template <int NC>
static void launch_add_rmsnorm_warp(float* resid, const void* delta, const int* rows, const float* w, float eps, void* out,
                                    int n_rows, cudaStream_t stream) {
  const int warps = 4;
  qe_launch(add_rmsnorm_bf16_warp_kernel<NC>, dim3((n_rows + warps - 1) / warps), dim3(warps * 32), 0, stream, resid,
            (const __nv_bfloat16*)delta, rows, w, eps, (__nv_bfloat16*)out, n_rows);
}

extern "C" int qe_add_rmsnorm(float* resid, const void* delta, const int* rows, const float* w,
                              float eps, void* out, int n_rows, int H, int dtype, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const int threads = H >= 1024 ? 256 : (H >= 256 ? 128 : 64);
  if (dtype == QE_DTYPE_BF16 && H % 8 == 0 &&
      (((uintptr_t)resid | (uintptr_t)delta | (uintptr_t)w | (uintptr_t)out) & 15) == 0) {
    if (H % 256 == 0 && H <= 2048) {
      switch (H / 256) {
        case 1: launch_add_rmsnorm_warp<1>(resid, delta, rows, w, eps, out, n_rows, stream); break;
        case 2: launch_add_rmsnorm_warp<2>(resid, delta, rows, w, eps, out, n_rows, stream); break;
        case 3: launch_add_rmsnorm_warp<3>(resid, delta, rows, w, eps, out, n_rows, stream); break;
        case 4: launch_add_rmsnorm_warp<4>(resid, delta, rows, w, eps, out, n_rows, stream); break;
        case 5: launch_add_rmsnorm_warp<5>(resid, delta, rows, w, eps, out, n_rows, stream); break;
        case 6: launch_add_rmsnorm_warp<6>(resid, delta, rows, w, eps, out, n_rows, stream); break;
        case 7: launch_add_rmsnorm_warp<7>(resid, delta, rows, w, eps, out, n_rows, stream); break;
        default: launch_add_rmsnorm_warp<8>(resid, delta, rows, w, eps, out, n_rows, stream); break;
      }
      QE_CHECK_LAUNCH("add_rmsnorm");
      return 0;
    }
    const int vthreads = H >= 2048 ? 256 : 128;
    qe_launch(add_rmsnorm_bf16x8_kernel, dim3(n_rows), dim3(vthreads), 0, stream, resid, (const __nv_bfloat16*)delta,
              rows, w, eps, (__nv_bfloat16*)out, H);
    QE_CHECK_LAUNCH("add_rmsnorm");
    return 0;
  }
  if (dtype == QE_DTYPE_F32)
    qe_launch(add_rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, resid, (const float*)delta, rows, w, eps, (float*)out, H);
  else if (dtype == QE_DTYPE_BF16)
    qe_launch(add_rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, resid, (const __nv_bfloat16*)delta, rows, w, eps, (__nv_bfloat16*)out, H);
  else QE_REFUSE("add_rmsnorm: unknown dtype %d", dtype);
  QE_CHECK_LAUNCH("add_rmsnorm");
  return 0;
}

// ---------------------------------------------------------------------------------------
// out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i],  silu(g) = g / (1 + exp(-g))
// (reference src/layers/fused_ops/silumul.py:50-53), all in float32, rounded once.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int I, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
    const size_t t = e / I;
    const int i = (int)(e - t * I);
    const float g = to_f32(gate_up[t * 2 * I + i]);
    const float u = to_f32(gate_up[t * 2 * I + I + i]);
    out[e] = from_f32<T>(g / (1.f + expf(-g)) * u);
  }
}

__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out,
                                       int I, size_t total8) {
  pdl_launch_dependents();
  pdl_wait();
  // two 16-byte pieces per thread and turn, all four loads in flight before the arithmetic; the
  // exponential and the quotient by the fast hardware forms (the result is rounded to bfloat16)
  const int I8 = I / 8;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t e0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e0 < total8; e0 += 2 * stride) {
    const size_t e1 = e0 + stride;
    const bool two = e1 < total8;
    const size_t t0 = e0 / I8, t1 = two ? e1 / I8 : t0;
    const int i0 = (int)(e0 - t0 * I8) * 8, i1 = two ? (int)(e1 - t1 * I8) * 8 : i0;
    const uint4 rg0 = __ldcg(reinterpret_cast<const uint4*>(gate_up + t0 * 2 * I + i0));
    const uint4 ru0 = __ldcg(reinterpret_cast<const uint4*>(gate_up + t0 * 2 * I + I + i0));
    const uint4 rg1 = __ldcg(reinterpret_cast<const uint4*>(gate_up + t1 * 2 * I + i1));
    const uint4 ru1 = __ldcg(reinterpret_cast<const uint4*>(gate_up + t1 * 2 * I + I + i1));
    float g[8], u[8];
    bf16x8_to_f32(rg0, g);
    bf16x8_to_f32(ru0, u);
#pragma unroll
    for (int k = 0; k < 8; ++k) g[k] = __fdividef(g[k], 1.f + __expf(-g[k])) * u[k];
    *reinterpret_cast<uint4*>(out + t0 * I + i0) = f32_to_bf16x8(g);
    if (two) {
      bf16x8_to_f32(rg1, g);
      bf16x8_to_f32(ru1, u);
#pragma unroll
      for (int k = 0; k < 8; ++k) g[k] = __fdividef(g[k], 1.f + __expf(-g[k])) * u[k];
      *reinterpret_cast<uint4*>(out + t1 * I + i1) = f32_to_bf16x8(g);
    }
  }
}

extern "C" int qe_silu_mul(const void* gate_up, void* out, int T, int I, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  const size_t total = (size_t)T * I;
  if (dtype == QE_DTYPE_BF16 && I % 8 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0) {
    const size_t total8 = total / 8;
    const int vblocks = (int)((total8 + 255) / 256 < 148 * 8 ? (total8 + 255) / 256 : 148 * 8);
    qe_launch(silu_mul_bf16x8_kernel, dim3(vblocks), dim3(256), 0, stream, (const __nv_bfloat16*)gate_up,
              (__nv_bfloat16*)out, I, total8);
    QE_CHECK_LAUNCH("silu_mul");
    return 0;
  }
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  if (dtype == QE_DTYPE_F32)
    qe_launch(silu_mul_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float*)gate_up, (float*)out, I, total);
  else if (dtype == QE_DTYPE_BF16)
    qe_launch(silu_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, I, total);
  else QE_REFUSE("silu_mul: unknown dtype %d", dtype);
  QE_CHECK_LAUNCH("silu_mul");
  return 0;
}

// ---------------------------------------------------------------------------------------
// One warp per (token, head).  For q and k heads: optional RMS norm over the head
// (src/layers/ops/layernorm.py:127-134), then optional half-split rotation by
// angle = position * inv_freq[j] computed in float32 (src/layers/ops/rope.py:37-121), written
// back in place; k is also written to the token's slot of the cache, v is copied there.
// Cache layout of one layer: [page][K or V][kv head][offset in page][D].
// ---------------------------------------------------------------------------------------
#define QKR_MAX_D 512
template <typename T>
__global__ void qk_norm_rope_kv_write_kernel(T* __restrict__ q, T* __restrict__ k, const T* __restrict__ v,
                                             long q_stride, long k_stride, long v_stride,
                                             const int* __restrict__ positions,
                                             const float* __restrict__ qw, const float* __restrict__ kw, float eps,
                                             const float* __restrict__ inv_freq, int rotary_dim,
                                             T* __restrict__ pages, const int* __restrict__ slot_mapping,
                                             int T_tokens, int Hq, int Hkv, int D, int page_size, int write_kv) {
  extern __shared__ float smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads_total = Hq + 2 * Hkv;
  const long item = (long)blockIdx.x * warps_per_block + warp;
  if (item >= (long)T_tokens * heads_total) return;
  const int t = (int)(item / heads_total);
  const int head = (int)(item % heads_total);
  float* buf = smem + (size_t)warp * D;

  if (head >= Hq + Hkv) {           // a value head: copy into the cache
    if (!write_kv) return;
    const int h = head - Hq - Hkv;
    const int slot = slot_mapping[t];
    const int page = slot / page_size, off = slot % page_size;
    const T* src = v + (size_t)t * v_stride + (size_t)h * D;
    T* dst = pages + ((((size_t)page * 2 + 1) * Hkv + h) * page_size + off) * D;
    for (int d = lane; d < D; d += 32) dst[d] = src[d];
    return;
  }
  const bool is_q = head < Hq;
  const int h = is_q ? head : head - Hq;
  T* x = is_q ? q + (size_t)t * q_stride + (size_t)h * D : k + (size_t)t * k_stride + (size_t)h * D;
  const float* w = is_q ? qw : kw;
  float ss = 0.f;
  for (int d = lane; d < D; d += 32) {
    const float val = to_f32(x[d]);
    buf[d] = val;
    ss += val * val;
  }
  if (w) {
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)D + eps);
    for (int d = lane; d < D; d += 32) buf[d] = buf[d] * rstd * w[d];
  }
  __syncwarp();
  T* cache_dst = nullptr;
  if (!is_q && write_kv) {
    const int slot = slot_mapping[t];
    const int page = slot / page_size, off = slot % page_size;
    cache_dst = pages + ((((size_t)page * 2 + 0) * Hkv + h) * page_size + off) * D;
  }
  const int half = rotary_dim >> 1;
  const float pos = (float)positions[t];
  for (int d = lane; d < D; d += 32) {
    float o = buf[d];
    if (inv_freq && d < rotary_dim) {
      const int j = d < half ? d : d - half;
      const float ang = pos * inv_freq[j];
      float s, c;
      sincosf(ang, &s, &c);
      o = d < half ? c * buf[d] - s * buf[d + half] : s * buf[d - half] + c * buf[d];
    }
    const T r = from_f32<T>(o);
    x[d] = r;
    if (cache_dst) cache_dst[d] = r;
  }
}

// U consecutive (token, head) per warp, their loads in flight together (large steps: U = 4)
template <int U>
__global__ void qk_norm_rope_kv_write_d128_kernel(RopeD128Args args) {
  pdl_launch_dependents();
  // the launcher keeps tokens x heads below 2^31
  const int heads_total = args.Hq + 2 * args.Hkv;
  const int item0 = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * U;
  const int t0 = item0 / heads_total, head0 = item0 - t0 * heads_total;
  if constexpr (U == 1) {
    // a small step (a decode step): position, angles, norm weights and cache slot are fetched and worked
    // out while the kernel before this one (the QKV product) is still running
    RopeD128Pre pre;
    rope_d128_prepare(args, t0, head0, pre);
    pdl_wait();
    rope_d128_finish(args, t0, head0, rope_d128_load(args, t0, head0), &pre);
    return;
  }
  pdl_wait();
  uint2 raw[U];
  int t[U], head[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    head[u] = head0 + u; t[u] = t0;
    while (head[u] >= heads_total) { head[u] -= heads_total; ++t[u]; }
    raw[u] = rope_d128_load(args, t[u], head[u]);
  }
#pragma unroll
  for (int u = 0; u < U; ++u) rope_d128_finish(args, t[u], head[u], raw[u]);
}

// cos_sin[t, j] = (cos, sin)(positions[t] * inv_freq[j]) in float32: the angles of a step, computed
// once and shared by every layer and head (the reference keeps such a table for every position of
// the model in every layer, src/models/qwen3/model.py:75-84).
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float2* __restrict__ cos_sin, int T, int half) {
  pdl_launch_dependents();
  pdl_wait();
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= T * half) return;
  const int t = e / half, j = e - t * half;
  float s, c;
  sincosf((float)positions[t] * inv_freq[j], &s, &c);
  cos_sin[e] = make_float2(c, s);
}

extern "C" int qe_rope_table(const int* positions, const float* inv_freq, void* cos_sin, int T, int half,
                             cudaStream_t stream) {
  if (T <= 0 || half <= 0) return 0;
  const int n = T * half;
  qe_launch(rope_table_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, positions, inv_freq, (float2*)cos_sin, T, half);
  QE_CHECK_LAUNCH("rope_table");
  return 0;
}

extern "C" int qe_qk_norm_rope_kv_write(void* q, void* k, const void* v, long q_stride, long k_stride, long v_stride,
                                        const int* positions, const float* qw, const float* kw, float eps,
                                        const float* inv_freq, const void* cos_sin, int rotary_dim, void* pages,
                                        const int* slot_mapping, int T, int Hq, int Hkv, int D, int page_size,
                                        int write_kv, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D > QKR_MAX_D) QE_REFUSE("qk_norm_rope_kv_write: head_dim %d is above %d", D, QKR_MAX_D);
  if (inv_freq && (rotary_dim % 2 || rotary_dim > D || rotary_dim <= 0))
    QE_REFUSE("qk_norm_rope_kv_write: rotary_dim %d does not fit head_dim %d", rotary_dim, D);
  if (write_kv && (!pages || !slot_mapping)) QE_REFUSE("qk_norm_rope_kv_write: cache write without cache");
  if (dtype == QE_DTYPE_BF16 && D == 128 && (!inv_freq || rotary_dim == D) &&
      ((q_stride | k_stride | v_stride) % 4) == 0 &&
      (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)pages) & 7) == 0) {
    const long n_items = (long)T * (Hq + 2 * Hkv);
    if (n_items > 0x7fffff00L) QE_REFUSE("qk_norm_rope_kv_write: %d tokens x %d heads are too many for one launch", T, Hq + 2 * Hkv);
    const int vwarps = 8;
    RopeD128Args ra{(__nv_bfloat16*)q, (__nv_bfloat16*)k, (const __nv_bfloat16*)v, q_stride, k_stride, v_stride, positions,
                    qw, kw, eps, inv_freq, (const float2*)cos_sin, (__nv_bfloat16*)pages, slot_mapping, T, Hq, Hkv, page_size, write_kv};
    if (n_items >= 4096)
      qe_launch(qk_norm_rope_kv_write_d128_kernel<4>, dim3((unsigned)((n_items + 4 * vwarps - 1) / (4 * vwarps))),
                dim3(vwarps * 32), 0, stream, ra);
    else
      qe_launch(qk_norm_rope_kv_write_d128_kernel<1>, dim3((unsigned)((n_items + vwarps - 1) / vwarps)), dim3(vwarps * 32), 0,
                stream, ra);
    QE_CHECK_LAUNCH("qk_norm_rope_kv_write");
    return 0;
  }
  const int warps = 4;
  const long items = (long)T * (Hq + 2 * Hkv);
  const int blocks = (int)((items + warps - 1) / warps);
  const size_t smem = (size_t)warps * D * sizeof(float);
  if (dtype == QE_DTYPE_F32)
    qe_launch(qk_norm_rope_kv_write_kernel<float>, dim3(blocks), dim3(warps * 32), smem, stream,
        (float*)q, (float*)k, (const float*)v, q_stride, k_stride, v_stride, positions, qw, kw, eps, inv_freq,
        rotary_dim, (float*)pages, slot_mapping, T, Hq, Hkv, D, page_size, write_kv);
  else if (dtype == QE_DTYPE_BF16)
    qe_launch(qk_norm_rope_kv_write_kernel<__nv_bfloat16>, dim3(blocks), dim3(warps * 32), smem, stream,
        (__nv_bfloat16*)q, (__nv_bfloat16*)k, (const __nv_bfloat16*)v, q_stride, k_stride, v_stride, positions, qw, kw,
        eps, inv_freq, rotary_dim, (__nv_bfloat16*)pages, slot_mapping, T, Hq, Hkv, D, page_size, write_kv);
  else QE_REFUSE("qk_norm_rope_kv_write: unknown dtype %d", dtype);
  QE_CHECK_LAUNCH("qk_norm_rope_kv_write");
  return 0;
}

// ---------------------------------------------------------------------------------------
// dst[rows[i]] = src[src_index[i]]: token ids that the step before this one sampled and that the host
// has not read yet are put into this step's token list on the device (a step launched ahead).
// ---------------------------------------------------------------------------------------
__global__ void place_tokens_kernel(int* __restrict__ dst, const int* __restrict__ rows, const int* __restrict__ src,
                                    const int* __restrict__ src_index, int n) {
  // No early start of the kernels behind this one (no griddepcontrol.launch_dependents): they begin when this grid
  // has completed.  The step's kernels do what reads only "the step's index data" before their own wait, and the
  // token ids that this kernel writes are such data: a dependent that started early, and its dependents after it,
  // could read an id before it is here.
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[rows[i]] = src[src_index[i]];
}

extern "C" int qe_place_tokens(int* dst, const int* rows, const int* src, const int* src_index, int n, cudaStream_t stream) {
  if (n <= 0) return 0;
  qe_launch(place_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, dst, rows, src, src_index, n);
  QE_CHECK_LAUNCH("place_tokens");
  return 0;
}

// ---------------------------------------------------------------------------------------
// Copies of whole cache pages: for every pair (src, dst) the page src of every cache slot of a group is
// copied to page dst of the same slot (a request that found its whole prompt in shared pages gets a private
// copy of the last one before it writes there).  cache: [slots, pages, page_bytes]; pairs: int32 [n, 2] on the
// device.  A pair that names a page outside the group is passed over.
// ---------------------------------------------------------------------------------------
template <typename U>
__global__ void copy_pages_kernel(U* __restrict__ cache, long slot_units, long page_units, const int* __restrict__ pairs,
                                  int n_pages) {
  // No early start of the kernels behind this one (as place_tokens): the attention kernels ask for keys and values of
  // earlier steps before their own wait, and a page copied here holds such keys.
  pdl_wait();
  const int src = pairs[2 * blockIdx.z], dst = pairs[2 * blockIdx.z + 1];
  if (src < 0 || dst < 0 || src >= n_pages || dst >= n_pages || src == dst) return;
  U* base = cache + (long)blockIdx.y * slot_units;
  const U* s = base + (long)src * page_units;
  U* d = base + (long)dst * page_units;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < page_units; i += (long)gridDim.x * blockDim.x) d[i] = s[i];
}

extern "C" int qe_copy_pages(void* cache, int n_slots, int n_pages, long page_bytes, const int* pairs, int n_pairs,
                             cudaStream_t stream) {
  if (n_pairs <= 0 || n_slots <= 0) return 0;
  if (page_bytes <= 0 || n_pages <= 0) QE_REFUSE("copy_pages: a group of %d pages of %ld bytes", n_pages, page_bytes);
  if (n_slots > 65535 || n_pairs > 65535) QE_REFUSE("copy_pages: %d slots x %d pairs are too many for one launch", n_slots, n_pairs);
  const int threads = 256;
  if (page_bytes % 16 == 0 && ((uintptr_t)cache & 15) == 0) {
    const long units = page_bytes / 16;
    const unsigned blocks = (unsigned)((units + threads - 1) / threads < 64 ? (units + threads - 1) / threads : 64);
    qe_launch(copy_pages_kernel<uint4>, dim3(blocks, n_slots, n_pairs), dim3(threads), 0, stream, (uint4*)cache,
              (long)n_pages * units, units, pairs, n_pages);
  } else if (page_bytes % 2 == 0 && ((uintptr_t)cache & 1) == 0) {
    const long units = page_bytes / 2;
    const unsigned blocks = (unsigned)((units + threads - 1) / threads < 64 ? (units + threads - 1) / threads : 64);
    qe_launch(copy_pages_kernel<unsigned short>, dim3(blocks, n_slots, n_pairs), dim3(threads), 0, stream,
              (unsigned short*)cache, (long)n_pages * units, units, pairs, n_pages);
  } else {
    QE_REFUSE("copy_pages: pages of %ld bytes", page_bytes);
  }
  QE_CHECK_LAUNCH("copy_pages");
  return 0;
}
