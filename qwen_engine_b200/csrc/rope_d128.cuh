// The fused per-head norm + rotary encoding + cache write for head size 128 in bfloat16 as a device
// function (see elementwise.cu), as a header so that another kernel can do the same for its own rows.
#pragma once
#include "common.cuh"

// The common case in bfloat16, head size 128 with all of it rotated (or none): a lane holds 4
// consecutive elements, its rotation partner (d +- 64) is held by lane +- 16, no shared memory.
struct RopeD128Args {
  __nv_bfloat16* q; __nv_bfloat16* k; const __nv_bfloat16* v;
  long q_stride, k_stride, v_stride;
  const int* positions; const float* qw; const float* kw; float eps; const float* inv_freq;
  const float2* cos_sin;            // optional [T, 64] (cos, sin) of position * inv_freq, made once per step
  __nv_bfloat16* pages; const int* slot_mapping;
  int T_tokens, Hq, Hkv, page_size, write_kv;
};

// One (token, head) by the calling warp.  In two halves, so that
// a warp can have the loads of several items in flight before it works on the first: the load of the
// lane's 4 elements, and the rest.  Loads of q, k, v bypass L1 (they are another kernel's or an
// earlier phase's output).
__device__ __forceinline__ uint2 rope_d128_load(const RopeD128Args& A, int t, int head) {
  constexpr int D = 128;
  const int lane = threadIdx.x & 31;
  if (t >= A.T_tokens) return make_uint2(0u, 0u);
  const __nv_bfloat16* src;
  if (head < A.Hq) src = A.q + (size_t)t * A.q_stride + (size_t)head * D;
  else if (head < A.Hq + A.Hkv) src = A.k + (size_t)t * A.k_stride + (size_t)(head - A.Hq) * D;
  else {
    if (!A.write_kv) return make_uint2(0u, 0u);
    src = A.v + (size_t)t * A.v_stride + (size_t)(head - A.Hq - A.Hkv) * D;
  }
  return __ldcg(reinterpret_cast<const uint2*>(src + 4 * lane));
}

// What a lane needs besides the head's elements, none of it written by a kernel of the step (positions and
// slots come with the step's host copy, the rest are weights): a kernel may fetch it before it waits for
// its predecessor.  Angles only where the step has no table of them.
struct RopeD128Pre {
  float cs[4], sn[4];
  float4 wv;
  int slot;
};
__device__ __forceinline__ void rope_d128_prepare(const RopeD128Args& A, int t, int head, RopeD128Pre& P) {
  const int lane = threadIdx.x & 31;
  P.slot = 0;
  P.wv = make_float4(1.f, 1.f, 1.f, 1.f);
#pragma unroll
  for (int i = 0; i < 4; ++i) { P.cs[i] = 1.f; P.sn[i] = 0.f; }
  if (t >= A.T_tokens) return;
  if (A.write_kv && head >= A.Hq) P.slot = __ldg(A.slot_mapping + t);
  if (head >= A.Hq + A.Hkv) return;
  const float* w = head < A.Hq ? A.qw : A.kw;
  if (w) P.wv = __ldg(reinterpret_cast<const float4*>(w + 4 * lane));
  if (A.inv_freq && !A.cos_sin) {
    const float pos = (float)__ldg(A.positions + t);
#pragma unroll
    for (int i = 0; i < 4; ++i) sincosf(pos * __ldg(A.inv_freq + ((4 * lane + i) & 63)), &P.sn[i], &P.cs[i]);
  }
}

__device__ __forceinline__ void rope_d128_finish(const RopeD128Args& A, int t, int head, const uint2 raw,
                                                 const RopeD128Pre* pre = nullptr) {
  constexpr int D = 128;
  __nv_bfloat16* q = A.q; __nv_bfloat16* k = A.k;
  const long q_stride = A.q_stride, k_stride = A.k_stride;
  const int* positions = A.positions; const float* qw = A.qw; const float* kw = A.kw; const float eps = A.eps;
  const float* inv_freq = A.inv_freq; __nv_bfloat16* pages = A.pages; const int* slot_mapping = A.slot_mapping;
  const int Hq = A.Hq, Hkv = A.Hkv, page_size = A.page_size, write_kv = A.write_kv;
  const int lane = threadIdx.x & 31;
  if (t >= A.T_tokens) return;
  if (head >= Hq + Hkv) {           // a value head: copy into the cache
    if (!write_kv) return;
    const int h = head - Hq - Hkv;
    const int slot = pre ? pre->slot : slot_mapping[t];
    // slot = page * page_size + off: the row of (page, V, h, off) is slot + (page * (2 Hkv - 1) + Hkv + h) * page_size
    const int page = (page_size & (page_size - 1)) == 0 ? slot >> (__ffs(page_size) - 1) : slot / page_size;
    *reinterpret_cast<uint2*>(pages + ((size_t)slot + ((size_t)page * (2 * Hkv - 1) + Hkv + h) * page_size) * D + 4 * lane) = raw;
    return;
  }
  const bool is_q = head < Hq;
  const int h = is_q ? head : head - Hq;
  __nv_bfloat16* x = (is_q ? q + (size_t)t * q_stride : k + (size_t)t * k_stride) + (size_t)h * D + 4 * lane;
  const float* w = is_q ? qw : kw;
  float f[4];
  {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  }
  if (w) {
    const float ss = warp_sum(f[0] * f[0] + f[1] * f[1] + f[2] * f[2] + f[3] * f[3]);
    const float rstd = rsqrtf(ss / (float)D + eps);
    const float4 wv = pre ? pre->wv : *reinterpret_cast<const float4*>(w + 4 * lane);
    f[0] = f[0] * rstd * wv.x; f[1] = f[1] * rstd * wv.y; f[2] = f[2] * rstd * wv.z; f[3] = f[3] * rstd * wv.w;
  }
  if (inv_freq) {
    float cs[4], sn[4];
    if (A.cos_sin) {
      // the lane's four (cos, sin) pairs lie side by side in the step's table: two 16-byte loads
      const float4* tp = reinterpret_cast<const float4*>(A.cos_sin + (size_t)t * 64 + ((4 * lane) & 63));
      const float4 t01 = __ldg(tp), t23 = __ldg(tp + 1);
      cs[0] = t01.x; sn[0] = t01.y; cs[1] = t01.z; sn[1] = t01.w;
      cs[2] = t23.x; sn[2] = t23.y; cs[3] = t23.z; sn[3] = t23.w;
    } else if (pre) {
#pragma unroll
      for (int i = 0; i < 4; ++i) { cs[i] = pre->cs[i]; sn[i] = pre->sn[i]; }
    } else {
      const float pos = (float)positions[t];
#pragma unroll
      for (int i = 0; i < 4; ++i) sincosf(pos * inv_freq[(4 * lane + i) & 63], &sn[i], &cs[i]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float partner = __shfl_xor_sync(0xffffffffu, f[i], 16);
      f[i] = lane < 16 ? cs[i] * f[i] - sn[i] * partner : sn[i] * partner + cs[i] * f[i];
    }
  }
  uint2 res;
  {
    __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
    res.x = *reinterpret_cast<uint32_t*>(&a);
    res.y = *reinterpret_cast<uint32_t*>(&b);
  }
  *reinterpret_cast<uint2*>(x) = res;
  if (!is_q && write_kv) {
    const int slot = pre ? pre->slot : slot_mapping[t];
    const int page = (page_size & (page_size - 1)) == 0 ? slot >> (__ffs(page_size) - 1) : slot / page_size;
    *reinterpret_cast<uint2*>(pages + ((size_t)slot + ((size_t)page * (2 * Hkv - 1) + h) * page_size) * D + 4 * lane) = res;
  }
}


// `item` = token * (Hq + 2 Hkv) + head
__device__ __forceinline__ void rope_d128_item(const RopeD128Args& A, long item) {
  const int heads_total = A.Hq + 2 * A.Hkv;
  if (item >= (long)A.T_tokens * heads_total) return;
  const int t = (int)(item / heads_total), head = (int)(item - (long)t * heads_total);
  rope_d128_finish(A, t, head, rope_d128_load(A, t, head));
}
