// Next-token choice on float32 logits: argmax (the reference's only sampler,
// src/engine/executor.py:51-54) and temperature / top-k sampling by inverse CDF with a uniform
// number that the host supplies per row, so that a row's token does not depend on what else is
// in the batch.
#include "common.cuh"
#include <math.h>

#define SM_THREADS 1024

// order-preserving map float -> uint32 (larger float, larger key)
__device__ __forceinline__ unsigned int float_key(float f) {
  const unsigned int u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// (max value, lowest index that holds it) over a row; result in every thread.
__device__ void block_argmax(const float* __restrict__ row, int V, float& best_v, int& best_i,
                             float* sv, int* si) {
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float x = row[i];
    if (x > bv || (x == bv && i < bi)) { bv = x; bi = i; }   // NaN never wins
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    bv = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { sv[32] = bv; si[32] = bi; }
  }
  __syncthreads();
  best_v = sv[32];
  best_i = si[32] == 0x7fffffff ? 0 : si[32];
}

__global__ void __launch_bounds__(SM_THREADS)
argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int V) {
  __shared__ float sv[33];
  __shared__ int si[33];
  pdl_launch_dependents();
  pdl_wait();
  float bv; int bi;
  block_argmax(logits + (size_t)blockIdx.x * V, V, bv, bi, sv, si);
  if (threadIdx.x == 0) out[blockIdx.x] = bi;
}

// A long row shared by the AM_CLUSTER CTAs of a cluster: each takes a contiguous share of the row, the first
// CTA reads the others' results from their shared memory in rank order (lower shares hold lower indices, so
// "larger, or equal and earlier" keeps the lowest index on a tie).  One CTA reads a row of 150 000 logits in
// some tens of microseconds; eight take a few.
#define AM_CLUSTER 8
#define AM_MIN_V 16384     // rows at least this long go to the clusters

__global__ void __launch_bounds__(SM_THREADS)
argmax_cluster_kernel(const float* __restrict__ logits, int* __restrict__ out, int V) {
  __shared__ float sv[33];
  __shared__ int si[33];
  __shared__ float res_v;
  __shared__ int res_i;
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t rank = cluster_cta_rank();
  const int row = blockIdx.y;
  const int share = (V + AM_CLUSTER - 1) / AM_CLUSTER;
  const int lo = min(V, (int)rank * share), hi = min(V, lo + share);
  float bv; int bi;
  block_argmax(logits + (size_t)row * V + lo, hi - lo, bv, bi, sv, si);
  if (threadIdx.x == 0) { res_v = hi > lo ? bv : -INFINITY; res_i = lo + bi; }
  cluster_sync_all();
  if (rank == 0 && threadIdx.x == 0) {
    float best = res_v;
    int at = res_i;
    for (uint32_t r = 1; r < AM_CLUSTER; ++r) {
      const float v = cluster_ld_f32(cluster_map_shared(&res_v, r));
      const int i = __float_as_int(cluster_ld_f32(cluster_map_shared(&res_i, r)));
      if (v > best) { best = v; at = i; }
    }
    out[row] = at;
  }
  cluster_sync_all();     // the others' shared memory stays until it has been read
}

extern "C" int qe_argmax(const float* logits, int* out, int N, int V, cudaStream_t stream) {
  if (N <= 0) return 0;
  if (V <= 0) QE_REFUSE("argmax: empty vocabulary");
  if (V >= AM_MIN_V && N <= 65535) {
    qe_launch_cluster(argmax_cluster_kernel, dim3(AM_CLUSTER, N), dim3(SM_THREADS), 0, stream, AM_CLUSTER, logits, out, V);
    QE_CHECK_LAUNCH("argmax");
    return 0;
  }
  qe_launch(argmax_kernel, dim3(N), dim3(SM_THREADS), 0, stream, logits, out, V);
  QE_CHECK_LAUNCH("argmax");
  return 0;
}

// Row n: temperature[n] <= 0 -> argmax.  Otherwise keep the logits that are >= the top_k[n]-th
// largest value (all of them when top_k is 0 or >= V; ties at the threshold are all kept),
// p_i = exp((logit_i - max) / temperature) in float32, and return the first index whose running
// sum of p (in index order, float64) exceeds uniform[n] * total.
__global__ void __launch_bounds__(SM_THREADS)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ uniform, int* __restrict__ out, int V) {
  __shared__ float sv[33];
  __shared__ int si[33];
  __shared__ unsigned int s_count[33];
  __shared__ double s_part[SM_THREADS];
  __shared__ int s_result;
  __shared__ double s_total;
  pdl_launch_dependents();
  pdl_wait();
  const int n = blockIdx.x;
  const float* row = logits + (size_t)n * V;
  float mx; int arg;
  block_argmax(row, V, mx, arg, sv, si);
  const float temp = temperature[n];
  if (!(temp > 0.f)) { if (threadIdx.x == 0) out[n] = arg; return; }

  // threshold key: the largest key t such that count(key >= t) >= k, by bits from the top
  unsigned int thr = 0u;
  const int k = top_k[n];
  if (k > 0 && k < V) {
    for (int bit = 31; bit >= 0; --bit) {
      const unsigned int cand = thr | (1u << bit);
      unsigned int c = 0;
      for (int i = threadIdx.x; i < V; i += blockDim.x) c += float_key(row[i]) >= cand;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
      __syncthreads();
      if ((threadIdx.x & 31) == 0) s_count[threadIdx.x >> 5] = c;
      __syncthreads();
      if (threadIdx.x == 0) {
        unsigned int tot = 0;
        for (int w = 0; w < (int)((blockDim.x + 31) >> 5); ++w) tot += s_count[w];
        s_count[32] = tot;
      }
      __syncthreads();
      if (s_count[32] >= (unsigned int)k) thr = cand;
    }
  }
  // each thread owns a contiguous range of indices
  const int chunk = (V + blockDim.x - 1) / blockDim.x;
  const int lo = min(V, (int)threadIdx.x * chunk), hi = min(V, lo + chunk);
  double part = 0.0;
  for (int i = lo; i < hi; ++i) {
    const float x = row[i];
    if (float_key(x) >= thr) part += (double)expf((x - mx) / temp);
  }
  s_part[threadIdx.x] = part;
  if (threadIdx.x == 0) s_result = -1;
  __syncthreads();
  if (threadIdx.x == 0) {          // exclusive scan over the threads' partial sums, in order
    double run = 0.0;
    for (int t = 0; t < (int)blockDim.x; ++t) { const double p = s_part[t]; s_part[t] = run; run += p; }
    s_total = run;
  }
  __syncthreads();
  const double total = s_total;
  const double target = (double)uniform[n] * total;
  const double before = s_part[threadIdx.x];
  if (before <= target && target < before + part) {
    double run = before;
    int found = -1;
    for (int i = lo; i < hi; ++i) {
      const float x = row[i];
      if (float_key(x) >= thr) {
        run += (double)expf((x - mx) / temp);
        if (run > target) { found = i; break; }
      }
    }
    if (found >= 0) atomicMax(&s_result, found);
  }
  __syncthreads();
  if (threadIdx.x == 0) out[n] = s_result >= 0 ? s_result : arg;
}

extern "C" int qe_sample(const float* logits, const float* temperature, const int* top_k,
                         const float* uniform, int* out, int N, int V, cudaStream_t stream) {
  if (N <= 0) return 0;
  if (V <= 0) QE_REFUSE("sample: empty vocabulary");
  qe_launch(sample_kernel, dim3(N), dim3(SM_THREADS), 0, stream, logits, temperature, top_k, uniform, out, V);
  QE_CHECK_LAUNCH("sample");
  return 0;
}
