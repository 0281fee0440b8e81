// Shared helpers of the sm_100a kernels: element types, error reporting, reductions.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define QE_DTYPE_F32 0
#define QE_DTYPE_BF16 1

// Every entry point returns 0 on success; otherwise qe_last_error() has the text.
extern "C" const char* qe_last_error();
void qe_set_error(const char* fmt, ...);

#define QE_REFUSE(...) do { qe_set_error(__VA_ARGS__); return 1; } while (0)
#define QE_CHECK_LAUNCH(name) do { cudaError_t e_ = cudaGetLastError(); \
    if (e_ != cudaSuccess) { qe_set_error("%s: launch failed: %s", name, cudaGetErrorString(e_)); return 2; } \
  } while (0)

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads, in a fixed order; every thread gets the result.
// `scratch` has 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// ---- programmatic dependent launch --------------------------------------------------------------------
// Kernels of a step form a chain on one stream.  Launched with the attribute below, a kernel may
// start while its predecessor is still running; it must call pdl_wait() before it touches anything
// the predecessor reads or writes, and may do independent work first (a matrix product starts to
// fetch its weights, which no kernel of the step writes).  pdl_launch_dependents() lets the next
// kernel of the chain start early in turn.  Every kernel of this library calls pdl_wait() in all of
// its threads, so a kernel never completes before its predecessor has, and waiting on the
// predecessor alone is enough.  qe_set_pdl(0) turns the attribute off (plain stream order).
#ifndef QE_TIMELINE
#define QE_TL_MARK(kind) do { } while (0)
#define QE_TL_STAMPS(n) do { } while (0)
#define QE_TL_STAMP(i) do { } while (0)
#define QE_TL_FLUSH_STAMPS() do { } while (0)
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
#else
// ---- timeline build (-DQE_TIMELINE; QE_TIMELINE=1 in the environment of the build) ------------------------
// Every kernel of the library passes these two calls, so they double as probes: thread 0 of every CTA
// writes the GPU's global timer when it lets its dependents start (about when the CTA started) and
// when its wait for the predecessor returns (the predecessor has completed).  That is enough to lay a
// step's kernels, their overlaps and the gaps between them on one time axis without a profiler.  An
// event is four 64-bit words: (hash of the source file's name << 32 | line << 16 | kind), (the CTA's
// linear index << 32 | CTAs of the grid), the time in ns, the SM.  Word 0 of the buffer counts the
// events, word 1 is its capacity in events; the events follow from word 4 on.
// Every translation unit keeps its own copy of the buffer's address; qe_timeline_begin sets them all.
static __device__ unsigned long long* qe_tl_buf = nullptr;
__host__ __device__ constexpr unsigned qe_tl_hash(const char* s) {
  unsigned h = 2166136261u;
  const char* base = s;
  for (const char* p = s; *p; ++p) if (*p == '/') base = p + 1;       // the file's name without its folder
  for (const char* p = base; *p; ++p) h = (h ^ (unsigned)*p) * 16777619u;
  return h;
}
__device__ __forceinline__ void qe_tl_event(unsigned file_hash, unsigned line, unsigned kind) {
  if (threadIdx.x != 0 || threadIdx.y != 0 || threadIdx.z != 0 || qe_tl_buf == nullptr) return;
  unsigned long long t;
  unsigned sm;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  asm volatile("mov.u32 %0, %%smid;\n" : "=r"(sm));
  const unsigned long long idx = atomicAdd(qe_tl_buf, 1ull);
  if (idx < qe_tl_buf[1]) {
    const unsigned long long cta = blockIdx.x + (unsigned long long)gridDim.x * (blockIdx.y + (unsigned long long)gridDim.y * blockIdx.z);
    const unsigned long long total = (unsigned long long)gridDim.x * gridDim.y * gridDim.z;
    unsigned long long* e = qe_tl_buf + 4 + 4 * idx;
    e[0] = ((unsigned long long)file_hash << 32) | ((unsigned long long)(line & 0xffffu) << 16) | (kind & 3u);
    e[1] = (cta << 32) | (total & 0xffffffffull);
    e[2] = t;
    e[3] = sm;
  }
}
__device__ __forceinline__ void pdl_wait_at(unsigned file_hash, unsigned line) {
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  qe_tl_event(file_hash, line, 1);
}
__device__ __forceinline__ void pdl_launch_dependents_at(unsigned file_hash, unsigned line) {
  qe_tl_event(file_hash, line, 0);
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
}
#define QE_TL_MARK(kind) qe_tl_event(qe_tl_hash(__FILE__), __LINE__, kind)   // a kernel's own marks: kinds 2 and 3
// Marks inside a loop, where an event (an atomic's round trip to L2) would cost as much as what it measures: a CTA
// keeps up to n times in shared memory (QE_TL_STAMP(i) by whichever thread the kernel chooses: the i-th stamp;
// indices outside 0..n-1 are dropped) and thread 0 writes those that were set as events of kind 2, with the stamp's
// index in the place of the line, when the kernel calls QE_TL_FLUSH_STAMPS at its end (after a barrier).
#define QE_TL_STAMPS(n) __shared__ unsigned long long qe_tl_stamps[n]; constexpr int qe_tl_max_stamps = n; \
  for (int i_ = threadIdx.x; i_ < n; i_ += blockDim.x) qe_tl_stamps[i_] = 0ull      /* (a __syncthreads follows before the first stamp) */
#define QE_TL_STAMP(i) do { if ((i) >= 0 && (i) < qe_tl_max_stamps) { unsigned long long t_; \
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t_)); qe_tl_stamps[i] = t_; } } while (0)
#define QE_TL_FLUSH_STAMPS() do { if (threadIdx.x == 0 && qe_tl_buf != nullptr) for (int i_ = 0; i_ < qe_tl_max_stamps; ++i_) { \
  if (qe_tl_stamps[i_] == 0ull) continue; \
  const unsigned long long idx_ = atomicAdd(qe_tl_buf, 1ull); if (idx_ < qe_tl_buf[1]) { unsigned long long* e_ = qe_tl_buf + 4 + 4 * idx_; \
  e_[0] = ((unsigned long long)qe_tl_hash(__FILE__) << 32) | ((unsigned long long)(i_ & 0xffff) << 16) | 2ull; \
  e_[1] = ((unsigned long long)(blockIdx.x + gridDim.x * (blockIdx.y + (unsigned long long)gridDim.y * blockIdx.z)) << 32) | (((unsigned long long)gridDim.x * gridDim.y * gridDim.z) & 0xffffffffull); \
  e_[2] = qe_tl_stamps[i_]; e_[3] = 0; } } } while (0)
#define pdl_wait() pdl_wait_at(qe_tl_hash(__FILE__), __LINE__)
#define pdl_launch_dependents() pdl_launch_dependents_at(qe_tl_hash(__FILE__), __LINE__)
void qe_tl_register(void (*setter)(unsigned long long*));
static void qe_tl_set_here(unsigned long long* p) { cudaMemcpyToSymbol(qe_tl_buf, &p, sizeof(p)); }
static const int qe_tl_registered = (qe_tl_register(qe_tl_set_here), 0);
#endif

// ---- thread-block clusters ------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_num_ctas() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;\n" : "=r"(r));
  return r;
}
// all threads of all CTAs of the cluster
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// the address, in the cluster's shared window, of CTA `cta`'s copy of this CTA's shared variable
__device__ __forceinline__ uint32_t cluster_map_shared(const void* local, uint32_t cta) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n"
               : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(cta));
  return remote;
}
__device__ __forceinline__ float cluster_ld_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ float4 cluster_ld_f32x4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];\n"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}

extern "C" void qe_set_pdl(int enabled);
int qe_pdl_enabled();

template <typename... KArgs, typename... Args>
static inline cudaError_t qe_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = qe_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same for a kernel whose CTAs form clusters of `cluster_x` (a divisor of grid.x).
template <typename... KArgs, typename... Args>
static inline cudaError_t qe_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                            unsigned cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster_x;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = qe_pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
