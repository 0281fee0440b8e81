// Flash attention over the paged cache in bfloat16: the stand-alone kernels and their launchers.
// The device code is in attention_flash.cuh.
#include "attention_flash.cuh"

template <int D, int STAGES, int QROWS>
__global__ void __launch_bounds__(2 * FA_THREADS, (D <= 128 ? 2 : 1))
flash_attention_kernel(FaArgs args) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  flash_attention_cta<D, STAGES, QROWS, false>(args, blockIdx.x, blockIdx.y, smem_raw);
}

// out = sum_s 2^(m_s - m) acc_s / sum_s 2^(m_s - m) l_s  (reference attn.py:520-594), float32.
template <int D>
__global__ void flash_merge_kernel(const int* __restrict__ merge_items, const int* __restrict__ cu_q,
                                   const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                   int part_rows, __nv_bfloat16* __restrict__ out, int Hq, int Hkv) {
  pdl_launch_dependents();
  pdl_wait();
  const int* it = merge_items + 4 * blockIdx.x;
  const int req = it[0], q0 = it[1], first = it[2], n = it[3];
  const int hkv = blockIdx.y;
  const int G = Hq / Hkv;
  const int row0 = cu_q[req];
  const int q_len = cu_q[req + 1] - row0;
  const int nrows = min(FA_BM / G, q_len - q0) * G;
  for (int r = threadIdx.y; r < nrows; r += blockDim.y) {
    float m = -INFINITY;
    for (int s = 0; s < n; ++s) m = fmaxf(m, part_ml[2 * ((((size_t)first + s) * Hkv + hkv) * part_rows + r)]);
    if (m == -INFINITY) m = 0.f;          // every part of the row empty: weights 0, not exp2(-inf + inf)
    float l = 0.f;
    for (int s = 0; s < n; ++s) {
      const size_t slot = (((size_t)first + s) * Hkv + hkv) * part_rows + r;
      l += exp2f(part_ml[2 * slot] - m) * part_ml[2 * slot + 1];
    }
    const int ti = r / G, hg = r - ti * G;
    __nv_bfloat16* dst = out + (size_t)(row0 + q0 + ti) * ((size_t)Hq * D) + (size_t)(hkv * G + hg) * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      float acc = 0.f;
      for (int s = 0; s < n; ++s) {
        const size_t slot = (((size_t)first + s) * Hkv + hkv) * part_rows + r;
        acc += exp2f(part_ml[2 * slot] - m) * part_acc[slot * D + d];
      }
      dst[d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    }
  }
}

template <int D, int STAGES, int QROWS>
static int launch_flash(const void* q, long q_stride, const void* pages, const int* block_tables, int max_blocks,
                        const int* cu_q, const int* ctx_lens, const int* items, int n_items,
                        const int* merge_items, int n_merge, void* out, float* part_acc, float* part_ml,
                        int part_rows, int* counters, float scale, int window, int Hq, int Hkv, int page_size,
                        cudaStream_t stream) {
  constexpr int LD = D + 8;
  const size_t smem = (size_t)(QROWS + 2 * STAGES * FA_BN) * LD * sizeof(__nv_bfloat16);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(flash_attention_kernel<D, STAGES, QROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) QE_REFUSE("flash_attention: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(n_items, Hkv);
  FaArgs fa{(const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)pages, block_tables, max_blocks, items,
            (__nv_bfloat16*)out, part_acc, part_ml, part_rows, counters, scale_log2, window, Hq, Hkv, page_size};
  qe_launch(flash_attention_kernel<D, STAGES, QROWS>, grid, dim3(2 * FA_THREADS), smem, stream, fa);
  QE_CHECK_LAUNCH("flash_attention");
  if (n_merge > 0 && counters == nullptr) {
    dim3 mgrid(n_merge, Hkv), mblock(32, 4);
    qe_launch(flash_merge_kernel<D>, mgrid, mblock, 0, stream, merge_items, cu_q, (const float*)part_acc,
              (const float*)part_ml, part_rows, (__nv_bfloat16*)out, Hq, Hkv);
    QE_CHECK_LAUNCH("flash_merge");
  }
  return 0;
}

// 0 if no bounded wait of the attention kernel's tile pipeline ever ran out (1: a slot never came
// free, 2: a tile never landed).  Synchronises the device.
extern "C" int qe_flash_attention_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_fa_status, sizeof(int));
  return v;
}
extern "C" void qe_flash_attention_clear_status() {
  int v = 0;
  cudaMemcpyToSymbol(g_fa_status, &v, sizeof(int));
}

extern "C" int qe_flash_attention_supported(int Hq, int Hkv, int D) {
  return (D % 16 == 0 && D >= 16 && D <= 256 && Hkv >= 1 && Hq % Hkv == 0 && Hq / Hkv <= FA_BM && Hkv <= 65535) ? 1 : 0;
}

// The entry point with a counter array (see the kernel): parts are combined by the CTA that finishes
// last, without a merge kernel.  counters: n_parts * Hkv ints, zero before the first use.
extern "C" int qe_flash_attention_fused_merge(const void* q, long q_stride, const void* pages, const int* block_tables,
                                              int max_blocks, const int* cu_q, const int* ctx_lens, const int* items,
                                              int n_items, const int* merge_items, int n_merge, void* out,
                                              float* part_acc, float* part_ml, int part_rows, int* counters,
                                              int small_tiles, float scale, int window, int Hq, int Hkv, int D,
                                              int page_size, cudaStream_t stream);

extern "C" int qe_flash_attention(const void* q, long q_stride, const void* pages, const int* block_tables,
                                  int max_blocks, const int* cu_q, const int* ctx_lens, const int* items,
                                  int n_items, const int* merge_items, int n_merge, void* out, float* part_acc,
                                  float* part_ml, int part_rows, float scale, int window, int Hq, int Hkv, int D,
                                  int page_size, cudaStream_t stream) {
  return qe_flash_attention_fused_merge(q, q_stride, pages, block_tables, max_blocks, cu_q, ctx_lens, items, n_items,
                                        merge_items, n_merge, out, part_acc, part_ml, part_rows, nullptr, 0, scale,
                                        window, Hq, Hkv, D, page_size, stream);
}

extern "C" int qe_flash_attention_fused_merge(const void* q, long q_stride, const void* pages, const int* block_tables,
                                              int max_blocks, const int* cu_q, const int* ctx_lens, const int* items,
                                              int n_items, const int* merge_items, int n_merge, void* out,
                                              float* part_acc, float* part_ml, int part_rows, int* counters,
                                              int small_tiles, float scale, int window, int Hq, int Hkv, int D,
                                              int page_size, cudaStream_t stream) {
  // small_tiles: every item has at most 16 rows (a decode step): 16 query rows are staged and the key
  // tiles run through a deeper pipeline
  if (n_items <= 0) return 0;
  if (!qe_flash_attention_supported(Hq, Hkv, D))
    QE_REFUSE("flash_attention: heads %d/%d with head_dim %d are not supported", Hq, Hkv, D);
  if (((uintptr_t)q | (uintptr_t)pages) & 15 || (q_stride % 8)) QE_REFUSE("flash_attention: operands must be 16-byte aligned");
#define FA_ARGS q, q_stride, pages, block_tables, max_blocks, cu_q, ctx_lens, items, n_items, merge_items, n_merge, out, \
      part_acc, part_ml, part_rows, counters, scale, window, Hq, Hkv, page_size, stream
#define FA_CASE(DD) case DD: return small_tiles ? launch_flash<DD, 3, 16>(FA_ARGS) : launch_flash<DD, 2, FA_BM>(FA_ARGS);
  switch (D) {
    FA_CASE(16) FA_CASE(32) FA_CASE(48) FA_CASE(64) FA_CASE(80) FA_CASE(96) FA_CASE(112) FA_CASE(128)
    FA_CASE(144) FA_CASE(160) FA_CASE(176) FA_CASE(192) FA_CASE(208) FA_CASE(224) FA_CASE(240) FA_CASE(256)
  }
#undef FA_CASE
#undef FA_ARGS
  QE_REFUSE("flash_attention: head_dim %d is not supported", D);
}

// ---------------------------------------------------------------------------------------------------
// The same attention for callers that must not allocate (see no_alloc.h): the parts of split
// contexts go to a fixed array of this library instead of to memory the caller provides.
// ---------------------------------------------------------------------------------------------------
#include "no_alloc.h"

// Device memory of the library itself: present on every GPU that loads it, until the process ends.
static __device__ __align__(256) unsigned char g_noalloc_scratch[QE_NOALLOC_SCRATCH_BYTES];

#define QE_NOALLOC_MAX_DEVICES 64
// In host code the name g_noalloc_scratch is only a handle for the runtime, not an address a kernel
// can use; the device address is asked for once per device and kept here.
static float* g_noalloc_scratch_addr[QE_NOALLOC_MAX_DEVICES] = {nullptr};

extern "C" int qe_flash_attention_noalloc(const void* q, long q_stride, const void* pages, const int* block_tables,
                                          int max_blocks, const int* cu_q, const int* ctx_lens, const int* items,
                                          int n_items, const int* merge_items, int n_merge, void* out, int n_parts,
                                          int part_rows, float scale, int window, int Hq, int Hkv, int D,
                                          int page_size, cudaStream_t stream) {
  if (n_items <= 0) return 0;
  if (n_parts < 0 || part_rows < 1) QE_REFUSE("flash_attention_noalloc: bad part counts (%d parts of %d rows)", n_parts, part_rows);
  if (!qe_flash_attention_supported(Hq, Hkv, D))
    QE_REFUSE("flash_attention_noalloc: heads %d/%d with head_dim %d are not supported", Hq, Hkv, D);
  // accumulators [slots][D] first, then (max, sum) pairs [slots][2], all float32
  const size_t slots = (size_t)n_parts * Hkv * part_rows;
  const size_t acc_bytes = (slots * D * sizeof(float) + 255) / 256 * 256;
  const size_t need = acc_bytes + slots * 2 * sizeof(float);
  if (need > QE_NOALLOC_SCRATCH_BYTES)
    QE_REFUSE("flash_attention_noalloc: %d parts x %d kv heads x %d rows of head size %d need %zu bytes of scratch; "
              "the library's fixed array holds %u", n_parts, Hkv, part_rows, D, need, QE_NOALLOC_SCRATCH_BYTES);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { qe_set_error("flash_attention_noalloc: cudaGetDevice: %s", cudaGetErrorString(e)); return 2; }
  if (dev < 0 || dev >= QE_NOALLOC_MAX_DEVICES) QE_REFUSE("flash_attention_noalloc: device %d is outside 0..%d", dev, QE_NOALLOC_MAX_DEVICES - 1);
  if (g_noalloc_scratch_addr[dev] == nullptr) {
    // set-up, once per device, with that device current: the device address of the array
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      qe_set_error("flash_attention_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      return 2;
    }
    g_noalloc_scratch_addr[dev] = static_cast<float*>(p);
  }
  float* part_acc = g_noalloc_scratch_addr[dev];
  float* part_ml = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(part_acc) + acc_bytes);
  return qe_flash_attention(q, q_stride, pages, block_tables, max_blocks, cu_q, ctx_lens, items, n_items, merge_items,
                            n_merge, out, part_acc, part_ml, part_rows, scale, window, Hq, Hkv, D, page_size, stream);
}
