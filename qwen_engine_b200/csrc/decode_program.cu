// A decode step's operations run as a program by one persistent kernel.
//
// A decode step of a small model is a chain of ~170 short, dependent operations (products over a few
// rows, rotary + cache write, attention).  Launched one by one, each costs several microseconds of
// launch, ramp-up and drain even from a CUDA graph, far more than its memory traffic.  Here the host
// records the operations of a step as a list of descriptors, and ONE cooperative kernel (two CTAs
// per SM, all resident) walks the list: every CTA takes its share of an operation's work items, then
// all CTAs meet at a grid barrier (a counter in global memory) before the next operation starts.
// Before it waits at the barrier, a CTA already fetches the first weights of its share of the next
// product: weights are nobody's output.
//
// The operations are the device functions of the stand-alone kernels (gemm_small_m.cuh,
// rope_d128.cuh, attention_flash.cuh); they read what earlier operations wrote with loads that
// bypass L1, since no kernel boundary invalidates L1 between them.
//
// The barrier's wait is bounded: if the counter does not reach its target, the CTA records a code in
// a status word and the kernel returns (every CTA's wait runs out alike).
#include "gemm_small_m.cuh"
#include "rope_d128.cuh"
#include "attention_flash.cuh"

enum { OP_GEMM = 1, OP_ROPE = 2, OP_ATTN = 3 };

// One operation; 192 bytes, written by the host (qwen_engine_b200/ops: struct format "<ii14i2f4q10Q8x").
struct alignas(16) QeOp {
  int type;
  int n_vblocks;          // work items of the size of a CTA
  int i[14];
  float f[2];
  long long l[4];
  const void* p[10];
  long long pad;
};
static_assert(sizeof(QeOp) == 192, "QeOp layout");

#define PROG_THREADS 256
#define PROG_BARRIER_LIMIT (1u << 21)

__device__ int g_program_status = 0;

__device__ __forceinline__ bool grid_barrier(unsigned* counter, unsigned target, int* s_ok) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();                               // this CTA's writes are visible before it is counted
    atomicAdd(counter, 1u);
    int ok = 1;
    unsigned spins = 0;
    for (;;) {
      unsigned v;
      asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(counter) : "memory");
      if (v >= target) break;
      if (++spins > PROG_BARRIER_LIMIT) { ok = 0; atomicCAS(&g_program_status, 0, 1); break; }
    }
    __threadfence();                               // what the other CTAs wrote before they were counted is visible
    *s_ok = ok;
  }
  __syncthreads();
  return *s_ok != 0;
}

// Asks L2 for the weights of work item `vb` of a product (16 rows of K bfloat16 each), one 128-byte
// line per thread and step.  No register holds anything: after the barrier the loads hit L2.
__device__ __forceinline__ void prefetch_weights_l2(const __nv_bfloat16* w, int N, int K, int vb) {
  const int lines_per_row = (K * 2 + 127) / 128;
  const int rows = min(16, N - vb * 16);
  for (int e = threadIdx.x; e < rows * lines_per_row; e += PROG_THREADS) {
    const int r = e / lines_per_row, l = e - r * lines_per_row;
    const char* p = reinterpret_cast<const char*>(w + (size_t)(vb * 16 + r) * K) + (size_t)l * 128;
    asm volatile("prefetch.global.L2 [%0];\n" :: "l"(p));
  }
}

template <int MT>
__device__ __forceinline__ void run_gemm(const QeOp& op, float* red, float* s_rstd) {
  const int M = op.i[0], N = op.i[1], K = op.i[2], kpw = op.i[3], xmode = op.i[4], resid = op.i[5], out_f32 = op.i[6];
  const __nv_bfloat16* x = (const __nv_bfloat16*)op.p[0];
  const __nv_bfloat16* w = (const __nv_bfloat16*)op.p[1];
  void* out = const_cast<void*>(op.p[2]);
  FuseArgs na{};
  na.resid = (const float*)op.p[3];
  na.ssq = (const float*)op.p[4];
  na.norm_w = (const float*)op.p[5];
  na.ssq_out = (float*)const_cast<void*>(op.p[6]);
  na.n_ssq = op.i[7];
  na.ssq_ld = op.i[8];
  na.eps = op.f[0];
  for (int vb = blockIdx.x; vb < op.n_vblocks; vb += gridDim.x) {
    GsmChunk c0, c1;
    gsm_prefetch(w, N, K, kpw, vb, c0, c1);
    if (xmode == X_NORM) {
      if (out_f32) gsm_cta<MT, float, X_NORM, false>(x, w, (float*)out, M, N, K, kpw, na, vb, red, s_rstd, c0, c1);
      else gsm_cta<MT, __nv_bfloat16, X_NORM, false>(x, w, (__nv_bfloat16*)out, M, N, K, kpw, na, vb, red, s_rstd, c0, c1);
    } else if (xmode == X_SILU) {
      if (resid) gsm_cta<MT, float, X_SILU, true>(x, w, (float*)out, M, N, K, kpw, na, vb, red, s_rstd, c0, c1);
      else gsm_cta<MT, __nv_bfloat16, X_SILU, false>(x, w, (__nv_bfloat16*)out, M, N, K, kpw, na, vb, red, s_rstd, c0, c1);
    } else {
      if (resid) gsm_cta<MT, float, X_PLAIN, true>(x, w, (float*)out, M, N, K, kpw, na, vb, red, s_rstd, c0, c1);
      else if (out_f32) gsm_cta<MT, float, X_PLAIN, false>(x, w, (float*)out, M, N, K, kpw, na, vb, red, s_rstd, c0, c1);
      else gsm_cta<MT, __nv_bfloat16, X_PLAIN, false>(x, w, (__nv_bfloat16*)out, M, N, K, kpw, na, vb, red, s_rstd, c0, c1);
    }
    __syncthreads();                               // the reduction buffer is free for the next item
  }
}

__global__ void __launch_bounds__(PROG_THREADS, 2)
decode_program_kernel(const QeOp* __restrict__ ops, int n_ops, unsigned* barrier) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ QeOp s_ops[2];                        // this operation and the next (fetched while this one runs)
  __shared__ float s_rstd[16];
  __shared__ int s_ok;
  float* red = reinterpret_cast<float*>(smem_raw);
  constexpr int OP_INTS = (int)(sizeof(QeOp) / sizeof(int));
  if (threadIdx.x < OP_INTS) reinterpret_cast<int*>(&s_ops[0])[threadIdx.x] = __ldg(reinterpret_cast<const int*>(ops) + threadIdx.x);
  for (int oi = 0; oi < n_ops; ++oi) {
    __syncthreads();                               // s_ops[oi & 1] is complete; s_ops[(oi + 1) & 1] is free
    if (oi + 1 < n_ops && threadIdx.x < OP_INTS)
      reinterpret_cast<int*>(&s_ops[(oi + 1) & 1])[threadIdx.x] = __ldg(reinterpret_cast<const int*>(ops + oi + 1) + threadIdx.x);
    const QeOp& op = s_ops[oi & 1];
    // weights of this CTA's first item of a product: on their way to L2 before the barrier
    if (op.type == OP_GEMM && (int)blockIdx.x < op.n_vblocks)
      prefetch_weights_l2((const __nv_bfloat16*)op.p[1], op.i[1], op.i[2], blockIdx.x);
    if (oi > 0 && !grid_barrier(barrier, (unsigned)oi * gridDim.x, &s_ok)) return;
    if (op.type == OP_GEMM) {
      if (op.i[0] <= 8) run_gemm<1>(op, red, s_rstd);
      else run_gemm<2>(op, red, s_rstd);
    } else if (op.type == OP_ROPE) {
      RopeD128Args ra{(__nv_bfloat16*)const_cast<void*>(op.p[0]), (__nv_bfloat16*)const_cast<void*>(op.p[1]),
                      (const __nv_bfloat16*)op.p[2], (long)op.l[0], (long)op.l[1], (long)op.l[2], (const int*)op.p[3],
                      (const float*)op.p[4], (const float*)op.p[5], op.f[0], (const float*)op.p[6], nullptr,
                      (__nv_bfloat16*)const_cast<void*>(op.p[7]), (const int*)op.p[8],
                      op.i[0], op.i[1], op.i[2], op.i[3], op.i[4]};
      for (int vb = blockIdx.x; vb < op.n_vblocks; vb += gridDim.x)
        rope_d128_item(ra, (long)vb * (PROG_THREADS / 32) + (threadIdx.x >> 5));
    } else if (op.type == OP_ATTN) {
      FaArgs fa{(const __nv_bfloat16*)op.p[0], (long)op.l[0], (const __nv_bfloat16*)op.p[1], (const int*)op.p[2],
                op.i[4], (const int*)op.p[3], (__nv_bfloat16*)const_cast<void*>(op.p[4]),
                (float*)const_cast<void*>(op.p[5]), (float*)const_cast<void*>(op.p[6]), op.i[5],
                (int*)const_cast<void*>(op.p[7]), op.f[0], op.i[6], op.i[2], op.i[1], op.i[3]};
      const int Hkv = op.i[1];
      for (int vb = blockIdx.x; vb < op.n_vblocks; vb += gridDim.x)
        flash_attention_cta<128, 3, 16, true>(fa, vb / Hkv, vb % Hkv, smem_raw);
    }
  }
}

extern "C" int qe_program_op_bytes() { return (int)sizeof(QeOp); }

extern "C" int qe_decode_program_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_program_status, sizeof(int));
  return v;
}

// Shared memory of a CTA: the attention's tiles (16 query rows + 3 stages of 64 keys and values of
// head size 128); the product's reduction buffer (8 warps x 16 x 16 floats) fits in the same bytes.
static constexpr size_t kProgramSmem = (size_t)(16 + 2 * 3 * FA_BN) * (128 + 8) * sizeof(__nv_bfloat16);

// Runs n_ops operations from ops_dev (device memory, QeOp each).  `barrier`: one unsigned in device
// memory for the grid barrier (set to zero here, on the stream).  Returns 0, or 1 with a message.
extern "C" int qe_run_decode_program(const void* ops_dev, int n_ops, unsigned* barrier, cudaStream_t stream) {
  if (n_ops <= 0) return 0;
  static int grid = 0;
  if (grid == 0) {
    cudaError_t e = cudaFuncSetAttribute(decode_program_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kProgramSmem);
    if (e != cudaSuccess) QE_REFUSE("decode_program: shared memory %zu: %s", kProgramSmem, cudaGetErrorString(e));
    int dev = 0, sms = 0, per_sm = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_program_kernel, PROG_THREADS, kProgramSmem);
    if (e != cudaSuccess || per_sm < 1) QE_REFUSE("decode_program: the kernel does not fit an SM (%s)", cudaGetErrorString(e));
    grid = sms * (per_sm > 2 ? 2 : per_sm);
  }
  cudaError_t e = cudaMemsetAsync(barrier, 0, sizeof(unsigned), stream);
  if (e != cudaSuccess) { qe_set_error("decode_program: memset: %s", cudaGetErrorString(e)); return 2; }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(PROG_THREADS);
  cfg.dynamicSmemBytes = kProgramSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;     // all CTAs resident at once: the grid barrier needs it
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, decode_program_kernel, (const QeOp*)ops_dev, n_ops, barrier);
  if (e != cudaSuccess) { qe_set_error("decode_program: launch failed: %s", cudaGetErrorString(e)); return 2; }
  return 0;
}
