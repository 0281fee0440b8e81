// An attention entry point for callers that must not allocate.
//
// This entry point has no counterpart in kzw3933/Qwen-Engine (whose attention allocates its
// split buffers with torch.empty on every call); it exists for users of this library.
//
// Who needs it: code that runs where device memory cannot be requested.  Examples are a host
// program that has handed the whole device to its own pool and forbids any further cudaMalloc, a
// real-time loop in which an allocation (which may synchronise the device) would break its
// timing, or a plug-in loaded into a process whose allocator it cannot reach.  Such a caller can
// still supply its inputs and outputs, but it has nowhere to take the scratch memory from that
// flash decoding needs when a long context is cut into parts (each part leaves an unnormalised
// float32 accumulator with its running maximum and sum, which a merge step combines).
//
// qe_flash_attention_noalloc does exactly what qe_flash_attention does, with that scratch taken
// from a fixed array inside the library instead of from pointers the caller passes:
//
//   * The array is QE_NOALLOC_SCRATCH_BYTES (8 MiB) of device memory per GPU, reserved when the
//     library is loaded on a GPU and kept until the process exits.  A call whose parts need more
//     (parts x kv heads x rows per part x (head size + 2) x 4 bytes) is refused with return code
//     1 and a message in qe_last_error(); nothing is launched then.
//   * It calls no cudaMalloc, cudaFree or any other allocating routine.
//   * The first call on a device looks up the array's device address (once per device, with that
//     device current).  Make that first call outside of any stream capture; later calls only
//     launch kernels.
//   * All calls share the one array, and it keeps what the last call left in it.  Nothing in it
//     has to start at zero: every value the merge step reads was written by the same call's
//     attention kernel before.  Two calls that may run on the GPU at the same time (different
//     streams, or different host threads on one device) race on the array; order them.
#pragma once
#include <cuda_runtime.h>

#define QE_NOALLOC_SCRATCH_BYTES (8u << 20)

#ifdef __cplusplus
extern "C" {
#endif

// Arguments as qe_flash_attention, without part_acc and part_ml; n_parts is the number of parts the
// work items name (0 if no context is split) and part_rows the rows each part holds.  The work items
// live in device memory, where this call cannot look: every part index in them must be below n_parts
// and no item may bring more rows than part_rows, or a part is written past the space sized from
// these two numbers (the same holds for the pointers given to qe_flash_attention).
// Returns 0 on success, 1 if refused (sizes, alignment, scratch too small), 2 on a CUDA error.
int qe_flash_attention_noalloc(const void* q, long q_stride, const void* pages, const int* block_tables,
                               int max_blocks, const int* cu_q, const int* ctx_lens, const int* items,
                               int n_items, const int* merge_items, int n_merge, void* out, int n_parts,
                               int part_rows, float scale, int window, int Hq, int Hkv, int D, int page_size,
                               cudaStream_t stream);

#ifdef __cplusplus
}
#endif
