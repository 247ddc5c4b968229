// Allocation-free entry point of the kernel library.
//
// This entry point has no counterpart in the reference engine.
//
// Who it is for: hosts that are not allowed to allocate device memory at the moment they need
// attention — a plugin running inside another runtime's memory pool, a real-time loop that must
// not call into the allocator, a process whose memory budget was fixed at start-up.  Such a
// caller cannot hand the split-KV decode kernel the scratch buffer it needs, and must not have
// the library call cudaMalloc (or any allocating routine) on its behalf.
//
// What it does: the same paged GQA decode attention as xllm_paged_decode_attn, but the partial
// outputs and log-sum-exps of the KV splits are kept in a fixed array that lives inside the
// library image (file scope, `static __device__`).  Every GPU on which the library's kernels are
// loaded holds that array (XLLM_NO_ALLOC_SCRATCH_BYTES, 8 MiB) until the process exits.  The caller
// still passes every input and the output.
//
// When the memory is taken: CUDA loads modules lazily by default, so the array (and the kernel
// image) get their device memory when the library is first USED on a device, not when the shared
// object is opened.  A host that freezes its memory budget, or that must not see driver-side
// allocation later, makes one call of this entry point per device at start-up (or runs with
// CUDA_MODULE_LOADING=EAGER); from then on calls neither allocate nor load anything.
//
// Contract:
//   * nothing is allocated or freed, by this call or by anything it calls;
//   * the scratch needed is batch * nq * splits * (d + 1) * 4 bytes; a request beyond
//     XLLM_NO_ALLOC_SCRATCH_BYTES is refused with XLLM_NO_ALLOC_TOO_LARGE and the reason can be
//     read with xllm_no_alloc_last_error();
//   * the first call on a device looks up the device address of the array (one
//     cudaGetSymbolAddress, with that device current), sets the kernel's shared-memory attribute
//     and triggers the driver's module load.  Make that first call at start-up, outside of any
//     stream capture and before a memory budget is frozen.  It is safe from several host threads
//     at once;
//   * arguments are validated before any CUDA call: head_dim must be 64, 128 or 256, batch > 0;
//   * all calls on a device share the one array, which keeps whatever the previous call left in
//     it.  The kernels overwrite every slot they later read, so nothing has to be cleared between
//     calls — but two calls that overlap in time on the same GPU (different streams) race on it.
//     Order them on one stream or with events.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define XLLM_NO_ALLOC_SCRATCH_BYTES (8u << 20)
#define XLLM_NO_ALLOC_TOO_LARGE (-2)
#define XLLM_NO_ALLOC_SETUP_FAILED (-3)

// Arguments as for xllm_paged_decode_attn minus the workspace.  Returns 0, a cudaError_t value
// (> 0) from the launch, or one of the negative codes above.
int xllm_paged_decode_attn_noalloc(void* out, const void* q, int64_t q_stride, const void* k_cache,
                                   const void* v_cache, const void* block_table, int bt_stride,
                                   const void* seq_lens, int batch, int nq, int nkv, int d, int page_size,
                                   float scale, int splits, void* stream);

// Human-readable reason of the last refusal on the calling thread ("" when there was none).
const char* xllm_no_alloc_last_error(void);

#ifdef __cplusplus
}
#endif
