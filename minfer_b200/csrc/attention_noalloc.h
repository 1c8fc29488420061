// Attention over the paged cache for callers that must not allocate device memory.
//
// This entry point has no counterpart in yusiwen/minfer; it exists for users of this
// library's C interface.
//
// Who needs it: code that runs where cudaMalloc is off limits.  Examples are a real-time
// loop that may not block on the allocator, a plug-in that lives inside a host application
// which owns all device memory and hands out none, and a process that has pinned its memory
// budget and treats any later allocation as a fault.  mf_attention_paged needs float32 scratch to merge the key chunks
// of a long sequence, and its callers normally allocate that scratch themselves; here the
// scratch is a fixed array that is part of the loaded library image instead.
//
// What it costs and what its limits are:
//   * The array holds MF_ATTENTION_NOALLOC_FLOATS float32 values (16 MiB).  Every GPU on
//     which the library is loaded keeps that much memory until the process exits.
//   * A call needs rows * n_heads * n_chunks * (head_dim + 2) floats.  A call that needs more
//     is refused with MF_ERR_SCRATCH_LIMIT (2005) before anything is launched.
//   * The first call on each device does the set-up for that device, with that device
//     current: it looks up the array's device address (cudaGetSymbolAddress), opens the
//     shared memory of every kernel variant a later call may pick (cudaFuncSetAttribute) and
//     reads the environment.  Make that first call before any stream capture begins.  Two host
//     threads that make their first calls on a device at the same moment both do the set-up
//     and store the same values, which is harmless.
//   * It calls no cudaMalloc, no cudaFree and no routine of an allocating library.
//   * All calls share the one array, and the array keeps what the last call left in it.
//     Nothing in it has to start at zero: the kernels write every entry they later read.
//     Two calls that overlap on the GPU (different streams, or graphs replayed
//     concurrently) would write the same entries and race; run them one after another.
//
// Arguments and results are those of mf_attention_paged without `partial`; inputs and
// outputs are still the caller's own buffers.
#pragma once
#include <cuda_runtime.h>

#define MF_ATTENTION_NOALLOC_FLOATS (4u << 20)
#define MF_ERR_SCRATCH_LIMIT 2005

#ifdef __cplusplus
extern "C" {
#endif

int mf_attention_paged_noalloc(const void* q, const void* k_cache, const void* v_cache,
                               const int* row_seq, const int* row_pos, const int* page_table,
                               int table_stride, int ring, void* out, int rows, int n_heads,
                               int n_kv, int hd, int window, int chunk, int n_chunks, float scale,
                               int dtype, cudaStream_t stream);

// The number of float32 values the fixed scratch array holds.
long long mf_attention_noalloc_capacity(void);

#ifdef __cplusplus
}
#endif
