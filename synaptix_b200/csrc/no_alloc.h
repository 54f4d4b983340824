// sx_attn_decode_noalloc: split-KV decode attention that allocates nothing.
//
// This entry point has no counterpart in the reference project; it is an addition of this library.
//
// Who it is for.  sx_attn_decode needs float32 scratch for the partial results of its splits, and
// its caller has to bring that memory.  Some callers cannot: a host program that drives these
// kernels through the C symbols without torch, in a process where another component (an inference
// server's memory pool, say) has already taken the whole device, so that a cudaMalloc of its own
// fails or eats into someone else's budget; or a latency-bound loop that must not call cudaMalloc or
// cudaFree because both synchronise the device.  For them the scratch lives inside the library: a
// file-scope device array of SX_NOALLOC_SCRATCH_BYTES (4 MiB) that every GPU which loads the
// library holds until the process exits.
//
// Contract.
//   * Inputs and outputs are the caller's, exactly as for sx_attn_decode (q [S, nh, hd] bfloat16,
//     paged K/V, out [S, nh*hd] bfloat16, seq_lens and block_table int32 on the device).
//   * S * nh * n_splits * (hd + 2) * 4 bytes must fit into SX_NOALLOC_SCRATCH_BYTES; a larger
//     problem is refused with SX_ERR_NOALLOC_TOO_LARGE (10005) and nothing is launched.  With
//     n_splits == 1 no scratch is used and any size that sx_attn_decode takes is taken.  More than
//     4,096 splits are refused (10002) by both entry points, also before anything is launched.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress) with
//     that device current and remembers it; make that first call outside any stream capture.
//     Host threads may make their first calls at the same time.
//     No call allocates or frees memory, on the device or through any library.
//   * All calls share the one array and it keeps what the last call left.  Nothing in it has to
//     start at zero: every slot a merge reads is written by the split kernel of the same call.
//     Two calls whose kernels may run at the same time on one GPU (different streams) race on the
//     array; keep them on one stream or order them with events.
#pragma once
#include <cuda_runtime.h>

#define SX_NOALLOC_SCRATCH_BYTES (4u << 20)
#define SX_ERR_NOALLOC_TOO_LARGE 10005

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0, an SX_ERR_* code of the argument checks, or the cudaError_t of set-up or launch.
int sx_attn_decode_noalloc(const void* q, const void* k_pages, const void* v_pages, void* out,
                           const int* seq_lens, const int* block_table, int maxp, int S, int nh, int nkv, int hd,
                           float scale, int window, int n_splits, cudaStream_t stream);

// Bytes of the built-in scratch array (SX_NOALLOC_SCRATCH_BYTES), for callers that size their splits by it.
unsigned long long sx_attn_decode_noalloc_capacity(void);

#ifdef __cplusplus
}
#endif
