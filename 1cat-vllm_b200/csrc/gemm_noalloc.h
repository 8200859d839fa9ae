// Split-K bf16 GEMM for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for embedders of this library whose call sites cannot reach an
// allocator: code running inside another framework's memory-planned region (all device memory handed out up front), real-time loops that forbid
// the latency and the implicit device synchronisation of cudaMalloc/cudaFree, and plain C callers that link the shared object without
// PyTorch (so there is no caching allocator to hand out a workspace). The normal entry point takes the split-K workspace (fp32 partial
// tiles plus one counter per output tile) from the caller; this one keeps that scratch in a fixed array inside the library image.
//
//   out[t, n] = sum_k x[t, k] * w[n, k]      bf16 in, fp32 accumulate, bf16 out; all matrices row-major
//
// Limits and rules
//   * The scratch array is ONECAT_NOALLOC_SCRATCH_BYTES (16 MiB + 8 KiB) of device memory per GPU that loads the library, held until
//     the process exits. A call needs tiles * splits * 128 * token_tile * 4 bytes of it (tiles = ceil(N/128) * ceil(T/token_tile),
//     token_tile = 32/64/128/256 chosen from T) and at most 1024 output tiles; larger problems are rejected with
//     ONECAT_NOALLOC_TOO_LARGE and nothing is launched.
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress with that device current) and raises the
//     kernel's shared-memory limit on that device (both are remembered per device; concurrent first calls from several host threads
//     are serialised inside). Make that first call outside any stream capture.
//   * Every call uses the same array. The tile counters are cleared on the given stream before each launch; partial tiles are always
//     written before they are read. Two calls whose kernels may overlap on the GPU (for example on different streams) race on the
//     scratch: serialise them.
//   * No cudaMalloc, cudaFree or allocating library routine is called, here or in anything this calls.
// Returns 0 on success, a negative ONECAT_NOALLOC_* code otherwise. K must be a multiple of 64; x, w and out 16-byte aligned with
// 16-byte row pitches (ldx, ldw, ldo are in elements).
#pragma once
#include <cuda_runtime.h>

#define ONECAT_NOALLOC_SCRATCH_BYTES ((16u << 20) + 8192u)
#define ONECAT_NOALLOC_BAD_ARGUMENT (-1)
#define ONECAT_NOALLOC_TOO_LARGE (-2)
#define ONECAT_NOALLOC_SETUP_FAILED (-3)
#define ONECAT_NOALLOC_LAUNCH_FAILED (-4)

#ifdef __cplusplus
extern "C" {
#endif

int onecat_gemm_bf16_splitk_noalloc(const void* x, const void* w, void* out, int T, int N, int K, int ldx, int ldw, int ldo, int splits,
                                    cudaStream_t stream);

#ifdef __cplusplus
}
#endif
