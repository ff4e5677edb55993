// An entry point for callers that may not allocate device memory.
//
// This function has no counterpart in the reference parameter server. It exists
// for hosts that embed the localise step (unique keys, CSC offsets, CSR remap,
// owner offsets) where a device allocation is impossible or forbidden: code that
// runs after the application has handed all free device memory to its own pool,
// real-time loops that must not take the allocator's lock, and plug-ins that are
// given device pointers but no allocator handle. The regular entry point,
// psb_localize, needs a caller-provided scratch buffer; here that scratch lives
// inside the library, in a fixed device array.
//
// Limits and rules:
//   * at most PSB_LOCALIZE_STATIC_MAX_N sorted (key, position) pairs per call;
//     larger inputs are rejected with cudaErrorInvalidValue and nothing is
//     launched;
//   * the scratch array (PSB_LOCALIZE_STATIC_SCRATCH_WORDS 32-bit words, about
//     16 KB) is part of the library image: every GPU that loads the library
//     holds it until the process exits;
//   * the first call on a device looks up the array's device address (no
//     allocation, but a runtime query), so make that first call before starting
//     any stream capture. The address is remembered per device for the life of
//     the process: after a cudaDeviceReset in the same process the remembered
//     address is stale, so do not call this function again in a process that
//     has reset the device;
//   * all calls on one device share the array and it keeps the previous call's
//     contents. Nothing in it has to start at zero (every word that is read is
//     written earlier in the same call), but two calls that overlap on the GPU
//     (different streams, no dependency) race on it: serialise them;
//   * inputs and outputs are still the caller's buffers, exactly as for
//     psb_localize. No cudaMalloc, cudaFree or allocating library call is made.
#pragma once
#include "psb_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

#define PSB_LOCALIZE_STATIC_MAX_N (16u * 1024u * 1024u)
#define PSB_LOCALIZE_STATIC_SCRATCH_WORDS (PSB_LOCALIZE_STATIC_MAX_N / 4096u + 16u)

// Same contract and outputs as psb_localize (see psb_cuda.h), without the
// scratch argument. Returns 0, or minus a cudaError.
int psb_localize_static(const psb_u64* sorted_keys, uint32_t* sorted_pos, uint32_t n,
                        const uint32_t* row_ptr, uint32_t n_rows, uint32_t fixed_z, const float* vals,
                        const psb_u64* bounds, int S, psb_u64* ukeys, uint32_t* seg_off,
                        uint32_t* csr_col, float* csc_val, uint32_t* flagbits, uint32_t* wordbase,
                        uint32_t* n_unique, uint32_t* own_off, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
