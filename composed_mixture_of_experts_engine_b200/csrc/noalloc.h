// Allocation-free entry point for the MoE row plan.  This entry point has no counterpart in the reference.
//
// Who needs it: code that drives this library from a place where calling cudaMalloc is not an option.
// Examples are a plugin that runs inside another framework's executor under a fixed memory budget, a
// real-time inference loop that must not take the allocator lock (cudaMalloc synchronises the device and can
// block for milliseconds), or a host program that pre-allocated the whole GPU and has nothing left to give.
// Those callers can hand over input and output buffers they already own, but they cannot provide the
// temporary histogram the plan kernels need, and the regular entry point gets that from a torch allocation.
//
// cmoe_moe_plan_noalloc builds the same expert-sorted, 128-row-padded row plan as launch_moe_plan (ops.cuh),
// but its temporary storage is a fixed array that lives inside the library image on every GPU that loads it
// (CMOE_NOALLOC_SCRATCH_WORDS 32-bit words = 4 MiB per device, held until the process exits).  The call performs no
// cudaMalloc, cudaFree or any other allocating call.
//
// Limits and rules:
//   * The problem must fit the fixed array: ceil(n_slots / 256) * bins + 2 * bins <= CMOE_NOALLOC_SCRATCH_WORDS,
//     where bins = n_local * (per_k_bins ? K : 1).  Larger problems are rejected with CMOE_NOALLOC_TOO_LARGE
//     and nothing is launched.
//   * The first call on each device looks up the device address of the array (one cudaGetSymbolAddress, with
//     that device current).  Make that first call outside any stream capture.  Two host threads may make their
//     first calls on a device at the same time: the address is published through an atomic and both arrive at
//     the same value.
//   * The experts planned are [expert_lo, expert_lo + n_local), which must lie inside [0, num_experts);
//     capacity must not be negative.  Anything else is CMOE_NOALLOC_BAD_ARGUMENT.
//   * overflow (optional, may be null): a device counter to which the kernels add the number of (token, k)
//     slots that found no row because cap_rows was too small for the routing.  The caller clears it.
//   * Every call on a device shares the one array, and the array keeps whatever the previous call left in it;
//     the kernels clear the part they use before reading it.  Two calls whose kernels overlap on the same GPU
//     (different streams, or different threads) would race on the array: issue them on one stream, or order
//     them yourself.
//   * All pointers are device pointers of the current device; see MoePlanArgs in ops.cuh for their shapes.
#pragma once
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  CMOE_NOALLOC_OK = 0,
  CMOE_NOALLOC_BAD_ARGUMENT = 1,
  CMOE_NOALLOC_TOO_LARGE = 2,  // the fixed scratch array cannot hold this problem
  CMOE_NOALLOC_CUDA_ERROR = 3, // a CUDA call failed; *cuda_error (if given) holds the cudaError_t
};

#define CMOE_NOALLOC_SCRATCH_WORDS (1u << 20)

// Number of 32-bit scratch words the plan needs (the same formula the regular entry point uses).
size_t cmoe_moe_plan_noalloc_words(long long n_slots, int n_local, int K, int per_k_bins);

int cmoe_moe_plan_noalloc(const int* topk_idx, long long n_slots, int K, int num_experts, int expert_lo, int n_local,
                          int per_k_bins, int capacity, long long cap_rows, int* slot_row, int* row_slot,
                          int* group_offsets, int* tile_group, int* num_m_tiles, int* counts_kept, int* overflow,
                          void* cuda_stream, int* cuda_error);

#ifdef __cplusplus
}
#endif
