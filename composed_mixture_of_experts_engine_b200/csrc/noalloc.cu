// cmoe_moe_plan_noalloc: the MoE row plan with its temporary storage in a fixed device array, for callers that
// cannot allocate GPU memory (see noalloc.h for who they are and for the rules).  No counterpart in the
// reference.
#include "noalloc.h"

#include <cuda_runtime.h>

#include <atomic>

#include "ops.cuh"

namespace {

// The scratch itself.  In host code this name is only a handle for the runtime, not a device address: handing
// `g_plan_scratch` to a kernel would make it touch the wrong memory.  Host code below asks the runtime for the
// real address once per device and passes that.
static __device__ __align__(256) int g_plan_scratch[CMOE_NOALLOC_SCRATCH_WORDS];

constexpr int kMaxDevices = 64;
std::atomic<int*> g_scratch_addr[kMaxDevices];  // zero-initialised; filled on the first call per device

// Device address of the scratch array on the current device (looked up on the first call per device).
cudaError_t scratch_for_current_device(int** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  int* ptr = g_scratch_addr[dev].load(std::memory_order_acquire);
  if (ptr == nullptr) {  // two threads racing here both ask the runtime and both get the same address
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_plan_scratch);
    if (e != cudaSuccess) return e;
    g_scratch_addr[dev].store(ptr, std::memory_order_release);
  }
  *out = ptr;
  return cudaSuccess;
}

}  // namespace

extern "C" size_t cmoe_moe_plan_noalloc_words(long long n_slots, int n_local, int K, int per_k_bins) {
  return cmoe::moe_plan_scratch_words(n_slots, n_local, K, per_k_bins);
}

extern "C" int cmoe_moe_plan_noalloc(const int* topk_idx, long long n_slots, int K, int num_experts, int expert_lo,
                                     int n_local, int per_k_bins, int capacity, long long cap_rows, int* slot_row,
                                     int* row_slot, int* group_offsets, int* tile_group, int* num_m_tiles,
                                     int* counts_kept, int* overflow, void* cuda_stream, int* cuda_error) {
  if (cuda_error) *cuda_error = 0;
  if (topk_idx == nullptr || slot_row == nullptr || row_slot == nullptr || group_offsets == nullptr ||
      tile_group == nullptr || num_m_tiles == nullptr || counts_kept == nullptr || n_slots <= 0 || K <= 0 ||
      n_local <= 0 || num_experts <= 0 || cap_rows <= 0 || cap_rows % 128 != 0 || expert_lo < 0 ||
      static_cast<long long>(expert_lo) + n_local > num_experts || capacity < 0)
    return CMOE_NOALLOC_BAD_ARGUMENT;
  if (cmoe::moe_plan_scratch_words(n_slots, n_local, K, per_k_bins) > CMOE_NOALLOC_SCRATCH_WORDS)
    return CMOE_NOALLOC_TOO_LARGE;

  int* scratch = nullptr;
  cudaError_t e = scratch_for_current_device(&scratch);
  if (e == cudaSuccess) {
    cmoe::MoePlanArgs a;
    a.topk_idx = topk_idx;
    a.n_slots = n_slots;
    a.K = K;
    a.num_experts = num_experts;
    a.expert_lo = expert_lo;
    a.n_local = n_local;
    a.per_k_bins = per_k_bins;
    a.capacity = capacity;
    a.cap_rows = cap_rows;
    a.slot_row = slot_row;
    a.row_slot = row_slot;
    a.group_offsets = group_offsets;
    a.tile_group = tile_group;
    a.num_m_tiles = num_m_tiles;
    a.counts_kept = counts_kept;
    a.overflow = overflow;  // may be null: the kernels then only skip the slots that do not fit
    a.scratch = scratch;  // the histogram pass zeroes the words it uses, so stale contents do no harm
    e = cmoe::launch_moe_plan(a, static_cast<cudaStream_t>(cuda_stream));
  }
  if (e != cudaSuccess) {
    if (cuda_error) *cuda_error = static_cast<int>(e);
    return CMOE_NOALLOC_CUDA_ERROR;
  }
  return CMOE_NOALLOC_OK;
}
