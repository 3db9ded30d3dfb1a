// Host-side interface of the tcgen05 GEMM family (dense, grouped by rows, grouped by K).
// The kernels live in gemm.cu; this header is torch-free so that both the pybind layer and
// plain C callers can use it.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "ep.cuh"

namespace cmoe {

enum GemmMode : int {
  GEMM_DENSE = 0,      // D[M,N] = A[M,K] * B
  GEMM_GROUPED_M = 1,  // rows of A come in 128-row tiles, each tile owned by one group (expert)
  GEMM_GROUPED_K = 2,  // D[g] = A[:, rows of g]^T-style contraction over the rows of group g
};

enum GemmEpilogue : int {
  EPI_STORE = 0,       // D = acc (bf16 or fp32), optional accumulate into D
  EPI_SWIGLU_FWD = 1,  // acc = [gate | up] halves; D = silu(gate) * up, optional copy of gate/up to aux_out
  EPI_SWIGLU_BWD = 2,  // acc = dH; reads gate/up from aux_in, writes [dGate | dUp] to D
};

// One launch description.  All matrices are bf16 unless said otherwise.
//
// Operand A is a 2-D row-major view [a_rows, a_cols] with leading dimension a_ld (elements):
//   a_mn == 0 (K-major):  a_rows index M, a_cols index K.
//   a_mn == 1 (M-major):  a_rows index K, a_cols index M   (A is used transposed).
// Operand B likewise:
//   b_mn == 0 (K-major):  b_rows index N (stacked per group), b_cols index K   (nn.Linear weight [out, in]).
//   b_mn == 1 (N-major):  b_rows index K (stacked per group), b_cols index N.
struct GemmArgs {
  const void* A = nullptr;
  long long a_rows = 0, a_cols = 0, a_ld = 0;
  int a_mn = 0;
  const void* B = nullptr;
  long long b_rows = 0, b_cols = 0, b_ld = 0;
  int b_mn = 0;

  int mode = GEMM_DENSE;
  int epilogue = EPI_STORE;
  int M = 0, N = 0, K = 0;  // dense: problem size.  grouped-M: N, K per group (M unused).
                            // grouped-K: M, N per group output (K comes from group_offsets).
  int groups = 1;
  long long b_group_rows = 0;  // rows of B's 2-D view that belong to one group
  int split_n = 0;             // SWIGLU_FWD: row offset of the "up" half inside one group's B rows

  const int* tile_group = nullptr;     // grouped-M: group of each 128-row tile (-1: skip), device memory
  const int* num_m_tiles = nullptr;    // grouped-M: number of live 128-row tiles, device scalar
  int max_m_tiles = 0;                 // grouped-M: upper bound on *num_m_tiles (sizes the grid)
  const int* group_offsets = nullptr;  // grouped-K: [groups+1] row offsets (multiples of 64), device memory

  void* D = nullptr;
  long long ldd = 0;
  long long d_group_stride = 0;  // grouped-K: elements between consecutive groups' outputs
  int d_fp32 = 0;
  int accumulate = 0;

  const void* aux_in = nullptr;  // SWIGLU_BWD: [rows, 2N] gate|up saved by the forward
  long long ld_aux_in = 0;
  void* aux_out = nullptr;  // SWIGLU_FWD: optional [rows, 2N] gate|up
  long long ld_aux_out = 0;

  // Optional readiness flags (fused dispatch): before the first load of a 128-row tile the
  // producer waits until ready_flags[tile_group * ready_stride + s] >= ready_target for all
  // s < ready_count.  nullptr disables the wait.
  const uint32_t* ready_flags = nullptr;
  int ready_stride = 0;
  int ready_count = 0;
  uint32_t ready_target = 0;

  // Fused expert-parallel dispatch (grouped-M only).  When pull_row_slot is set, four extra warps per CTA fill
  // the rows of A themselves before the tiles that need them run: row r of A is the token row
  // (slot % pull_slots_per_src) / pull_K of rank slot / pull_slots_per_src (slot = pull_row_slot[r]), read with
  // plain loads from that rank's buffer in pull_src (peer memory over NVLink, or local), times pull_slot_scale[slot]
  // if given; padding rows are zero filled.  tile_ready[4 m + q] (uint32, this GPU's memory, kPullFlagsPerTile words
  // per tile) is set to pull_epoch when quarter q of 128-row tile m is complete, and the TMA producer of every
  // tile waits (bounded) for its four flags.  The transfer of later tiles overlaps the MMAs of earlier ones.
  const int* pull_row_slot = nullptr;
  PeerTable pull_src = {};
  long long pull_slots_per_src = 0;
  int pull_K = 1;
  const float* pull_slot_scale = nullptr;
  long long pull_ld_src = 0;
  uint32_t* tile_ready = nullptr;
  uint32_t pull_epoch = 0;
  // Optional device timestamps of a launch with the fused row pull (4 x uint64 of `%globaltimer` nanoseconds, the
  // caller presets {max, 0, max, 0}): [0] first row pulled, [1] last tile of rows complete, [2] first MMA issued,
  // [3] last accumulator committed; min / max over all CTAs.  Telemetry derives from them how much of the transfer
  // ran under the tensor-core work.  nullptr: nothing is recorded.
  unsigned long long* pull_stamps = nullptr;

  // Fused scatter (EPI_STORE, bf16, no accumulate).  When scatter_row_slot is set, output row r is not written to D
  // but to the buffer of rank  slot / scatter_slots_per_rank  in scatter_out, at row  slot % scatter_slots_per_rank
  // (slot = scatter_row_slot[r], leading dimension scatter_ld), with stores from the epilogue's staging area (peer
  // memory over NVLink, or local); rows with a negative slot are skipped.  This is the combine push of expert
  // parallelism (the slot of a row is the (token, k) pair it came from) and the scatter half of a reduce-scatter.
  const int* scatter_row_slot = nullptr;
  long long scatter_slots_per_rank = 0;
  PeerTable scatter_out = {};
  long long scatter_ld = 0;

  int* status = nullptr;  // device int, set to a StatusCode when a wait ran out
  unsigned long long timeout_ns = 0;  // 0: default
  int num_sms = 0;                    // 0: query the current device
};

// Enqueues the GEMM on `stream`.  Returns cudaSuccess or the first CUDA error met while
// encoding tensor maps or launching.
cudaError_t launch_gemm(const GemmArgs& args, cudaStream_t stream);

// Two-SM variant (clusters of two CTAs, `tcgen05.mma.cta_group::2`, 256 x 256 tiles) for dense GEMMs and grouped-K
// weight-gradient GEMMs with plain results; `gemm_2cta_supported` says whether a launch description qualifies.
bool gemm_2cta_supported(const GemmArgs& args);
constexpr int kPullFlagsPerTile = 4;  // words of GemmArgs::tile_ready per 128-row tile
cudaError_t launch_gemm_2cta(const GemmArgs& args, cudaStream_t stream);

}  // namespace cmoe
