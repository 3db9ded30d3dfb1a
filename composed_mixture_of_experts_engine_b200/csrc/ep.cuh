// Host-side interface of the peer-memory (NVLink P2P) kernels used by expert, tensor and data parallelism.
// All "peer tables" hold one device pointer per rank of the group, each pointing at the same symmetric buffer
// on that rank (the rank's own entry points at local memory).  Plain loads/stores only: no TMA on peer memory.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace cmoe {

constexpr int kMaxPeers = 16;

struct PeerTable {
  void* ptr[kMaxPeers];
};

// Device int where the row kernels below record ST_BAD_INDEX when a row plan or routing table names a rank that has
// no buffer in the peer table (the access is skipped).  Set once per process; nullptr switches the record off.
cudaError_t set_peer_status_word(int* status);

// Group barrier over 32-bit flag words in symmetric memory.  Rank `rank` writes `epoch` into word [rank] of
// every peer's flag array, then waits (bounded by timeout_ns) until all `world` words of its own array are
// >= epoch.  A wait that runs out records ST_TIMEOUT_PEER_FLAG in *status and the kernel returns normally.
cudaError_t launch_peer_barrier(const PeerTable& flags, int rank, int world, uint32_t epoch, int* status,
                                unsigned long long timeout_ns, cudaStream_t stream);

// out[r * n_bytes + i] = peers[r][i]: gathers one small buffer (n_bytes, multiple of 16) from every rank.
cudaError_t launch_peer_allgather(const PeerTable& src, int world, long long n_bytes, void* out, cudaStream_t stream);

// Expert-sorted row gather with remote sources.  Row r of `out` is token (slot % slots_per_src) / K of rank
// slot / slots_per_src, where slot = row_slot[r] (padding rows, slot < 0, are zero filled).  slot_scale
// (optional, fp32 per global slot, local memory) multiplies the row.
cudaError_t launch_gather_rows_peer(const PeerTable& src, long long slots_per_src, int K, const int* row_slot,
                                    const float* slot_scale, void* out, long long cap_rows, const int* num_m_tiles,
                                    int H, long long ld_src, long long ld_out, cudaStream_t stream);

// y[t,:] = sum_k w[t,k] * rows[owner][slot_row[owner][slot_base + t*K + k], :], owner = expert_rank[idx[t,k]].
// `rows` and `slot_row` are peer tables of the owners' result rows and row plans; w may be nullptr (weights 1).
// With local_rows != nullptr the rows were already pushed to this rank (row t*K+k of local_rows, by the owners'
// GEMM epilogues) and only the validity of each slot is looked up in the owners' plans.
cudaError_t launch_combine_rows_peer(const PeerTable& rows, const PeerTable& slot_row, const int* idx,
                                     const int* expert_rank, const float* w, void* y, long long n_tokens, int K, int H,
                                     long long slot_base, long long ld_rows, long long ld_y, const void* local_rows,
                                     cudaStream_t stream);

// dw[t,k] = <dy[t,:], rows[owner][row(t,k), :]>  (0 where the slot was dropped)
cudaError_t launch_combine_bwd_w_peer(const PeerTable& rows, const PeerTable& slot_row, const int* idx,
                                      const int* expert_rank, const void* dy, float* dw, long long n_tokens, int K,
                                      int H, long long slot_base, long long ld_rows, long long ld_dy,
                                      const void* local_rows, cudaStream_t stream);

// Gradient reduce-scatter fused with cast and scale: out[i] = scale * sum_r float(grads[r][shard_lo + i]) for
// i < n (fp32 out; grads are bf16 or fp32 flat buffers of every rank).
cudaError_t launch_reduce_scatter_cast(const PeerTable& grads, int world, int grad_is_bf16, long long shard_lo,
                                       long long n, float scale, float* out, cudaStream_t stream);

// out[i, :] = sum_r rows[r][row_map[i], :] for i < n_out (fp32 accumulation, bf16 out): the reduce-scatter of a
// row-parallel linear, each rank pulling and summing the partial results of its own rows.
cudaError_t launch_reduce_rows_peer(const PeerTable& rows, int world, const int* row_map, void* out, long long n_out,
                                    int H, long long ld_rows, long long ld_out, cudaStream_t stream);

// Parameter all-gather by push: copies n bf16 elements at offset shard_lo of the local flat buffer into the same
// offset of every peer's flat buffer.
cudaError_t launch_push_shard(const PeerTable& params, int rank, int world, long long shard_lo, long long n,
                              cudaStream_t stream);

}  // namespace cmoe
