// pybind11 registration of the peer-memory kernels (ep.cu).  Peer tables arrive as lists of integer addresses
// (one per rank of the group, from the symmetric-memory rendezvous).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <optional>
#include <vector>

#include "ep.cuh"

namespace {

using torch::Tensor;
using OptTensor = std::optional<Tensor>;

cmoe::PeerTable table(const std::vector<int64_t>& ptrs) {
  TORCH_CHECK(!ptrs.empty() && ptrs.size() <= static_cast<size_t>(cmoe::kMaxPeers), "peer table size");
  cmoe::PeerTable t;
  for (int i = 0; i < cmoe::kMaxPeers; ++i)
    t.ptr[i] = i < static_cast<int>(ptrs.size()) ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return t;
}
void check(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, "cmoe: ", what, " failed: ", cudaGetErrorString(e));
}
cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void peer_barrier(const std::vector<int64_t>& flags, int64_t rank, int64_t epoch, Tensor& status, int64_t timeout_ns) {
  const c10::cuda::CUDAGuard guard(status.device());
  check(cmoe::launch_peer_barrier(table(flags), static_cast<int>(rank), static_cast<int>(flags.size()),
                                  static_cast<uint32_t>(epoch), status.data_ptr<int>(),
                                  static_cast<unsigned long long>(timeout_ns), stream()),
        "peer_barrier");
}

void peer_allgather(const std::vector<int64_t>& src, int64_t n_bytes, Tensor& out) {
  const c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(out.is_contiguous() && out.nbytes() >= static_cast<size_t>(n_bytes) * src.size());
  check(cmoe::launch_peer_allgather(table(src), static_cast<int>(src.size()), n_bytes, out.data_ptr(), stream()),
        "peer_allgather");
}

void gather_rows_peer(const std::vector<int64_t>& src, int64_t slots_per_src, int64_t K, const Tensor& row_slot,
                      const OptTensor& slot_scale, Tensor& out, const OptTensor& num_m_tiles, int64_t ld_src) {
  const c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(out.dim() == 2 && out.stride(1) == 1 && out.scalar_type() == at::kBFloat16);
  check(cmoe::launch_gather_rows_peer(table(src), slots_per_src, static_cast<int>(K), row_slot.data_ptr<int>(),
                                      slot_scale.has_value() ? slot_scale->data_ptr<float>() : nullptr,
                                      out.data_ptr(), out.size(0),
                                      num_m_tiles.has_value() ? num_m_tiles->data_ptr<int>() : nullptr,
                                      static_cast<int>(out.size(1)), ld_src, out.stride(0), stream()),
        "gather_rows_peer");
}

void combine_rows_peer(const std::vector<int64_t>& rows, const std::vector<int64_t>& slot_row, const Tensor& idx,
                       const Tensor& expert_rank, const OptTensor& w, Tensor& y, int64_t K, int64_t slot_base,
                       int64_t ld_rows, const OptTensor& local_rows) {
  const c10::cuda::CUDAGuard guard(y.device());
  TORCH_CHECK(y.dim() == 2 && y.stride(1) == 1 && y.scalar_type() == at::kBFloat16);
  TORCH_CHECK(idx.scalar_type() == at::kInt && idx.is_contiguous() && expert_rank.scalar_type() == at::kInt);
  check(cmoe::launch_combine_rows_peer(table(rows), table(slot_row), idx.data_ptr<int>(), expert_rank.data_ptr<int>(),
                                       w.has_value() ? w->data_ptr<float>() : nullptr, y.data_ptr(), y.size(0),
                                       static_cast<int>(K), static_cast<int>(y.size(1)), slot_base, ld_rows,
                                       y.stride(0), local_rows.has_value() ? local_rows->data_ptr() : nullptr,
                                       stream()),
        "combine_rows_peer");
}

void combine_bwd_w_peer(const std::vector<int64_t>& rows, const std::vector<int64_t>& slot_row, const Tensor& idx,
                        const Tensor& expert_rank, const Tensor& dy, Tensor& dw, int64_t K, int64_t slot_base,
                        int64_t ld_rows, const OptTensor& local_rows) {
  const c10::cuda::CUDAGuard guard(dy.device());
  TORCH_CHECK(dy.dim() == 2 && dy.stride(1) == 1 && dy.scalar_type() == at::kBFloat16);
  check(cmoe::launch_combine_bwd_w_peer(table(rows), table(slot_row), idx.data_ptr<int>(),
                                        expert_rank.data_ptr<int>(), dy.data_ptr(), dw.data_ptr<float>(), dy.size(0),
                                        static_cast<int>(K), static_cast<int>(dy.size(1)), slot_base, ld_rows,
                                        dy.stride(0), local_rows.has_value() ? local_rows->data_ptr() : nullptr,
                                        stream()),
        "combine_bwd_w_peer");
}

void reduce_scatter_cast(const std::vector<int64_t>& grads, bool grad_is_bf16, int64_t shard_lo, int64_t n,
                         double scale, Tensor& out) {
  const c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(out.scalar_type() == at::kFloat && out.is_contiguous() && out.numel() >= n);
  check(cmoe::launch_reduce_scatter_cast(table(grads), static_cast<int>(grads.size()), grad_is_bf16, shard_lo, n,
                                         static_cast<float>(scale), out.data_ptr<float>(), stream()),
        "reduce_scatter_cast");
}

void reduce_rows_peer(const std::vector<int64_t>& rows, const OptTensor& row_map, Tensor& out, int64_t ld_rows) {
  const c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(out.dim() == 2 && out.stride(1) == 1 && out.scalar_type() == at::kBFloat16);
  check(cmoe::launch_reduce_rows_peer(table(rows), static_cast<int>(rows.size()),
                                      row_map.has_value() ? row_map->data_ptr<int>() : nullptr, out.data_ptr(),
                                      out.size(0), static_cast<int>(out.size(1)), ld_rows, out.stride(0), stream()),
        "reduce_rows_peer");
}

void push_shard(const std::vector<int64_t>& params, int64_t rank, int64_t shard_lo, int64_t n, const Tensor& anchor) {
  const c10::cuda::CUDAGuard guard(anchor.device());
  check(cmoe::launch_push_shard(table(params), static_cast<int>(rank), static_cast<int>(params.size()), shard_lo, n,
                                stream()),
        "push_shard");
}



void set_peer_status_word(Tensor& status) {
  const c10::cuda::CUDAGuard guard(status.device());
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 1);
  check(cmoe::set_peer_status_word(status.data_ptr<int>()), "set_peer_status_word");
}

}  // namespace

void register_ep(pybind11::module_& m) {
  m.def("set_peer_status_word", &set_peer_status_word);
  m.def("peer_barrier", &peer_barrier);
  m.def("peer_allgather", &peer_allgather);
  m.def("gather_rows_peer", &gather_rows_peer);
  m.def("combine_rows_peer", &combine_rows_peer);
  m.def("combine_bwd_w_peer", &combine_bwd_w_peer);
  m.def("reduce_scatter_cast", &reduce_scatter_cast);
  m.def("reduce_rows_peer", &reduce_rows_peer);
  m.def("push_shard", &push_shard);
}
