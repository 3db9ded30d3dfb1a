// pybind11 layer: torch tensors in, raw-pointer launchers of gemm.cu / router.cu / ops.cu / attention.cu /
// ep.cu out.  All launches go to the current CUDA stream of the calling thread.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstdlib>

#include <algorithm>
#include <optional>
#include <string>
#include <vector>

#include "gemm.cuh"
#include "ops.cuh"
#include "router.cuh"

namespace {

using torch::Tensor;
using OptTensor = std::optional<Tensor>;

void check_cuda(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, "cmoe: ", what, " failed: ", cudaGetErrorString(e));
}
cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_bf16_2d(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16, name, " must be a CUDA bf16 tensor");
  TORCH_CHECK(t.dim() == 2 && t.stride(1) == 1, name, " must be 2-D with unit inner stride");
}
template <typename T>
T* opt_ptr(const OptTensor& t) {
  return t.has_value() ? reinterpret_cast<T*>(t->data_ptr()) : nullptr;
}

// ------------------------------------------------------------------------------------------ GEMM
cmoe::GemmArgs gemm_args(const Tensor& A, const Tensor& B, Tensor& D, int64_t mode, int64_t epilogue, int64_t M, int64_t N, int64_t K,
          bool a_mn, bool b_mn, int64_t groups, int64_t b_group_rows, int64_t split_n, const OptTensor& tile_group,
          const OptTensor& num_m_tiles, int64_t max_m_tiles, const OptTensor& group_offsets, int64_t d_group_stride,
          bool accumulate, const OptTensor& aux_in, const OptTensor& aux_out, const OptTensor& ready_flags,
          int64_t ready_stride, int64_t ready_count, int64_t ready_target, const OptTensor& status,
          int64_t timeout_ns) {
  check_bf16_2d(A, "A");
  check_bf16_2d(B, "B");
  TORCH_CHECK(D.is_cuda() && D.dim() >= 2 && D.stride(-1) == 1, "D must be CUDA with unit inner stride");
  TORCH_CHECK(D.scalar_type() == at::kBFloat16 || D.scalar_type() == at::kFloat, "D must be bf16 or fp32");
  cmoe::GemmArgs g;
  g.A = A.data_ptr();
  g.a_rows = A.size(0);
  g.a_cols = A.size(1);
  g.a_ld = A.stride(0);
  g.a_mn = a_mn;
  g.B = B.data_ptr();
  g.b_rows = B.size(0);
  g.b_cols = B.size(1);
  g.b_ld = B.stride(0);
  g.b_mn = b_mn;
  g.mode = static_cast<int>(mode);
  g.epilogue = static_cast<int>(epilogue);
  g.M = static_cast<int>(M);
  g.N = static_cast<int>(N);
  g.K = static_cast<int>(K);
  g.groups = static_cast<int>(groups);
  g.b_group_rows = b_group_rows;
  g.split_n = static_cast<int>(split_n);
  g.tile_group = opt_ptr<const int>(tile_group);
  g.num_m_tiles = opt_ptr<const int>(num_m_tiles);
  g.max_m_tiles = static_cast<int>(max_m_tiles);
  g.group_offsets = opt_ptr<const int>(group_offsets);
  g.D = D.data_ptr();
  g.ldd = D.stride(-2);
  g.d_group_stride = d_group_stride;
  g.d_fp32 = D.scalar_type() == at::kFloat;
  g.accumulate = accumulate;
  if (aux_in.has_value()) {
    g.aux_in = aux_in->data_ptr();
    g.ld_aux_in = aux_in->stride(0);
  }
  if (aux_out.has_value()) {
    g.aux_out = aux_out->data_ptr();
    g.ld_aux_out = aux_out->stride(0);
  }
  g.ready_flags = opt_ptr<const uint32_t>(ready_flags);
  g.ready_stride = static_cast<int>(ready_stride);
  g.ready_count = static_cast<int>(ready_count);
  g.ready_target = static_cast<uint32_t>(ready_target);
  g.status = opt_ptr<int>(status);
  g.timeout_ns = static_cast<unsigned long long>(timeout_ns);
  return g;
}

void gemm(const Tensor& A, const Tensor& B, Tensor& D, int64_t mode, int64_t epilogue, int64_t M, int64_t N, int64_t K,
          bool a_mn, bool b_mn, int64_t groups, int64_t b_group_rows, int64_t split_n, const OptTensor& tile_group,
          const OptTensor& num_m_tiles, int64_t max_m_tiles, const OptTensor& group_offsets, int64_t d_group_stride,
          bool accumulate, const OptTensor& aux_in, const OptTensor& aux_out, const OptTensor& ready_flags,
          int64_t ready_stride, int64_t ready_count, int64_t ready_target, const OptTensor& status,
          int64_t timeout_ns) {
  const c10::cuda::CUDAGuard guard(A.device());
  cmoe::GemmArgs g = gemm_args(A, B, D, mode, epilogue, M, N, K, a_mn, b_mn, groups, b_group_rows, split_n, tile_group,
                               num_m_tiles, max_m_tiles, group_offsets, d_group_stride, accumulate, aux_in, aux_out,
                               ready_flags, ready_stride, ready_count, ready_target, status, timeout_ns);
  // dense and grouped-K launches with plain results run on the two-SM kernel (CMOE_GEMM_2CTA=0: one-CTA kernel)
  static const bool two_cta = [] {
    const char* v = std::getenv("CMOE_GEMM_2CTA");
    return v == nullptr || (v[0] != '\0' && v[0] != '0');
  }();
  if (two_cta && cmoe::gemm_2cta_supported(g)) {
    check_cuda(cmoe::launch_gemm_2cta(g, cur_stream()), "launch_gemm_2cta");
    return;
  }
  check_cuda(cmoe::launch_gemm(g, cur_stream()), "launch_gemm");
}

// GEMM (dense or grouped-M) whose output rows are scattered by the epilogue: row r goes to rank
// row_slot[r] / slots_per_rank, row row_slot[r] % slots_per_rank of that rank's buffer (negative slot: skipped)
void gemm_scatter(const Tensor& A, const Tensor& B, Tensor& D, int64_t mode, int64_t M, int64_t N, int64_t K, bool b_mn,
                  int64_t groups, int64_t b_group_rows, const OptTensor& tile_group, const OptTensor& num_m_tiles,
                  int64_t max_m_tiles, const Tensor& row_slot, int64_t slots_per_rank,
                  const std::vector<int64_t>& out_ptrs, int64_t out_ld, const OptTensor& status, int64_t timeout_ns) {
  const c10::cuda::CUDAGuard guard(A.device());
  cmoe::GemmArgs g = gemm_args(A, B, D, mode, cmoe::EPI_STORE, M, N, K, false, b_mn, groups, b_group_rows, 0, tile_group,
                               num_m_tiles, max_m_tiles, std::nullopt, 0, false, std::nullopt, std::nullopt,
                               std::nullopt, 0, 0, 0, status, timeout_ns);
  TORCH_CHECK(!out_ptrs.empty() && out_ptrs.size() <= static_cast<size_t>(cmoe::kMaxPeers), "peer table size");
  for (size_t i = 0; i < out_ptrs.size(); ++i) g.scatter_out.ptr[i] = reinterpret_cast<void*>(out_ptrs[i]);
  TORCH_CHECK(row_slot.scalar_type() == at::kInt && row_slot.is_contiguous() && row_slot.numel() >= A.size(0));
  g.scatter_row_slot = row_slot.data_ptr<int>();
  g.scatter_slots_per_rank = slots_per_rank;
  g.scatter_ld = out_ld;
  check_cuda(cmoe::launch_gemm(g, cur_stream()), "launch_gemm(scatter)");
}

// grouped-M GEMM whose A rows are pulled from peer buffers by the kernel itself (fused expert-parallel dispatch)
void gemm_pull(const Tensor& A, const Tensor& B, Tensor& D, int64_t epilogue, int64_t N, int64_t K, bool b_mn,
               int64_t groups, int64_t b_group_rows, int64_t split_n, const Tensor& tile_group,
               const Tensor& num_m_tiles, int64_t max_m_tiles, const OptTensor& aux_in, const OptTensor& aux_out,
               const Tensor& row_slot, const std::vector<int64_t>& src_ptrs, int64_t slots_per_src, int64_t pull_K,
               const OptTensor& slot_scale, int64_t ld_src, Tensor& tile_ready, int64_t epoch, const OptTensor& status,
               int64_t timeout_ns, const OptTensor& stamps) {
  const c10::cuda::CUDAGuard guard(A.device());
  cmoe::GemmArgs g = gemm_args(A, B, D, cmoe::GEMM_GROUPED_M, epilogue, 0, N, K, false, b_mn, groups, b_group_rows,
                               split_n, tile_group, num_m_tiles, max_m_tiles, std::nullopt, 0, false, aux_in, aux_out,
                               std::nullopt, 0, 0, 0, status, timeout_ns);
  TORCH_CHECK(!src_ptrs.empty() && src_ptrs.size() <= static_cast<size_t>(cmoe::kMaxPeers), "peer table size");
  for (size_t i = 0; i < src_ptrs.size(); ++i) g.pull_src.ptr[i] = reinterpret_cast<void*>(src_ptrs[i]);
  TORCH_CHECK(row_slot.scalar_type() == at::kInt && row_slot.numel() >= A.size(0));
  TORCH_CHECK(tile_ready.scalar_type() == at::kInt && tile_ready.numel() >= max_m_tiles * cmoe::kPullFlagsPerTile);
  g.pull_row_slot = row_slot.data_ptr<int>();
  g.pull_slots_per_src = slots_per_src;
  g.pull_K = static_cast<int>(pull_K);
  g.pull_slot_scale = slot_scale.has_value() ? slot_scale->data_ptr<float>() : nullptr;
  g.pull_ld_src = ld_src;
  g.tile_ready = reinterpret_cast<uint32_t*>(tile_ready.data_ptr<int>());
  g.pull_epoch = static_cast<uint32_t>(epoch);
  if (stamps.has_value()) {
    TORCH_CHECK(stamps->scalar_type() == at::kLong && stamps->numel() >= 4 && stamps->is_contiguous() &&
                    stamps->is_cuda(), "stamps must be a CUDA int64 tensor of 4 elements");
    g.pull_stamps = reinterpret_cast<unsigned long long*>(stamps->data_ptr<int64_t>());
  }
  check_cuda(cmoe::launch_gemm(g, cur_stream()), "launch_gemm(pull)");
}

// ------------------------------------------------------------------------------------------ router
void router_fwd(const Tensor& X, const Tensor& Wg, int64_t K, Tensor& logits, Tensor& topk_idx, Tensor& topk_w,
                Tensor& lse, Tensor& counts, Tensor& mean_prob, Tensor& stats, Tensor& workspace,
                const OptTensor& status, int64_t timeout_ns) {
  check_bf16_2d(X, "X");
  check_bf16_2d(Wg, "Wg");
  TORCH_CHECK(Wg.is_contiguous(), "Wg must be contiguous [H, E]");
  const c10::cuda::CUDAGuard guard(X.device());
  cmoe::RouterFwdArgs a;
  a.X = X.data_ptr();
  a.n_tokens = X.size(0);
  a.H = static_cast<int>(X.size(1));
  a.ldx = X.stride(0);
  a.Wg = Wg.data_ptr();
  a.E = static_cast<int>(Wg.size(1));
  a.K = static_cast<int>(K);
  TORCH_CHECK(Wg.size(0) == X.size(1), "gate weight / token hidden size mismatch");
  TORCH_CHECK(logits.scalar_type() == at::kFloat && logits.is_contiguous() && logits.numel() == a.n_tokens * a.E);
  TORCH_CHECK(topk_idx.scalar_type() == at::kInt && topk_idx.numel() == a.n_tokens * a.K);
  TORCH_CHECK(topk_w.scalar_type() == at::kFloat && topk_w.numel() == a.n_tokens * a.K);
  TORCH_CHECK(lse.scalar_type() == at::kFloat && lse.numel() == a.n_tokens);
  TORCH_CHECK(counts.scalar_type() == at::kInt && counts.numel() == a.E);
  TORCH_CHECK(mean_prob.scalar_type() == at::kFloat && mean_prob.numel() == a.E);
  TORCH_CHECK(stats.scalar_type() == at::kFloat && stats.numel() >= 4);
  TORCH_CHECK(workspace.scalar_type() == at::kInt &&
              static_cast<size_t>(workspace.numel()) >= cmoe::router_workspace_words(a.E));
  a.logits = logits.data_ptr<float>();
  a.topk_idx = topk_idx.data_ptr<int>();
  a.topk_w = topk_w.data_ptr<float>();
  a.lse = lse.data_ptr<float>();
  a.counts = counts.data_ptr<int>();
  a.mean_prob = mean_prob.data_ptr<float>();
  a.stats = stats.data_ptr<float>();
  a.workspace = reinterpret_cast<uint32_t*>(workspace.data_ptr());
  a.status = opt_ptr<int>(status);
  a.timeout_ns = static_cast<unsigned long long>(timeout_ns);
  check_cuda(cmoe::launch_router_fwd(a, cur_stream()), "launch_router_fwd");
}

void router_bwd(const Tensor& logits, const Tensor& lse, const Tensor& topk_idx, const OptTensor& grad_w,
                const Tensor& counts, const OptTensor& grad_aux, const OptTensor& grad_z, const OptTensor& gl_bf16,
                const OptTensor& gl_f32) {
  const c10::cuda::CUDAGuard guard(logits.device());
  cmoe::RouterBwdArgs a;
  a.logits = logits.data_ptr<float>();
  a.lse = lse.data_ptr<float>();
  a.topk_idx = topk_idx.data_ptr<int>();
  a.grad_w = opt_ptr<const float>(grad_w);
  a.counts = counts.data_ptr<int>();
  a.grad_aux = opt_ptr<const float>(grad_aux);
  a.grad_z = opt_ptr<const float>(grad_z);
  a.n_tokens = logits.size(0);
  a.E = static_cast<int>(logits.size(1));
  a.K = static_cast<int>(topk_idx.size(1));
  a.grad_logits_bf16 = gl_bf16.has_value() ? gl_bf16->data_ptr() : nullptr;
  a.grad_logits_f32 = opt_ptr<float>(gl_f32);
  check_cuda(cmoe::launch_router_bwd(a, cur_stream()), "launch_router_bwd");
}

// ------------------------------------------------------------------------------------------ elementwise
void rmsnorm_fwd(const Tensor& x, const Tensor& w, Tensor& y, Tensor& rstd, double eps) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous() && x.scalar_type() == at::kBFloat16 &&
              w.scalar_type() == at::kBFloat16);
  const int H = static_cast<int>(x.size(-1));
  check_cuda(cmoe::launch_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), x.numel() / H,
                                      H, static_cast<float>(eps), cur_stream()),
             "rmsnorm_fwd");
}
void rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& rstd, Tensor& dx, Tensor& dw) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(dy.is_contiguous() && x.is_contiguous() && dx.is_contiguous() && dw.scalar_type() == at::kFloat);
  const int H = static_cast<int>(x.size(-1));
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const int64_t rows = x.numel() / H;
  // scratch for the per-CTA column sums (stream-ordered caching allocation, no synchronisation)
  Tensor partial = at::empty({cmoe::rmsnorm_bwd_partial_rows(rows, sms), H}, dw.options());
  check_cuda(cmoe::launch_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), dx.data_ptr(),
                                      dw.data_ptr<float>(), partial.data_ptr<float>(), rows, H, sms, cur_stream()),
             "rmsnorm_bwd");
}
void rope(Tensor& t, const Tensor& cos_tab, const Tensor& sin_tab, int64_t seq, bool inverse) {
  // t: [rows, heads, head_dim] view with unit stride on head_dim and stride head_dim on heads
  const c10::cuda::CUDAGuard guard(t.device());
  TORCH_CHECK(t.dim() == 3 && t.stride(2) == 1 && t.stride(1) == t.size(2) && t.scalar_type() == at::kBFloat16);
  TORCH_CHECK(cos_tab.scalar_type() == at::kFloat && cos_tab.is_contiguous() && sin_tab.is_contiguous());
  TORCH_CHECK(cos_tab.size(0) >= seq && cos_tab.size(1) == t.size(2) / 2);
  check_cuda(cmoe::launch_rope(t.data_ptr(), cos_tab.data_ptr<float>(), sin_tab.data_ptr<float>(), t.size(0),
                               static_cast<int>(seq), static_cast<int>(t.size(1)), static_cast<int>(t.size(2)),
                               t.stride(0), inverse ? 1 : 0, cur_stream()),
             "rope");
}
void qkv_grad_pack(const Tensor& dq, const Tensor& dk, const Tensor& dv, Tensor& out, const Tensor& cos_tab,
                   const Tensor& sin_tab) {
  // dq [B, nh, S, hd], dk / dv [B, nkv, S, hd] (any batch / head / sequence strides); out [B, S, nh + 2 nkv, hd]
  const c10::cuda::CUDAGuard guard(out.device());
  TORCH_CHECK(dq.dim() == 4 && dk.dim() == 4 && dv.dim() == 4 && out.dim() == 4 && out.is_contiguous());
  for (const Tensor* t : {&dq, &dk, &dv})
    TORCH_CHECK(t->scalar_type() == at::kBFloat16 && t->stride(3) == 1 && t->is_cuda(), "bf16 CUDA, unit inner stride");
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && cos_tab.scalar_type() == at::kFloat && cos_tab.is_contiguous() &&
              sin_tab.is_contiguous());
  const int64_t B = dq.size(0), nh = dq.size(1), S = dq.size(2), hd = dq.size(3), nkv = dk.size(1);
  TORCH_CHECK(dv.size(1) == nkv && out.size(0) == B && out.size(1) == S && out.size(2) == nh + 2 * nkv &&
              out.size(3) == hd && cos_tab.size(0) >= S && cos_tab.size(1) == hd / 2);
  const long long sq[3] = {dq.stride(0), dq.stride(1), dq.stride(2)};
  const long long sk[3] = {dk.stride(0), dk.stride(1), dk.stride(2)};
  const long long sv[3] = {dv.stride(0), dv.stride(1), dv.stride(2)};
  check_cuda(cmoe::launch_qkv_grad_pack(dq.data_ptr(), sq, dk.data_ptr(), sk, dv.data_ptr(), sv, out.data_ptr(),
                                        cos_tab.data_ptr<float>(), sin_tab.data_ptr<float>(), B, static_cast<int>(S),
                                        static_cast<int>(nh), static_cast<int>(nkv), static_cast<int>(hd), cur_stream()),
             "qkv_grad_pack");
}
void adamw(Tensor& p32, const OptTensor& p16, Tensor& m, Tensor& v, Tensor& grad, double lr, double beta1, double beta2,
           double eps, double weight_decay, int64_t step, double grad_scale, double max_norm, const OptTensor& sumsq,
           bool zero_grad) {
  const c10::cuda::CUDAGuard guard(p32.device());
  TORCH_CHECK(p32.is_contiguous() && m.is_contiguous() && v.is_contiguous() && grad.is_contiguous());
  TORCH_CHECK(p32.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat);
  TORCH_CHECK(grad.numel() == p32.numel() && m.numel() == p32.numel() && v.numel() == p32.numel());
  cmoe::AdamWArgs a;
  a.p32 = p32.data_ptr<float>();
  if (p16.has_value()) {
    TORCH_CHECK(p16->scalar_type() == at::kBFloat16 && p16->is_contiguous() && p16->numel() == p32.numel());
    a.p16 = p16->data_ptr();
  }
  a.m = m.data_ptr<float>();
  a.v = v.data_ptr<float>();
  a.grad = grad.data_ptr();
  a.grad_is_bf16 = grad.scalar_type() == at::kBFloat16;
  TORCH_CHECK(a.grad_is_bf16 || grad.scalar_type() == at::kFloat);
  a.n = p32.numel();
  a.lr = static_cast<float>(lr);
  a.beta1 = static_cast<float>(beta1);
  a.beta2 = static_cast<float>(beta2);
  a.eps = static_cast<float>(eps);
  a.weight_decay = static_cast<float>(weight_decay);
  a.bias_corr1 = static_cast<float>(1.0 - std::pow(beta1, static_cast<double>(step)));
  a.bias_corr2 = static_cast<float>(1.0 - std::pow(beta2, static_cast<double>(step)));
  a.grad_scale = static_cast<float>(grad_scale);
  a.max_norm = static_cast<float>(max_norm);
  a.sumsq = opt_ptr<const float>(sumsq);
  a.zero_grad = zero_grad;
  check_cuda(cmoe::launch_adamw(a, cur_stream()), "adamw");
}
void sumsq(const Tensor& x, Tensor& out) {
  const c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && out.scalar_type() == at::kFloat);
  const bool bf = x.scalar_type() == at::kBFloat16;
  TORCH_CHECK(bf || x.scalar_type() == at::kFloat);
  // per-block partial sums, added in block order by a second kernel (stream-ordered caching allocation)
  Tensor partials = at::empty({std::max(1, cmoe::sumsq_partial_count(x.numel()))}, out.options());
  check_cuda(cmoe::launch_sumsq(x.data_ptr(), bf, x.numel(), out.data_ptr<float>(), partials.data_ptr<float>(),
                                cur_stream()),
             "sumsq");
}
void cross_entropy(Tensor& logits, const Tensor& targets, Tensor& loss_sum, double grad_scale) {
  const c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && logits.scalar_type() == at::kBFloat16);
  TORCH_CHECK(targets.scalar_type() == at::kLong && targets.is_contiguous() && targets.numel() == logits.size(0));
  // per-row losses, summed by a library reduction whose order is fixed: the loss value is reproducible bit for bit
  Tensor row_loss = at::empty({logits.size(0)}, loss_sum.options());
  check_cuda(cmoe::launch_cross_entropy(logits.data_ptr(), reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()),
                                        loss_sum.data_ptr<float>(), row_loss.data_ptr<float>(), logits.size(0),
                                        static_cast<int>(logits.size(1)), logits.stride(0),
                                        static_cast<float>(grad_scale), cur_stream()),
             "cross_entropy");
  loss_sum.add_(row_loss.sum());
}

// ------------------------------------------------------------------------------------------ MoE bookkeeping
int64_t moe_plan_scratch_words(int64_t n_slots, int64_t n_local, int64_t K, bool per_k_bins) {
  return static_cast<int64_t>(
      cmoe::moe_plan_scratch_words(n_slots, static_cast<int>(n_local), static_cast<int>(K), per_k_bins));
}
void moe_plan(const Tensor& topk_idx, int64_t K, int64_t num_experts, int64_t expert_lo, int64_t n_local,
              bool per_k_bins, int64_t capacity, Tensor& slot_row, Tensor& row_slot, Tensor& group_offsets,
              Tensor& tile_group, Tensor& num_m_tiles, Tensor& counts_kept, Tensor& scratch,
              const OptTensor& overflow) {
  const c10::cuda::CUDAGuard guard(topk_idx.device());
  TORCH_CHECK(topk_idx.scalar_type() == at::kInt && topk_idx.is_contiguous());
  cmoe::MoePlanArgs a;
  a.topk_idx = topk_idx.data_ptr<int>();
  a.n_slots = topk_idx.numel();
  a.K = static_cast<int>(K);
  a.num_experts = static_cast<int>(num_experts);
  a.expert_lo = static_cast<int>(expert_lo);
  a.n_local = static_cast<int>(n_local);
  a.per_k_bins = per_k_bins;
  a.capacity = static_cast<int>(capacity);
  a.cap_rows = row_slot.numel();
  TORCH_CHECK(slot_row.numel() == a.n_slots && tile_group.numel() >= (a.cap_rows + 127) / 128);
  TORCH_CHECK(group_offsets.numel() >= n_local + 1 && counts_kept.numel() >= n_local);
  TORCH_CHECK(static_cast<size_t>(scratch.numel()) >=
              cmoe::moe_plan_scratch_words(a.n_slots, a.n_local, a.K, a.per_k_bins));
  a.slot_row = slot_row.data_ptr<int>();
  a.row_slot = row_slot.data_ptr<int>();
  a.group_offsets = group_offsets.data_ptr<int>();
  a.tile_group = tile_group.data_ptr<int>();
  a.num_m_tiles = num_m_tiles.data_ptr<int>();
  a.counts_kept = counts_kept.data_ptr<int>();
  a.scratch = scratch.data_ptr<int>();
  a.overflow = opt_ptr<int>(overflow);
  check_cuda(cmoe::launch_moe_plan(a, cur_stream()), "moe_plan");
}
void gather_rows(const Tensor& src, const Tensor& row_slot, int64_t slot_div, const OptTensor& slot_scale, Tensor& out,
                 const OptTensor& num_m_tiles) {
  const c10::cuda::CUDAGuard guard(src.device());
  check_bf16_2d(src, "src");
  check_bf16_2d(out, "out");
  check_cuda(cmoe::launch_gather_rows(src.data_ptr(), row_slot.data_ptr<int>(), static_cast<int>(slot_div),
                                      opt_ptr<const float>(slot_scale), out.data_ptr(), out.size(0),
                                      opt_ptr<const int>(num_m_tiles), static_cast<int>(src.size(1)), src.stride(0),
                                      out.stride(0), cur_stream()),
             "gather_rows");
}
void combine_rows(const Tensor& rows, const Tensor& slot_row, const OptTensor& w, Tensor& y, int64_t K) {
  const c10::cuda::CUDAGuard guard(rows.device());
  check_bf16_2d(rows, "rows");
  check_bf16_2d(y, "y");
  check_cuda(cmoe::launch_combine_rows(rows.data_ptr(), slot_row.data_ptr<int>(), opt_ptr<const float>(w), y.data_ptr(),
                                       y.size(0), static_cast<int>(K), static_cast<int>(y.size(1)), rows.stride(0),
                                       y.stride(0), cur_stream()),
             "combine_rows");
}
void combine_bwd_w(const Tensor& rows, const Tensor& slot_row, const Tensor& dy, Tensor& dw, int64_t K) {
  const c10::cuda::CUDAGuard guard(rows.device());
  check_bf16_2d(rows, "rows");
  check_bf16_2d(dy, "dy");
  check_cuda(cmoe::launch_combine_bwd_w(rows.data_ptr(), slot_row.data_ptr<int>(), dy.data_ptr(), dw.data_ptr<float>(),
                                        dy.size(0), static_cast<int>(K), static_cast<int>(dy.size(1)), rows.stride(0),
                                        dy.stride(0), cur_stream()),
             "combine_bwd_w");
}

}  // namespace

void register_attention(pybind11::module_& m);
void register_ep(pybind11::module_& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "sm_100a kernels of the composed MoE engine";
  m.def("gemm", &gemm);
  m.def("gemm_pull", &gemm_pull);
  m.def("gemm_scatter", &gemm_scatter);
  m.def("router_fwd", &router_fwd);
  m.def("router_bwd", &router_bwd);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("rope", &rope);
  m.def("qkv_grad_pack", &qkv_grad_pack);
  m.def("adamw", &adamw);
  m.def("sumsq", &sumsq);
  m.def("cross_entropy", &cross_entropy);
  m.def("moe_plan_scratch_words", &moe_plan_scratch_words);
  m.def("moe_plan", &moe_plan);
  m.def("gather_rows", &gather_rows);
  m.def("combine_rows", &combine_rows);
  m.def("combine_bwd_w", &combine_bwd_w);
  register_attention(m);
  register_ep(m);
}
