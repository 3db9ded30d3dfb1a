// pybind11 registration of the attention kernels (attention.cu).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "attention.cuh"

namespace {

using torch::Tensor;

void check(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, "cmoe: ", what, " failed: ", cudaGetErrorString(e));
}
cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_packed(const Tensor& qkv, int64_t nh, int64_t nkv) {
  TORCH_CHECK(qkv.is_cuda() && qkv.scalar_type() == at::kBFloat16 && qkv.dim() == 4 && qkv.is_contiguous(),
              "qkv must be a contiguous CUDA bf16 tensor [B, S, nh + 2 nkv, hd]");
  TORCH_CHECK(qkv.size(2) == nh + 2 * nkv, "qkv holds ", qkv.size(2), " heads, expected nh + 2 nkv = ", nh + 2 * nkv);
  TORCH_CHECK(cmoe::attention_shape_supported(static_cast<int>(qkv.size(1)), static_cast<int>(nh),
                                              static_cast<int>(nkv), static_cast<int>(qkv.size(3))),
              "attention kernel: S must be a multiple of 128, hd 64 or 128, nh a multiple of nkv");
}

bool attention_supported(int64_t S, int64_t nh, int64_t nkv, int64_t hd) {
  return cmoe::attention_shape_supported(static_cast<int>(S), static_cast<int>(nh), static_cast<int>(nkv),
                                         static_cast<int>(hd));
}

// qkv [B, S, nh + 2 nkv, hd] -> out [B, S, nh, hd] (bf16), lse [B, nh, S] (fp32)
void attention_fwd(const Tensor& qkv, int64_t nh, int64_t nkv, Tensor& out, Tensor& lse, Tensor& status,
                   int64_t timeout_ns) {
  check_packed(qkv, nh, nkv);
  const c10::cuda::CUDAGuard guard(qkv.device());
  const int64_t B = qkv.size(0), S = qkv.size(1), hd = qkv.size(3);
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kBFloat16 && out.is_contiguous() && out.numel() == B * S * nh * hd,
              "out must be contiguous bf16 [B, S, nh, hd]");
  TORCH_CHECK(lse.is_cuda() && lse.scalar_type() == at::kFloat && lse.is_contiguous() && lse.numel() == B * nh * S,
              "lse must be contiguous fp32 [B, nh, S]");
  TORCH_CHECK(status.scalar_type() == at::kInt && status.numel() >= 1);
  cmoe::AttnFwdArgs a;
  a.qkv = qkv.data_ptr();
  a.out = out.data_ptr();
  a.lse = lse.data_ptr<float>();
  a.B = static_cast<int>(B);
  a.S = static_cast<int>(S);
  a.nh = static_cast<int>(nh);
  a.nkv = static_cast<int>(nkv);
  a.hd = static_cast<int>(hd);
  a.status = status.data_ptr<int>();
  a.timeout_ns = static_cast<unsigned long long>(timeout_ns);
  check(cmoe::launch_attention_fwd(a, stream()), "launch_attention_fwd");
}

// dq (fp32 [B, S, nh, hd]) must be zero on entry; dk / dv are bf16 [B, S, nkv, hd]; delta is fp32 scratch [B, nh, S]
void attention_bwd(const Tensor& qkv, int64_t nh, int64_t nkv, const Tensor& out, const Tensor& dout, const Tensor& lse,
                   Tensor& delta, Tensor& dq, Tensor& dk, Tensor& dv, Tensor& status, int64_t timeout_ns) {
  check_packed(qkv, nh, nkv);
  const c10::cuda::CUDAGuard guard(qkv.device());
  const int64_t B = qkv.size(0), S = qkv.size(1), hd = qkv.size(3);
  auto bf16_full = [&](const Tensor& t, int64_t heads) {
    return t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous() && t.numel() == B * S * heads * hd;
  };
  TORCH_CHECK(bf16_full(out, nh) && bf16_full(dout, nh), "out / dout must be contiguous bf16 [B, S, nh, hd]");
  TORCH_CHECK(bf16_full(dk, nkv) && bf16_full(dv, nkv), "dk / dv must be contiguous bf16 [B, S, nkv, hd]");
  TORCH_CHECK(dq.is_cuda() && dq.scalar_type() == at::kFloat && dq.is_contiguous() && dq.numel() == B * S * nh * hd,
              "dq must be contiguous fp32 [B, S, nh, hd]");
  TORCH_CHECK(lse.scalar_type() == at::kFloat && lse.is_contiguous() && lse.numel() == B * nh * S);
  TORCH_CHECK(delta.scalar_type() == at::kFloat && delta.is_contiguous() && delta.numel() == B * nh * S);
  TORCH_CHECK(status.scalar_type() == at::kInt && status.numel() >= 1);
  cmoe::AttnBwdArgs a;
  a.qkv = qkv.data_ptr();
  a.out = out.data_ptr();
  a.dout = dout.data_ptr();
  a.lse = lse.data_ptr<float>();
  a.delta = delta.data_ptr<float>();
  a.dq = dq.data_ptr<float>();
  a.dk = dk.data_ptr();
  a.dv = dv.data_ptr();
  a.B = static_cast<int>(B);
  a.S = static_cast<int>(S);
  a.nh = static_cast<int>(nh);
  a.nkv = static_cast<int>(nkv);
  a.hd = static_cast<int>(hd);
  a.status = status.data_ptr<int>();
  a.timeout_ns = static_cast<unsigned long long>(timeout_ns);
  check(cmoe::launch_attention_bwd(a, stream()), "launch_attention_bwd");
}

}  // namespace

void register_attention(pybind11::module_& m) {
  m.def("attention_supported", &attention_supported);
  m.def("attention_fwd", &attention_fwd);
  m.def("attention_bwd", &attention_bwd);
}
