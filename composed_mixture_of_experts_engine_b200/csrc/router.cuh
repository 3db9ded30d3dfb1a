// Host-side interface of the fused top-k router kernels (forward and analytic backward).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace cmoe {

constexpr int kRouterMaxExperts = 256;
constexpr int kRouterMaxTopK = 8;
// Workspace layout (32-bit words, 8-byte aligned base): E + 1 unsigned 64-bit fixed-point accumulators (the sums of
// the probabilities of each expert, scaled by 2^40, then the sum of lse^2 scaled by 2^24), followed by E int counts
// and the finished-CTA counter.  The sums are integers so that the order in which the CTAs add to them cannot
// change the result (same inputs, same bits).  3*E+4 words in total, zero before the first launch; the kernel
// leaves it zeroed again.
inline size_t router_workspace_words(int num_experts) { return 3 * static_cast<size_t>(num_experts) + 4; }
constexpr float kRouterProbScale = 1099511627776.f;  // 2^40
constexpr float kRouterZScale = 16777216.f;          // 2^24

struct RouterFwdArgs {
  const void* X = nullptr;  // [n_tokens, H] bf16, leading dimension ldx
  long long n_tokens = 0;
  int H = 0;
  long long ldx = 0;
  const void* Wg = nullptr;  // [H, E] bf16 row-major (E contiguous)
  int E = 0;
  int K = 0;
  float* logits = nullptr;   // [n_tokens, E] fp32
  int* topk_idx = nullptr;   // [n_tokens, K] int32, descending probability, ties -> lowest index
  float* topk_w = nullptr;   // [n_tokens, K] fp32, renormalised over the K picks
  float* lse = nullptr;      // [n_tokens] fp32 log-sum-exp of the logits (saved for the backward)
  int* counts = nullptr;     // [E] int32 number of (token, slot) pairs routed to each expert
  float* mean_prob = nullptr;  // [E] fp32 mean softmax probability of each expert (P_i)
  float* stats = nullptr;    // [4]: E*sum_i f_i*P_i (aux loss), mean lse^2 (z loss), max/mean load, sum(counts)
  uint32_t* workspace = nullptr;  // router_workspace_words(E) zeroed words
  int* status = nullptr;
  unsigned long long timeout_ns = 0;
};

cudaError_t launch_router_fwd(const RouterFwdArgs& args, cudaStream_t stream);

// grad_logits[t, i] for
//   L = sum_tk gw[t,k] * w[t,k]  +  aux_coeff * E * sum_i f_i * P_i  +  z_coeff * mean_t lse_t^2
// with f_i (the routed fraction) treated as a constant, as in Switch-style load-balance losses.
struct RouterBwdArgs {
  const float* logits = nullptr;  // [n_tokens, E]
  const float* lse = nullptr;     // [n_tokens]
  const int* topk_idx = nullptr;  // [n_tokens, K]
  const float* grad_w = nullptr;  // [n_tokens, K] fp32 (may be nullptr: treated as zero)
  const int* counts = nullptr;    // [E]
  const float* grad_aux = nullptr;  // device scalar: upstream gradient of the aux loss (nullptr: 0)
  const float* grad_z = nullptr;    // device scalar: upstream gradient of the z loss (nullptr: 0)
  long long n_tokens = 0;
  int E = 0;
  int K = 0;
  void* grad_logits_bf16 = nullptr;  // [n_tokens, E] bf16 (operand of the two backward GEMMs), may be nullptr
  float* grad_logits_f32 = nullptr;  // [n_tokens, E] fp32, may be nullptr
};

cudaError_t launch_router_bwd(const RouterBwdArgs& args, cudaStream_t stream);

}  // namespace cmoe
