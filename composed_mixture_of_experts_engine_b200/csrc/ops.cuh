// Host-side interface of the bandwidth-bound kernels: RMSNorm, RoPE, fused AdamW, sum of squares,
// cross-entropy, and the MoE routing bookkeeping (expert-sorted row map, row gather, weighted
// combine).  Torch-free; pointers are device pointers of the current device.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace cmoe {

// ---- RMSNorm ------------------------------------------------------------------------------
// y = x * rsqrt(mean(x^2) + eps) * w, fp32 math, bf16 in/out.  rstd [rows] is saved for the backward.
cudaError_t launch_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int H, float eps,
                               cudaStream_t stream);
// dx (bf16) and dw (fp32, added to: zero it first unless accumulation is wanted).  With dw_partial (fp32
// [rmsnorm_bwd_partial_rows(rows, num_sms), H] scratch) every CTA writes its column sums there and a second small
// kernel adds them to dw; without it the CTAs add to dw with atomics.
long long rmsnorm_bwd_partial_rows(long long rows, int num_sms);
cudaError_t launch_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw,
                               float* dw_partial, long long rows, int H, int num_sms, cudaStream_t stream);

// ---- RoPE (rotate-half pairing: element i pairs with i + head_dim/2), in place -----------------
// t: [batch*seq, heads, head_dim] bf16; cos/sin: [seq, head_dim/2] fp32; position of row r is r % seq.
// inverse != 0 applies the transposed rotation (the backward).
cudaError_t launch_rope(void* t, const float* cos_tab, const float* sin_tab, long long rows, int seq, int heads,
                        int head_dim, long long row_stride, int inverse, cudaStream_t stream);

// dqkv[b*seq + s, h, :] = un-rotated dq / dk (first nh, next nkv heads) or dv (last nkv heads); each source is a
// [batch, heads, seq, head_dim] view given by its (batch, head, seq) strides in elements, unit stride on head_dim.
cudaError_t launch_qkv_grad_pack(const void* dq, const long long* dq_strides, const void* dk, const long long* dk_strides,
                                 const void* dv, const long long* dv_strides, void* out, const float* cos_tab,
                                 const float* sin_tab, long long batch, int seq, int nh, int nkv, int head_dim,
                                 cudaStream_t stream);

// ---- fused AdamW ---------------------------------------------------------------------------
// Decoupled weight decay; p32 is the fp32 master copy, p16 (optional) the bf16 copy that the model
// computes with.  grad is fp32 or bf16.  The gradient is first multiplied by
//   grad_scale * min(1, max_norm / (sqrt(*sumsq) + 1e-6))      (max_norm <= 0: no clipping)
// where sumsq is a device scalar holding the squared global norm of the already scaled gradients
// (launch_sumsq over the raw gradients, times grad_scale^2, summed over all parameter groups).
struct AdamWArgs {
  float* p32 = nullptr;
  void* p16 = nullptr;
  float* m = nullptr;
  float* v = nullptr;
  const void* grad = nullptr;
  int grad_is_bf16 = 0;
  long long n = 0;
  float lr = 0.f, beta1 = 0.9f, beta2 = 0.95f, eps = 1e-8f, weight_decay = 0.f;
  float bias_corr1 = 1.f, bias_corr2 = 1.f;  // 1 - beta^t
  float grad_scale = 1.f;
  float max_norm = 0.f;
  const float* sumsq = nullptr;
  int zero_grad = 0;  // != 0: the gradient buffer is cleared after it has been read
};
cudaError_t launch_adamw(const AdamWArgs& a, cudaStream_t stream);
// *out += sum(x^2) (out must be zeroed by the caller before the first call of a step).  With `partials` (room for
// sumsq_partial_count(n) floats) the per-block sums are added in a fixed order, so that equal inputs give equal bits
// (the clipping factor, and with it the whole update, hangs on this number); nullptr: fp32 atomics.
int sumsq_partial_count(long long n);
cudaError_t launch_sumsq(const void* x, int is_bf16, long long n, float* out, float* partials, cudaStream_t stream);

// ---- cross-entropy, forward and gradient in one pass ------------------------------------------
// logits [rows, V] bf16 are overwritten with d(loss)/d(logits) = (softmax - onehot) * grad_scale;
// *loss_sum += sum over rows of the per-row loss (fp32), or, with `row_loss` [rows], the per-row losses are written
// there for the caller to sum in a fixed order (*loss_sum is then left alone).  targets are int64; target < 0 is
// ignored (its row loss is 0).
cudaError_t launch_cross_entropy(void* logits, const long long* targets, float* loss_sum, float* row_loss,
                                 long long rows, int V, long long ld, float grad_scale, cudaStream_t stream);

// ---- MoE routing bookkeeping -------------------------------------------------------------------
// Builds the expert-sorted, 128-row-padded row layout for `n_slots` (token, k) slots.
//   topk_idx   [n_slots] expert of each slot (slot = token * K + k)
//   per_k_bins != 0: rows are ordered by (expert, k, token) and at most `capacity` slots per
//                    (expert, k) are kept - first come first served in token order; the rest get row -1.
//   expert_lo / n_local: only experts in [expert_lo, expert_lo + n_local) get rows (others: row -1).
// Outputs:
//   slot_row      [n_slots]      destination row of each slot, or -1
//   row_slot      [cap_rows]     source slot of each row, or -1 for padding rows
//   group_offsets [n_local + 1]  first row of each local expert (multiples of 128)
//   tile_group    [cap_rows/128] local expert of each 128-row tile, -1 beyond the last tile
//   num_m_tiles   [1]            number of live tiles;  counts_kept [n_local] rows per local expert
// scratch: int32 words, see moe_plan_scratch_words().  Deterministic (no atomics on the order).
struct MoePlanArgs {
  const int* topk_idx = nullptr;
  long long n_slots = 0;
  int K = 1;
  int num_experts = 0;
  int expert_lo = 0;
  int n_local = 0;
  int per_k_bins = 0;
  int capacity = 0;  // <= 0: unlimited
  long long cap_rows = 0;
  int* slot_row = nullptr;
  int* row_slot = nullptr;
  int* group_offsets = nullptr;
  int* tile_group = nullptr;
  int* num_m_tiles = nullptr;
  int* counts_kept = nullptr;
  int* scratch = nullptr;
  int* overflow = nullptr;  // optional counter: slots dropped because cap_rows was too small for the routing
};
size_t moe_plan_scratch_words(long long n_slots, int n_local, int K, int per_k_bins);
cudaError_t launch_moe_plan(const MoePlanArgs& a, cudaStream_t stream);

// out[r, :] = scale * src[row_slot[r] / slot_div, :]  (zeros where row_slot[r] < 0), for r < *n_rows_dev * 128
// (n_rows_dev = num_m_tiles) or r < cap_rows when n_rows_dev is nullptr.  slot_scale (fp32 per slot) optional.
cudaError_t launch_gather_rows(const void* src, const int* row_slot, int slot_div, const float* slot_scale, void* out,
                               long long cap_rows, const int* num_m_tiles, int H, long long ld_src, long long ld_out,
                               cudaStream_t stream);
// y[t, :] = sum_k w[t,k] * rows[slot_row[t*K+k], :]  (slots with row -1 skipped), fp32 accumulate, bf16 out
cudaError_t launch_combine_rows(const void* rows, const int* slot_row, const float* w, void* y, long long n_tokens,
                                int K, int H, long long ld_rows, long long ld_y, cudaStream_t stream);
// dw[t,k] = <dy[t,:], rows[slot_row[t*K+k], :]>
cudaError_t launch_combine_bwd_w(const void* rows, const int* slot_row, const void* dy, float* dw, long long n_tokens,
                                 int K, int H, long long ld_rows, long long ld_dy, cudaStream_t stream);

}  // namespace cmoe
