// Host-side interface of the causal attention kernels (attention.cu): tcgen05 / TMEM forward and backward on a
// packed projection.  Torch-free.
//
// The reference has no attention operator (pkg/models/moe.py:148-186 is a decoder of norm + MoE blocks only); these
// kernels exist because the benchmark configurations name heads, grouped-query attention and rotary embedding.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace cmoe {

// qkv is a bf16 buffer [B, S, nh + 2 nkv, hd]: q heads, then k heads, then v heads (already rotated).
// S must be a multiple of 128, hd is 64 or 128, nh a multiple of nkv.
struct AttnFwdArgs {
  const void* qkv = nullptr;
  void* out = nullptr;    // bf16 [B, S, nh, hd]
  float* lse = nullptr;   // fp32 [B, nh, S]: natural-log sum of exp of the scaled scores of every query row
  int B = 0, S = 0, nh = 0, nkv = 0, hd = 0;
  float scale = 0.f;      // 0: 1 / sqrt(hd)
  int* status = nullptr;  // device int, set to a StatusCode when a wait ran out
  unsigned long long timeout_ns = 0;  // 0: default
};

struct AttnBwdArgs {
  const void* qkv = nullptr;
  const void* out = nullptr;   // bf16 [B, S, nh, hd] of the forward
  const void* dout = nullptr;  // bf16 [B, S, nh, hd]
  const float* lse = nullptr;  // fp32 [B, nh, S] of the forward
  float* delta = nullptr;      // fp32 [B, nh, S] scratch: row sums of dout * out (written by the launch)
  float* dq = nullptr;         // fp32 [B, S, nh, hd], must be zero on entry (query gradients are accumulated)
  void* dk = nullptr;          // bf16 [B, S, nkv, hd]
  void* dv = nullptr;          // bf16 [B, S, nkv, hd]
  int B = 0, S = 0, nh = 0, nkv = 0, hd = 0;
  float scale = 0.f;
  int* status = nullptr;
  unsigned long long timeout_ns = 0;
};

bool attention_shape_supported(int S, int nh, int nkv, int hd);
// The forward picks the two-query-tile kernel (attention_fwd2.cu) when the head dimension is 128, S is a multiple
// of 256 and the default scale is used; CMOE_ATTN_FWD2=0 keeps the one-tile kernel.
cudaError_t launch_attention_fwd(const AttnFwdArgs& a, cudaStream_t stream);
cudaError_t launch_attention_bwd(const AttnBwdArgs& a, cudaStream_t stream);

}  // namespace cmoe

// Raw-pointer entry of the two-query-tile forward kernel (attention_fwd2.cu): S % 256 == 0, hd 128.  Returns a
// cudaError_t as int.
extern "C" int cmoe_attention_fwd2(const void* qkv, void* out, float* lse, int B, int S, int nh, int nkv, int hd,
                                   int* status, unsigned long long timeout_ns, void* stream);
