// Bandwidth-bound kernels of the training step: RMSNorm, RoPE, fused AdamW (+ global-norm clipping
// without a host round trip), cross-entropy with in-place gradient, and the MoE bookkeeping kernels
// (deterministic expert-sorted row plan, row gather, weighted combine).
//
// Reference counterparts: RMSNorm eager ops (pkg/models/moe.py:83-86); torch.optim.AdamW +
// clip_grad_norm_ + F.cross_entropy (train.py:207-212, 297-303, 322-323); argsort /
// repeat_interleave / per-k scatter loop of the MoE layer (pkg/distributed/moe_layer.py:309-353);
// capacity dropping (moe_layer.py:64-155).  RoPE has no counterpart there.
#include "ops.cuh"

#include <cstdlib>

#include "common.cuh"

namespace cmoe {

namespace {

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 x = *reinterpret_cast<const uint4*>(p);
  const float2 a = unpack_bf16x2(x.x), b = unpack_bf16x2(x.y), c = unpack_bf16x2(x.z), d = unpack_bf16x2(x.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 o;
  o.x = pack_bf16x2(f[0], f[1]);
  o.y = pack_bf16x2(f[2], f[3]);
  o.z = pack_bf16x2(f[4], f[5]);
  o.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = o;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (threadIdx.x < THREADS / 32) ? red[threadIdx.x] : 0.f;
  if (warp == 0) {
    t = warp_sum(t);
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

// ------------------------------------------------------------------------------------ RMSNorm
// One CTA of 128 threads per row; each thread keeps VEC vectors of 8 columns in registers
// (VEC = 1, 2, 4, 8 covers H <= 1024, 2048, 4096, 8192).  Small CTAs keep 16 rows in flight per SM.
constexpr int RN_THREADS = 128;

template <int VEC>
__global__ void __launch_bounds__(RN_THREADS) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                                 const __nv_bfloat16* __restrict__ w,
                                                                 __nv_bfloat16* __restrict__ y,
                                                                 float* __restrict__ rstd, long long rows, int H,
                                                                 float eps) {
  __shared__ float red[RN_THREADS / 32];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* xr = x + row * H;
    float v[VEC][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = (i * RN_THREADS + threadIdx.x) * 8;
      if (c < H) {
        load8(xr + c, v[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
      }
    }
    ss = block_sum<RN_THREADS>(ss, red);
    const float r = rsqrtf(ss / H + eps);
    if (threadIdx.x == 0 && rstd) rstd[row] = r;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = (i * RN_THREADS + threadIdx.x) * 8;
      if (c < H) {
        float wv[8], o[8];
        load8(w + c, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = v[i][j] * r * wv[j];
        store8(y + row * H + c, o);
      }
    }
  }
}

// rows of x / dy that a CTA of the backward kernel keeps in flight (shared-memory ring)
__host__ __device__ constexpr int rn_bwd_stages(int vec) { return vec <= 2 ? 4 : 2; }
__host__ __device__ constexpr int rn_bwd_smem(int vec) { return rn_bwd_stages(vec) * 2 * vec * RN_THREADS * 16; }

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))),
               "l"(gsrc)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int VEC>
__global__ void __launch_bounds__(RN_THREADS) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                                 const __nv_bfloat16* __restrict__ x,
                                                                 const __nv_bfloat16* __restrict__ w,
                                                                 const float* __restrict__ rstd,
                                                                 __nv_bfloat16* __restrict__ dx, float* __restrict__ dw,
                                                                 float* __restrict__ dw_partial, long long rows,
                                                                 int H) {
  __shared__ float red[RN_THREADS / 32];
  extern __shared__ uint4 rn_ring[];  // [stages][x | dy][VEC][RN_THREADS]: every thread's own 16-byte pieces
  constexpr int S = rn_bwd_stages(VEC);
  float wv[VEC][8], dwacc[VEC][8];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = (i * RN_THREADS + threadIdx.x) * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dwacc[i][j] = 0.f;
      wv[i][j] = 0.f;
    }
    if (c < H) load8(w + c, wv[i]);
  }
  // The rows of x and dy stream through a ring of S rows in shared memory, filled by per-thread asynchronous copies
  // (`cp.async`, 16 bytes each, past L1): a CTA keeps S rows of loads in flight without holding them in registers,
  // and every thread reads back only the pieces it copied itself, so the ring needs no barrier.  One commit group per
  // row (an empty one past the end), so that "all but the newest S - 1 groups" is always the row about to be used.
  auto slot = [&](int s, int which, int i) { return rn_ring + ((s * 2 + which) * VEC + i) * RN_THREADS + threadIdx.x; };
  auto issue = [&](long long row, int s) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = (i * RN_THREADS + threadIdx.x) * 8;
      if (row < rows && c < H) {
        cp_async_16(slot(s, 0, i), x + row * H + c);
        cp_async_16(slot(s, 1, i), dy + row * H + c);
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int s = 0; s < S; ++s) issue(blockIdx.x + static_cast<long long>(s) * gridDim.x, s);
  int s = 0;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    cp_async_wait<S - 1>();
    const float r = rstd[row];
    float xh[VEC][8], g[VEC][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = (i * RN_THREADS + threadIdx.x) * 8;
      if (c < H) {
        const uint4 nx = *slot(s, 0, i), nd = *slot(s, 1, i);
        const uint32_t xw[4] = {nx.x, nx.y, nx.z, nx.w};
        const uint32_t dw4[4] = {nd.x, nd.y, nd.z, nd.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 xv = unpack_bf16x2(xw[q]), dv = unpack_bf16x2(dw4[q]);
          xh[i][2 * q] = xv.x * r;
          xh[i][2 * q + 1] = xv.y * r;
          g[i][2 * q] = dv.x * wv[i][2 * q];
          g[i][2 * q + 1] = dv.y * wv[i][2 * q + 1];
          dot += g[i][2 * q] * xh[i][2 * q] + g[i][2 * q + 1] * xh[i][2 * q + 1];
          dwacc[i][2 * q] += dv.x * xh[i][2 * q];
          dwacc[i][2 * q + 1] += dv.y * xh[i][2 * q + 1];
        }
      }
    }
    // the slot's values are in registers (the arithmetic above used them): refill it with the row S steps ahead
    issue(row + static_cast<long long>(S) * gridDim.x, s);
    s = (s + 1 == S) ? 0 : s + 1;
    dot = block_sum<RN_THREADS>(dot, red) / H;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = (i * RN_THREADS + threadIdx.x) * 8;
      if (c < H) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = r * (g[i][j] - xh[i][j] * dot);
        store8(dx + row * H + c, o);
      }
    }
  }
  if (dw_partial) {
    // one row of partial column sums per CTA, summed in a fixed order by the colsum kernels: CTAs adding atomically to
    // the same H addresses serialise in L2 and cost more than the whole row pass
    float* out = dw_partial + static_cast<long long>(blockIdx.x) * H;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = (i * RN_THREADS + threadIdx.x) * 8;
      if (c < H) {
        *reinterpret_cast<float4*>(out + c) = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
        *reinterpret_cast<float4*>(out + c + 4) = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
      }
    }
  } else if (dw) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int c = (i * RN_THREADS + threadIdx.x) * 8;
      if (c < H) {
#pragma unroll
        for (int j = 0; j < 8; ++j) atomicAdd(dw + c + j, dwacc[i][j]);
      }
    }
  }
}

// Column sums of the per-CTA partial rows in a fixed order (the same inputs give the same bits, whichever CTA
// finishes first).  Stage 1, grid (ceil(H / 128), slices): slice y adds the rows y, y + slices, ... in that order and
// leaves the result in row y (only slice y ever touches those rows).  Stage 2, grid (ceil(H / 128)): dw[c] += the
// `slices` stage-1 rows, again in order.
__global__ void __launch_bounds__(128) colsum_stage1_kernel(float* __restrict__ partial, int n_rows, int H) {
  const int c = blockIdx.x * 128 + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
#pragma unroll 8
  for (int b = blockIdx.y; b < n_rows; b += gridDim.y) s += partial[static_cast<long long>(b) * H + c];  // loads ahead, adds in order
  partial[static_cast<long long>(blockIdx.y) * H + c] = s;
}
__global__ void __launch_bounds__(128) colsum_stage2_kernel(const float* __restrict__ partial, float* __restrict__ dw,
                                                            int slices, int H) {
  const int c = blockIdx.x * 128 + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
#pragma unroll 8
  for (int y = 0; y < slices; ++y) s += partial[static_cast<long long>(y) * H + c];
  dw[c] += s;
}

// ------------------------------------------------------------------------------------ RoPE
__global__ void rope_kernel(__nv_bfloat16* __restrict__ t, const float* __restrict__ cos_tab,
                            const float* __restrict__ sin_tab, long long rows, int seq, int heads, int head_dim,
                            long long row_stride, int inverse) {
  const int half = head_dim / 2;
  const int vec_per_head = half / 8;
  const long long total = rows * heads * vec_per_head;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int vi = static_cast<int>(i % vec_per_head);
    const long long rh = i / vec_per_head;
    const int h = static_cast<int>(rh % heads);
    const long long r = rh / heads;
    const int pos = static_cast<int>(r % seq);
    __nv_bfloat16* base = t + r * row_stride + static_cast<long long>(h) * head_dim + vi * 8;
    float a[8], b[8], oa[8], ob[8];
    load8(base, a);
    load8(base + half, b);
    const float* cp = cos_tab + static_cast<long long>(pos) * half + vi * 8;
    const float* sp = sin_tab + static_cast<long long>(pos) * half + vi * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float c = cp[j];
      const float s = inverse ? -sp[j] : sp[j];
      oa[j] = a[j] * c - b[j] * s;
      ob[j] = b[j] * c + a[j] * s;
    }
    store8(base, oa);
    store8(base + half, ob);
  }
}

// Packs the three attention gradients into one [rows, heads, head_dim] buffer (q heads, k heads, v heads) and undoes
// the rotary embedding on the q and k heads on the way: one read and one write of every element instead of three
// strided copies plus an in-place rotation pass.  Sources are [B, h, S, head_dim] views with arbitrary batch / head /
// sequence strides and unit stride on head_dim.
struct QkvGradSrc {
  const __nv_bfloat16* ptr;
  long long sb, sh, ss;  // strides (elements) of batch, head, sequence position
};

__global__ void qkv_grad_pack_kernel(QkvGradSrc dq, QkvGradSrc dk, QkvGradSrc dv, __nv_bfloat16* __restrict__ out,
                                     const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                                     long long rows, int seq, int nh, int nkv, int head_dim) {
  const int heads = nh + 2 * nkv;
  const int half = head_dim / 2;
  const int vec_per_head = half / 8;
  const long long total = rows * heads * vec_per_head;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int vi = static_cast<int>(i % vec_per_head);
    const long long rh = i / vec_per_head;
    const int h = static_cast<int>(rh % heads);
    const long long r = rh / heads;
    const int pos = static_cast<int>(r % seq);
    const long long b = r / seq;
    const QkvGradSrc& s = h < nh ? dq : (h < nh + nkv ? dk : dv);
    const int hh = h < nh ? h : (h < nh + nkv ? h - nh : h - nh - nkv);
    const __nv_bfloat16* src = s.ptr + b * s.sb + hh * s.sh + pos * s.ss + vi * 8;
    __nv_bfloat16* dst = out + (r * heads + h) * head_dim + vi * 8;
    const uint4 ra = __ldcs(reinterpret_cast<const uint4*>(src));
    const uint4 rb = __ldcs(reinterpret_cast<const uint4*>(src + half));
    if (h >= nh + nkv) {  // v heads: plain copy
      *reinterpret_cast<uint4*>(dst) = ra;
      *reinterpret_cast<uint4*>(dst + half) = rb;
      continue;
    }
    const uint32_t aw[4] = {ra.x, ra.y, ra.z, ra.w}, bw[4] = {rb.x, rb.y, rb.z, rb.w};
    uint32_t oa[4], ob[4];
    const float* cp = cos_tab + static_cast<long long>(pos) * half + vi * 8;
    const float* sp = sin_tab + static_cast<long long>(pos) * half + vi * 8;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 a = unpack_bf16x2(aw[q]), bb = unpack_bf16x2(bw[q]);
      const float c0 = cp[2 * q], c1 = cp[2 * q + 1], s0 = sp[2 * q], s1 = sp[2 * q + 1];
      // the transpose of the rotation: [a; b] -> [a c + b s; b c - a s]
      oa[q] = pack_bf16x2(a.x * c0 + bb.x * s0, a.y * c1 + bb.y * s1);
      ob[q] = pack_bf16x2(bb.x * c0 - a.x * s0, bb.y * c1 - a.y * s1);
    }
    *reinterpret_cast<uint4*>(dst) = make_uint4(oa[0], oa[1], oa[2], oa[3]);
    *reinterpret_cast<uint4*>(dst + half) = make_uint4(ob[0], ob[1], ob[2], ob[3]);
  }
}

// ------------------------------------------------------------------------------------ AdamW
__global__ void adamw_kernel(const AdamWArgs a) {
  float gs = a.grad_scale;
  if (a.max_norm > 0.f && a.sumsq != nullptr) {
    const float norm = sqrtf(*a.sumsq);  // sumsq already refers to the scaled gradients
    gs *= fminf(1.f, a.max_norm / (norm + 1e-6f));
  }
  const float inv_bc1 = 1.f / a.bias_corr1;
  const float inv_sqrt_bc2 = rsqrtf(a.bias_corr2);
  const long long n4 = a.n / 4;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  float4* __restrict__ p32v = reinterpret_cast<float4*>(a.p32);
  float4* __restrict__ mv = reinterpret_cast<float4*>(a.m);
  float4* __restrict__ vv4 = reinterpret_cast<float4*>(a.v);
  uint2* __restrict__ p16v = reinterpret_cast<uint2*>(a.p16);
  float4* __restrict__ g32v = reinterpret_cast<float4*>(const_cast<void*>(a.grad));
  uint2* __restrict__ g16v = reinterpret_cast<uint2*>(const_cast<void*>(a.grad));
  const float decay = 1.f - a.lr * a.weight_decay;
  const float omb1 = 1.f - a.beta1, omb2 = 1.f - a.beta2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4; i += stride) {
    // all loads first (streaming: nothing here is read twice), then the math, then the stores
    const float4 p = __ldcs(p32v + i);
    const float4 m = __ldcs(mv + i);
    const float4 v = __ldcs(vv4 + i);
    float g[4];
    if (a.grad_is_bf16) {
      const uint2 raw = __ldcs(g16v + i);
      const float2 g0 = unpack_bf16x2(raw.x), g1 = unpack_bf16x2(raw.y);
      g[0] = g0.x; g[1] = g0.y; g[2] = g1.x; g[3] = g1.y;
    } else {
      const float4 raw = __ldcs(g32v + i);
      g[0] = raw.x; g[1] = raw.y; g[2] = raw.z; g[3] = raw.w;
    }
    float pp[4] = {p.x, p.y, p.z, p.w}, mm[4] = {m.x, m.y, m.z, m.w}, vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = g[j] * gs;
      mm[j] = a.beta1 * mm[j] + omb1 * gj;
      vv[j] = a.beta2 * vv[j] + omb2 * gj * gj;
      const float denom = sqrtf(vv[j]) * inv_sqrt_bc2 + a.eps;
      pp[j] = pp[j] * decay - a.lr * (mm[j] * inv_bc1) * __frcp_rn(denom);
    }
    __stcs(p32v + i, make_float4(pp[0], pp[1], pp[2], pp[3]));
    __stcs(mv + i, make_float4(mm[0], mm[1], mm[2], mm[3]));
    __stcs(vv4 + i, make_float4(vv[0], vv[1], vv[2], vv[3]));
    if (a.p16) p16v[i] = make_uint2(pack_bf16x2(pp[0], pp[1]), pack_bf16x2(pp[2], pp[3]));
    if (a.zero_grad) {
      if (a.grad_is_bf16) __stcs(g16v + i, make_uint2(0u, 0u));
      else __stcs(g32v + i, make_float4(0.f, 0.f, 0.f, 0.f));
    }
  }
  // tail (n not a multiple of 4)
  const long long tail0 = n4 * 4;
  const long long gi = tail0 + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (gi < a.n) {
    float g = a.grad_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.grad)[gi])
                             : reinterpret_cast<const float*>(a.grad)[gi];
    if (a.zero_grad) {
      if (a.grad_is_bf16) reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(a.grad))[gi] = __float2bfloat16(0.f);
      else reinterpret_cast<float*>(const_cast<void*>(a.grad))[gi] = 0.f;
    }
    g *= gs;
    const float m = a.beta1 * a.m[gi] + (1.f - a.beta1) * g;
    const float v = a.beta2 * a.v[gi] + (1.f - a.beta2) * g * g;
    const float denom = sqrtf(v) * inv_sqrt_bc2 + a.eps;
    const float p = a.p32[gi] * (1.f - a.lr * a.weight_decay) - a.lr * (m * inv_bc1) / denom;
    a.p32[gi] = p;
    a.m[gi] = m;
    a.v[gi] = v;
    if (a.p16) reinterpret_cast<__nv_bfloat16*>(a.p16)[gi] = __float2bfloat16(p);
  }
}

__global__ void __launch_bounds__(256) sumsq_kernel(const void* x, int is_bf16, long long n, float* out,
                                                    float* __restrict__ partials) {
  __shared__ float red[8];
  float acc = 0.f;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  if (is_bf16) {
    const long long n8 = n / 8;
    const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(x);
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8; i += stride) {
      float f[8];
      load8(xb + i * 8, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += f[j] * f[j];
    }
    const long long gi = n8 * 8 + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (gi < n) {
      const float f = __bfloat162float(xb[gi]);
      acc += f * f;
    }
  } else {
    const long long n4 = n / 4;
    const float* xf = reinterpret_cast<const float*>(x);
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4; i += stride) {
      const float4 f = reinterpret_cast<const float4*>(xf)[i];
      acc += f.x * f.x + f.y * f.y + f.z * f.z + f.w * f.w;
    }
    const long long gi = n4 * 4 + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    if (gi < n) acc += xf[gi] * xf[gi];
  }
  acc = block_sum<256>(acc, red);
  if (threadIdx.x == 0) {
    if (partials != nullptr)
      partials[blockIdx.x] = acc;  // summed in block order by sumsq_final_kernel
    else
      atomicAdd(out, acc);
  }
}

// out += sum of `n` per-block partial sums, always in the same order (one block, fixed tree)
__global__ void __launch_bounds__(256) sumsq_final_kernel(const float* __restrict__ partials, int n,
                                                          float* __restrict__ out) {
  __shared__ float red[8];
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += 256) acc += partials[i];
  acc = block_sum<256>(acc, red);
  if (threadIdx.x == 0) *out += acc;
}

// ------------------------------------------------------------------------------------ cross-entropy
constexpr int CE_THREADS = 512;
__global__ void __launch_bounds__(CE_THREADS) cross_entropy_kernel(__nv_bfloat16* __restrict__ logits,
                                                                   const long long* __restrict__ targets,
                                                                   float* __restrict__ loss_sum,
                                                                   float* __restrict__ row_loss, long long rows, int V,
                                                                   long long ld, float grad_scale) {
  __shared__ float red[CE_THREADS / 32];
  __shared__ float s_max, s_sum;
  const long long row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const long long tgt = targets[row];
  const int nvec = V / 8;
  // online max / sum-exp per thread, then merged across the block
  float mx = -INFINITY, se = 0.f;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    float f[8];
    load8(lr + i * 8, f);
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
    if (lm > mx) {
      se *= __expf(mx - lm);
      mx = lm;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) se += __expf(f[j] - mx);
  }
  for (int c = nvec * 8 + threadIdx.x; c < V; c += CE_THREADS) {
    const float f = __bfloat162float(lr[c]);
    if (f > mx) {
      se *= __expf(mx - f);
      mx = f;
    }
    se += __expf(f - mx);
  }
  // block max
  float bm = warp_max(mx);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = bm;
  __syncthreads();
  if (warp == 0) {
    float t = lane < CE_THREADS / 32 ? red[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) s_max = t;
  }
  __syncthreads();
  bm = s_max;
  se = (mx == -INFINITY) ? 0.f : se * __expf(mx - bm);
  se = block_sum<CE_THREADS>(se, red);
  if (threadIdx.x == 0) s_sum = se;
  __syncthreads();
  const float lse = bm + logf(s_sum);
  const bool ignore = tgt < 0 || tgt >= V;
  if (threadIdx.x == 0) {
    const float l = ignore ? 0.f : lse - __bfloat162float(lr[tgt]);
    if (row_loss != nullptr)
      row_loss[row] = l;  // the caller sums the rows in a fixed order
    else if (!ignore)
      atomicAdd(loss_sum, l);
  }
  __syncthreads();
  const float gs = ignore ? 0.f : grad_scale;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    float f[8], o[8];
    load8(lr + i * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float p = __expf(f[j] - lse);
      o[j] = (p - ((i * 8 + j) == tgt ? 1.f : 0.f)) * gs;
    }
    store8(lr + i * 8, o);
  }
  for (int c = nvec * 8 + threadIdx.x; c < V; c += CE_THREADS) {
    const float p = __expf(__bfloat162float(lr[c]) - lse);
    lr[c] = __float2bfloat16((p - (c == tgt ? 1.f : 0.f)) * gs);
  }
}

// ------------------------------------------------------------------------------------ MoE plan
constexpr int PLAN_UNIT_SLOTS = 256;  // slots ranked by one warp
constexpr int PLAN_WARPS = 8;

__device__ __forceinline__ int plan_bin(const MoePlanArgs& a, long long slot) {
  const int e = a.topk_idx[slot] - a.expert_lo;
  if (e < 0 || e >= a.n_local) return -1;
  return a.per_k_bins ? e * a.K + static_cast<int>(slot % a.K) : e;
}

// pass 1: per-unit histogram.  hist[unit][bin]
__global__ void __launch_bounds__(PLAN_WARPS * 32) moe_plan_hist_kernel(const MoePlanArgs a, int nbins, int n_units) {
  const int unit = blockIdx.x * PLAN_WARPS + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (unit >= n_units) return;
  int* hist = a.scratch + static_cast<long long>(unit) * nbins;
  for (int b = lane; b < nbins; b += 32) hist[b] = 0;
  __syncwarp();
  const long long s0 = static_cast<long long>(unit) * PLAN_UNIT_SLOTS;
  for (int r = 0; r < PLAN_UNIT_SLOTS / 32; ++r) {
    const long long slot = s0 + r * 32 + lane;
    const int bin = slot < a.n_slots ? plan_bin(a, slot) : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, bin);
    if (bin >= 0 && (peers & ((1u << lane) - 1u)) == 0u) hist[bin] += __popc(peers);
    __syncwarp();
  }
}

// pass 2 (one CTA): exclusive prefix of hist over units within each bin, clipped bin totals,
// 128-row-padded expert offsets, tile table
__global__ void __launch_bounds__(1024) moe_plan_scan_kernel(const MoePlanArgs a, int nbins, int n_units) {
  int* hist = a.scratch;
  int* bin_base = a.scratch + static_cast<long long>(n_units) * nbins;
  int* bin_total = bin_base + nbins;
  __shared__ int s_part[1024];
  if (nbins <= 1024) {
    // all 1024 threads: thread = (chunk of units, bin).  Chunk sums, a short serial prefix over the chunks of the
    // bin in shared memory, then the exclusive prefix inside the chunk.  Loads of neighbouring threads are
    // neighbouring bins (coalesced) and independent of the running sum.
    int chunks = 1024 / nbins;
    if (chunks > n_units) chunks = n_units;
    const int per = (n_units + chunks - 1) / chunks;
    const int b = threadIdx.x % nbins, c = threadIdx.x / nbins;
    const bool live = c < chunks;
    const int u0 = c * per, u1 = min(n_units, u0 + per);
    int sum = 0;
    if (live) {
#pragma unroll 8
      for (int u = u0; u < u1; ++u) sum += hist[static_cast<long long>(u) * nbins + b];
    }
    s_part[threadIdx.x] = sum;
    __syncthreads();
    if (live) {
      int run = 0;
      for (int cc = 0; cc < c; ++cc) run += s_part[cc * nbins + b];
#pragma unroll 8
      for (int u = u0; u < u1; ++u) {
        const int cnt = hist[static_cast<long long>(u) * nbins + b];
        hist[static_cast<long long>(u) * nbins + b] = run;
        run += cnt;
      }
      if (c == chunks - 1) {  // the last chunk's running sum is the bin total
        for (int cc = c + 1; cc < chunks; ++cc) run += s_part[cc * nbins + b];
        bin_total[b] = (a.capacity > 0 && run > a.capacity) ? a.capacity : run;
      }
    }
  } else {
    for (int b = threadIdx.x; b < nbins; b += blockDim.x) {
      int run = 0;
      for (int u = 0; u < n_units; ++u) {
        const int c = hist[static_cast<long long>(u) * nbins + b];
        hist[static_cast<long long>(u) * nbins + b] = run;
        run += c;
      }
      bin_total[b] = (a.capacity > 0 && run > a.capacity) ? a.capacity : run;
    }
  }
  __syncthreads();
  __shared__ int s_total_rows;
  if (threadIdx.x == 0) {
    const int kb = a.per_k_bins ? a.K : 1;
    int off = 0;
    for (int e = 0; e < a.n_local; ++e) {
      a.group_offsets[e] = off;
      int cnt = 0;
      for (int k = 0; k < kb; ++k) {
        bin_base[e * kb + k] = off + cnt;
        cnt += bin_total[e * kb + k];
      }
      // rows that do not fit the buffer are dropped by the assign pass (and counted in `overflow`)
      const long long room = a.cap_rows - off;
      if (cnt > room) cnt = room > 0 ? static_cast<int>(room) : 0;
      a.counts_kept[e] = cnt;
      off += (cnt + 127) / 128 * 128;
      if (off > a.cap_rows) off = static_cast<int>(a.cap_rows / 128 * 128);
    }
    a.group_offsets[a.n_local] = off;
    *a.num_m_tiles = off / 128;
    s_total_rows = off;
  }
  __syncthreads();
  const int tiles = s_total_rows / 128;
  for (int t = threadIdx.x; t < tiles; t += blockDim.x) {
    const int row = t * 128;
    int lo = 0, hi = a.n_local;  // largest e with group_offsets[e] <= row
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (a.group_offsets[mid] <= row) lo = mid; else hi = mid;
    }
    a.tile_group[t] = lo;
  }
}

// pass 3: destination row of every slot
__global__ void __launch_bounds__(PLAN_WARPS * 32) moe_plan_assign_kernel(const MoePlanArgs a, int nbins, int n_units) {
  const int unit = blockIdx.x * PLAN_WARPS + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (unit >= n_units) return;
  int* hist = a.scratch + static_cast<long long>(unit) * nbins;
  const int* bin_base = a.scratch + static_cast<long long>(n_units) * nbins;
  const long long s0 = static_cast<long long>(unit) * PLAN_UNIT_SLOTS;
  for (int r = 0; r < PLAN_UNIT_SLOTS / 32; ++r) {
    const long long slot = s0 + r * 32 + lane;
    const int bin = slot < a.n_slots ? plan_bin(a, slot) : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, bin);
    int row = -1;
    if (bin >= 0) {
      const int rank = hist[bin] + __popc(peers & ((1u << lane) - 1u));
      if (a.capacity <= 0 || rank < a.capacity) row = bin_base[bin] + rank;
      if (row >= a.cap_rows) {  // the row buffer is full: drop the slot and report it
        row = -1;
        if (a.overflow) atomicAdd(a.overflow, 1);
      }
    }
    __syncwarp();
    if (bin >= 0 && (peers & ((1u << lane) - 1u)) == 0u) hist[bin] += __popc(peers);
    __syncwarp();
    if (slot < a.n_slots) {
      a.slot_row[slot] = row;
      if (row >= 0 && row < a.cap_rows) a.row_slot[row] = static_cast<int>(slot);
    }
  }
}

// ------------------------------------------------------------------------------------ gather / combine
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ row_slot,
                                   int slot_div, const float* __restrict__ slot_scale,
                                   __nv_bfloat16* __restrict__ out, long long cap_rows,
                                   const int* __restrict__ num_m_tiles, int H, long long ld_src, long long ld_out) {
  const long long n_rows = num_m_tiles ? min(static_cast<long long>(*num_m_tiles) * 128, cap_rows) : cap_rows;
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (long long r = blockIdx.x * static_cast<long long>(warps_per_block) + (threadIdx.x >> 5); r < n_rows;
       r += static_cast<long long>(gridDim.x) * warps_per_block) {
    const int slot = row_slot[r];
    __nv_bfloat16* o = out + r * ld_out;
    if (slot < 0) {
      for (int c = lane * 8; c < H; c += 256) *reinterpret_cast<uint4*>(o + c) = make_uint4(0u, 0u, 0u, 0u);
    } else {
      const __nv_bfloat16* s = src + static_cast<long long>(slot / slot_div) * ld_src;
      if (slot_scale == nullptr) {
        for (int c = lane * 8; c < H; c += 256) *reinterpret_cast<uint4*>(o + c) = *reinterpret_cast<const uint4*>(s + c);
      } else {
        const float sc = slot_scale[slot];
        for (int c = lane * 8; c < H; c += 256) {
          float f[8];
          load8(s + c, f);
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] *= sc;
          store8(o + c, f);
        }
      }
    }
  }
}

__global__ void combine_rows_kernel(const __nv_bfloat16* __restrict__ rows, const int* __restrict__ slot_row,
                                    const float* __restrict__ w, __nv_bfloat16* __restrict__ y, long long n_tokens,
                                    int K, int H, long long ld_rows, long long ld_y) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (long long t = blockIdx.x * static_cast<long long>(warps_per_block) + (threadIdx.x >> 5); t < n_tokens;
       t += static_cast<long long>(gridDim.x) * warps_per_block) {
    for (int c = lane * 8; c < H; c += 256) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int k = 0; k < K; ++k) {
        const int r = slot_row[t * K + k];
        if (r < 0) continue;
        const float wk = w ? w[t * K + k] : 1.f;
        float f[8];
        load8(rows + static_cast<long long>(r) * ld_rows + c, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += wk * f[j];
      }
      store8(y + t * ld_y + c, acc);
    }
  }
}

// Same sum for a compile-time K: the K (row, weight) pairs of a token are looked up once (lane k loads pair k, the
// warp shares them by shuffle) and the loads of all K rows of a column block are issued before the first use, so a
// lane keeps K x 16 bytes in flight instead of 16.  The order of the additions is that of the kernel above.
template <int KK>
__global__ void combine_rows_k_kernel(const __nv_bfloat16* __restrict__ rows, const int* __restrict__ slot_row,
                                      const float* __restrict__ w, __nv_bfloat16* __restrict__ y, long long n_tokens,
                                      int H, long long ld_rows, long long ld_y) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (long long t = blockIdx.x * static_cast<long long>(warps_per_block) + (threadIdx.x >> 5); t < n_tokens;
       t += static_cast<long long>(gridDim.x) * warps_per_block) {
    int my_r = -1;
    float my_w = 0.f;
    if (lane < KK) {
      my_r = slot_row[t * KK + lane];
      my_w = w ? w[t * KK + lane] : 1.f;
    }
    const __nv_bfloat16* src[KK];
    float wk[KK];
#pragma unroll
    for (int k = 0; k < KK; ++k) {
      const int r = __shfl_sync(0xffffffffu, my_r, k);
      wk[k] = __shfl_sync(0xffffffffu, my_w, k);
      src[k] = r >= 0 ? rows + static_cast<long long>(r) * ld_rows : nullptr;
    }
    for (int c = lane * 8; c < H; c += 256) {
      uint4 v[KK];
#pragma unroll
      for (int k = 0; k < KK; ++k)
        v[k] = src[k] != nullptr ? *reinterpret_cast<const uint4*>(src[k] + c) : make_uint4(0u, 0u, 0u, 0u);
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
      for (int k = 0; k < KK; ++k) {
        if (src[k] == nullptr) continue;  // a dropped slot adds nothing (and no signed zero)
        const float2 a = unpack_bf16x2(v[k].x), b = unpack_bf16x2(v[k].y), cc = unpack_bf16x2(v[k].z),
                     d = unpack_bf16x2(v[k].w);
        acc[0] += wk[k] * a.x; acc[1] += wk[k] * a.y; acc[2] += wk[k] * b.x; acc[3] += wk[k] * b.y;
        acc[4] += wk[k] * cc.x; acc[5] += wk[k] * cc.y; acc[6] += wk[k] * d.x; acc[7] += wk[k] * d.y;
      }
      store8(y + t * ld_y + c, acc);
    }
  }
}

__global__ void combine_bwd_w_kernel(const __nv_bfloat16* __restrict__ rows, const int* __restrict__ slot_row,
                                     const __nv_bfloat16* __restrict__ dy, float* __restrict__ dw, long long n_tokens,
                                     int K, int H, long long ld_rows, long long ld_dy) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long n_slots = n_tokens * K;
  for (long long s = blockIdx.x * static_cast<long long>(warps_per_block) + (threadIdx.x >> 5); s < n_slots;
       s += static_cast<long long>(gridDim.x) * warps_per_block) {
    const int r = slot_row[s];
    float acc = 0.f;
    if (r >= 0) {
      const __nv_bfloat16* a = rows + static_cast<long long>(r) * ld_rows;
      const __nv_bfloat16* b = dy + (s / K) * ld_dy;
      for (int c = lane * 8; c < H; c += 256) {
        float fa[8], fb[8];
        load8(a + c, fa);
        load8(b + c, fb);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += fa[j] * fb[j];
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) dw[s] = acc;
  }
}

inline unsigned grid_for(long long work_items, int per_block, int max_blocks) {
  long long b = (work_items + per_block - 1) / per_block;
  if (b < 1) b = 1;
  if (b > max_blocks) b = max_blocks;
  return static_cast<unsigned>(b);
}

}  // namespace

inline int rn_vec_for(int H) {
  const int per = RN_THREADS * 8;
  const int need = (H + per - 1) / per;
  return need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 8;
}

cudaError_t launch_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int H, float eps,
                               cudaStream_t stream) {
  if (H % 8 != 0 || H > RN_THREADS * 8 * 8 || rows <= 0) return cudaErrorInvalidValue;
  const unsigned grid = grid_for(rows, 1, 148 * 32);
  auto xb = reinterpret_cast<const __nv_bfloat16*>(x);
  auto wb = reinterpret_cast<const __nv_bfloat16*>(w);
  auto yb = reinterpret_cast<__nv_bfloat16*>(y);
  switch (rn_vec_for(H)) {
    case 1: rmsnorm_fwd_kernel<1><<<grid, RN_THREADS, 0, stream>>>(xb, wb, yb, rstd, rows, H, eps); break;
    case 2: rmsnorm_fwd_kernel<2><<<grid, RN_THREADS, 0, stream>>>(xb, wb, yb, rstd, rows, H, eps); break;
    case 4: rmsnorm_fwd_kernel<4><<<grid, RN_THREADS, 0, stream>>>(xb, wb, yb, rstd, rows, H, eps); break;
    default: rmsnorm_fwd_kernel<8><<<grid, RN_THREADS, 0, stream>>>(xb, wb, yb, rstd, rows, H, eps); break;
  }
  return cudaGetLastError();
}

long long rmsnorm_bwd_partial_rows(long long rows, int num_sms) {
  return grid_for(rows, 1, (num_sms > 0 ? num_sms : 148) * 4);  // one wave of persistent CTAs
}

cudaError_t launch_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw,
                               float* dw_partial, long long rows, int H, int num_sms, cudaStream_t stream) {
  if (H % 8 != 0 || H > RN_THREADS * 8 * 8 || rows <= 0) return cudaErrorInvalidValue;
  const unsigned grid = static_cast<unsigned>(rmsnorm_bwd_partial_rows(rows, num_sms));
  if (dw == nullptr) dw_partial = nullptr;
  auto dyb = reinterpret_cast<const __nv_bfloat16*>(dy);
  auto xb = reinterpret_cast<const __nv_bfloat16*>(x);
  auto wb = reinterpret_cast<const __nv_bfloat16*>(w);
  auto dxb = reinterpret_cast<__nv_bfloat16*>(dx);
  static bool configured = false;
  if (!configured) {  // the largest ring (H up to 8192) is above the default 48 KiB of dynamic shared memory
    cudaError_t e = cudaFuncSetAttribute(rmsnorm_bwd_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, rn_bwd_smem(8));
    if (e != cudaSuccess) return e;
    configured = true;
  }
  switch (rn_vec_for(H)) {
    case 1: rmsnorm_bwd_kernel<1><<<grid, RN_THREADS, rn_bwd_smem(1), stream>>>(dyb, xb, wb, rstd, dxb, dw, dw_partial, rows, H); break;
    case 2: rmsnorm_bwd_kernel<2><<<grid, RN_THREADS, rn_bwd_smem(2), stream>>>(dyb, xb, wb, rstd, dxb, dw, dw_partial, rows, H); break;
    case 4: rmsnorm_bwd_kernel<4><<<grid, RN_THREADS, rn_bwd_smem(4), stream>>>(dyb, xb, wb, rstd, dxb, dw, dw_partial, rows, H); break;
    default: rmsnorm_bwd_kernel<8><<<grid, RN_THREADS, rn_bwd_smem(8), stream>>>(dyb, xb, wb, rstd, dxb, dw, dw_partial, rows, H); break;
  }
  if (dw_partial != nullptr) {
    const unsigned slices = grid < 16u ? grid : 16u;
    colsum_stage1_kernel<<<dim3((H + 127) / 128, slices), 128, 0, stream>>>(dw_partial, static_cast<int>(grid), H);
    colsum_stage2_kernel<<<(H + 127) / 128, 128, 0, stream>>>(dw_partial, dw, static_cast<int>(slices), H);
  }
  return cudaGetLastError();
}

cudaError_t launch_rope(void* t, const float* cos_tab, const float* sin_tab, long long rows, int seq, int heads,
                        int head_dim, long long row_stride, int inverse, cudaStream_t stream) {
  if (head_dim % 16 != 0 || rows <= 0) return cudaErrorInvalidValue;
  const long long total = rows * heads * (head_dim / 16);
  rope_kernel<<<grid_for(total, 256, 148 * 16), 256, 0, stream>>>(reinterpret_cast<__nv_bfloat16*>(t), cos_tab, sin_tab,
                                                                  rows, seq, heads, head_dim, row_stride, inverse);
  return cudaGetLastError();
}

cudaError_t launch_qkv_grad_pack(const void* dq, const long long* dq_strides, const void* dk, const long long* dk_strides,
                                 const void* dv, const long long* dv_strides, void* out, const float* cos_tab,
                                 const float* sin_tab, long long batch, int seq, int nh, int nkv, int head_dim,
                                 cudaStream_t stream) {
  if (head_dim % 16 != 0 || batch <= 0 || seq <= 0 || nh <= 0 || nkv <= 0) return cudaErrorInvalidValue;
  auto mk = [](const void* p, const long long* st) {
    return QkvGradSrc{reinterpret_cast<const __nv_bfloat16*>(p), st[0], st[1], st[2]};
  };
  for (const long long* st : {dq_strides, dk_strides, dv_strides})
    if (st[0] % 8 != 0 || st[1] % 8 != 0 || st[2] % 8 != 0) return cudaErrorInvalidValue;  // 16-byte vector loads
  const long long rows = batch * seq;
  const long long total = rows * (nh + 2 * nkv) * (head_dim / 16);
  qkv_grad_pack_kernel<<<grid_for(total, 256, 148 * 16), 256, 0, stream>>>(
      mk(dq, dq_strides), mk(dk, dk_strides), mk(dv, dv_strides), reinterpret_cast<__nv_bfloat16*>(out), cos_tab,
      sin_tab, rows, seq, nh, nkv, head_dim);
  return cudaGetLastError();
}

cudaError_t launch_adamw(const AdamWArgs& a, cudaStream_t stream) {
  if (a.n <= 0) return cudaSuccess;
  adamw_kernel<<<grid_for(a.n / 4 + 1, 256, 148 * 16), 256, 0, stream>>>(a);
  return cudaGetLastError();
}

int sumsq_partial_count(long long n) { return n <= 0 ? 0 : static_cast<int>(grid_for(n / 8 + 1, 256, 148 * 8)); }

cudaError_t launch_sumsq(const void* x, int is_bf16, long long n, float* out, float* partials, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  const unsigned grid = static_cast<unsigned>(sumsq_partial_count(n));
  sumsq_kernel<<<grid, 256, 0, stream>>>(x, is_bf16, n, out, partials);
  if (partials != nullptr) sumsq_final_kernel<<<1, 256, 0, stream>>>(partials, static_cast<int>(grid), out);
  return cudaGetLastError();
}

cudaError_t launch_cross_entropy(void* logits, const long long* targets, float* loss_sum, float* row_loss,
                                 long long rows, int V, long long ld, float grad_scale, cudaStream_t stream) {
  if (rows <= 0) return cudaSuccess;
  if (ld % 8 != 0) return cudaErrorInvalidValue;
  cross_entropy_kernel<<<static_cast<unsigned>(rows), CE_THREADS, 0, stream>>>(
      reinterpret_cast<__nv_bfloat16*>(logits), targets, loss_sum, row_loss, rows, V, ld, grad_scale);
  return cudaGetLastError();
}

size_t moe_plan_scratch_words(long long n_slots, int n_local, int K, int per_k_bins) {
  const long long nbins = static_cast<long long>(n_local) * (per_k_bins ? K : 1);
  const long long n_units = (n_slots + PLAN_UNIT_SLOTS - 1) / PLAN_UNIT_SLOTS;
  return static_cast<size_t>(n_units * nbins + 2 * nbins);
}

cudaError_t launch_moe_plan(const MoePlanArgs& a, cudaStream_t stream) {
  if (a.n_slots <= 0 || a.n_local <= 0) return cudaErrorInvalidValue;
  const int nbins = a.n_local * (a.per_k_bins ? a.K : 1);
  const int n_units = static_cast<int>((a.n_slots + PLAN_UNIT_SLOTS - 1) / PLAN_UNIT_SLOTS);
  cudaError_t e = cudaMemsetAsync(a.row_slot, 0xFF, sizeof(int) * a.cap_rows, stream);
  if (e != cudaSuccess) return e;
  e = cudaMemsetAsync(a.tile_group, 0xFF, sizeof(int) * ((a.cap_rows + 127) / 128), stream);
  if (e != cudaSuccess) return e;
  const unsigned blocks = static_cast<unsigned>((n_units + PLAN_WARPS - 1) / PLAN_WARPS);
  moe_plan_hist_kernel<<<blocks, PLAN_WARPS * 32, 0, stream>>>(a, nbins, n_units);
  moe_plan_scan_kernel<<<1, 1024, 0, stream>>>(a, nbins, n_units);
  moe_plan_assign_kernel<<<blocks, PLAN_WARPS * 32, 0, stream>>>(a, nbins, n_units);
  return cudaGetLastError();
}

cudaError_t launch_gather_rows(const void* src, const int* row_slot, int slot_div, const float* slot_scale, void* out,
                               long long cap_rows, const int* num_m_tiles, int H, long long ld_src, long long ld_out,
                               cudaStream_t stream) {
  if (H % 8 != 0 || cap_rows <= 0 || slot_div <= 0) return cudaErrorInvalidValue;
  gather_rows_kernel<<<grid_for(cap_rows, 8, 148 * 8), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(src), row_slot, slot_div, slot_scale,
      reinterpret_cast<__nv_bfloat16*>(out), cap_rows, num_m_tiles, H, ld_src, ld_out);
  return cudaGetLastError();
}

cudaError_t launch_combine_rows(const void* rows, const int* slot_row, const float* w, void* y, long long n_tokens,
                                int K, int H, long long ld_rows, long long ld_y, cudaStream_t stream) {
  if (H % 8 != 0 || n_tokens <= 0) return cudaErrorInvalidValue;
  static const bool generic_only = [] {
    const char* v = std::getenv("CMOE_COMBINE_GENERIC");  // A/B switch: the kernel with a run-time K for every K
    return v != nullptr && v[0] != '\0' && v[0] != '0';
  }();
  if (!generic_only && (K == 8 || K == 6 || K == 4 || K == 2)) {
    const unsigned grid = grid_for(n_tokens, 8, 148 * 8);
    auto rb = reinterpret_cast<const __nv_bfloat16*>(rows);
    auto yb = reinterpret_cast<__nv_bfloat16*>(y);
    switch (K) {
      case 8: combine_rows_k_kernel<8><<<grid, 256, 0, stream>>>(rb, slot_row, w, yb, n_tokens, H, ld_rows, ld_y); break;
      case 6: combine_rows_k_kernel<6><<<grid, 256, 0, stream>>>(rb, slot_row, w, yb, n_tokens, H, ld_rows, ld_y); break;
      case 4: combine_rows_k_kernel<4><<<grid, 256, 0, stream>>>(rb, slot_row, w, yb, n_tokens, H, ld_rows, ld_y); break;
      default: combine_rows_k_kernel<2><<<grid, 256, 0, stream>>>(rb, slot_row, w, yb, n_tokens, H, ld_rows, ld_y); break;
    }
    return cudaGetLastError();
  }
  combine_rows_kernel<<<grid_for(n_tokens, 8, 148 * 8), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(rows), slot_row, w, reinterpret_cast<__nv_bfloat16*>(y), n_tokens, K, H,
      ld_rows, ld_y);
  return cudaGetLastError();
}

cudaError_t launch_combine_bwd_w(const void* rows, const int* slot_row, const void* dy, float* dw, long long n_tokens,
                                 int K, int H, long long ld_rows, long long ld_dy, cudaStream_t stream) {
  if (H % 8 != 0 || n_tokens <= 0) return cudaErrorInvalidValue;
  combine_bwd_w_kernel<<<grid_for(n_tokens * K, 8, 148 * 8), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(rows), slot_row, reinterpret_cast<const __nv_bfloat16*>(dy), dw, n_tokens,
      K, H, ld_rows, ld_dy);
  return cudaGetLastError();
}

}  // namespace cmoe
