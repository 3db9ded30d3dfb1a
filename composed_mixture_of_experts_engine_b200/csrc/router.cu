// Fused top-k router for sm_100a.
//
// Forward, one launch: gate GEMM (tokens [N,H] x gate_w [H,E]) on tcgen05 with the fp32 logits in
// tensor memory, then per token row (one thread per row, straight out of TMEM): fp32 softmax
// statistics, top-k with lowest-index tie break, renormalised gate weights, per-expert counts,
// per-expert probability sums (load-balance loss), z-loss, and a last-CTA finalisation that turns
// those sums into the loss values.  The tokens are read from HBM exactly once.
//
// Backward: the analytic gradient of the gate weights, load-balance loss and z-loss with respect
// to the logits (one warp per token); the two contractions with it (grad_tokens, grad_gate_w) run
// on the tcgen05 GEMM of gemm.cu.
//
// Counterpart in the reference: the Triton kernels _router_fwd_kernel / _router_bwd_kernel plus the
// bincount, the second logits GEMM for the z-loss and the two cuBLAS GEMMs of the backward
// (pkg/kernels/moe_router.py:102-251, 545-546, 690-734).
#include "router.cuh"

#include <cstdio>
#include <mutex>

#include "common.cuh"

namespace cmoe {

namespace {

constexpr int RT_BM = 128;
constexpr int RT_BK = 64;
constexpr int RT_A_BYTES = RT_BM * RT_BK * 2;  // 16 KiB
constexpr int RT_CHUNK_BYTES = 64 * RT_BK * 2;  // 8 KiB: 64 experts x 64 k
constexpr int RT_THREADS = 192;
constexpr int RT_MAX_STAGES = 8;
constexpr int RT_SMEM_BUDGET = 200 * 1024;

struct RouterParams {
  long long n_tokens;
  int H, E, K;
  int n_chunks;  // ceil(E / 64)
  int stages;
  int umma_n;  // E rounded up to 16
  int tmem_cols;
  float* logits;
  int* topk_idx;
  float* topk_w;
  float* lse;
  int* counts;
  float* mean_prob;
  float* stats;
  uint32_t* workspace;
  int* status;
  unsigned long long timeout_ns;
};

// sum v[i] over the 32 lanes of the warp for all 32 i at once (31 shuffles); afterwards lane L
// holds the total of column L in v[0]
__device__ __forceinline__ void warp_transpose_reduce(float (&v)[32], int lane) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < off; ++i) {
      const float send = upper ? v[i] : v[i + off];
      const float keep = upper ? v[i + off] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
}

__global__ void __launch_bounds__(RT_THREADS, 1)
router_fwd_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                  const RouterParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int b_bytes = p.n_chunks * RT_CHUNK_BYTES;
  const int stage_bytes = RT_A_BYTES + b_bytes;
  uint8_t* tail = smem + p.stages * stage_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);   // [RT_MAX_STAGES]
  uint64_t* empty_bar = full_bar + RT_MAX_STAGES;           // [RT_MAX_STAGES]
  uint64_t* tfull_bar = empty_bar + RT_MAX_STAGES;          // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfull_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_last = const_cast<int*>(abort_flag) + 1;
  // per-tile sums as 64-bit fixed point (integer adds commute: the result does not depend on the order of the warps)
  unsigned long long* s_prob = reinterpret_cast<unsigned long long*>(
      (reinterpret_cast<uintptr_t>(s_last + 1) + 7) & ~uintptr_t(7));  // [256]
  unsigned long long* s_z = s_prob + kRouterMaxExperts;
  int* s_cnt = reinterpret_cast<int*>(s_z + 1);  // [256]
  int* s_topi = s_cnt + kRouterMaxExperts;                      // [kRouterMaxTopK][128] chosen experts, one column per row
  float* s_topp = reinterpret_cast<float*>(s_topi + kRouterMaxTopK * 128);  // [kRouterMaxTopK][128] their probabilities

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long row0 = static_cast<long long>(blockIdx.x) * RT_BM;
  const int k_blocks = (p.H + RT_BK - 1) / RT_BK;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    *s_last = 0;
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tfull_bar, 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmW);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  WaitCtx wc;
  wc.abort_flag = abort_flag;
  wc.status = p.status;
  wc.timeout_ns = p.timeout_ns;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = 0; kb < k_blocks; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1u, wc, ST_TIMEOUT_SMEM_EMPTY)) break;
        mbar_arrive_expect_tx(&full_bar[stage], stage_bytes);
        uint8_t* a_dst = smem + stage * stage_bytes;
        uint8_t* b_dst = a_dst + RT_A_BYTES;
        tma_load_2d(a_dst, &tmX, &full_bar[stage], kb * RT_BK, static_cast<int>(row0));
        for (int j = 0; j < p.n_chunks; ++j)
          tma_load_2d(b_dst + j * RT_CHUNK_BYTES, &tmW, &full_bar[stage], 64 * j, kb * RT_BK);
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(RT_BM, p.umma_n, 0, 1);
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = 0; kb < k_blocks; ++kb) {
        if (!mbar_wait(&full_bar[stage], phase, wc, ST_TIMEOUT_SMEM_FULL)) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + stage * stage_bytes);
        const uint32_t b_addr = a_addr + RT_A_BYTES;
#pragma unroll
        for (int k = 0; k < RT_BK / 16; ++k) {
          const uint64_t ad = make_smem_desc_sw128(a_addr + k * 32, 16, 1024);
          const uint64_t bd = make_smem_desc_sw128(b_addr + k * 2048, RT_CHUNK_BYTES, 1024);
          umma_bf16_ss(tmem_base, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
        }
        umma_commit(&empty_bar[stage]);
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      umma_commit(tfull_bar);
    }
  } else {
    // ---------------------------------------------------------------- epilogue: one thread per token row
    const int et = threadIdx.x - 64;  // 0..127
    const int quad = warp & 3;
    const long long row = row0 + quad * 32 + lane;
    const bool row_ok = row < p.n_tokens;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const int E = p.E;
    const int nch = (E + 31) / 32;
    for (int e = et; e < kRouterMaxExperts; e += 128) {
      s_prob[e] = 0ull;
      s_cnt[e] = 0;
    }
    if (et == 0) *s_z = 0ull;
    asm volatile("bar.sync 1, 128;" ::: "memory");

    const bool ok = mbar_wait(tfull_bar, 0, wc, ST_TIMEOUT_TMEM_FULL);
    tc_fence_after();
    if (ok) {
      // pass 1: row maximum, and the logits go out to global memory
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < nch; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (c * 32 + j < E) mx = fmaxf(mx, __uint_as_float(r[j]));
        if (row_ok) {
          float* dst = p.logits + row * E + c * 32;
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            if (c * 32 + j < E)
              *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                                __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
        }
      }
      // pass 2: log-sum-exp
      float se = 0.f;
#pragma unroll 1
      for (int c = 0; c < nch; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (c * 32 + j < E) se += expf(__uint_as_float(r[j]) - mx);
      }
      const float lse = mx + logf(se);
      if (row_ok) p.lse[row] = lse;
      // pass 3: per-expert probability sums over the 128 rows of this tile
#pragma unroll 1
      for (int c = 0; c < nch; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c * 32, r);
        tmem_ld_wait();
        float pv[32];
#pragma unroll
        for (int j = 0; j < 32; ++j)
          pv[j] = (row_ok && (c * 32 + j < E)) ? expf(__uint_as_float(r[j]) - lse) : 0.f;
        warp_transpose_reduce(pv, lane);
        if (c * 32 + lane < E) atomicAdd(&s_prob[c * 32 + lane], __float2ull_rn(pv[0] * kRouterProbScale));
      }
      // pass 4: top-k by repeated arg-max over TMEM (already chosen experts are masked by bit sets).  The loops
      // over k and over the 32-expert chunks stay rolled: this code runs once per CTA, so every instruction is a
      // cold fetch, and eight unrolled copies of the compare block cost more in instruction fetches than they
      // save in loop overhead.  The K results wait in shared memory (one column per thread) for the renormalisation.
      uint32_t sel[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) sel[c] = 0u;
      float psum = 0.f;
#pragma unroll 1
      for (int kk = 0; kk < p.K; ++kk) {
        float best = -INFINITY;
        int bi = -1;
#pragma unroll 1
        for (int c = 0; c < nch; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_row + c * 32, r);
          tmem_ld_wait();
          uint32_t m = 0u;
#pragma unroll
          for (int q = 0; q < 8; ++q) m = (q == c) ? sel[q] : m;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float v = __uint_as_float(r[j]);
            const bool cand = (c * 32 + j < E) && (((m >> j) & 1u) == 0u);
            if (cand && (bi < 0 || v > best)) {
              best = v;
              bi = c * 32 + j;
            }
          }
        }
#pragma unroll
        for (int c = 0; c < 8; ++c)
          if (c == (bi >> 5)) sel[c] |= 1u << (bi & 31);
        const float pk = expf(best - lse);
        psum += pk;
        s_topi[kk * 128 + et] = bi;
        s_topp[kk * 128 + et] = pk;
      }
      if (row_ok) {
        const float inv = 1.f / psum;
#pragma unroll 1
        for (int kk = 0; kk < p.K; ++kk) {
          const int e = s_topi[kk * 128 + et];
          p.topk_idx[row * p.K + kk] = e;
          p.topk_w[row * p.K + kk] = s_topp[kk * 128 + et] * inv;
          atomicAdd(&s_cnt[e], 1);
        }
      }
      const float z = warp_sum(row_ok ? lse * lse : 0.f);
      if (lane == 0) atomicAdd(s_z, __float2ull_rn(z * kRouterZScale));
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    // flush this tile's sums; the last CTA to finish turns them into the loss values
    unsigned long long* ws_prob = reinterpret_cast<unsigned long long*>(p.workspace);
    unsigned long long* ws_z = ws_prob + E;
    int* ws_cnt = reinterpret_cast<int*>(ws_z + 1);
    unsigned int* ws_done = reinterpret_cast<unsigned int*>(ws_cnt + E);
    for (int e = et; e < E; e += 128) {
      if (s_prob[e] != 0ull) atomicAdd(&ws_prob[e], s_prob[e]);
      if (s_cnt[e] != 0) atomicAdd(&ws_cnt[e], s_cnt[e]);
    }
    if (et == 0) atomicAdd(ws_z, *s_z);
    __threadfence();
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (et == 0) {
      const unsigned int ticket = atomicAdd(ws_done, 1u);
      *s_last = (ticket == gridDim.x - 1) ? 1 : 0;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (*s_last && et < 32) {
      __threadfence();
      const float n_tok = static_cast<float>(p.n_tokens);
      float aux = 0.f, mxc = 0.f, sumc = 0.f;
      for (int e = lane; e < E; e += 32) {
        const float pr = static_cast<float>(static_cast<double>(__ldcg(&ws_prob[e])) / kRouterProbScale);
        const int cn = __ldcg(&ws_cnt[e]);
        p.counts[e] = cn;
        p.mean_prob[e] = pr / n_tok;
        aux += (static_cast<float>(cn) / (n_tok * p.K)) * (pr / n_tok);
        mxc = fmaxf(mxc, static_cast<float>(cn));
        sumc += static_cast<float>(cn);
        ws_prob[e] = 0ull;
        ws_cnt[e] = 0;
      }
      aux = warp_sum(aux);
      mxc = warp_max(mxc);
      sumc = warp_sum(sumc);
      if (lane == 0) {
        p.stats[0] = aux * E;
        p.stats[1] = static_cast<float>(static_cast<double>(__ldcg(ws_z)) / kRouterZScale) / n_tok;
        p.stats[2] = sumc > 0.f ? mxc / (sumc / E) : 1.f;
        p.stats[3] = sumc;
        *ws_z = 0ull;
        *ws_done = 0u;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag) {
      for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
}

// one warp per token
__global__ void router_bwd_kernel(const RouterBwdArgs a) {
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= a.n_tokens) return;
  const int E = a.E, K = a.K;
  const float* l = a.logits + row * E;
  const float lse = a.lse[row];
  const float ga = a.grad_aux ? *a.grad_aux : 0.f;
  const float gz = a.grad_z ? *a.grad_z : 0.f;
  const float n_tok = static_cast<float>(a.n_tokens);

  int idx[kRouterMaxTopK];
  float gw[kRouterMaxTopK];
  float S = 0.f, gwv = 0.f;
#pragma unroll
  for (int k = 0; k < kRouterMaxTopK; ++k) {
    idx[k] = -1;
    gw[k] = 0.f;
    if (k < K) {
      idx[k] = a.topk_idx[row * K + k];
      gw[k] = a.grad_w ? a.grad_w[row * K + k] : 0.f;
      const float pk = expf(l[idx[k]] - lse);
      S += pk;
      gwv += gw[k] * pk;
    }
  }
  const float invS = 1.f / S;
  const float aux_c = ga * E / (n_tok * n_tok * K);  // d(aux)/dp[t,i] = ga * E * (counts_i / (N K)) / N

  float pe[kRouterMaxExperts / 32], gp[kRouterMaxExperts / 32];
  float dot = 0.f;
#pragma unroll
  for (int q = 0; q < kRouterMaxExperts / 32; ++q) {
    const int e = q * 32 + lane;
    pe[q] = 0.f;
    gp[q] = 0.f;
    if (e < E) {
      pe[q] = expf(l[e] - lse);
      float g = aux_c * static_cast<float>(a.counts[e]);
#pragma unroll
      for (int k = 0; k < kRouterMaxTopK; ++k)
        if (k < K && idx[k] == e) g += gw[k] * invS - gwv * invS * invS;
      gp[q] = g;
      dot += g * pe[q];
    }
  }
  dot = warp_sum(dot);
  const float zc = gz * 2.f * lse / n_tok;
#pragma unroll
  for (int q = 0; q < kRouterMaxExperts / 32; ++q) {
    const int e = q * 32 + lane;
    if (e < E) {
      const float gl = pe[q] * (gp[q] - dot) + zc * pe[q];
      if (a.grad_logits_f32) a.grad_logits_f32[row * E + e] = gl;
      if (a.grad_logits_bf16)
        reinterpret_cast<__nv_bfloat16*>(a.grad_logits_bf16)[row * E + e] = __float2bfloat16(gl);
    }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn router_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

cudaError_t encode_bf16_2d(CUtensorMap* out, const void* ptr, long long rows, long long cols, long long ld,
                           int box_rows) {
  EncodeTiledFn enc = router_encode_fn();
  if (enc == nullptr) return cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0 || (ld * 2) % 16 != 0) return cudaErrorInvalidValue;
  cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t gstride[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estride[2] = {1u, 1u};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estride,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

}  // namespace

cudaError_t launch_router_fwd(const RouterFwdArgs& a, cudaStream_t stream) {
  if (a.E <= 0 || a.E > kRouterMaxExperts || a.E % 8 != 0 || a.K <= 0 || a.K > kRouterMaxTopK || a.K > a.E ||
      a.H % 8 != 0 || a.n_tokens <= 0)
    return cudaErrorInvalidValue;
  CUtensorMap tmX, tmW;
  cudaError_t e = encode_bf16_2d(&tmX, a.X, a.n_tokens, a.H, a.ldx, 128);
  if (e != cudaSuccess) return e;
  e = encode_bf16_2d(&tmW, a.Wg, a.H, a.E, a.E, 64);
  if (e != cudaSuccess) return e;

  RouterParams p;
  p.n_tokens = a.n_tokens;
  p.H = a.H;
  p.E = a.E;
  p.K = a.K;
  p.n_chunks = (a.E + 63) / 64;
  const int stage_bytes = RT_A_BYTES + p.n_chunks * RT_CHUNK_BYTES;
  int stages = RT_SMEM_BUDGET / stage_bytes;
  if (stages > RT_MAX_STAGES) stages = RT_MAX_STAGES;
  p.stages = stages;
  p.umma_n = ((a.E + 15) / 16) * 16;
  int cols = 32;
  while (cols < p.umma_n) cols <<= 1;
  p.tmem_cols = cols;
  p.logits = a.logits;
  p.topk_idx = a.topk_idx;
  p.topk_w = a.topk_w;
  p.lse = a.lse;
  p.counts = a.counts;
  p.mean_prob = a.mean_prob;
  p.stats = a.stats;
  p.workspace = a.workspace;
  p.status = a.status;
  p.timeout_ns = a.timeout_ns ? a.timeout_ns : kDefaultTimeoutNs;

  const int smem = stages * stage_bytes + 1024 + 512 + kRouterMaxExperts * (8 + 4) + kRouterMaxTopK * 128 * 8 + 64;
  static int configured_smem = 0;
  if (smem > configured_smem) {
    e = cudaFuncSetAttribute(router_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    configured_smem = smem;
  }
  const unsigned grid = static_cast<unsigned>((a.n_tokens + RT_BM - 1) / RT_BM);
  router_fwd_kernel<<<grid, RT_THREADS, smem, stream>>>(tmX, tmW, p);
  return cudaGetLastError();
}

cudaError_t launch_router_bwd(const RouterBwdArgs& a, cudaStream_t stream) {
  if (a.E <= 0 || a.E > kRouterMaxExperts || a.K <= 0 || a.K > kRouterMaxTopK || a.n_tokens <= 0)
    return cudaErrorInvalidValue;
  const int threads = 256;
  const long long warps = a.n_tokens;
  const unsigned grid = static_cast<unsigned>((warps * 32 + threads - 1) / threads);
  router_bwd_kernel<<<grid, threads, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace cmoe
