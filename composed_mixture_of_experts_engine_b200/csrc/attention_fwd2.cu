// Causal attention forward with two query tiles per CTA: 256 query rows share every K / V tile (half the L2 and
// shared-memory traffic per FLOP of the one-tile kernel in attention.cu), probabilities and output accumulators live
// in tensor memory.
//
// TMEM: S_a [0,128)  S_b [128,256)  O_a [256,256+HD)  O_b [384,384+HD).  P (bf16, two per 32-bit column, written
// with tcgen05.st) overwrites the first 64 columns of its tile's S and is the A operand of P V straight from tensor
// memory (tcgen05.mma with A in TMEM); O accumulates in TMEM across key tiles and is rescaled in place (tcgen05.ld /
// tcgen05.st) only when a row's maximum has grown by more than 2^8 since the value the probabilities are taken
// against was last moved.  Warp 0: TMA (Q twice, K and V rings).  Warp 1: MMA, in the order P V_a, S_a(next),
// P V_b, S_b(next), so that each tile's softmax runs under the other tile's products.  Warps 2-5: softmax of the
// upper query tile, one thread per row; warps 6-9: lower tile.  Every wait is bounded.
//
// Used by launch_attention_fwd for head dimension 128 and sequence lengths that are multiples of 256.
// The reference has no attention operator (pkg/models/moe.py:148-186).
#include <cuda.h>
#include <cuda_bf16.h>
#include "attention.cuh"
#include "common.cuh"

namespace cmoe {
namespace {
constexpr int BLK = 128;
constexpr int BLOCK_BYTES = BLK * 128;
constexpr int THREADS2 = 320;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.f;  // base-2: probabilities stay below 2^8 while the maximum is stale

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t block_addr, int k16) {
  return make_smem_desc_sw128(block_addr + static_cast<uint32_t>(k16) * 32u, 16, 1024);
}
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile_addr, int k16) {
  return make_smem_desc_sw128(tile_addr + static_cast<uint32_t>(k16) * 2048u, BLOCK_BYTES, 1024);
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

struct Fwd2Params {
  __nv_bfloat16* out;
  float* lse;
  int S, nh, nkv;
  float scale_log2;
  int* status;
  unsigned long long timeout_ns;
};

template <int HD>
struct Fwd2Smem {
  static constexpr int TILE_BYTES = (HD / 64) * BLOCK_BYTES;
  static constexpr int Q = 0;                   // [2]
  static constexpr int K = Q + 2 * TILE_BYTES;  // [2]
  static constexpr int V = K + 2 * TILE_BYTES;  // [2]
  static constexpr int BARS = V + 2 * TILE_BYTES;
  static constexpr int END = BARS + 192;
};

template <int HD>
__global__ void __launch_bounds__(THREADS2, 1)
attention_fwd2_kernel(const __grid_constant__ CUtensorMap tmQKV, const Fwd2Params p, const int smem_bytes) {
  using L = Fwd2Smem<HD>;
  constexpr int KB = HD / 64;
  constexpr int TILE_BYTES = L::TILE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  if (smem + L::END > smem_raw + smem_bytes) {
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, ST_BAD_ARGUMENT);
    return;
  }
  uint8_t* sQ = smem + L::Q;  // [2]: tile a, tile b
  uint8_t* sK = smem + L::K;  // [2]
  uint8_t* sV = smem + L::V;  // [2]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BARS);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;   // [2]
  uint64_t* k_empty = bars + 3;  // [2]
  uint64_t* v_full = bars + 5;   // [2]
  uint64_t* v_empty = bars + 7;  // [2]
  uint64_t* s_full = bars + 9;   // [2] per query tile
  uint64_t* p_full = bars + 11;  // [2] per query tile: P is in tensor memory and O carries the current maximum
  uint64_t* o_full = bars + 13;  // [2] per query tile: P V has been added to O
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int pair = gridDim.x - 1 - blockIdx.x;  // 256-row block of queries, long rows first
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int hk = h / (p.nh / p.nkv);
  const int n_a = 2 * pair + 1;  // key tiles of the upper query tile (the last one is its diagonal)
  const int n_b = 2 * pair + 2;
  const int row0 = b * p.S;
  const int q_col = h * HD;
  const int k_col = (p.nh + hk) * HD;
  const int v_col = (p.nh + p.nkv + hk) * HD;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 128);
      mbar_init(&o_full[s], 1);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmQKV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
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
      mbar_arrive_expect_tx(q_full, 2 * TILE_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
          tma_load_2d(sQ + t * TILE_BYTES + kb * BLOCK_BYTES, &tmQKV, q_full, q_col + 64 * kb,
                      row0 + pair * 2 * BLK + t * BLK);
      for (int i = 0; i <= n_b; ++i) {
        if (i < n_b) {
          const int st = i & 1;
          if (!mbar_wait(&k_empty[st], ((i >> 1) & 1) ^ 1u, wc, ST_TIMEOUT_SMEM_EMPTY)) break;
          mbar_arrive_expect_tx(&k_full[st], TILE_BYTES);
#pragma unroll
          for (int kb = 0; kb < KB; ++kb)
            tma_load_2d(sK + st * TILE_BYTES + kb * BLOCK_BYTES, &tmQKV, &k_full[st], k_col + 64 * kb, row0 + i * BLK);
        }
        if (i >= 1) {
          const int j = i - 1;
          const int st = j & 1;
          if (!mbar_wait(&v_empty[st], ((j >> 1) & 1) ^ 1u, wc, ST_TIMEOUT_SMEM_EMPTY)) break;
          mbar_arrive_expect_tx(&v_full[st], TILE_BYTES);
#pragma unroll
          for (int kb = 0; kb < KB; ++kb)
            tma_load_2d(sV + st * TILE_BYTES + kb * BLOCK_BYTES, &tmQKV, &v_full[st], v_col + 64 * kb, row0 + j * BLK);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(BLK, BLK, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(BLK, HD, 0, 1);
      auto issue_s = [&](int t, int i) {  // S_t = Q_t K_i^T; the caller has waited for K_i
        const uint32_t q_addr = smem_u32(sQ + t * TILE_BYTES);
        const uint32_t k_addr = smem_u32(sK + (i & 1) * TILE_BYTES);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss(tmem_base + t * BLK, desc_kmajor(q_addr + kb * BLOCK_BYTES, k),
                         desc_kmajor(k_addr + kb * BLOCK_BYTES, k), idesc_s, (kb | k) != 0 ? 1u : 0u);
        umma_commit(&s_full[t]);
      };
      auto issue_pv = [&](int t, int i) {  // O_t (+)= P_t V_i, P from tensor memory (two bf16 per column)
        const uint32_t v_addr = smem_u32(sV + (i & 1) * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16_ts(tmem_base + (2 + t) * BLK, tmem_base + t * BLK + k * 8, desc_mnmajor(v_addr, k), idesc_pv,
                       (i | k) != 0 ? 1u : 0u);
        umma_commit(&o_full[t]);
      };
      bool ok = mbar_wait(q_full, 0, wc, ST_TIMEOUT_SMEM_FULL) && mbar_wait(&k_full[0], 0, wc, ST_TIMEOUT_SMEM_FULL);
      if (ok) {
        tc_fence_after();
        issue_s(0, 0);
        issue_s(1, 0);
        umma_commit(&k_empty[0]);
      }
      for (int i = 0; ok && i < n_b; ++i) {
        const int st = i & 1;
        const int nx = i + 1;
        if (!mbar_wait(&v_full[st], (i >> 1) & 1, wc, ST_TIMEOUT_SMEM_FULL)) break;
        if (i < n_a) {
          if (!mbar_wait(&p_full[0], i & 1, wc, ST_TIMEOUT_TMEM_FULL)) break;
          tc_fence_after();
          issue_pv(0, i);
        }
        if (nx < n_b && !mbar_wait(&k_full[nx & 1], (nx >> 1) & 1, wc, ST_TIMEOUT_SMEM_FULL)) break;
        if (nx < n_a) {
          tc_fence_after();
          issue_s(0, nx);  // after P V of this tile in the pipe: S_a and P_a share columns
        }
        if (!mbar_wait(&p_full[1], i & 1, wc, ST_TIMEOUT_TMEM_FULL)) break;
        tc_fence_after();
        issue_pv(1, i);
        umma_commit(&v_empty[st]);
        if (nx < n_b) {
          issue_s(1, nx);
          umma_commit(&k_empty[nx & 1]);
        }
      }
    }
  } else {
    const int quad = warp & 3;
    const int t = (warp - 2) >> 2;  // 0: upper query tile, 1: lower
    const int n_t = t == 0 ? n_a : n_b;
    const int r = quad * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_base + t * BLK;
    const uint32_t o_tmem = tmem_base + lane_base + (2 + t) * BLK;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int i = 0; i < n_t; ++i) {
      if (!mbar_wait(&s_full[t], i & 1, wc, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int limit = (i == n_t - 1) ? r : BLK;
      uint32_t v[32];
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        tmem_ld_32x32b_x32(s_tmem + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) mx = fmaxf(mx, (c * 32 + j <= limit) ? __uint_as_float(v[j]) : -INFINITY);
      }
      // The maximum that the probabilities are taken against moves only when the row maximum has grown by more
      // than 2^8 since it was last moved: O in tensor memory is rescaled rarely
      const float m_new = fmaxf(m_used, mx * p.scale_log2);
      const bool grow = (m_new - m_used) > kRescaleThreshold;
      float alpha = 1.f;
      if (grow) {
        alpha = ex2_approx(m_used - m_new);
        m_used = m_new;
      }
      uint32_t w[64];
      float lsum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        tmem_ld_32x32b_x32(s_tmem + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          float p0 = ex2_approx(fmaf(__uint_as_float(v[j]), p.scale_log2, -m_used));
          float p1 = ex2_approx(fmaf(__uint_as_float(v[j + 1]), p.scale_log2, -m_used));
          if (c * 32 + j > limit) p0 = 0.f;
          if (c * 32 + j + 1 > limit) p1 = 0.f;
          lsum += p0 + p1;
          w[c * 16 + (j >> 1)] = pack_bf16x2(p0, p1);
        }
      }
      l = fmaf(l, alpha, lsum);
      if (i > 0) {
        if (!mbar_wait(&o_full[t], (i - 1) & 1, wc, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, grow)) {
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            tmem_ld_32x32b_x32(o_tmem + c * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * alpha);
            tmem_st_32x32b_x32(o_tmem + c * 32, v);
          }
        }
      }
      {
        uint32_t lo[32], hi[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          lo[j] = w[j];
          hi[j] = w[32 + j];
        }
        tmem_st_32x32b_x32(s_tmem, lo);
        tmem_st_32x32b_x32(s_tmem + 32, hi);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_full[t]);
    }
    if (ok && mbar_wait(&o_full[t], (n_t - 1) & 1, wc, ST_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      const float inv = 1.f / l;
      const long long grow_ = static_cast<long long>(row0) + pair * 2 * BLK + t * BLK + r;
      __nv_bfloat16* dst = p.out + (grow_ * p.nh + h) * HD;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(o_tmem + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 o;
          o.x = pack_bf16x2(__uint_as_float(v[j]) * inv, __uint_as_float(v[j + 1]) * inv);
          o.y = pack_bf16x2(__uint_as_float(v[j + 2]) * inv, __uint_as_float(v[j + 3]) * inv);
          o.z = pack_bf16x2(__uint_as_float(v[j + 4]) * inv, __uint_as_float(v[j + 5]) * inv);
          o.w = pack_bf16x2(__uint_as_float(v[j + 6]) * inv, __uint_as_float(v[j + 7]) * inv);
          *reinterpret_cast<uint4*>(dst + c * 32 + j) = o;
        }
      }
      p.lse[(static_cast<long long>(b) * p.nh + h) * p.S + pair * 2 * BLK + t * BLK + r] = (m_used + log2f(l)) * kLn2;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template __global__ void attention_fwd2_kernel<128>(const __grid_constant__ CUtensorMap, const Fwd2Params, const int);
}  // namespace
}  // namespace cmoe

// ---- C entry point (raw pointers; also what launch_attention_fwd calls): returns a cudaError_t ----
#include <cstdio>
namespace {
typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
}
extern "C" int cmoe_attention_fwd2(const void* qkv, void* out, float* lse, int B, int S, int nh, int nkv, int hd,
                                   int* status, unsigned long long timeout_ns, void* stream) {
  using namespace cmoe;
  if (S % 256 != 0 || hd != 128 || nkv <= 0 || nh % nkv != 0 || B <= 0 || B > 65535 || nh > 65535)
    return (int)cudaErrorInvalidValue;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn)
    return (int)cudaErrorNotSupported;
  const long long rows = (long long)B * S, cols = (long long)(nh + 2 * nkv) * hd;
  CUtensorMap tm;
  cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64u, 128u};
  cuuint32_t estride[2] = {1u, 1u};
  if (reinterpret_cast<EncodeTiledFn2>(fn)(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(qkv), gdim,
                                           gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return (int)cudaErrorInvalidValue;
  Fwd2Params p;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.S = S;
  p.nh = nh;
  p.nkv = nkv;
  p.scale_log2 = 1.4426950408889634f / sqrtf((float)hd);
  p.status = status;
  p.timeout_ns = timeout_ns ? timeout_ns : kDefaultTimeoutNs;
  dim3 grid(S / 256, nh, B);
  cudaError_t e;
  constexpr int smem = Fwd2Smem<128>::END + 1024;
  e = cudaFuncSetAttribute(attention_fwd2_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  attention_fwd2_kernel<128><<<grid, THREADS2, smem, (cudaStream_t)stream>>>(tm, p, smem);
  return (int)cudaGetLastError();
}
