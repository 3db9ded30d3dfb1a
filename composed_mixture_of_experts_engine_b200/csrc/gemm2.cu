// Two-SM variant of the tcgen05 GEMM (`tcgen05.mma.cta_group::2`): a cluster of two CTAs on neighbouring SMs works on
// one 256 x 256 output tile.  Each CTA loads its own 128 rows of A and its own 128-column half of B (ordinary TMA
// loads, every CTA its own, no cluster broadcast), the leader CTA issues one MMA per 16 k that reads both CTAs'
// shared memory and accumulates 128 rows in each CTA's tensor memory.  Per CTA and k-block that is 32 KiB of
// operands for 128 x 256 x 64 multiply-adds instead of the 48 KiB of the one-CTA kernel, so the L2 -> SM traffic per
// FLOP drops by a third and six stages fit where four did.
//
// Scope: dense GEMMs and the grouped-K weight-gradient GEMMs with plain (staged, TMA-stored or TMA-reduced) results.
// Everything that needs the fused epilogues, the row pull or the scatter stays on the one-CTA kernel in gemm.cu.
// The host side sends every launch that qualifies here (`CMOE_GEMM_2CTA=0` keeps them on the one-CTA kernel).
// Measured on a B200: dense 8192^3 1543 TFLOP/s against 1407 for the one-CTA kernel (cuBLAS in the same run: 1707),
// grouped weight gradient with fp32 accumulation 1352 against 1144.
//
// CTA layout (192 threads): warp 0 TMA producer, warp 1 TMEM allocation (both CTAs) + MMA issue (leader only),
// warps 2..5 epilogue of this CTA's 128 rows.  Barriers:
//   full[s]   in the leader: one arrival with the byte count of both CTAs' loads; both CTAs' TMA loads complete on it
//   empty[s]  in each CTA: the leader's MMA commits to its own and to the peer's barrier
//   tfull[a]  in each CTA: committed by the leader to both when an accumulator is complete
//   tempty[a] in the leader: 256 arrivals, the epilogue threads of both CTAs
// Every wait is bounded as in gemm.cu; a wait that runs out ends the kernel normally with a status code.
#include "gemm.cuh"

#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace cmoe {

namespace {

constexpr int T_BM = 256;   // tile rows (128 per CTA)
constexpr int T_BN = 256;   // tile columns (each CTA loads 128 of B's rows / columns)
constexpr int T_BK = 64;
constexpr int T_STAGES = 6;
constexpr int T_A_BYTES = 128 * T_BK * 2;  // 16 KiB
constexpr int T_B_BYTES = 128 * T_BK * 2;  // 16 KiB
constexpr int T_STAGE_BYTES = T_A_BYTES + T_B_BYTES;
constexpr int T_CHUNK_BYTES = 64 * T_BK * 2;  // one 64 x 64 bf16 box of an MN-major operand
constexpr int T_STAGING_BUF = 128 * 128;
constexpr int T_STAGING = 2 * T_STAGING_BUF;
constexpr int T_THREADS = 192;
constexpr int T_TMEM_COLS = 512;
constexpr int T_SMEM = T_STAGES * T_STAGE_BYTES + T_STAGING + 1024 + 256;
constexpr int T_SWIZZLE = 4;  // band of row tiles walked together
constexpr int T_EPI_FIRST = 64;

struct K2Params {
  int mode, M, N, K, groups;
  int a_mn, b_mn;
  const int* group_offsets;
  int d_fp32, reduce;  // reduce: TMA reduce-add (fp32 accumulate) instead of store
  int* status;
  unsigned long long timeout_ns;
};

struct Tile2 {
  int m0, n0, group, a_k0, b_k0, k_blocks;
};

__device__ __forceinline__ Tile2 decode2(const K2Params& p, int t, int m_tiles, int n_tiles) {
  Tile2 ti;
  int g = 0;
  if (p.mode == GEMM_GROUPED_K) {
    g = t / (m_tiles * n_tiles);
    t -= g * m_tiles * n_tiles;
  }
  const int band = t / (T_SWIZZLE * n_tiles);
  const int r = t - band * T_SWIZZLE * n_tiles;
  const int band_rows = min(T_SWIZZLE, m_tiles - band * T_SWIZZLE);
  ti.m0 = (band * T_SWIZZLE + r % band_rows) * T_BM;
  ti.n0 = (r / band_rows) * T_BN;
  ti.group = g;
  if (p.mode == GEMM_GROUPED_K) {
    const int r0 = p.group_offsets[g], r1 = p.group_offsets[g + 1];
    ti.a_k0 = ti.b_k0 = r0;
    ti.k_blocks = (r1 - r0 + T_BK - 1) / T_BK;
  } else {
    ti.a_k0 = ti.b_k0 = 0;
    ti.k_blocks = (p.K + T_BK - 1) / T_BK;
  }
  return ti;
}

// ---- cluster / two-SM PTX -------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_addr), "r"(rank));
  return a;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load of this CTA's operand piece whose bytes are counted on a barrier that may live in the peer CTA
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* tmap, uint32_t bar_cluster_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// arrives once on the barrier at `cluster_addr` (own or peer CTA) when all MMAs issued so far have completed
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}
__device__ __forceinline__ void umma_bf16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                  uint32_t accumulate) {
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(T_THREADS, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
             const __grid_constant__ CUtensorMap tmD, const K2Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + T_STAGES * T_A_BYTES;
  uint8_t* stg = smem + T_STAGES * T_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + T_STAGES * T_STAGE_BYTES + T_STAGING);
  uint64_t* full_bar = bars;                    // [T_STAGES]  (used in the leader)
  uint64_t* empty_bar = bars + T_STAGES;        // [T_STAGES]
  uint64_t* tfull_bar = bars + 2 * T_STAGES;    // [2]
  uint64_t* tempty_bar = bars + 2 * T_STAGES + 2;  // [2]       (used in the leader)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * T_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0: leader (issues the MMAs), 1: peer
  const bool leader = cta == 0;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < T_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 256);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmD);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, T_TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anybody signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  WaitCtx wc;
  wc.abort_flag = abort_flag;
  wc.status = p.status;
  wc.timeout_ns = p.timeout_ns;

  const int m_tiles = (p.M + T_BM - 1) / T_BM;
  const int n_tiles = (p.N + T_BN - 1) / T_BN;
  const int n_total = (p.mode == GEMM_GROUPED_K ? p.groups : 1) * m_tiles * n_tiles;
  const int cluster_id = blockIdx.x >> 1;
  const int n_clusters = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      const int moff = static_cast<int>(cta) * 128;  // this CTA's rows of A and its half of B
      for (int t = cluster_id; t < n_total; t += n_clusters) {
        const Tile2 ti = decode2(p, t, m_tiles, n_tiles);
        if (ti.k_blocks == 0) continue;
        for (int kb = 0; kb < ti.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, wc, ST_TIMEOUT_SMEM_EMPTY)) break;
          const uint32_t fb = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * T_STAGE_BYTES);
          uint8_t* a_dst = sA + stage * T_A_BYTES;
          uint8_t* b_dst = sB + stage * T_B_BYTES;
          const int k = kb * T_BK;
          if (p.a_mn) {
            tma_load_2d_pair(a_dst, &tmA, fb, ti.m0 + moff, ti.a_k0 + k);
            tma_load_2d_pair(a_dst + T_CHUNK_BYTES, &tmA, fb, ti.m0 + moff + 64, ti.a_k0 + k);
          } else {
            tma_load_2d_pair(a_dst, &tmA, fb, ti.a_k0 + k, ti.m0 + moff);
          }
          if (p.b_mn) {
            tma_load_2d_pair(b_dst, &tmB, fb, ti.n0 + moff, ti.b_k0 + k);
            tma_load_2d_pair(b_dst + T_CHUNK_BYTES, &tmB, fb, ti.n0 + moff + 64, ti.b_k0 + k);
          } else {
            tma_load_2d_pair(b_dst, &tmB, fb, ti.b_k0 + k, ti.n0 + moff);
          }
          if (++stage == T_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (*abort_flag) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader && lane == 0) {
      const uint32_t idesc = make_idesc_bf16(T_BM, T_BN, p.a_mn, p.b_mn);
      const uint32_t a_lbo = p.a_mn ? T_CHUNK_BYTES : 16;
      const uint32_t b_lbo = p.b_mn ? T_CHUNK_BYTES : 16;
      const uint32_t a_kstep = p.a_mn ? 2048u : 32u;
      const uint32_t b_kstep = p.b_mn ? 2048u : 32u;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = cluster_id; t < n_total; t += n_clusters) {
        const Tile2 ti = decode2(p, t, m_tiles, n_tiles);
        if (ti.k_blocks == 0) continue;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, wc, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * T_BN;
        for (int kb = 0; kb < ti.k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, wc, ST_TIMEOUT_SMEM_FULL)) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + stage * T_A_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * T_B_BYTES);
#pragma unroll
          for (int k = 0; k < T_BK / 16; ++k) {
            const uint64_t ad = make_smem_desc_sw128(a_addr + k * a_kstep, a_lbo, 1024);
            const uint64_t bd = make_smem_desc_sw128(b_addr + k * b_kstep, b_lbo, 1024);
            umma_bf16_ss_pair(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // the stage is free in both CTAs once these MMAs have read it
          const uint32_t eb = smem_u32(&empty_bar[stage]);
          umma_commit_pair(eb);
          umma_commit_pair(map_to_cta(eb, 1));
          if (++stage == T_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        const uint32_t tb = smem_u32(&tfull_bar[acc]);
        umma_commit_pair(tb);
        umma_commit_pair(map_to_cta(tb, 1));
        if (*abort_flag) break;
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (this CTA's 128 rows)
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const int sw = row_in_tile & 7;
    const int unit_cols = p.d_fp32 ? 32 : 64;
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t stage_ctr = 0;
    for (int t = cluster_id; t < n_total; t += n_clusters) {
      const Tile2 ti = decode2(p, t, m_tiles, n_tiles);
      const int row0 = ti.m0 + static_cast<int>(cta) * 128;
      const bool have_acc = ti.k_blocks != 0;
      if (!have_acc && p.reduce) continue;  // adding zero: nothing to do
      bool ok = true;
      if (have_acc) {
        ok = mbar_wait(&tfull_bar[acc], acc_phase, wc, ST_TIMEOUT_TMEM_FULL);
        tc_fence_after();
      }
      const uint32_t t_acc = tmem_base + acc * T_BN + lane_base;
      bool any_bad = false;
#pragma unroll 1
      for (int u = 0; u < T_BN / unit_cols; ++u) {
        const int col0 = ti.n0 + u * unit_cols;
        if (col0 >= p.N) break;  // uniform
        uint8_t* buf = stg + (stage_ctr & 1) * T_STAGING_BUF;
        uint8_t* myrow = buf + row_in_tile * 128;
        if (ok) {
          if (p.d_fp32) {
            uint32_t r[32];
            if (have_acc) {
              tmem_ld_32x32b_x32(t_acc + u * 32, r);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) r[j] = 0u;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<uint4*>(myrow + ((j ^ sw) << 4)) =
                  make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
          } else {
            uint32_t r0[32], r1[32];
            if (have_acc) {
              tmem_ld_32x32b_x32(t_acc + u * 64, r0);
              tmem_ld_32x32b_x32(t_acc + u * 64 + 32, r1);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) r0[j] = r1[j] = 0u;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r0[8 * j]), __uint_as_float(r0[8 * j + 1]));
              o.y = pack_bf16x2(__uint_as_float(r0[8 * j + 2]), __uint_as_float(r0[8 * j + 3]));
              o.z = pack_bf16x2(__uint_as_float(r0[8 * j + 4]), __uint_as_float(r0[8 * j + 5]));
              o.w = pack_bf16x2(__uint_as_float(r0[8 * j + 6]), __uint_as_float(r0[8 * j + 7]));
              *reinterpret_cast<uint4*>(myrow + ((j ^ sw) << 4)) = o;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r1[8 * j]), __uint_as_float(r1[8 * j + 1]));
              o.y = pack_bf16x2(__uint_as_float(r1[8 * j + 2]), __uint_as_float(r1[8 * j + 3]));
              o.z = pack_bf16x2(__uint_as_float(r1[8 * j + 4]), __uint_as_float(r1[8 * j + 5]));
              o.w = pack_bf16x2(__uint_as_float(r1[8 * j + 6]), __uint_as_float(r1[8 * j + 7]));
              *reinterpret_cast<uint4*>(myrow + (((j + 4) ^ sw) << 4)) = o;
            }
          }
        }
        fence_proxy_async_smem();
        if (threadIdx.x == T_EPI_FIRST) bulk_wait_group_read<0>();
        {
          const int bad = (!ok || *abort_flag) ? 1 : 0;
          int any;
          asm volatile(
              "{\n\t.reg .pred q, r;\n\tsetp.ne.s32 q, %1, 0;\n\tbar.red.or.pred r, 1, 128, q;\n\t"
              "selp.s32 %0, 1, 0, r;\n\t}"
              : "=r"(any)
              : "r"(bad)
              : "memory");
          any_bad = any != 0;
        }
        if (any_bad) break;
        if (threadIdx.x == T_EPI_FIRST && row0 < p.M) {
          const int zgrp = (p.mode == GEMM_GROUPED_K) ? ti.group : 0;
          if (p.reduce)
            tma_reduce_add_3d(&tmD, buf, col0, row0, zgrp);
          else
            tma_store_3d(&tmD, buf, col0, row0, zgrp);
          bulk_commit_group();
        }
        ++stage_ctr;
      }
      if (have_acc) {
        // the leader's MMA warp may reuse this accumulator once all 256 epilogue threads of the pair have read it
        tc_fence_before();
        mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[acc]), 0));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (any_bad) break;
    }
    if (threadIdx.x == T_EPI_FIRST) bulk_wait_group<0>();
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves (or frees tensor memory) while the other may still touch it
  if (warp == 1) {
    if (*abort_flag) {
      for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, T_TMEM_COLS);
  }
}

}  // namespace

// bf16 row-major [rows, cols], box 64 columns x box_rows rows, 128-byte swizzle (same layout as gemm.cu's operand maps)
static cudaError_t encode_operand_map(CUtensorMap* out, const void* ptr, long long rows, long long cols, long long ld,
                                      int box_rows);
static cudaError_t encode_output_map(CUtensorMap* out, const void* ptr, int fp32, long long groups, long long rows,
                                     long long cols, long long ld, long long gstride);

typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn2 encode_fn2() {
  static EncodeTiledFn2 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn2>(ptr);
  });
  return fn;
}

static cudaError_t encode_operand_map(CUtensorMap* out, const void* ptr, long long rows, long long cols, long long ld,
                                      int box_rows) {
  EncodeTiledFn2 enc = encode_fn2();
  if (enc == nullptr) return cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0 || (ld * 2) % 16 != 0 || cols <= 0 || rows <= 0)
    return cudaErrorInvalidValue;
  cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t gstride[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estride[2] = {1u, 1u};
  return enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estride,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
             ? cudaSuccess
             : cudaErrorInvalidValue;
}

static cudaError_t encode_output_map(CUtensorMap* out, const void* ptr, int fp32, long long groups, long long rows,
                                     long long cols, long long ld, long long gstride) {
  EncodeTiledFn2 enc = encode_fn2();
  if (enc == nullptr) return cudaErrorNotSupported;
  const long long es = fp32 ? 4 : 2;
  cuuint64_t gdim[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(groups)};
  cuuint64_t gstr[2] = {static_cast<cuuint64_t>(ld * es), static_cast<cuuint64_t>(gstride * es)};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(128 / es), 128u, 1u};
  cuuint32_t estride[3] = {1u, 1u, 1u};
  return enc(out, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
             const_cast<void*>(ptr), gdim, gstr, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS
             ? cudaSuccess
             : cudaErrorInvalidValue;
}

bool gemm_2cta_supported(const GemmArgs& a) {
  if (a.epilogue != EPI_STORE || a.scatter_row_slot != nullptr || a.pull_row_slot != nullptr ||
      a.ready_flags != nullptr)
    return false;
  if (a.mode == GEMM_DENSE) {
    if (a.a_mn) return false;
  } else if (a.mode == GEMM_GROUPED_K) {
    if (!(a.a_mn && a.b_mn)) return false;
  } else {
    return false;
  }
  if (a.accumulate && !a.d_fp32) return false;
  if (a.N % 8 != 0 || a.N <= 0 || a.M <= 0) return false;
  const long long es = a.d_fp32 ? 4 : 2;
  const long long gstride = a.mode == GEMM_GROUPED_K ? a.d_group_stride : static_cast<long long>(a.M) * a.ldd;
  return (reinterpret_cast<uintptr_t>(a.D) & 15u) == 0 && (a.ldd * es) % 16 == 0 && (gstride * es) % 16 == 0 &&
         a.ldd >= a.N;
}

cudaError_t launch_gemm_2cta(const GemmArgs& a, cudaStream_t stream) {
  if (!gemm_2cta_supported(a)) return cudaErrorInvalidValue;
  CUtensorMap tmA, tmB, tmD;
  cudaError_t e = encode_operand_map(&tmA, a.A, a.a_rows, a.a_cols, a.a_ld, a.a_mn ? 64 : 128);
  if (e != cudaSuccess) return e;
  e = encode_operand_map(&tmB, a.B, a.b_rows, a.b_cols, a.b_ld, a.b_mn ? 64 : 128);
  if (e != cudaSuccess) return e;
  const long long groups = a.mode == GEMM_GROUPED_K ? a.groups : 1;
  const long long gstride = a.mode == GEMM_GROUPED_K ? a.d_group_stride : static_cast<long long>(a.M) * a.ldd;
  e = encode_output_map(&tmD, a.D, a.d_fp32, groups, a.M, a.N, a.ldd, gstride);
  if (e != cudaSuccess) return e;

  K2Params kp;
  kp.mode = a.mode;
  kp.M = a.M;
  kp.N = a.N;
  kp.K = a.K;
  kp.groups = a.groups;
  kp.a_mn = a.a_mn;
  kp.b_mn = a.b_mn;
  kp.group_offsets = a.group_offsets;
  kp.d_fp32 = a.d_fp32;
  kp.reduce = a.accumulate;
  kp.status = a.status;
  kp.timeout_ns = a.timeout_ns ? a.timeout_ns : kDefaultTimeoutNs;

  int num_sms = a.num_sms;
  if (num_sms <= 0) {
    int dev = 0;
    e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    e = cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
  }
  const long long m_tiles = (a.M + T_BM - 1) / T_BM, n_tiles = (a.N + T_BN - 1) / T_BN;
  const long long tiles = m_tiles * n_tiles * groups;
  if (tiles <= 0) return cudaSuccess;
  long long clusters = num_sms / 2;
  if (tiles < clusters) clusters = tiles;
  static bool configured = false;
  if (!configured) {
    e = cudaFuncSetAttribute(gemm2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T_SMEM);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  gemm2_kernel<<<static_cast<unsigned>(2 * clusters), T_THREADS, T_SMEM, stream>>>(tmA, tmB, tmD, kp);
  return cudaGetLastError();
}

}  // namespace cmoe
