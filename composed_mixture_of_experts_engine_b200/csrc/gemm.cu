// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma with
// the fp32 accumulator in tensor memory -> tcgen05.ld epilogue.  One kernel serves the dense
// projections, the grouped expert GEMMs (rows grouped in 128-row tiles per expert), the grouped
// weight-gradient GEMMs (contraction over each expert's rows) and the fused SwiGLU epilogues.
//
// Replaces the per-expert Python loop of three cuBLAS calls in the reference
// (pkg/distributed/moe_layer.py:197-198, 327-337) with one launch per GEMM of the layer.
//
// CTA layout (192 threads, one CTA per SM):
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocation + MMA issue (one lane)
//   warps 2..5  epilogue: each warp owns the TMEM lane quadrant (warp_id % 4)
// Tile 128 x 256 x 64, 4 shared-memory stages (48 KiB each), two accumulators of 256 TMEM
// columns so that the epilogue of tile i overlaps the main loop of tile i+1.
// Plain results leave through a 32 KiB swizzled staging area and TMA: `cp.async.bulk.tensor` stores, or
// `cp.reduce.async.bulk.tensor ... add` when the fp32 result accumulates into global memory (weight gradients),
// so the SM never reads the old values; rows that scatter to other ranks are copied out of the staging area
// with whole-row coalesced stores.  The SwiGLU epilogues use the same area in 64-byte-swizzled pieces of 32 columns:
// the forward stages h / gate / up and stores them with TMA, the backward receives the saved gate / up pieces by TMA
// one piece ahead, overwrites them in place with dGate / dUp and stores those with TMA.
#include "gemm.cuh"

#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace cmoe {

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int CHUNK_BYTES = 64 * BK * 2;  // one 64 x 64 bf16 box (MN-major operands) = 8 KiB
constexpr int GEMM_THREADS = 192;
constexpr int GEMM_THREADS_PULL = 320;  // + four row-pull warps (fused expert-parallel dispatch)
constexpr int PULL_SUBS = 4;            // the pull warps fill a 128-row tile in quarters, each with its own ready flag
constexpr int TMEM_COLS = 2 * BN;  // 512: two accumulators
constexpr int GROUP_M_SWIZZLE = 8;
// epilogue staging: two buffers of 128 rows x 128 bytes (32 fp32 or 64 bf16 columns) in the 128-byte swizzle, from
// which finished pieces of a tile leave through TMA stores (or coalesced row copies when rows scatter to peers)
constexpr int STAGING_BUF_BYTES = BM * 128;
constexpr int STAGING_BYTES = 2 * STAGING_BUF_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int EPI_FIRST_THREAD = 64;  // warp 2, lane 0: issues the TMA stores of the epilogue

enum OutMode : int {
  OUT_DIRECT = 0,      // each thread stores its own row from registers
  OUT_TMA_STORE = 1,   // staged in shared memory, written by TMA
  OUT_TMA_REDUCE = 2,  // staged, added to global memory by TMA (fp32 accumulate)
  OUT_SCATTER = 3,     // staged, then whole rows are copied to their (rank, row) homes with coalesced stores
};

struct KParams {
  int mode, M, N, K, groups;
  int a_mn, b_mn;
  int b_group_rows, split_n;
  const int* tile_group;
  const int* num_m_tiles;
  const int* group_offsets;
  void* D;
  long long ldd, d_group_stride;
  int d_fp32, accumulate;
  const __nv_bfloat16* aux_in;
  long long ld_aux_in;
  __nv_bfloat16* aux_out;
  long long ld_aux_out;
  const uint32_t* ready_flags;
  int ready_stride, ready_count;
  uint32_t ready_target;
  int* status;
  unsigned long long timeout_ns;
  int n_cols_per_tile;  // output columns covered by one tile (256, or 128 with the SwiGLU forward)
  // fused dispatch: rows of A are pulled from peers by the extra warps
  const int* pull_row_slot;
  PeerTable pull_src;
  long long pull_slots_per_src;
  int pull_K;
  const float* pull_slot_scale;
  long long pull_ld_src;
  __nv_bfloat16* pull_dst;
  long long pull_ld_dst;
  int pull_cols;
  uint32_t* tile_ready;
  uint32_t pull_epoch;
  unsigned long long* pull_stamps;
  // fused scatter: the slot of every output row gives its destination (rank, row)
  const int* scatter_row_slot;
  long long scatter_slots_per_rank;
  PeerTable scatter_out;
  long long scatter_ld;
  int out_mode;    // OutMode (EPI_STORE only)
  int fwd_staged;  // SwiGLU forward: h (tmD) and gate|up (tmE) leave through the staging area and TMA stores
  int bwd_staged;  // SwiGLU backward: dGate|dUp (tmE) leave through the piece's own staging buffer and TMA stores
};

struct Tile {
  int m0, n0;    // origin of the output tile (rows are group-local in grouped-K mode)
  int group;     // expert / group id (0 when dense)
  int a_mn0;     // A: first M index of the tile (row coordinate if K-major, inner coordinate if M-major)
  int a_k0;      // A: first K index
  int b_n0;      // B K-major: row coordinate of the first 128 tile rows; N-major: inner coordinate
  int b_n1;      // B K-major: row coordinate of tile rows 128..255
  int b_k0;      // B: first K index (inner coordinate if K-major, row coordinate if N-major)
  int k_blocks;  // number of 64-wide K blocks
  bool skip;
};

__device__ __forceinline__ int total_tiles(const KParams& p, int m_tiles, int n_tiles) {
  return (p.mode == GEMM_GROUPED_K ? p.groups : 1) * m_tiles * n_tiles;
}

__device__ __forceinline__ Tile decode_tile(const KParams& p, int t, int m_tiles, int n_tiles) {
  Tile ti;
  ti.skip = false;
  int g = 0;
  if (p.mode == GEMM_GROUPED_K) {
    g = t / (m_tiles * n_tiles);
    t -= g * m_tiles * n_tiles;
  }
  // walk the tile grid in bands of GROUP_M_SWIZZLE row tiles so that concurrently running CTAs
  // share both A and B tiles in L2
  const int band = t / (GROUP_M_SWIZZLE * n_tiles);
  const int r = t - band * GROUP_M_SWIZZLE * n_tiles;
  const int band_rows = min(GROUP_M_SWIZZLE, m_tiles - band * GROUP_M_SWIZZLE);
  const int mt = band * GROUP_M_SWIZZLE + r % band_rows;
  const int nt = r / band_rows;
  ti.m0 = mt * BM;
  ti.n0 = nt * p.n_cols_per_tile;
  ti.group = g;
  if (p.mode == GEMM_DENSE) {
    ti.a_mn0 = ti.m0;
    ti.a_k0 = 0;
    ti.b_n0 = ti.n0;
    ti.b_n1 = ti.n0 + 128;
    ti.b_k0 = 0;
    ti.k_blocks = (p.K + BK - 1) / BK;
  } else if (p.mode == GEMM_GROUPED_M) {
    g = p.tile_group[mt];
    ti.group = g;
    if (g < 0) {
      ti.skip = true;
      g = 0;
    }
    ti.a_mn0 = ti.m0;
    ti.a_k0 = 0;
    if (p.b_mn) {
      ti.b_n0 = ti.n0;
      ti.b_n1 = 0;
      ti.b_k0 = g * p.b_group_rows;
    } else {
      ti.b_n0 = g * p.b_group_rows + ti.n0;
      ti.b_n1 = p.split_n ? (g * p.b_group_rows + p.split_n + ti.n0) : (ti.b_n0 + 128);
      ti.b_k0 = 0;
    }
    ti.k_blocks = (p.K + BK - 1) / BK;
  } else {  // grouped-K: both operands are MN-major, contraction over the rows of group g
    const int r0 = p.group_offsets[g];
    const int r1 = p.group_offsets[g + 1];
    ti.a_mn0 = ti.m0;
    ti.a_k0 = r0;
    ti.b_n0 = ti.n0;
    ti.b_n1 = 0;
    ti.b_k0 = r0;
    ti.k_blocks = (r1 - r0 + BK - 1) / BK;
  }
  return ti;
}

// ex2.approx + rcp.approx: two special-function instructions instead of an IEEE division (the epilogue warps are
// issue-bound: one warp per scheduler, so every instruction saved per element shortens the tile)
__device__ __forceinline__ float sigmoidf_fast(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

// 32 fp32 values of one output row -> bf16 (or fp32) in global memory, columns [col, col+32) masked by n_limit
__device__ __forceinline__ void store_row_chunk(void* D, long long ldd, int d_fp32, int accumulate, long long row,
                                                int col, int n_limit, const float (&v)[32]) {
  if (col >= n_limit) return;
  if (d_fp32) {
    float* dst = reinterpret_cast<float*>(D) + row * ldd + col;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      if (col + j < n_limit) {  // N is a multiple of 8, so groups of 4 are all-in or all-out
        if (accumulate) {
          // fire-and-forget vector reduction: the add happens in L2, the SM never waits for the old value
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + j), "f"(v[j]), "f"(v[j + 1]),
                       "f"(v[j + 2]), "f"(v[j + 3])
                       : "memory");
        } else {
          *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        }
      }
    }
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(D) + row * ldd + col;
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      if (col + j < n_limit) {
        float f[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) f[q] = v[j + q];
        if (accumulate) {
          const uint4 old = *reinterpret_cast<const uint4*>(dst + j);
          const float2 o0 = unpack_bf16x2(old.x), o1 = unpack_bf16x2(old.y), o2 = unpack_bf16x2(old.z),
                       o3 = unpack_bf16x2(old.w);
          f[0] += o0.x; f[1] += o0.y; f[2] += o1.x; f[3] += o1.y;
          f[4] += o2.x; f[5] += o2.y; f[6] += o3.x; f[7] += o3.y;
        }
        uint4 o;
        o.x = pack_bf16x2(f[0], f[1]);
        o.y = pack_bf16x2(f[2], f[3]);
        o.z = pack_bf16x2(f[4], f[5]);
        o.w = pack_bf16x2(f[6], f[7]);
        *reinterpret_cast<uint4*>(dst + j) = o;
      }
    }
  }
}

// 32 fp32 values of one row starting at column `col` (groups of 4 beyond n_limit are skipped)
__device__ __forceinline__ void prefetch_f32_chunk(const float* row_ptr, int col, int n_limit, bool row_ok,
                                                   float4 (&v)[8]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row_ok && col + j * 4 < n_limit) v[j] = *reinterpret_cast<const float4*>(row_ptr + col + j * 4);
  }
}

// SwiGLU backward for 32 columns of one row: dH (fp32 bits in r) with the saved gate / up values (bf16, packed in
// cg / cu) -> dGate / dUp (bf16, packed) written over cg / cu.  Eight columns at a time, straight from the packed
// inputs to the packed outputs.
__device__ __forceinline__ void swiglu_bwd_math(const uint32_t (&r)[32], uint4 (&cg)[4], uint4 (&cu)[4]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t gw[4] = {cg[j].x, cg[j].y, cg[j].z, cg[j].w};
    const uint32_t uw[4] = {cu[j].x, cu[j].y, cu[j].z, cu[j].w};
    uint32_t og[4], ou[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 g = unpack_bf16x2(gw[q]);
      const float2 u = unpack_bf16x2(uw[q]);
      const float dh0 = __uint_as_float(r[8 * j + 2 * q]), dh1 = __uint_as_float(r[8 * j + 2 * q + 1]);
      const float s0 = sigmoidf_fast(g.x), s1 = sigmoidf_fast(g.y);
      // d silu(g)/dg = s (1 + g (1 - s))
      const float dg0 = dh0 * u.x * (s0 * fmaf(g.x, 1.f - s0, 1.f));
      const float dg1 = dh1 * u.y * (s1 * fmaf(g.y, 1.f - s1, 1.f));
      og[q] = pack_bf16x2(dg0, dg1);
      ou[q] = pack_bf16x2(dh0 * (g.x * s0), dh1 * (g.y * s1));
    }
    cg[j] = make_uint4(og[0], og[1], og[2], og[3]);
    cu[j] = make_uint4(ou[0], ou[1], ou[2], ou[3]);
  }
}

// ... and its results stored from registers: dGate at D[row, col..], dUp at D[row, N + col..]; columns past N hold
// garbage and are not stored.
__device__ __forceinline__ void swiglu_bwd_chunk(const uint32_t (&r)[32], uint4 (&cg)[4], uint4 (&cu)[4], int col,
                                                 int N, void* Dg, long long ldd, long long row) {
  swiglu_bwd_math(r, cg, cu);
  __nv_bfloat16* dgp = reinterpret_cast<__nv_bfloat16*>(Dg) + row * ldd + col;
  __nv_bfloat16* dup = dgp + N;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (col + j * 8 < N) {  // N is a multiple of 8
      *reinterpret_cast<uint4*>(dgp + j * 8) = cg[j];
      *reinterpret_cast<uint4*>(dup + j * 8) = cu[j];
    }
  }
}

template <int EPI>
__global__ void __launch_bounds__(GEMM_THREADS_PULL, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmE, const KParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint8_t* stg = smem + STAGES * STAGE_BYTES;  // 1024-byte aligned, as the swizzle pattern needs
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES + STAGING_BYTES);
  uint64_t* full_bar = bars;                 // [STAGES]
  uint64_t* empty_bar = bars + STAGES;       // [STAGES]
  uint64_t* tfull_bar = bars + 2 * STAGES;   // [2]
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;  // [2]
  uint64_t* gfull_bar = bars + 2 * STAGES + 4;   // [2] saved gate/up pieces landed (SwiGLU backward)
  uint64_t* gempty_bar = bars + 2 * STAGES + 6;  // [2] ... and were consumed by all epilogue threads
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 128);
      mbar_init(&gfull_bar[a], 1);
      mbar_init(&gempty_bar[a], 128);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmD);
    tma_prefetch_desc(&tmE);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
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

  int m_tiles;
  if (p.mode == GEMM_GROUPED_M) {
    m_tiles = *p.num_m_tiles;
  } else {
    m_tiles = (p.M + BM - 1) / BM;
  }
  const int n_tiles = (p.N + p.n_cols_per_tile - 1) / p.n_cols_per_tile;
  const int n_total = total_tiles(p, m_tiles, n_tiles);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // One elected lane issues the loads.  With the fused row pull the whole warp walks the tiles: lanes 0..3 each
    // poll one of the tile's four quarter flags at the same time (one L2 round trip per tile instead of four in a
    // row, which the four buffered stages hide), then lane 0 goes on alone.
    const bool pulling = p.pull_row_slot != nullptr;
    if (lane == 0 || pulling) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < n_total; t += gridDim.x) {
        const Tile ti = decode_tile(p, t, m_tiles, n_tiles);
        if (ti.skip || ti.k_blocks == 0) continue;
        if (lane == 0 && p.ready_flags != nullptr) {
          const uint32_t* f = p.ready_flags + (long long)ti.group * p.ready_stride;
          for (int s = 0; s < p.ready_count; ++s) flag_wait_ge(f + s, p.ready_target, wc);
        }
        if (pulling) {
          // the rows of this tile are written by the pull warps of some CTAs of this launch
          if (lane < PULL_SUBS) flag_wait_ge_gpu(p.tile_ready + (ti.m0 / BM) * PULL_SUBS + lane, p.pull_epoch, wc);
          __syncwarp();
          if (lane == 0) asm volatile("fence.proxy.async.global;" ::: "memory");  // generic-proxy writes -> TMA reads
        }
        if (lane == 0) {
          for (int kb = 0; kb < ti.k_blocks; ++kb) {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1u, wc, ST_TIMEOUT_SMEM_EMPTY)) break;
            mbar_arrive_expect_tx(&full_bar[stage], STAGE_BYTES);
            uint8_t* a_dst = sA + stage * A_STAGE_BYTES;
            uint8_t* b_dst = sB + stage * B_STAGE_BYTES;
            const int k = kb * BK;
            if (p.a_mn) {
              tma_load_2d(a_dst, &tmA, &full_bar[stage], ti.a_mn0, ti.a_k0 + k);
              tma_load_2d(a_dst + CHUNK_BYTES, &tmA, &full_bar[stage], ti.a_mn0 + 64, ti.a_k0 + k);
            } else {
              tma_load_2d(a_dst, &tmA, &full_bar[stage], ti.a_k0 + k, ti.a_mn0);
            }
            if (p.b_mn) {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                tma_load_2d(b_dst + j * CHUNK_BYTES, &tmB, &full_bar[stage], ti.b_n0 + 64 * j, ti.b_k0 + k);
            } else {
              tma_load_2d(b_dst, &tmB, &full_bar[stage], ti.b_k0 + k, ti.b_n0);
              tma_load_2d(b_dst + 128 * BK * 2, &tmB, &full_bar[stage], ti.b_k0 + k, ti.b_n1);
            }
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
        if (pulling) __syncwarp();
        if (*abort_flag) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(BM, BN, p.a_mn, p.b_mn);
      const uint32_t a_lbo = p.a_mn ? CHUNK_BYTES : 16;
      const uint32_t b_lbo = p.b_mn ? CHUNK_BYTES : 16;
      const uint32_t a_kstep = p.a_mn ? 2048u : 32u;  // bytes per UMMA_K = 16 step
      const uint32_t b_kstep = p.b_mn ? 2048u : 32u;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool stamped = false;
      for (int t = blockIdx.x; t < n_total; t += gridDim.x) {
        const Tile ti = decode_tile(p, t, m_tiles, n_tiles);
        if (ti.skip || ti.k_blocks == 0) continue;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, wc, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < ti.k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, wc, ST_TIMEOUT_SMEM_FULL)) break;
          tc_fence_after();
          if (p.pull_stamps != nullptr && !stamped) {
            atomicMin(p.pull_stamps + 2, global_timer_ns());
            stamped = true;
          }
          const uint32_t a_addr = smem_u32(sA + stage * A_STAGE_BYTES);
          const uint32_t b_addr = smem_u32(sB + stage * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t ad = make_smem_desc_sw128(a_addr + k * a_kstep, a_lbo, 1024);
            const uint64_t bd = make_smem_desc_sw128(b_addr + k * b_kstep, b_lbo, 1024);
            umma_bf16_ss(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // the stage is free once these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        umma_commit(&tfull_bar[acc]);
        if (*abort_flag) break;
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (p.pull_stamps != nullptr && stamped) atomicMax(p.pull_stamps + 3, global_timer_ns());
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------------ row-pull warps (fused dispatch)
    if (p.pull_row_slot != nullptr) {
      const int pw = warp - 6;  // 0..3: each warp brings in a quarter of the rows of a work item
      if (p.pull_stamps != nullptr && threadIdx.x == 6 * 32 && static_cast<int>(blockIdx.x) < m_tiles * PULL_SUBS)
        atomicMin(p.pull_stamps + 0, global_timer_ns());
      // Work items are quarter tiles (32 rows, 8 per warp) handed out in tile order: all CTAs first work on the
      // earliest tiles, so the rows that the first wave of MMA tiles needs are complete after one or two rounds
      // of loads instead of after a whole 128-row tile per CTA (one CTA moves ~16 GB/s at NVLink latency)
      for (int item = blockIdx.x; item < m_tiles * PULL_SUBS; item += gridDim.x) {
        const int mt = item / PULL_SUBS, sub = item % PULL_SUBS;
        if (p.tile_group[mt] >= 0) {
          // Two rows at a time and up to eight 16-byte loads per lane and row in flight (16 KiB per warp): remote
          // loads over NVLink take microseconds, so the transfer rate is set by the bytes in flight
          for (int i = 0; i < 32 / PULL_SUBS; i += 2) {
            const long long r0 = static_cast<long long>(mt) * BM + sub * 32 + pw * (32 / PULL_SUBS) + i;
            int slot[2];
            const __nv_bfloat16* src[2];
            float sc[2];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              slot[q] = p.pull_row_slot[r0 + q];
              src[q] = nullptr;
              sc[q] = 1.f;
              if (slot[q] >= 0) {
                const int src_rank = static_cast<int>(slot[q] / p.pull_slots_per_src);
                if (static_cast<unsigned>(src_rank) >= static_cast<unsigned>(kMaxPeers) ||
                    p.pull_src.ptr[src_rank] == nullptr) {
                  // the plan names a rank without a buffer: record it and leave the row zero instead of faulting
                  if (p.status != nullptr) atomicCAS(p.status, 0, ST_BAD_INDEX);
                } else {
                  const long long tok = (slot[q] - src_rank * p.pull_slots_per_src) / p.pull_K;
                  src[q] = reinterpret_cast<const __nv_bfloat16*>(p.pull_src.ptr[src_rank]) + tok * p.pull_ld_src;
                  if (p.pull_slot_scale) sc[q] = p.pull_slot_scale[slot[q]];
                }
              }
            }
            for (int c0 = lane * 8; c0 < p.pull_cols; c0 += 2048) {
              uint4 v[2][8];
#pragma unroll
              for (int q = 0; q < 2; ++q) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  v[q][j] = make_uint4(0u, 0u, 0u, 0u);  // padding rows are zero filled
                  if (src[q] != nullptr && c0 + j * 256 < p.pull_cols)
                    v[q][j] = *reinterpret_cast<const uint4*>(src[q] + c0 + j * 256);
                }
              }
#pragma unroll
              for (int q = 0; q < 2; ++q) {
                __nv_bfloat16* o = p.pull_dst + (r0 + q) * p.pull_ld_dst;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  if (c0 + j * 256 < p.pull_cols) {
                    uint4 w = v[q][j];
                    if (p.pull_slot_scale) {
                      const float2 a = unpack_bf16x2(w.x), b = unpack_bf16x2(w.y), c = unpack_bf16x2(w.z),
                                   d = unpack_bf16x2(w.w);
                      w.x = pack_bf16x2(a.x * sc[q], a.y * sc[q]);
                      w.y = pack_bf16x2(b.x * sc[q], b.y * sc[q]);
                      w.z = pack_bf16x2(c.x * sc[q], c.y * sc[q]);
                      w.w = pack_bf16x2(d.x * sc[q], d.y * sc[q]);
                    }
                    *reinterpret_cast<uint4*>(o + c0 + j * 256) = w;
                  }
                }
              }
            }
          }
        }
        __threadfence();
        asm volatile("fence.proxy.async.global;" ::: "memory");
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (threadIdx.x == 6 * 32) {
          asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.tile_ready + mt * PULL_SUBS + sub),
                       "r"(p.pull_epoch)
                       : "memory");
        }
      }
      if (p.pull_stamps != nullptr && threadIdx.x == 6 * 32 && static_cast<int>(blockIdx.x) < m_tiles * PULL_SUBS)
        atomicMax(p.pull_stamps + 1, global_timer_ns());
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int quad = warp & 3;
    const int row_in_tile = quad * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t stage_ctr = 0;  // pieces staged so far: picks the staging buffer
    const int m_limit = (p.mode == GEMM_GROUPED_M) ? (m_tiles * BM) : p.M;
    for (int t = blockIdx.x; t < n_total; t += gridDim.x) {
      const Tile ti = decode_tile(p, t, m_tiles, n_tiles);
      if (ti.skip) continue;
      const long long row = ti.m0 + row_in_tile;
      const bool row_ok = (ti.m0 + row_in_tile) < m_limit;
      void* Dg = p.D;
      if (p.mode == GEMM_GROUPED_K) {
        Dg = p.d_fp32 ? static_cast<void*>(reinterpret_cast<float*>(p.D) + ti.group * p.d_group_stride)
                      : static_cast<void*>(reinterpret_cast<__nv_bfloat16*>(p.D) + ti.group * p.d_group_stride);
      }
      if (ti.k_blocks == 0) {
        // nothing to contract over: the product is zero
        if (EPI == EPI_STORE && !p.accumulate && row_ok) {
          float z[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) z[j] = 0.f;
          for (int c = 0; c < BN / 32; ++c) store_row_chunk(Dg, p.ldd, p.d_fp32, 0, row, ti.n0 + c * 32, p.N, z);
        }
        continue;
      }
      // SwiGLU backward: pieces of 128 rows x 32 columns of the saved gate and up values are brought into the
      // staging area by TMA, one piece ahead of the one being processed; the first piece of a tile is requested
      // before the wait for its accumulator
      auto gu_issue = [&](uint32_t ctr, int col) {
        const uint32_t b = ctr & 1u;
        // direct stores: the buffer is free once all 128 threads have read it.  Staged stores: the caller has
        // waited for the TMA store that last read it.
        if (!p.bwd_staged && !mbar_wait(&gempty_bar[b], ((ctr >> 1) & 1u) ^ 1u, wc, ST_TIMEOUT_SMEM_EMPTY)) return;
        uint8_t* dst = stg + b * STAGING_BUF_BYTES;
        mbar_arrive_expect_tx(&gfull_bar[b], STAGING_BUF_BYTES);
        tma_load_2d(dst, &tmD, &gfull_bar[b], col, ti.m0);
        tma_load_2d(dst + STAGING_BUF_BYTES / 2, &tmD, &gfull_bar[b], p.N + col, ti.m0);
      };
      if (EPI == EPI_SWIGLU_BWD && threadIdx.x == EPI_FIRST_THREAD) {
        // staged: this piece's buffer was last read by the store issued two pieces ago
        if (p.bwd_staged) bulk_wait_group_read<1>();
        gu_issue(stage_ctr, ti.n0);
      }
      const bool ok = mbar_wait(&tfull_bar[acc], acc_phase, wc, ST_TIMEOUT_TMEM_FULL);
      tc_fence_after();
      const uint32_t t_acc = tmem_base + acc * BN + lane_base;
      if (EPI == EPI_STORE && p.out_mode != OUT_DIRECT) {
        // ---- staged epilogue.  Every piece of 128 rows x 128 bytes goes registers -> swizzled shared memory ->
        // global memory.  One named barrier per piece: it carries the OR of "my wait failed / abort seen", so all
        // 128 threads leave the loop together and no barrier is ever left waiting for a thread that gave up.
        const int unit_cols = p.d_fp32 ? 32 : 64;
        const int sw = row_in_tile & 7;
        bool any_bad = false;
        int2 dest[8];
        if (p.out_mode == OUT_SCATTER) {
          // copy-out assignment: thread t moves 16-byte chunk (t & 7) of rows (t >> 3) + 16 i
          const int t = threadIdx.x - EPI_FIRST_THREAD;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const long long rr = ti.m0 + (t >> 3) + 16 * i;
            dest[i] = make_int2(-1, 0);
            if (rr < m_limit) {
              const int slot = p.scatter_row_slot[rr];
              if (slot >= 0) {
                const int dr = static_cast<int>(slot / p.scatter_slots_per_rank);
                if (static_cast<unsigned>(dr) < static_cast<unsigned>(kMaxPeers) && p.scatter_out.ptr[dr] != nullptr)
                  dest[i] = make_int2(dr, static_cast<int>(slot - dr * p.scatter_slots_per_rank));
                else if (p.status != nullptr)
                  atomicCAS(p.status, 0, ST_BAD_INDEX);  // no such destination: recorded, the row is not stored
              }
            }
          }
        }
#pragma unroll 1
        for (int u = 0; u < BN / unit_cols; ++u) {
          const int col0 = ti.n0 + u * unit_cols;
          if (col0 >= p.N) break;  // uniform
          uint8_t* buf = stg + (stage_ctr & 1) * STAGING_BUF_BYTES;
          uint8_t* myrow = buf + row_in_tile * 128;
          if (ok) {
            if (p.d_fp32) {
              uint32_t r[32];
              tmem_ld_32x32b_x32(t_acc + u * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 8; ++j)
                *reinterpret_cast<uint4*>(myrow + ((j ^ sw) << 4)) =
                    make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            } else {
              uint32_t r0[32], r1[32];
              tmem_ld_32x32b_x32(t_acc + u * 64, r0);
              tmem_ld_32x32b_x32(t_acc + u * 64 + 32, r1);
              tmem_ld_wait();
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
          if (p.out_mode != OUT_SCATTER) {
            fence_proxy_async_smem();
            // the store issued one piece ago has read the other buffer before anybody writes it again
            if (threadIdx.x == EPI_FIRST_THREAD) bulk_wait_group_read<0>();
          }
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
          if (any_bad) break;  // uniform over the 128 epilogue threads
          if (p.out_mode == OUT_SCATTER) {
            const int t = threadIdx.x - EPI_FIRST_THREAD;
            const int ch = t & 7;
            if (col0 + ch * 8 < p.N) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                if (dest[i].x >= 0) {
                  const int rr = (t >> 3) + 16 * i;
                  const uint4 v = *reinterpret_cast<const uint4*>(buf + rr * 128 + ((ch ^ (rr & 7)) << 4));
                  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.scatter_out.ptr[dest[i].x]) +
                                     static_cast<long long>(dest[i].y) * p.scatter_ld + col0 + ch * 8;
                  *reinterpret_cast<uint4*>(o) = v;
                }
              }
            }
          } else if (threadIdx.x == EPI_FIRST_THREAD) {
            const int zgrp = (p.mode == GEMM_GROUPED_K) ? ti.group : 0;
            if (p.out_mode == OUT_TMA_REDUCE)
              tma_reduce_add_3d(&tmD, buf, col0, ti.m0, zgrp);  // rows and columns past the edge are clipped
            else
              tma_store_3d(&tmD, buf, col0, ti.m0, zgrp);
            bulk_commit_group();
          }
          ++stage_ctr;
        }
        tc_fence_before();
        mbar_arrive(&tempty_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
        if (any_bad) break;
        continue;
      }
      if (EPI == EPI_SWIGLU_FWD && p.fwd_staged) {
        // ---- staged SwiGLU forward: 32 output columns at a time, h / gate / up as three pieces of 128 rows x 64
        // bytes (64-byte swizzle) in one staging buffer; two named barriers per piece (buffer free, buffer filled)
        const int gsw = (row_in_tile >> 1) & 3;
        uint8_t* hrow = stg + row_in_tile * 64;
        bool any_bad = false;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          const int col = ti.n0 + c * 32;
          if (col >= p.N) break;  // uniform
          uint32_t ph[16], pg[16], pu[16];
          if (ok) {
            uint32_t rg[32], ru[32];
            tmem_ld_32x32b_x32(t_acc + c * 32, rg);
            tmem_ld_32x32b_x32(t_acc + 128 + c * 32, ru);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float g0 = __uint_as_float(rg[2 * j]), g1 = __uint_as_float(rg[2 * j + 1]);
              const float u0 = __uint_as_float(ru[2 * j]), u1 = __uint_as_float(ru[2 * j + 1]);
              ph[j] = pack_bf16x2(g0 * sigmoidf_fast(g0) * u0, g1 * sigmoidf_fast(g1) * u1);
              pg[j] = pack_bf16x2(g0, g1);
              pu[j] = pack_bf16x2(u0, u1);
            }
          }
          // the stores issued for the previous piece have read the buffer
          if (threadIdx.x == EPI_FIRST_THREAD) bulk_wait_group_read<0>();
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
          if (any_bad) break;  // uniform over the 128 epilogue threads
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int o = (j ^ gsw) << 4;
            *reinterpret_cast<uint4*>(hrow + o) = make_uint4(ph[4 * j], ph[4 * j + 1], ph[4 * j + 2], ph[4 * j + 3]);
            if (p.aux_out != nullptr) {
              *reinterpret_cast<uint4*>(hrow + STAGING_BUF_BYTES / 2 + o) =
                  make_uint4(pg[4 * j], pg[4 * j + 1], pg[4 * j + 2], pg[4 * j + 3]);
              *reinterpret_cast<uint4*>(hrow + STAGING_BUF_BYTES + o) =
                  make_uint4(pu[4 * j], pu[4 * j + 1], pu[4 * j + 2], pu[4 * j + 3]);
            }
          }
          fence_proxy_async_smem();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (threadIdx.x == EPI_FIRST_THREAD) {
            tma_store_3d(&tmD, stg, col, ti.m0, 0);
            if (p.aux_out != nullptr) {
              tma_store_3d(&tmE, stg + STAGING_BUF_BYTES / 2, col, 0, ti.m0);  // gate half
              tma_store_3d(&tmE, stg + STAGING_BUF_BYTES, col, 1, ti.m0);      // up half
            }
            bulk_commit_group();
          }
        }
        tc_fence_before();
        mbar_arrive(&tempty_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
        if (any_bad) break;
        continue;
      }
      if (ok) {
        if (EPI == EPI_STORE) {
          if (p.accumulate && p.d_fp32) {
            // D += acc in fp32: the old values of chunk c+1 are fetched while chunk c is being processed, so
            // the global-load latency hides behind the TMEM read and the stores (software pipeline of depth 1)
            float* drow = reinterpret_cast<float*>(Dg) + row * p.ldd;
            float4 cur[8], nxt[8];
            prefetch_f32_chunk(drow, ti.n0, p.N, row_ok, cur);
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
              const int col = ti.n0 + c * 32;
              if (col >= p.N) break;
              uint32_t r[32];
              tmem_ld_32x32b_x32(t_acc + c * 32, r);
              prefetch_f32_chunk(drow, col + 32, p.N, row_ok, nxt);
              tmem_ld_wait();
              if (row_ok) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  if (col + j * 4 < p.N) {
                    float4 o = cur[j];
                    o.x += __uint_as_float(r[4 * j]);
                    o.y += __uint_as_float(r[4 * j + 1]);
                    o.z += __uint_as_float(r[4 * j + 2]);
                    o.w += __uint_as_float(r[4 * j + 3]);
                    *reinterpret_cast<float4*>(drow + col + j * 4) = o;
                  }
                }
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) cur[j] = nxt[j];
            }
          } else {
            // direct bf16 / fp32 stores (and bf16 accumulate) from registers, one row per thread
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
              if (ti.n0 + c * 32 >= p.N) break;  // uniform across the warp
              uint32_t r[32];
              tmem_ld_32x32b_x32(t_acc + c * 32, r);
              tmem_ld_wait();
              if (row_ok) {
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                store_row_chunk(Dg, p.ldd, p.d_fp32, p.accumulate, row, ti.n0 + c * 32, p.N, v);
              }
            }
          }
        } else if (EPI == EPI_SWIGLU_FWD) {
          // accumulator columns [0,128) = gate, [128,256) = up for output columns n0 .. n0+127
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            if (ti.n0 + c * 32 >= p.N) break;
            uint32_t rg[32], ru[32];
            tmem_ld_32x32b_x32(t_acc + c * 32, rg);
            tmem_ld_32x32b_x32(t_acc + 128 + c * 32, ru);
            tmem_ld_wait();
            if (row_ok) {
              float g[32], u[32], h[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                g[j] = __uint_as_float(rg[j]);
                u[j] = __uint_as_float(ru[j]);
                h[j] = g[j] * sigmoidf_fast(g[j]) * u[j];
              }
              const int col = ti.n0 + c * 32;
              store_row_chunk(Dg, p.ldd, 0, 0, row, col, p.N, h);
              if (p.aux_out != nullptr) {
                store_row_chunk(p.aux_out, p.ld_aux_out, 0, 0, row, col, p.N, g);
                store_row_chunk(p.aux_out + p.N, p.ld_aux_out, 0, 0, row, col, p.N, u);
              }
            }
          }
        }
      }
      if (EPI == EPI_SWIGLU_BWD && p.bwd_staged) {
        // acc = dH; [dGate | dUp] = f(dH, gate, up).  Every thread reads its own row of the gate / up piece from the
        // staging buffer, writes its results over it, and the piece leaves through two TMA stores (each thread's
        // direct 16-byte stores at a row stride were the largest single cost of this epilogue).  One named barrier
        // per piece, carrying the OR of "a wait failed / abort seen" so that all 128 threads leave together.
        const int gsw = (row_in_tile >> 1) & 3;  // 64-byte swizzle: 16-byte chunk j of row r sits at j ^ ((r / 2) % 4)
        bool any_bad = false;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col = ti.n0 + c * 32;
          if (col >= p.N) break;
          const uint32_t b = stage_ctr & 1u;
          if (threadIdx.x == EPI_FIRST_THREAD && c + 1 < BN / 32 && col + 32 < p.N) {
            bulk_wait_group_read<0>();  // the store of the previous piece has read the other buffer
            gu_issue(stage_ctr + 1, col + 32);
          }
          const bool got = mbar_wait(&gfull_bar[b], (stage_ctr >> 1) & 1u, wc, ST_TIMEOUT_SMEM_FULL);
          uint32_t r[32];
          if (ok) {
            tmem_ld_32x32b_x32(t_acc + c * 32, r);
            tmem_ld_wait();
          }
          uint4 cg[4], cu[4];
          uint8_t* grow = stg + b * STAGING_BUF_BYTES + row_in_tile * 64;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            cg[j] = *reinterpret_cast<const uint4*>(grow + ((j ^ gsw) << 4));
            cu[j] = *reinterpret_cast<const uint4*>(grow + STAGING_BUF_BYTES / 2 + ((j ^ gsw) << 4));
          }
          if (ok && got) {
            swiglu_bwd_math(r, cg, cu);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              *reinterpret_cast<uint4*>(grow + ((j ^ gsw) << 4)) = cg[j];
              *reinterpret_cast<uint4*>(grow + STAGING_BUF_BYTES / 2 + ((j ^ gsw) << 4)) = cu[j];
            }
          }
          fence_proxy_async_smem();
          {
            const int bad = (!ok || !got || *abort_flag) ? 1 : 0;
            int any;
            asm volatile(
                "{\n\t.reg .pred q, r;\n\tsetp.ne.s32 q, %1, 0;\n\tbar.red.or.pred r, 1, 128, q;\n\t"
                "selp.s32 %0, 1, 0, r;\n\t}"
                : "=r"(any)
                : "r"(bad)
                : "memory");
            any_bad = any != 0;
          }
          if (any_bad) break;  // uniform over the 128 epilogue threads
          if (threadIdx.x == EPI_FIRST_THREAD) {
            tma_store_3d(&tmE, stg + b * STAGING_BUF_BYTES, col, 0, ti.m0);                          // dGate
            tma_store_3d(&tmE, stg + b * STAGING_BUF_BYTES + STAGING_BUF_BYTES / 2, col, 1, ti.m0);  // dUp
            bulk_commit_group();
          }
          ++stage_ctr;
        }
        tc_fence_before();
        mbar_arrive(&tempty_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
        if (any_bad) break;
        continue;
      }
      if (EPI == EPI_SWIGLU_BWD) {
        // direct stores.  acc = dH; D = [dGate | dUp] with row stride ldd (>= 2N).  Runs whether or not the
        // accumulator wait succeeded, so that every requested piece is also consumed
        const int gsw = (row_in_tile >> 1) & 3;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col = ti.n0 + c * 32;
          if (col >= p.N) break;
          if (threadIdx.x == EPI_FIRST_THREAD && c + 1 < BN / 32 && col + 32 < p.N) gu_issue(stage_ctr + 1, col + 32);
          const uint32_t b = stage_ctr & 1u;
          const bool got = mbar_wait(&gfull_bar[b], (stage_ctr >> 1) & 1u, wc, ST_TIMEOUT_SMEM_FULL);
          uint32_t r[32];
          if (ok) {
            tmem_ld_32x32b_x32(t_acc + c * 32, r);
            tmem_ld_wait();
          }
          uint4 cg[4], cu[4];
          const uint8_t* grow = stg + b * STAGING_BUF_BYTES + row_in_tile * 64;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            cg[j] = *reinterpret_cast<const uint4*>(grow + ((j ^ gsw) << 4));
            cu[j] = *reinterpret_cast<const uint4*>(grow + STAGING_BUF_BYTES / 2 + ((j ^ gsw) << 4));
          }
          mbar_arrive(&gempty_bar[b]);
          if (ok && got && row_ok) swiglu_bwd_chunk(r, cg, cu, col, p.N, Dg, p.ldd, row);
          ++stage_ctr;
        }
      }
      tc_fence_before();
      mbar_arrive(&tempty_bar[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
      if (*abort_flag) break;
    }
    // shared memory and the kernel's results must outlive the TMA stores still in flight
    if (threadIdx.x == EPI_FIRST_THREAD &&
        (p.out_mode == OUT_TMA_STORE || p.out_mode == OUT_TMA_REDUCE || (EPI == EPI_SWIGLU_FWD && p.fwd_staged) ||
         (EPI == EPI_SWIGLU_BWD && p.bwd_staged)))
      bulk_wait_group<0>();
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag) {
      // a wait ran out: give copies and MMAs that are still in flight time to land before the
      // shared and tensor memory of this CTA are handed back
      for (int i = 0; i < 64; ++i) __nanosleep(2000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ----------------------------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  });
  return fn;
}

struct TmapKey {
  const void* ptr;
  long long rows, cols, ld;
  int box_rows, box_cols;
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows &&
           box_cols == o.box_cols;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h = h * 1000003u ^ static_cast<size_t>(k.rows);
    h = h * 1000003u ^ static_cast<size_t>(k.cols);
    h = h * 1000003u ^ static_cast<size_t>(k.ld);
    h = h * 1000003u ^ static_cast<size_t>(k.box_rows);
    h = h * 1000003u ^ static_cast<size_t>(k.box_cols);
    return h;
  }
};

// bf16 row-major [rows, cols] (leading dimension ld), box = box_cols columns x box_rows rows; 64 columns use the
// 128-byte swizzle (operands), 32 columns the 64-byte swizzle (epilogue pieces)
cudaError_t make_tmap(CUtensorMap* out, const void* ptr, long long rows, long long cols, long long ld, int box_rows,
                      int box_cols = 64) {
  static std::mutex mu;
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  if (box_cols != 64 && box_cols != 32) return cudaErrorInvalidValue;
  TmapKey key{ptr, rows, cols, ld, box_rows, box_cols};
  {
    std::lock_guard<std::mutex> lk(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return cudaSuccess;
    }
  }
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0 || (ld * 2) % 16 != 0 || cols <= 0 || rows <= 0)
    return cudaErrorInvalidValue;
  cuuint64_t gdim[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t gstride[1] = {static_cast<cuuint64_t>(ld) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estride[2] = {1u, 1u};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estride,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   box_cols == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    std::fprintf(stderr, "cmoe: cuTensorMapEncodeTiled failed (%d) rows=%lld cols=%lld ld=%lld box_rows=%d\n",
                 static_cast<int>(r), rows, cols, ld, box_rows);
    return cudaErrorInvalidValue;
  }
  {
    std::lock_guard<std::mutex> lk(mu);
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, *out);
  }
  return cudaSuccess;
}

// Output map: [groups, rows, cols] of fp32 or bf16 with row stride ld and group stride gstride (elements); the box
// is one staging buffer, 128 rows x 128 bytes, 128-byte swizzle.
cudaError_t make_tmap_out(CUtensorMap* out, const void* ptr, int fp32, long long groups, long long rows,
                          long long cols, long long ld, long long gstride, int box_bytes = 128) {
  struct Key {
    const void* ptr;
    long long groups, rows, cols, ld, gstride;
    int fp32, box_bytes;
    bool operator==(const Key& o) const {
      return ptr == o.ptr && groups == o.groups && rows == o.rows && cols == o.cols && ld == o.ld &&
             gstride == o.gstride && fp32 == o.fp32 && box_bytes == o.box_bytes;
    }
  };
  struct KeyHash {
    size_t operator()(const Key& k) const {
      size_t h = reinterpret_cast<size_t>(k.ptr);
      for (long long v : {k.groups, k.rows, k.cols, k.ld, k.gstride, static_cast<long long>(k.fp32),
                          static_cast<long long>(k.box_bytes)})
        h = h * 1000003u ^ static_cast<size_t>(v);
      return h;
    }
  };
  static std::mutex mu;
  static std::unordered_map<Key, CUtensorMap, KeyHash> cache;
  if (box_bytes != 128 && box_bytes != 64) return cudaErrorInvalidValue;
  Key key{ptr, groups, rows, cols, ld, gstride, fp32, box_bytes};
  {
    std::lock_guard<std::mutex> lk(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return cudaSuccess;
    }
  }
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return cudaErrorNotSupported;
  const long long es = fp32 ? 4 : 2;
  cuuint64_t gdim[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(groups)};
  cuuint64_t gstr[2] = {static_cast<cuuint64_t>(ld * es), static_cast<cuuint64_t>(gstride * es)};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(box_bytes / es), static_cast<cuuint32_t>(BM), 1u};
  cuuint32_t estride[3] = {1u, 1u, 1u};
  CUresult r = enc(out, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                   const_cast<void*>(ptr), gdim, gstr, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   box_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    std::fprintf(stderr, "cmoe: cuTensorMapEncodeTiled (output) failed (%d) groups=%lld rows=%lld cols=%lld ld=%lld\n",
                 static_cast<int>(r), groups, rows, cols, ld);
    return cudaErrorInvalidValue;
  }
  {
    std::lock_guard<std::mutex> lk(mu);
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, *out);
  }
  return cudaSuccess;
}

// bf16 [rows, 2N] viewed as [rows, 2 halves, N] (gate | up): dims (N, 2, rows), box 32 columns x 1 half x 128 rows,
// 64-byte swizzle; a store of columns [c, c+32) of one half is clipped at N and never reaches into the other half
cudaError_t make_tmap_halves(CUtensorMap* out, const void* ptr, long long rows, long long n, long long ld) {
  struct Key {
    const void* ptr;
    long long rows, n, ld;
    bool operator==(const Key& o) const { return ptr == o.ptr && rows == o.rows && n == o.n && ld == o.ld; }
  };
  struct KeyHash {
    size_t operator()(const Key& k) const {
      size_t h = reinterpret_cast<size_t>(k.ptr);
      for (long long v : {k.rows, k.n, k.ld}) h = h * 1000003u ^ static_cast<size_t>(v);
      return h;
    }
  };
  static std::mutex mu;
  static std::unordered_map<Key, CUtensorMap, KeyHash> cache;
  Key key{ptr, rows, n, ld};
  {
    std::lock_guard<std::mutex> lk(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return cudaSuccess;
    }
  }
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return cudaErrorNotSupported;
  cuuint64_t gdim[3] = {static_cast<cuuint64_t>(n), 2u, static_cast<cuuint64_t>(rows)};
  cuuint64_t gstr[2] = {static_cast<cuuint64_t>(n * 2), static_cast<cuuint64_t>(ld * 2)};
  cuuint32_t box[3] = {32u, 1u, static_cast<cuuint32_t>(BM)};
  cuuint32_t estride[3] = {1u, 1u, 1u};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), gdim, gstr, box, estride,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  {
    std::lock_guard<std::mutex> lk(mu);
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, *out);
  }
  return cudaSuccess;
}

// CMOE_GEMM_DIRECT_EPILOGUE=1 keeps every epilogue on per-thread stores from registers (for A/B measurements)
bool direct_epilogue_forced() {
  static const bool forced = [] {
    const char* v = std::getenv("CMOE_GEMM_DIRECT_EPILOGUE");
    return v != nullptr && v[0] != '\0' && v[0] != '0';
  }();
  return forced;
}

template <int EPI>
cudaError_t launch_variant(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmD,
                           const CUtensorMap& tmE, const KParams& kp, int grid, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  const int threads = kp.pull_row_slot != nullptr ? GEMM_THREADS_PULL : GEMM_THREADS;
  gemm_kernel<EPI><<<grid, threads, SMEM_BYTES, stream>>>(tmA, tmB, tmD, tmE, kp);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_gemm(const GemmArgs& a, cudaStream_t stream) {
  if (a.N % 8 != 0 || a.N <= 0) return cudaErrorInvalidValue;
  if (a.mode == GEMM_GROUPED_K && !(a.a_mn && a.b_mn)) return cudaErrorInvalidValue;
  if (a.mode == GEMM_GROUPED_M && a.a_mn) return cudaErrorInvalidValue;
  if (a.epilogue == EPI_SWIGLU_FWD && (a.b_mn || a.split_n <= 0)) return cudaErrorInvalidValue;

  CUtensorMap tmA, tmB;
  cudaError_t e = make_tmap(&tmA, a.A, a.a_rows, a.a_cols, a.a_ld, a.a_mn ? 64 : 128);
  if (e != cudaSuccess) return e;
  e = make_tmap(&tmB, a.B, a.b_rows, a.b_cols, a.b_ld, a.b_mn ? 64 : 128);
  if (e != cudaSuccess) return e;

  KParams kp;
  kp.mode = a.mode;
  kp.M = a.M;
  kp.N = a.N;
  kp.K = a.K;
  kp.groups = a.groups;
  kp.a_mn = a.a_mn;
  kp.b_mn = a.b_mn;
  kp.b_group_rows = static_cast<int>(a.b_group_rows);
  kp.split_n = a.split_n;
  kp.tile_group = a.tile_group;
  kp.num_m_tiles = a.num_m_tiles;
  kp.group_offsets = a.group_offsets;
  kp.D = a.D;
  kp.ldd = a.ldd;
  kp.d_group_stride = a.d_group_stride;
  kp.d_fp32 = a.d_fp32;
  kp.accumulate = a.accumulate;
  kp.aux_in = reinterpret_cast<const __nv_bfloat16*>(a.aux_in);
  kp.ld_aux_in = a.ld_aux_in;
  kp.aux_out = reinterpret_cast<__nv_bfloat16*>(a.aux_out);
  kp.ld_aux_out = a.ld_aux_out;
  kp.pull_row_slot = a.pull_row_slot;
  kp.pull_src = a.pull_src;
  kp.pull_slots_per_src = a.pull_slots_per_src;
  kp.pull_K = a.pull_K;
  kp.pull_slot_scale = a.pull_slot_scale;
  kp.pull_ld_src = a.pull_ld_src;
  kp.pull_dst = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(a.A));
  kp.pull_ld_dst = a.a_ld;
  kp.pull_cols = static_cast<int>(a.a_cols);
  kp.tile_ready = a.tile_ready;
  kp.pull_epoch = a.pull_epoch;
  kp.pull_stamps = a.pull_stamps;
  if (a.pull_row_slot != nullptr &&
      (a.mode != GEMM_GROUPED_M || a.a_mn || a.tile_ready == nullptr || a.a_cols % 8 != 0))
    return cudaErrorInvalidValue;
  kp.scatter_row_slot = a.scatter_row_slot;
  kp.scatter_slots_per_rank = a.scatter_slots_per_rank;
  kp.scatter_out = a.scatter_out;
  kp.scatter_ld = a.scatter_ld;
  if (a.scatter_row_slot != nullptr &&
      (a.epilogue != EPI_STORE || a.d_fp32 || a.accumulate || a.mode == GEMM_GROUPED_K ||
       a.scatter_slots_per_rank <= 0 || a.scatter_ld % 8 != 0))
    return cudaErrorInvalidValue;
  // how the EPI_STORE epilogue leaves the SM
  kp.out_mode = OUT_DIRECT;
  CUtensorMap tmD = tmA;  // placeholder when no output map is needed
  if (a.epilogue == EPI_STORE && !direct_epilogue_forced()) {
    if (a.scatter_row_slot != nullptr) {
      kp.out_mode = OUT_SCATTER;
    } else if (!(a.accumulate && !a.d_fp32)) {
      const long long es = a.d_fp32 ? 4 : 2;
      const long long d_rows = a.mode == GEMM_GROUPED_M ? a.a_rows : a.M;
      const long long groups = a.mode == GEMM_GROUPED_K ? a.groups : 1;
      const long long gstride = a.mode == GEMM_GROUPED_K ? a.d_group_stride : d_rows * a.ldd;
      const bool aligned = (reinterpret_cast<uintptr_t>(a.D) & 15u) == 0 && (a.ldd * es) % 16 == 0 &&
                           (gstride * es) % 16 == 0 && a.ldd >= a.N && d_rows > 0;
      if (aligned && make_tmap_out(&tmD, a.D, a.d_fp32, groups, d_rows, a.N, a.ldd, gstride) == cudaSuccess)
        kp.out_mode = a.accumulate ? OUT_TMA_REDUCE : OUT_TMA_STORE;
    }
  }
  CUtensorMap tmE = tmA;  // placeholder unless the SwiGLU forward stages its gate|up output
  kp.fwd_staged = 0;
  kp.bwd_staged = 0;
  if (a.epilogue == EPI_SWIGLU_FWD && !direct_epilogue_forced() && a.mode != GEMM_GROUPED_K) {
    // h [rows, N] and the optional gate|up copy [rows, 2N] (as [2 halves, rows, N]) leave through TMA stores
    const long long d_rows = a.mode == GEMM_GROUPED_M ? a.a_rows : a.M;
    bool okmaps = !a.d_fp32 && (reinterpret_cast<uintptr_t>(a.D) & 15u) == 0 && (a.ldd * 2) % 16 == 0 && d_rows > 0 &&
                  make_tmap_out(&tmD, a.D, 0, 1, d_rows, a.N, a.ldd, d_rows * a.ldd, 64) == cudaSuccess;
    if (okmaps && a.aux_out != nullptr) {
      okmaps = (reinterpret_cast<uintptr_t>(a.aux_out) & 15u) == 0 && (a.ld_aux_out * 2) % 16 == 0 &&
               a.ld_aux_out >= 2LL * a.N &&
               make_tmap_halves(&tmE, a.aux_out, d_rows, a.N, a.ld_aux_out) == cudaSuccess;
    }
    kp.fwd_staged = okmaps ? 1 : 0;
  }
  if (a.epilogue == EPI_SWIGLU_BWD) {
    // the saved gate|up matrix [rows, 2N] comes into the epilogue through TMA (pieces of 128 rows x 32 columns)
    if (a.aux_in == nullptr || a.ld_aux_in < 2LL * a.N) return cudaErrorInvalidValue;
    const long long aux_rows = a.mode == GEMM_GROUPED_M ? a.a_rows : a.M;
    e = make_tmap(&tmD, a.aux_in, aux_rows, 2LL * a.N, a.ld_aux_in, BM, 32);
    if (e != cudaSuccess) return e;
    // [dGate | dUp] leaves through TMA stores of the same 128 x 32 pieces (as [rows, 2 halves, N], clipped at N)
    if (!direct_epilogue_forced() && !a.d_fp32 && !a.accumulate && a.mode != GEMM_GROUPED_K &&
        (reinterpret_cast<uintptr_t>(a.D) & 15u) == 0 && (a.ldd * 2) % 16 == 0 && a.ldd >= 2LL * a.N &&
        make_tmap_halves(&tmE, a.D, aux_rows, a.N, a.ldd) == cudaSuccess)
      kp.bwd_staged = 1;
  }
  kp.ready_flags = a.ready_flags;
  kp.ready_stride = a.ready_stride;
  kp.ready_count = a.ready_count;
  kp.ready_target = a.ready_target;
  kp.status = a.status;
  kp.timeout_ns = a.timeout_ns ? a.timeout_ns : kDefaultTimeoutNs;
  kp.n_cols_per_tile = (a.epilogue == EPI_SWIGLU_FWD) ? 128 : BN;

  int num_sms = a.num_sms;
  if (num_sms <= 0) {
    int dev = 0;
    e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    static int cached_dev = -1, cached_sms = 0;
    if (cached_dev != dev) {
      e = cudaDeviceGetAttribute(&cached_sms, cudaDevAttrMultiProcessorCount, dev);
      if (e != cudaSuccess) return e;
      cached_dev = dev;
    }
    num_sms = cached_sms;
  }
  const long long n_tiles = (a.N + kp.n_cols_per_tile - 1) / kp.n_cols_per_tile;
  long long m_tiles = (a.mode == GEMM_GROUPED_M) ? a.max_m_tiles : (a.M + BM - 1) / BM;
  long long tiles = m_tiles * n_tiles * (a.mode == GEMM_GROUPED_K ? a.groups : 1);
  if (tiles <= 0) return cudaSuccess;
  const int grid = static_cast<int>(tiles < num_sms ? tiles : num_sms);

  switch (a.epilogue) {
    case EPI_STORE:
      return launch_variant<EPI_STORE>(tmA, tmB, tmD, tmE, kp, grid, stream);
    case EPI_SWIGLU_FWD:
      return launch_variant<EPI_SWIGLU_FWD>(tmA, tmB, tmD, tmE, kp, grid, stream);
    case EPI_SWIGLU_BWD:
      return launch_variant<EPI_SWIGLU_BWD>(tmA, tmB, tmD, tmE, kp, grid, stream);
    default:
      return cudaErrorInvalidValue;
  }
}

}  // namespace cmoe
