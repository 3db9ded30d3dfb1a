// Peer-memory kernels over NVLink 5 / NVSwitch: the expert-parallel dispatch (row gather from peers) and
// combine (weighted row pull from the owners), the bounded group barrier between their phases, and the
// data-parallel gradient reduce-scatter (fused with cast + scale) and parameter push.
//
// They replace the reference's NCCL call sites C1-C3 (all_to_all_single for counts, dispatch and combine,
// pkg/distributed/expert_parallel.py:104-218) and C10 (FSDP2 reduce-scatter / all-gather,
// pkg/distributed/data_parallel.py:91-97).  Every remote access is a plain ld/st on a peer-mapped address;
// there is no TMA on peer memory and no wait without a bound anywhere in this file.
#include <cstdlib>
#include "ep.cuh"

#include "common.cuh"

namespace cmoe {

namespace {

// Where the kernels of this file record that a table pointed outside the peer buffers (set once per process with
// set_peer_status_word; the kernels skip the access and go on, the host finds the code at its next status check).
static __device__ int* g_peer_status = nullptr;

__device__ __forceinline__ bool peer_ok(const PeerTable& t, int rank) {
  if (static_cast<unsigned>(rank) < static_cast<unsigned>(kMaxPeers) && t.ptr[rank] != nullptr) return true;
  if (g_peer_status != nullptr) atomicCAS(g_peer_status, 0, ST_BAD_INDEX);
  return false;
}

__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 x = *reinterpret_cast<const uint4*>(p);
  const float2 a = unpack_bf16x2(x.x), b = unpack_bf16x2(x.y), c = unpack_bf16x2(x.z), d = unpack_bf16x2(x.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 o;
  o.x = pack_bf16x2(f[0], f[1]);
  o.y = pack_bf16x2(f[2], f[3]);
  o.z = pack_bf16x2(f[4], f[5]);
  o.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = o;
}

__global__ void peer_barrier_kernel(const PeerTable flags, int rank, int world, uint32_t epoch, int* status,
                                    unsigned long long timeout_ns) {
  const int r = threadIdx.x;
  if (r >= world) return;
  __threadfence_system();  // everything this GPU wrote before the barrier is visible before the flag is
  st_release_sys(reinterpret_cast<uint32_t*>(flags.ptr[r]) + rank, epoch);
  WaitCtx wc;
  wc.abort_flag = nullptr;
  wc.status = status;
  wc.timeout_ns = timeout_ns;
  flag_wait_ge(reinterpret_cast<const uint32_t*>(flags.ptr[rank]) + r, epoch, wc);
}

__global__ void peer_allgather_kernel(const PeerTable src, int world, long long n_vec, uint4* __restrict__ out) {
  const long long total = n_vec * world;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / n_vec);
    out[i] = reinterpret_cast<const uint4*>(src.ptr[r])[i - r * n_vec];
  }
}

// one warp per row; 16-byte loads from the (possibly remote) source row, up to four in flight per lane
__global__ void __launch_bounds__(256) gather_rows_peer_kernel(const PeerTable src, long long slots_per_src, int K,
                                                               const int* __restrict__ row_slot,
                                                               const float* __restrict__ slot_scale,
                                                               __nv_bfloat16* __restrict__ out, long long cap_rows,
                                                               const int* __restrict__ num_m_tiles, int H,
                                                               long long ld_src, long long ld_out) {
  const long long n_rows = num_m_tiles ? min(static_cast<long long>(*num_m_tiles) * 128, cap_rows) : cap_rows;
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  for (long long r = blockIdx.x * static_cast<long long>(warps) + (threadIdx.x >> 5); r < n_rows;
       r += static_cast<long long>(gridDim.x) * warps) {
    const int slot = row_slot[r];
    __nv_bfloat16* o = out + r * ld_out;
    if (slot < 0) {
      for (int c = lane * 8; c < H; c += 256) *reinterpret_cast<uint4*>(o + c) = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const int rank = static_cast<int>(slot / slots_per_src);
    if (!peer_ok(src, rank)) {  // a slot that names no source buffer: recorded, the row is left zero
      for (int c = lane * 8; c < H; c += 256) *reinterpret_cast<uint4*>(o + c) = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const long long tok = (slot - rank * slots_per_src) / K;
    const __nv_bfloat16* s = reinterpret_cast<const __nv_bfloat16*>(src.ptr[rank]) + tok * ld_src;
    const float sc = slot_scale ? slot_scale[slot] : 1.f;
    for (int c0 = lane * 8; c0 < H; c0 += 1024) {
      uint4 v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (c0 + j * 256 < H) v[j] = *reinterpret_cast<const uint4*>(s + c0 + j * 256);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (c0 + j * 256 < H) {
          if (slot_scale) {
            float2 a = unpack_bf16x2(v[j].x), b = unpack_bf16x2(v[j].y), c = unpack_bf16x2(v[j].z),
                   d = unpack_bf16x2(v[j].w);
            v[j].x = pack_bf16x2(a.x * sc, a.y * sc);
            v[j].y = pack_bf16x2(b.x * sc, b.y * sc);
            v[j].z = pack_bf16x2(c.x * sc, c.y * sc);
            v[j].w = pack_bf16x2(d.x * sc, d.y * sc);
          }
          *reinterpret_cast<uint4*>(o + c0 + j * 256) = v[j];
        }
      }
    }
  }
}

// one warp per token: look up the K (owner, row) pairs first, then stream the K rows
__global__ void __launch_bounds__(256) combine_rows_peer_kernel(const PeerTable rows, const PeerTable slot_row,
                                                                const int* __restrict__ idx,
                                                                const int* __restrict__ expert_rank,
                                                                const float* __restrict__ w,
                                                                __nv_bfloat16* __restrict__ y, long long n_tokens,
                                                                int K, int H, long long slot_base, long long ld_rows,
                                                                long long ld_y,
                                                                const __nv_bfloat16* __restrict__ local_rows) {
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  for (long long t = blockIdx.x * static_cast<long long>(warps) + (threadIdx.x >> 5); t < n_tokens;
       t += static_cast<long long>(gridDim.x) * warps) {
    int my_owner = 0, my_row = -1;
    float my_w = 0.f;
    if (lane < K) {
      const int e = idx[t * K + lane];
      my_owner = expert_rank[e];
      if (peer_ok(slot_row, my_owner) && (local_rows != nullptr || peer_ok(rows, my_owner)))
        my_row = reinterpret_cast<const int*>(slot_row.ptr[my_owner])[slot_base + t * K + lane];
      my_w = w ? w[t * K + lane] : 1.f;
    }
    for (int cb = 0; cb < H; cb += 256) {  // the same trip count on every lane: the shuffles below need all 32
      const int c = cb + lane * 8;
      const bool act = c < H;
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int k = 0; k < K; ++k) {
        const int owner = __shfl_sync(0xffffffffu, my_owner, k);
        const int row = __shfl_sync(0xffffffffu, my_row, k);
        const float wk = __shfl_sync(0xffffffffu, my_w, k);
        if (row < 0 || !act) continue;
        float f[8];
        // rows pushed here by the owners' GEMM epilogues sit at [t*K + k]; otherwise pull from the owner
        const __nv_bfloat16* src = local_rows ? local_rows + (t * K + k) * ld_rows
                                              : reinterpret_cast<const __nv_bfloat16*>(rows.ptr[owner]) +
                                                    static_cast<long long>(row) * ld_rows;
        ld8(src + c, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += wk * f[j];
      }
      if (act) st8(y + t * ld_y + c, acc);
    }
  }
}

// Same sum for a compile-time K: the K source rows of a token are resolved once (lane k looks pair k up, the warp
// shares the results by shuffle) and the loads of all K rows of a column block are issued before the first use, so
// a lane keeps K x 16 bytes in flight instead of 16.  The order of the additions is that of the kernel above.
template <int KK>
__global__ void __launch_bounds__(256) combine_rows_peer_k_kernel(const PeerTable rows, const PeerTable slot_row,
                                                                  const int* __restrict__ idx,
                                                                  const int* __restrict__ expert_rank,
                                                                  const float* __restrict__ w,
                                                                  __nv_bfloat16* __restrict__ y, long long n_tokens,
                                                                  int H, long long slot_base, long long ld_rows,
                                                                  long long ld_y,
                                                                  const __nv_bfloat16* __restrict__ local_rows) {
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  for (long long t = blockIdx.x * static_cast<long long>(warps) + (threadIdx.x >> 5); t < n_tokens;
       t += static_cast<long long>(gridDim.x) * warps) {
    const __nv_bfloat16* my_src = nullptr;
    float my_w = 0.f;
    if (lane < KK) {
      const int e = idx[t * KK + lane];
      const int owner = expert_rank[e];
      if (peer_ok(slot_row, owner) && (local_rows != nullptr || peer_ok(rows, owner))) {
        const int row = reinterpret_cast<const int*>(slot_row.ptr[owner])[slot_base + t * KK + lane];
        if (row >= 0)
          my_src = local_rows ? local_rows + (t * KK + lane) * ld_rows
                              : reinterpret_cast<const __nv_bfloat16*>(rows.ptr[owner]) +
                                    static_cast<long long>(row) * ld_rows;
      }
      my_w = w ? w[t * KK + lane] : 1.f;
    }
    const __nv_bfloat16* src[KK];
    float wk[KK];
#pragma unroll
    for (int k = 0; k < KK; ++k) {
      src[k] = reinterpret_cast<const __nv_bfloat16*>(
          __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_src), k));
      wk[k] = __shfl_sync(0xffffffffu, my_w, k);
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
        if (src[k] == nullptr) continue;  // a dropped slot adds nothing
        const float2 a = unpack_bf16x2(v[k].x), b = unpack_bf16x2(v[k].y), cc = unpack_bf16x2(v[k].z),
                     d = unpack_bf16x2(v[k].w);
        acc[0] += wk[k] * a.x; acc[1] += wk[k] * a.y; acc[2] += wk[k] * b.x; acc[3] += wk[k] * b.y;
        acc[4] += wk[k] * cc.x; acc[5] += wk[k] * cc.y; acc[6] += wk[k] * d.x; acc[7] += wk[k] * d.y;
      }
      st8(y + t * ld_y + c, acc);
    }
  }
}

__global__ void __launch_bounds__(256) combine_bwd_w_peer_kernel(const PeerTable rows, const PeerTable slot_row,
                                                                 const int* __restrict__ idx,
                                                                 const int* __restrict__ expert_rank,
                                                                 const __nv_bfloat16* __restrict__ dy,
                                                                 float* __restrict__ dw, long long n_tokens, int K,
                                                                 int H, long long slot_base, long long ld_rows,
                                                                 long long ld_dy,
                                                                 const __nv_bfloat16* __restrict__ local_rows) {
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  const long long n_slots = n_tokens * K;
  for (long long s = blockIdx.x * static_cast<long long>(warps) + (threadIdx.x >> 5); s < n_slots;
       s += static_cast<long long>(gridDim.x) * warps) {
    const int owner = expert_rank[idx[s]];
    const int row = (peer_ok(slot_row, owner) && (local_rows != nullptr || peer_ok(rows, owner)))
                        ? reinterpret_cast<const int*>(slot_row.ptr[owner])[slot_base + s]
                        : -1;
    float acc = 0.f;
    if (row >= 0) {
      const __nv_bfloat16* a = local_rows ? local_rows + s * ld_rows
                                          : reinterpret_cast<const __nv_bfloat16*>(rows.ptr[owner]) +
                                                static_cast<long long>(row) * ld_rows;
      const __nv_bfloat16* b = dy + (s / K) * ld_dy;
      for (int c = lane * 8; c < H; c += 256) {
        float fa[8], fb[8];
        ld8(a + c, fa);
        ld8(b + c, fb);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += fa[j] * fb[j];
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) dw[s] = acc;
  }
}

// out[i..i+7] = scale * sum over ranks; each lane keeps `world` 16-byte loads in flight
template <bool BF16>
__global__ void __launch_bounds__(256) reduce_scatter_cast_kernel(const PeerTable grads, int world, long long shard_lo,
                                                                  long long n, float scale, float* __restrict__ out) {
  constexpr int EPV = BF16 ? 8 : 4;  // elements per 16-byte vector
  const long long n_vec = n / EPV;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n_vec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    uint4 v[kMaxPeers];
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
      if (r < world) v[r] = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(grads.ptr[r]) +
                                                           (shard_lo + i * EPV) * (BF16 ? 2 : 4))[0];
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r) {
      if (r < world) {
        if (BF16) {
          const float2 a = unpack_bf16x2(v[r].x), b = unpack_bf16x2(v[r].y), c = unpack_bf16x2(v[r].z),
                       d = unpack_bf16x2(v[r].w);
          acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
          acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
        } else {
          acc[0] += __uint_as_float(v[r].x); acc[1] += __uint_as_float(v[r].y);
          acc[2] += __uint_as_float(v[r].z); acc[3] += __uint_as_float(v[r].w);
        }
      }
    }
    float4* o = reinterpret_cast<float4*>(out + i * EPV);
    o[0] = make_float4(acc[0] * scale, acc[1] * scale, acc[2] * scale, acc[3] * scale);
    if (BF16) o[1] = make_float4(acc[4] * scale, acc[5] * scale, acc[6] * scale, acc[7] * scale);
  }
}

// one warp per output row
__global__ void __launch_bounds__(256) reduce_rows_peer_kernel(const PeerTable rows, int world,
                                                               const int* __restrict__ row_map,
                                                               __nv_bfloat16* __restrict__ out, long long n_out, int H,
                                                               long long ld_rows, long long ld_out) {
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  for (long long i = blockIdx.x * static_cast<long long>(warps) + (threadIdx.x >> 5); i < n_out;
       i += static_cast<long long>(gridDim.x) * warps) {
    const long long src_row = row_map ? row_map[i] : i;
    for (int c = lane * 8; c < H; c += 256) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int r = 0; r < world; ++r) {
        float f[8];
        ld8(reinterpret_cast<const __nv_bfloat16*>(rows.ptr[r]) + src_row * ld_rows + c, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[j];
      }
      st8(out + i * ld_out + c, acc);
    }
  }
}

__global__ void __launch_bounds__(256) push_shard_kernel(const PeerTable params, int rank, int world, long long shard_lo,
                                                         long long n_vec) {
  const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(params.ptr[rank]) + shard_lo);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n_vec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 v = src[i];
    for (int r = 0; r < world; ++r) {
      if (r == rank) continue;
      reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.ptr[r]) + shard_lo)[i] = v;
    }
  }
}

inline unsigned blocks_for(long long items, int per_block, int max_blocks) {
  long long b = (items + per_block - 1) / per_block;
  if (b < 1) b = 1;
  if (b > max_blocks) b = max_blocks;
  return static_cast<unsigned>(b);
}

}  // namespace

cudaError_t set_peer_status_word(int* status) {
  return cudaMemcpyToSymbol(g_peer_status, &status, sizeof(status));
}

cudaError_t launch_peer_barrier(const PeerTable& flags, int rank, int world, uint32_t epoch, int* status,
                                unsigned long long timeout_ns, cudaStream_t stream) {
  if (world <= 0 || world > kMaxPeers || rank < 0 || rank >= world) return cudaErrorInvalidValue;
  peer_barrier_kernel<<<1, 32, 0, stream>>>(flags, rank, world, epoch, status,
                                            timeout_ns ? timeout_ns : kDefaultTimeoutNs);
  return cudaGetLastError();
}

cudaError_t launch_peer_allgather(const PeerTable& src, int world, long long n_bytes, void* out, cudaStream_t stream) {
  if (n_bytes % 16 != 0 || world <= 0 || world > kMaxPeers) return cudaErrorInvalidValue;
  const long long n_vec = n_bytes / 16;
  peer_allgather_kernel<<<blocks_for(n_vec * world, 256, 148 * 4), 256, 0, stream>>>(src, world, n_vec,
                                                                                     reinterpret_cast<uint4*>(out));
  return cudaGetLastError();
}

cudaError_t launch_gather_rows_peer(const PeerTable& src, long long slots_per_src, int K, const int* row_slot,
                                    const float* slot_scale, void* out, long long cap_rows, const int* num_m_tiles,
                                    int H, long long ld_src, long long ld_out, cudaStream_t stream) {
  if (H % 8 != 0 || cap_rows <= 0 || K <= 0 || slots_per_src <= 0) return cudaErrorInvalidValue;
  gather_rows_peer_kernel<<<blocks_for(cap_rows, 8, 148 * 8), 256, 0, stream>>>(
      src, slots_per_src, K, row_slot, slot_scale, reinterpret_cast<__nv_bfloat16*>(out), cap_rows, num_m_tiles, H,
      ld_src, ld_out);
  return cudaGetLastError();
}

cudaError_t launch_combine_rows_peer(const PeerTable& rows, const PeerTable& slot_row, const int* idx,
                                     const int* expert_rank, const float* w, void* y, long long n_tokens, int K, int H,
                                     long long slot_base, long long ld_rows, long long ld_y, const void* local_rows,
                                     cudaStream_t stream) {
  if (H % 8 != 0 || n_tokens <= 0 || K <= 0 || K > 32) return cudaErrorInvalidValue;
  static const bool generic_only = [] {
    const char* v = std::getenv("CMOE_COMBINE_GENERIC");  // A/B switch: the kernel with a run-time K for every K
    return v != nullptr && v[0] != '\0' && v[0] != '0';
  }();
  if (!generic_only) {
    const unsigned grid = blocks_for(n_tokens, 8, 148 * 8);
    auto yb = reinterpret_cast<__nv_bfloat16*>(y);
    auto lr = reinterpret_cast<const __nv_bfloat16*>(local_rows);
#define CMOE_COMBINE_PEER_CASE(KK)                                                                                  \
  case KK:                                                                                                          \
    combine_rows_peer_k_kernel<KK><<<grid, 256, 0, stream>>>(rows, slot_row, idx, expert_rank, w, yb, n_tokens, H,  \
                                                             slot_base, ld_rows, ld_y, lr);                         \
    return cudaGetLastError();
    switch (K) {
      CMOE_COMBINE_PEER_CASE(2)
      CMOE_COMBINE_PEER_CASE(4)
      CMOE_COMBINE_PEER_CASE(6)
      CMOE_COMBINE_PEER_CASE(8)
      CMOE_COMBINE_PEER_CASE(12)
      CMOE_COMBINE_PEER_CASE(16)
      default: break;
    }
#undef CMOE_COMBINE_PEER_CASE
  }
  combine_rows_peer_kernel<<<blocks_for(n_tokens, 8, 148 * 8), 256, 0, stream>>>(
      rows, slot_row, idx, expert_rank, w, reinterpret_cast<__nv_bfloat16*>(y), n_tokens, K, H, slot_base, ld_rows,
      ld_y, reinterpret_cast<const __nv_bfloat16*>(local_rows));
  return cudaGetLastError();
}

cudaError_t launch_combine_bwd_w_peer(const PeerTable& rows, const PeerTable& slot_row, const int* idx,
                                      const int* expert_rank, const void* dy, float* dw, long long n_tokens, int K,
                                      int H, long long slot_base, long long ld_rows, long long ld_dy,
                                      const void* local_rows, cudaStream_t stream) {
  if (H % 8 != 0 || n_tokens <= 0 || K <= 0) return cudaErrorInvalidValue;
  combine_bwd_w_peer_kernel<<<blocks_for(n_tokens * K, 8, 148 * 8), 256, 0, stream>>>(
      rows, slot_row, idx, expert_rank, reinterpret_cast<const __nv_bfloat16*>(dy), dw, n_tokens, K, H, slot_base,
      ld_rows, ld_dy, reinterpret_cast<const __nv_bfloat16*>(local_rows));
  return cudaGetLastError();
}

cudaError_t launch_reduce_scatter_cast(const PeerTable& grads, int world, int grad_is_bf16, long long shard_lo,
                                       long long n, float scale, float* out, cudaStream_t stream) {
  if (world <= 0 || world > kMaxPeers || n <= 0 || n % 8 != 0 || shard_lo % 8 != 0) return cudaErrorInvalidValue;
  const long long n_vec = n / (grad_is_bf16 ? 8 : 4);
  const unsigned grid = blocks_for(n_vec, 256, 148 * 8);
  if (grad_is_bf16)
    reduce_scatter_cast_kernel<true><<<grid, 256, 0, stream>>>(grads, world, shard_lo, n, scale, out);
  else
    reduce_scatter_cast_kernel<false><<<grid, 256, 0, stream>>>(grads, world, shard_lo, n, scale, out);
  return cudaGetLastError();
}

cudaError_t launch_reduce_rows_peer(const PeerTable& rows, int world, const int* row_map, void* out, long long n_out,
                                    int H, long long ld_rows, long long ld_out, cudaStream_t stream) {
  if (world <= 0 || world > kMaxPeers || n_out <= 0 || H % 8 != 0) return cudaErrorInvalidValue;
  reduce_rows_peer_kernel<<<blocks_for(n_out, 8, 148 * 8), 256, 0, stream>>>(
      rows, world, row_map, reinterpret_cast<__nv_bfloat16*>(out), n_out, H, ld_rows, ld_out);
  return cudaGetLastError();
}

cudaError_t launch_push_shard(const PeerTable& params, int rank, int world, long long shard_lo, long long n,
                              cudaStream_t stream) {
  if (world <= 0 || world > kMaxPeers || n <= 0 || n % 8 != 0 || shard_lo % 8 != 0) return cudaErrorInvalidValue;
  push_shard_kernel<<<blocks_for(n / 8, 256, 148 * 8), 256, 0, stream>>>(params, rank, world, shard_lo, n / 8);
  return cudaGetLastError();
}

}  // namespace cmoe
