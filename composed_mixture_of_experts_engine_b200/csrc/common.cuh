// Shared device-side building blocks for the sm_100a kernels of this package:
// mbarrier / TMA / tcgen05 (TMEM, UMMA) PTX wrappers, bounded waits and the
// status words through which a kernel reports that a wait ran out.
//
// Every wait in this package is bounded.  A wait that runs out records a
// status code in global memory, raises a CTA-wide abort flag (so that every
// later wait of the CTA returns at once) and the kernel then runs to its normal
// end: TMEM is freed and the context stays usable.  The host reads the status.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cmoe {

// ----------------------------------------------------------------------------
// status codes written to the int status word of a launch (0 = no error)
// ----------------------------------------------------------------------------
enum StatusCode : int {
  ST_OK = 0,
  ST_TIMEOUT_SMEM_FULL = 1,    // consumer waited for a TMA stage that never landed
  ST_TIMEOUT_SMEM_EMPTY = 2,   // producer waited for a stage that was never released
  ST_TIMEOUT_TMEM_FULL = 3,    // epilogue waited for an accumulator that was never committed
  ST_TIMEOUT_TMEM_EMPTY = 4,   // MMA warp waited for an accumulator that was never drained
  ST_TIMEOUT_PEER_FLAG = 5,    // waited for a flag that a peer GPU (or another CTA) never wrote
  ST_BAD_ARGUMENT = 6,
  ST_BAD_INDEX = 7,             // a row plan or routing table named a rank / row outside the buffers: access skipped
};

constexpr unsigned long long kDefaultTimeoutNs = 4000000000ull;  // 4 s

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " elect.sync _|p, 0xffffffff;\n"
      " selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ----------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      " selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Per-CTA wait context: the abort flag lives in shared memory, the status word
// in global memory.  `timeout_ns` bounds every single wait.
struct WaitCtx {
  volatile int* abort_flag;
  int* status;
  unsigned long long timeout_ns;
};

// Returns true when the phase completed, false when the wait ran out (or the
// CTA had already aborted).  Never spins without a limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtx& w, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*w.abort_flag) return false;
  const unsigned long long t0 = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if (((++spins) & 63u) == 0u) {
      if (*w.abort_flag) return false;
      if (global_timer_ns() - t0 > w.timeout_ns) {
        *w.abort_flag = 1;
        if (w.status) atomicCAS(w.status, 0, code);
        return false;
      }
    }
  }
  return true;
}

// Bounded wait on a 32-bit flag in global (possibly peer-written) memory:
// returns once *flag >= target (acquire at system scope).
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ bool flag_wait_ge(const uint32_t* flag, uint32_t target, const WaitCtx& w,
                                             int code = ST_TIMEOUT_PEER_FLAG) {
  if ((int32_t)(ld_acquire_sys(flag) - target) >= 0) return true;
  if (w.abort_flag && *w.abort_flag) return false;
  const unsigned long long t0 = global_timer_ns();
  uint32_t spins = 0;
  while ((int32_t)(ld_acquire_sys(flag) - target) < 0) {
    __nanosleep(64);
    if (((++spins) & 31u) == 0u) {
      if (w.abort_flag && *w.abort_flag) return false;
      if (global_timer_ns() - t0 > w.timeout_ns) {
        if (w.abort_flag) *w.abort_flag = 1;
        if (w.status) atomicCAS(w.status, 0, code);
        return false;
      }
    }
  }
  return true;
}

// The same bounded wait on a flag that a CTA of this GPU writes (gpu-scope acquire: cheaper than the system-scope
// one that flags written by peers need).
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool flag_wait_ge_gpu(const uint32_t* flag, uint32_t target, const WaitCtx& w,
                                                 int code = ST_TIMEOUT_PEER_FLAG) {
  if ((int32_t)(ld_acquire_gpu(flag) - target) >= 0) return true;
  if (w.abort_flag && *w.abort_flag) return false;
  const unsigned long long t0 = global_timer_ns();
  uint32_t spins = 0;
  while ((int32_t)(ld_acquire_gpu(flag) - target) < 0) {
    __nanosleep(64);
    if (((++spins) & 31u) == 0u) {
      if (w.abort_flag && *w.abort_flag) return false;
      if (global_timer_ns() - t0 > w.timeout_ns) {
        if (w.abort_flag) *w.abort_flag = 1;
        if (w.status) atomicCAS(w.status, 0, code);
        return false;
      }
    }
  }
  return true;
}

// ----------------------------------------------------------------------------
// TMA (tiled bulk tensor copies, this GPU's memory only; no cluster broadcast)
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
// x = innermost coordinate (elements).  x * sizeof(element) must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// Asks the TMA unit to bring the box at (x, y) into L2 without a destination in shared memory: a later load of the
// same box then pays L2 latency instead of DRAM latency.  No completion is tracked; same alignment rule for x.
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* tmap, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(x), "r"(y)
               : "memory");
}

// Tiled TMA stores (shared -> global) of a [1, rows, cols] box of a rank-3 tensor map, tracked by bulk async-groups.
// x = innermost coordinate (elements): x * sizeof(element) must be a multiple of 16 bytes; no coordinate may be negative.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* tmap, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
// same box, added element-wise to global memory (the addition happens in L2; the SM never reads the old values)
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* tmap, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// waits until the shared-memory sources of all but the N most recent bulk groups of this thread have been read
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// waits until all but the N most recent bulk groups of this thread have completed (writes performed)
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// ----------------------------------------------------------------------------
// tcgen05: tensor memory and UMMA
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrives once on `bar` when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], bf16 inputs, fp32 accumulate.  `accumulate` = 0 overwrites D.
__device__ __forceinline__ void umma_bf16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Instruction descriptor for kind::f16 with bf16 operands and an fp32 accumulator.
//   [4,6) D format (1 = f32)   [7,10) A format (1 = bf16)   [10,13) B format (1 = bf16)
//   [15] A major (0 = K, 1 = MN)   [16] B major   [17,23) N >> 3   [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc_bf16(int m, int n, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// Shared-memory matrix descriptor, 128-byte swizzle.
//   [0,14) start address >> 4   [16,30) leading byte offset >> 4   [32,46) stride byte offset >> 4
//   [46,48) descriptor version (1 on sm_100)   [61,64) layout (2 = SWIZZLE_128B)
// K-major operand (rows of 64 bf16 = 128 B): SBO = 1024 (eight rows), LBO unused.
// MN-major operand (k-rows of 64 contiguous MN elements): LBO = stride between 64-element MN
// chunks, SBO = 1024 (eight k-rows).
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// TMEM -> registers: each thread of the warp reads 32 consecutive fp32 columns of its own
// lane (lane = 32 * (warp_id % 4) + lane_id).  taddr = (lane_base << 16) | column.
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ----------------------------------------------------------------------------
// small numeric helpers
// ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t v) {
  __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&v);
  return __bfloat1622float2(b);
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace cmoe
