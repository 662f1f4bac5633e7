// Thin wrappers over the sm_100a PTX this library uses: mbarrier, TMA
// (cp.async.bulk.tensor, never with cluster multicast), tcgen05 (TMEM
// allocation, UMMA issue/commit, TMEM loads) and bounded waits.
//
// Every wait on an mbarrier goes through mbar_wait(), which gives up after a
// wall-clock limit, raises a CTA-wide abort flag and records where it gave up;
// callers leave their loop and fall through to the common teardown, so a
// kernel never spins forever and never traps.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nq {

// Device-visible status block (mapped pinned host memory, one per device).
struct DeviceStatus {
  int code;        // 0 = OK, else an NQ_ERR_* value written by the first failing CTA
  int where;       // site id of the wait that expired
  int block;       // blockIdx.x of the reporter
  int aux;         // site-specific (stage / K-tile index)
};

constexpr int kErrDeviceTimeout = -5;  // mirrors NQ_ERR_DEVICE_TIMEOUT in include/nq_fp8.h

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31; }

// ------------------------------- mbarrier --------------------------------- //
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking probe of the same condition (never suspends the thread).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}

// Shared by all roles of a CTA: raised once, never cleared during the launch.
struct AbortCtl {
  volatile int* flag;       // in shared memory
  DeviceStatus* status;     // mapped host memory (may be null)
  uint64_t limit_ns;        // wall-clock limit for one wait
  uint32_t wait_mode;       // 0 try_wait, 1 test_wait spin, >1 try_wait with that suspend-time hint (ns)
};

static __device__ __noinline__ void report_timeout(const AbortCtl& ac, int where, int aux) {
  *ac.flag = 1;
  if (ac.status != nullptr) {
    if (atomicCAS(&ac.status->code, 0, kErrDeviceTimeout) == 0) {
      ac.status->where = where;
      ac.status->block = static_cast<int>(blockIdx.x);
      ac.status->aux = aux;
      __threadfence_system();
    }
  }
}

// Waits for the phase with the given parity.  Returns false when the CTA is
// aborting (this wait or another one ran out of time).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const AbortCtl& ac, int where, int aux) {
  if (mbar_try_wait(bar, parity)) return true;
  // The limit is checked against the SM cycle counter (cheap to read; ~2 GHz, so
  // 2 cycles per nanosecond is a generous conversion of the wall-clock limit).
  const long long t0 = clock64();
  const long long limit_cycles = static_cast<long long>(ac.limit_ns) * 2;
  for (uint32_t spin = 1;; ++spin) {
    if (ac.wait_mode == 1) { if (mbar_test_wait(bar, parity)) return true; }
    else if (ac.wait_mode > 1) { if (mbar_try_wait_hint(bar, parity, ac.wait_mode)) return true; }
    else if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 255u) == 0u) {
      if (*ac.flag) return false;
      if (clock64() - t0 > limit_cycles) {
        report_timeout(ac, where, aux);
        return false;
      }
    }
  }
}

// Same bounded wait with cluster-scope acquire: the barrier is completed by another CTA of the cluster
// (remote arrivals, or copies issued by the peer).
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, const AbortCtl& ac, int where, int aux) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  const long long limit_cycles = static_cast<long long>(ac.limit_ns) * 2;
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((spin & 255u) == 0u) {
      if (*ac.flag) return false;
      if (clock64() - t0 > limit_cycles) {
        report_timeout(ac, where, aux);
        return false;
      }
    }
  }
}

// ---------------------------------- TMA ------------------------------------ //
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tiled load global -> shared::cta of this CTA; completes on `bar` by bytes.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_hint(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
// 2-D tiled store shared::cta -> global (bulk async group of the issuing thread); rows / columns outside the
// tensor are clipped by the hardware.  x * element size must be a multiple of 16 bytes, coordinates >= 0.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most N of this thread's store groups still READ their shared-memory source.
template <int N> __device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N> __device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// Programmatic dependent launch: wait for the kernels this one depends on /
// let the next kernel in the stream start its prologue.
__device__ __forceinline__ void pdl_wait_prior() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_next() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Register re-balancing between warpgroups (all four warps of a warpgroup must
// execute the same instruction).
template <int N> __device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N> __device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// -------------------------------- tcgen05 ---------------------------------- //
// TMEM allocation: whole warp, column count a power of two in [32, 512]; the
// base address lands in shared memory.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// All UMMAs issued so far by this thread arrive on `bar` when they complete.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ---- CTA-pair (cta_group::2) variants: one UMMA spans two SMs of a cluster of two CTAs ----
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Completion of all UMMAs issued so far by this thread (pair-wide) arrives on the barrier at this
// shared::cluster address, which may belong to either CTA of the pair.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}
// D[tmem, both CTAs] (+)= A * B^T, 256 x N x 32: each CTA supplies its own 128 rows of A and its half of
// the N rows of B from the same shared-memory offsets; issued by one thread of the leader CTA.
__device__ __forceinline__ void umma_f8_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 2-D tiled load into this CTA's shared memory whose completion bytes are counted on a barrier that may
// live in the other CTA of the pair (shared::cluster address).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t local_smem_addr, uint32_t cta_rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(cta_rank));
  return remote;
}
// Arrival on a barrier of another CTA of the cluster with the default (CTA-scope release) semantics: enough where the
// arrival only orders this thread's completed tensor-memory reads (tcgen05.wait::ld + fence::before_thread_sync).
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile whose rows are
// exactly 128 bytes (one 128-byte swizzle atom wide), rows 8-by-8 in 1024-byte
// groups, as written by a TMA load with CU_TENSOR_MAP_SWIZZLE_128B into a
// 1024-byte aligned buffer.
//   bits [0,14)  start address >> 4
//   bits [16,30) leading-dimension byte offset >> 4 (unused for this layout; 1)
//   bits [32,46) stride-dimension byte offset >> 4 = 1024 >> 4 (next 8-row group)
//   bits [46,48) descriptor version = 1 on sm_100
//   bits [61,64) layout type = 2 (128-byte swizzle)
__device__ __forceinline__ uint64_t umma_smem_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor for kind::f8f6f4, e4m3 x e4m3 -> fp32, both operands
// K-major, dense:  c_format(F32)=1 at [4,6); a/b format (E4M3)=0 at [7,10)/[10,13);
// a/b major (K)=0 at 15/16; N>>3 at [17,23); M>>4 at [24,29).
__host__ __device__ constexpr uint32_t umma_idesc_e4m3_f32(int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]^T, one 128 x N x 32 step; single thread issues.
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// TMEM -> registers: this warp's 32 lanes x 32 consecutive fp32 columns.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
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
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Same wait, tied to the destination registers of a load so that the compiler cannot
// schedule a consumer of those registers ahead of it.
__device__ __forceinline__ void tmem_ld_wait_on(uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.wait::ld.sync.aligned;"
      : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
        "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]),
        "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]),
        "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
      :
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait_on(uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.wait::ld.sync.aligned;"
      : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
        "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
      :
      : "memory");
}

// Global loads that stay where they are written.  A compiler under register pressure may move an ordinary (or
// __ldg) load down to its first use, which turns a software prefetch into an exposed round trip; a volatile asm
// statement keeps its place among the other volatile asm statements (barrier waits, arrivals).
__device__ __forceinline__ uint4 ld_global_v4_pinned(const void* p) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ float ld_global_f32_pinned(const float* p) {
  float v;
  asm volatile("ld.global.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}

// ------------------------- quantisation arithmetic (shared by the quantiser kernels and the fused GEMM) ---
__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) { return __uint_as_float(bits16 << 16); }

// x / s, correctly rounded, for many x and one s.  With y = RN(1/s): q0 = RN(x*y), r = x - s*q0 (exact in one
// FMA), q = RN(q0 + r*y) equals RN(x/s) unless the significand of s is all ones or an exponent is extreme
// (Markstein); those scales take the IEEE divide.  Three instructions per element instead of about ten.
struct ExactDivider {
  float s, y;
  bool slow;
  __device__ __forceinline__ explicit ExactDivider(float scale) : s(scale) {
    const uint32_t bits = __float_as_uint(scale);
    slow = !(scale >= 1e-30f && scale <= 1e30f) || ((bits & 0x7FFFFFu) == 0x7FFFFFu);
    y = __frcp_rn(scale);
  }
  __device__ __forceinline__ float operator()(float x) const {
    if (slow) return __fdiv_rn(x, s);
    const float q0 = __fmul_rn(x, y);
    const float r = __fmaf_rn(-s, q0, x);
    return __fmaf_rn(r, y, q0);
  }
  // Two quotients with packed two-wide instructions (same IEEE operations per lane); only for !slow.
  __device__ __forceinline__ float2 fast2(float2 x) const {
    const float2 y2 = make_float2(y, y);
    const float2 q0 = __fmul2_rn(x, y2);
    const float2 r = __ffma2_rn(make_float2(-s, -s), q0, x);
    return __ffma2_rn(r, y2, q0);
  }
};

// |a| max |b| element-wise on packed bf16 pairs (exact: a maximum never rounds).
__device__ __forceinline__ uint32_t bf16x2_absmax(uint32_t a, uint32_t b) {
  const __nv_bfloat162 x = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&a));
  const __nv_bfloat162 y = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&b));
  const __nv_bfloat162 m = __hmax2(x, y);
  return *reinterpret_cast<const uint32_t*>(&m);
}

__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}


}  // namespace nq
