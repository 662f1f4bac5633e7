// nq_row_reduce_pull: the SUM all-reduce that ends a row-parallel linear, for prefill-sized outputs, as ONE kernel
// per rank over peer-mapped ("symmetric") buffers: a two-shot exchange in which every transfer is a pull.
//
// Stands in for `dist.all_reduce(y)` of RowParallelLinear.forward (nano_qwen, src/nano_qwen/layers/linear.py:154-155)
// when y is large (bandwidth bound).  The row-parallel GEMM writes its partial output into a buffer that every
// GPU of the group has mapped; rank r owns the r-th slice of the message:
//   barrier A | own slice: y = S_own = sum over ranks (rank order, fp32) of S_q | fence, barrier B |
//   other slices q: y = S_q (the owner's sum) | barrier C (nobody reads this rank's buffer now)
// All transfers are bulk asynchronous copies (cp.async.bulk, no multicast, no tensor map) from the peers' buffers
// into shared memory, 64 KB per stage and three stages per block in flight: an SM sustains far more bytes in flight
// that way than with loads into registers (which topped out near 12 GB/s per SM over NVLink), so 16 blocks are
// enough to fill the links.
// Per GPU (tp-1)/tp of a message arrives in each of the two phases; the result lands in a private tensor y.  Every
// slice is summed once, by its owner, so all ranks end with the same bits.  A small grid is enough,
// which leaves the other SMs to a GEMM running beside it on another stream.
//
// Barriers: block b of rank r only ever waits for block b of its peers, through per-rank signal pads that the
// peers write with system-scope release stores; the call number (64-bit, in device memory, so that a CUDA graph
// replays correctly) tags the flags, nothing is ever reset.  Waits are bounded: on expiry the status block gets
// NQ_ERR_DEVICE_TIMEOUT (site 80/81/82, aux = the peer) and the kernel finishes.  All ranks must launch the same
// grid; no block waits for another block of its own grid.
//
// An in-switch variant of the same exchange (multimem.ld_reduce / multimem.st on an NVLS multicast mapping) was
// built and measured: 550-640 us for 64 MiB at 2 and 4 ranks against 130-190 us for this kernel and 150-185 us for
// NCCL, whatever the grid; it was removed.
#include "nq_internal.cuh"

namespace nq {
namespace {

constexpr int kMcMaxRanks = NQ_P2P_MAX_RANKS;
constexpr int kMcMaxBlocks = NQ_SYM_MAX_BLOCKS;
constexpr int kSiteMcBarrierA = 80;
constexpr int kSiteMcBarrierB = 81;
constexpr int kSiteMcBarrierC = 82;

struct McReduceParams {
  uint8_t* buf[kMcMaxRanks];     // the message in every rank's buffer as mapped here (peer pointers)
  uint4* y;                      // private result tensor
  int64_t n16;                   // 16-byte units in the message
  uint32_t* pad[kMcMaxRanks];    // signal pad of every rank as mapped here: [3][kMcMaxBlocks][kMcMaxRanks] words
  int rank, tp;
  uint64_t* state;               // [0] calls completed, [1] low half: ticket of the blocks of the call in flight
  DeviceStatus* status;
  uint64_t limit_ns;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Block b of this rank tells block b of every peer "I am at barrier `phase` of call `tag`" and waits for the same
// from each of them.  Threads 0..tp-1 each handle one peer.
__device__ __forceinline__ void mc_barrier(const McReduceParams& p, int phase, uint32_t tag, int site, int* s_abort) {
  const int t = threadIdx.x;
  if (t < p.tp) {
    const size_t slot = (static_cast<size_t>(phase) * kMcMaxBlocks + blockIdx.x) * kMcMaxRanks;
    st_release_sys(p.pad[t] + slot + p.rank, tag);                 // into peer t's pad (t == rank: my own)
    const uint32_t* mine = p.pad[p.rank] + slot + t;
    const long long t0 = clock64();
    const long long limit_cycles = static_cast<long long>(p.limit_ns) * 2;
    for (uint32_t spin = 1; ld_acquire_sys(mine) != tag; ++spin) {
      if ((spin & 63u) == 0u) {
        if (*reinterpret_cast<volatile int*>(s_abort)) break;
        if (clock64() - t0 > limit_cycles) {
          *reinterpret_cast<volatile int*>(s_abort) = 1;
          if (p.status != nullptr && atomicCAS(&p.status->code, 0, kErrDeviceTimeout) == 0) {
            p.status->where = site;
            p.status->block = static_cast<int>(blockIdx.x);
            p.status->aux = t;
            __threadfence_system();
          }
          break;
        }
      }
    }
  }
  __syncthreads();
}

__device__ __forceinline__ void acc_bf16x8(float (&acc)[8], const uint4& v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[2 * i] += bf16_bits_to_float(w[i] & 0xFFFFu);
    acc[2 * i + 1] += bf16_bits_to_float(w[i] >> 16);
  }
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ int64_t imin64(int64_t a, int64_t b) { return a < b ? a : b; }

// ---- bulk-copy helpers (non-tensor cp.async.bulk: 16-byte aligned addresses, sizes multiples of 16) ----
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gmem_dst), "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Bounded wait on a block-local mbarrier (same give-up rule as the cross-GPU barriers).
__device__ __forceinline__ bool sym_wait(uint64_t* bar, uint32_t parity, const McReduceParams& p, int* s_abort, int site,
                                         int aux) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  const long long limit_cycles = static_cast<long long>(p.limit_ns) * 2;
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 255u) == 0u) {
      if (*reinterpret_cast<volatile int*>(s_abort)) return false;
      if (clock64() - t0 > limit_cycles) {
        *reinterpret_cast<volatile int*>(s_abort) = 1;
        if (p.status != nullptr && atomicCAS(&p.status->code, 0, kErrDeviceTimeout) == 0) {
          p.status->where = site;
          p.status->block = static_cast<int>(blockIdx.x);
          p.status->aux = aux;
          __threadfence_system();
        }
        return false;
      }
    }
  }
}

constexpr int kSymStageBytes = 64 * 1024;
constexpr int kSymStages = 3;
constexpr int kSymConsumerWarps = 8;
constexpr int kSymThreads = 32 * (kSymConsumerWarps + 1);
constexpr int kSymSmemBytes = kSymStages * kSymStageBytes + 1024;
constexpr int kSiteSymPipe = 83;

struct SymBars {
  uint64_t full1[kSymStages], empty1[kSymStages], full2[kSymStages];
};

// This block's contiguous share of slice q, in 16-byte units.
__device__ __forceinline__ void sym_share(const McReduceParams& p, int tp, int q, int64_t& lo, int64_t& hi) {
  const int64_t per_rank = (p.n16 + tp - 1) / tp;
  const int64_t slo = min(per_rank * q, p.n16), shi = min(slo + per_rank, p.n16);
  const int64_t per_block = (shi - slo + gridDim.x - 1) / gridDim.x;
  lo = min(slo + per_block * blockIdx.x, shi);
  hi = min(lo + per_block, shi);
}

template <int TP>
__global__ void __launch_bounds__(kSymThreads, 1) row_reduce_pull_kernel(const McReduceParams p) {
  extern __shared__ __align__(128) uint8_t sym_smem[];
  __shared__ int s_abort;
  uint8_t* stages = sym_smem;
  SymBars* bars = reinterpret_cast<SymBars*>(sym_smem + kSymStages * kSymStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < kSymStages; ++s) {
      mbar_init(&bars->full1[s], 1);
      mbar_init(&bars->empty1[s], kSymConsumerWarps);
      mbar_init(&bars->full2[s], 1);
    }
    fence_mbar_init();
  }
  __syncthreads();
  const uint64_t call = *reinterpret_cast<volatile uint64_t*>(p.state) + 1ull;
  const uint32_t tag = static_cast<uint32_t>(call % 0xFFFFFFFFull) + 1u;

  mc_barrier(p, 0, tag, kSiteMcBarrierA, &s_abort);      // every rank's partial is complete

  // ---- phase 1: sum this block's share of the own slice.  One thread keeps bulk loads of the TP partials in
  //      flight (three stages of 64 KB), eight warps add them up from shared memory in rank order. ----
  constexpr int kChunk = kSymStageBytes / TP;             // bytes of one rank's partial per stage
  constexpr int kChunkUnits = kChunk / 16;
  int64_t lo, hi;
  sym_share(p, TP, p.rank, lo, hi);
  const int n_chunks = static_cast<int>((hi - lo + kChunkUnits - 1) / kChunkUnits);
  if (warp == kSymConsumerWarps) {
    if (lane == 0 && !s_abort) {
      fence_proxy_async_all();
      for (int k = 0; k < n_chunks; ++k) {
        const int s = k % kSymStages;
        const uint32_t ph = (k / kSymStages) & 1;
        if (!sym_wait(&bars->empty1[s], ph ^ 1, p, &s_abort, kSiteSymPipe, k)) break;
        const int64_t o = lo + static_cast<int64_t>(k) * kChunkUnits;
        const uint32_t bytes = static_cast<uint32_t>(imin64(kChunkUnits, hi - o)) * 16u;
        mbar_arrive_expect_tx(&bars->full1[s], bytes * TP);
#pragma unroll
        for (int r = 0; r < TP; ++r)
          bulk_load(stages + s * kSymStageBytes + r * kChunk, p.buf[r] + o * 16, bytes, &bars->full1[s]);
      }
    }
  } else {
    uint4* own = reinterpret_cast<uint4*>(p.buf[p.rank]);
    for (int k = 0; k < n_chunks; ++k) {
      const int s = k % kSymStages;
      const uint32_t ph = (k / kSymStages) & 1;
      if (!sym_wait(&bars->full1[s], ph, p, &s_abort, kSiteSymPipe, k)) break;
      const int64_t o = lo + static_cast<int64_t>(k) * kChunkUnits;
      const int units = static_cast<int>(imin64(kChunkUnits, hi - o));
      const uint8_t* st = stages + s * kSymStageBytes;
      for (int u = threadIdx.x; u < units; u += 32 * kSymConsumerWarps) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < TP; ++r)                                            // rank order
          acc_bf16x8(acc, *reinterpret_cast<const uint4*>(st + r * kChunk + u * 16));
        const uint4 v = make_uint4(pack2(acc[0], acc[1]), pack2(acc[2], acc[3]), pack2(acc[4], acc[5]), pack2(acc[6], acc[7]));
        own[o + u] = v;
        p.y[o + u] = v;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->empty1[s]);
    }
  }
  __threadfence_system();          // the sums written to this rank's buffer are performed before the flag is seen
  __syncthreads();

  mc_barrier(p, 1, tag, kSiteMcBarrierB, &s_abort);      // every owner's sums are in its buffer

  // ---- phase 2: fetch the other slices' sums from their owners: bulk load into shared memory, bulk store to y;
  //      one thread drives both, two loads ahead of the store ----
  if (warp == kSymConsumerWarps && lane == 0 && !s_abort) {
    fence_proxy_async_all();
    constexpr int kUnits2 = kSymStageBytes / 16;
    int issued = 0, stored = 0;                           // chunks over all peers, in one sequence
    // enumerate chunks lazily: (peer index d, chunk c)
    int d_i = 1, c_i = 0;                                  // issue cursor
    int d_s = 1, c_s = 0;                                  // store cursor
    int64_t lo_i = 0, hi_i = 0, lo_s = 0, hi_s = 0;
    if (TP > 1) { sym_share(p, TP, (p.rank + 1) % TP, lo_i, hi_i); lo_s = lo_i; hi_s = hi_i; }
    bool ok = true;
    auto advance = [&](int& d, int& c, int64_t& l, int64_t& h) {      // skips empty shares
      ++c;
      while (d < TP && l + static_cast<int64_t>(c) * kUnits2 >= h) {
        ++d; c = 0;
        if (d < TP) sym_share(p, TP, (p.rank + d) % TP, l, h);
      }
    };
    while (d_i < TP && lo_i >= hi_i) { ++d_i; if (d_i < TP) sym_share(p, TP, (p.rank + d_i) % TP, lo_i, hi_i); }
    while (d_s < TP && lo_s >= hi_s) { ++d_s; if (d_s < TP) sym_share(p, TP, (p.rank + d_s) % TP, lo_s, hi_s); }
    while (ok && d_s < TP) {
      // keep up to kSymStages - 1 loads ahead of the store
      while (d_i < TP && issued - stored < kSymStages - 1) {
        const int s = issued % kSymStages;
        if (issued >= kSymStages) {
          // the store that last read this stage was committed kSymStages chunks ago
          asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kSymStages - 2) : "memory");
        }
        const int64_t o = lo_i + static_cast<int64_t>(c_i) * kUnits2;
        const uint32_t bytes = static_cast<uint32_t>(imin64(kUnits2, hi_i - o)) * 16u;
        mbar_arrive_expect_tx(&bars->full2[s], bytes);
        bulk_load(stages + s * kSymStageBytes, p.buf[(p.rank + d_i) % TP] + o * 16, bytes, &bars->full2[s]);
        ++issued;
        advance(d_i, c_i, lo_i, hi_i);
      }
      const int s = stored % kSymStages;
      const uint32_t ph = (stored / kSymStages) & 1;
      if (!sym_wait(&bars->full2[s], ph, p, &s_abort, kSiteSymPipe + 1, stored)) { ok = false; break; }
      const int64_t o = lo_s + static_cast<int64_t>(c_s) * kUnits2;
      const uint32_t bytes = static_cast<uint32_t>(imin64(kUnits2, hi_s - o)) * 16u;
      bulk_store(reinterpret_cast<uint8_t*>(p.y) + o * 16, stages + s * kSymStageBytes, bytes);
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      ++stored;
      advance(d_s, c_s, lo_s, hi_s);
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // y is complete before the kernel ends
  }
  __syncthreads();

  mc_barrier(p, 2, tag, kSiteMcBarrierC, &s_abort);      // nobody reads this rank's buffer any more

  if (threadIdx.x == 0) {
    uint32_t* ticket = reinterpret_cast<uint32_t*>(p.state + 1);
    if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
      *ticket = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint64_t*>(p.state) = call;
    }
  }
}

}  // namespace
}  // namespace nq

namespace nq {
int setup_sym_kernels() {
  cudaError_t e = cudaFuncSetAttribute(row_reduce_pull_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSymSmemBytes);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(row_reduce_pull_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSymSmemBytes);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(row_reduce_pull_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSymSmemBytes);
  return check_cuda(e);
}
}  // namespace nq

using namespace nq;

extern "C" int nq_row_reduce_pull(void* const* bufs, void* y, int64_t count, void* const* pads, int rank, int tp,
                                  void* state, int blocks, void* stream) {
  if (count < 0 || tp < 2 || tp > kMcMaxRanks || rank < 0 || rank >= tp) return NQ_ERR_BAD_ARGUMENT;
  if (count == 0) return NQ_OK;
  if (!bufs || !y || !pads || !state) return NQ_ERR_BAD_ARGUMENT;
  if (count % 8 != 0 || reinterpret_cast<uintptr_t>(y) % 16) return NQ_ERR_BAD_ARGUMENT;
  if (blocks < 1 || blocks > kMcMaxBlocks) return NQ_ERR_BAD_ARGUMENT;
  if (tp != 2 && tp != 4 && tp != 8) return NQ_ERR_UNSUPPORTED;
  DeviceCtx* ctx = nullptr;
  const int st = ensure_init(&ctx);
  if (st != NQ_OK) return st;
  McReduceParams p;
  p.y = static_cast<uint4*>(y);
  p.n16 = count / 8;
  for (int r = 0; r < kMcMaxRanks; ++r) {
    p.pad[r] = r < tp ? static_cast<uint32_t*>(pads[r]) : nullptr;
    p.buf[r] = r < tp ? static_cast<uint8_t*>(bufs[r]) : nullptr;
    if (r < tp && (p.pad[r] == nullptr || p.buf[r] == nullptr || reinterpret_cast<uintptr_t>(p.buf[r]) % 16))
      return NQ_ERR_BAD_ARGUMENT;
  }
  p.rank = rank;
  p.tp = tp;
  p.state = static_cast<uint64_t*>(state);
  p.status = ctx->status_dev;
  p.limit_ns = wait_limit_ns();
  const dim3 grid(static_cast<unsigned>(blocks));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (tp == 2) row_reduce_pull_kernel<2><<<grid, kSymThreads, kSymSmemBytes, s>>>(p);
  else if (tp == 4) row_reduce_pull_kernel<4><<<grid, kSymThreads, kSymSmemBytes, s>>>(p);
  else row_reduce_pull_kernel<8><<<grid, kSymThreads, kSymSmemBytes, s>>>(p);
  count_launch();
  return check_cuda(cudaGetLastError());
}

