// nq_row_reduce_mc: the SUM all-reduce that ends a row-parallel linear, for prefill-sized outputs, done by ONE
// kernel per rank with the reduction inside the NVLink switch (NVLS: multimem.ld_reduce / multimem.st).
//
// Stands in for `dist.all_reduce(y)` of RowParallelLinear.forward (nano_qwen, src/nano_qwen/layers/linear.py:154-155)
// when y is large (bandwidth bound).  Every rank's partial sits at the same offset of a buffer that is mapped on
// all GPUs of the group and bound to one multicast address.  Rank r owns the r-th slice of the message:
//   1. barrier A with the same block index of every peer (their partials are complete and visible),
//   2. for each 16 bytes of its slice:  v = multimem.ld_reduce.add (the switch fetches the 16 bytes from every GPU
//      and adds them in fp32),  multimem.st v  (the switch writes the sum into every GPU's copy, in place),
//   3. system fence, barrier B (every slice of the local copy now holds the sum).
// Per GPU this moves one message out and one message in, whatever the number of ranks (a ring or a two-shot
// exchange over plain peer memory moves 2 (tp-1)/tp messages each way and reduces on the SMs).
// Every rank ends with the same bits (the sum is computed once, in the switch, and broadcast).
//
// Barriers: block b of rank r only ever waits for block b of its peers, through per-rank signal pads that the
// peers write with system-scope release stores; the call number (64-bit, in device memory, so that a CUDA graph
// replays correctly) tags the flags, nothing is ever reset.  Waits are bounded: on expiry the status block gets
// NQ_ERR_DEVICE_TIMEOUT (site 80/81, aux = the peer) and the kernel finishes.  All ranks must launch the same
// grid; the grid is small enough to be resident at once, and no block waits for another block of its own grid.
#include "nq_internal.cuh"

namespace nq {
namespace {

constexpr int kMcMaxRanks = NQ_P2P_MAX_RANKS;
constexpr int kMcThreads = 512;
constexpr int kMcMaxBlocks = NQ_MC_MAX_BLOCKS;
constexpr int kSiteMcBarrierA = 80;
constexpr int kSiteMcBarrierB = 81;
constexpr int kSiteMcBarrierC = 82;

struct McReduceParams {
  uint8_t* mc;                   // multicast address of the message (same offset on every GPU); NVLS kernel only
  uint8_t* buf[kMcMaxRanks];     // the message in every rank's buffer as mapped here (peer pointers); pull kernel only
  uint4* y;                      // private result tensor; pull kernel only
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
__device__ __forceinline__ uint4 mc_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void mc_st_16(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
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

__global__ void __launch_bounds__(kMcThreads) row_reduce_mc_kernel(const McReduceParams p) {
  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = 0;
  __syncthreads();
  const uint64_t call = *reinterpret_cast<volatile uint64_t*>(p.state) + 1ull;
  const uint32_t tag = static_cast<uint32_t>(call % 0xFFFFFFFFull) + 1u;      // never 0 (a pad that was never written)

  mc_barrier(p, 0, tag, kSiteMcBarrierA, &s_abort);

  // this rank's slice of the message, shared out over the blocks in interleaved chunks of kMcThreads * 4 units
  const int64_t per_rank = (p.n16 + p.tp - 1) / p.tp;
  const int64_t lo = min(per_rank * p.rank, p.n16), hi = min(lo + per_rank, p.n16);
  constexpr int kUnroll = 4;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kMcThreads * kUnroll;
  if (!s_abort) {
    for (int64_t base = lo + (static_cast<int64_t>(blockIdx.x) * kMcThreads + threadIdx.x) * kUnroll; base < hi;
         base += stride) {
      uint4 v[kUnroll];
#pragma unroll
      for (int j = 0; j < kUnroll; ++j)
        if (base + j < hi) v[j] = mc_ld_reduce_bf16x8(p.mc + (base + j) * 16);
#pragma unroll
      for (int j = 0; j < kUnroll; ++j)
        if (base + j < hi) mc_st_16(p.mc + (base + j) * 16, v[j]);
    }
  }
  __threadfence_system();          // this thread's broadcasts are performed before the flag below is seen
  __syncthreads();

  mc_barrier(p, 1, tag, kSiteMcBarrierB, &s_abort);

  if (threadIdx.x == 0) {          // the last block to finish closes the call
    uint32_t* ticket = reinterpret_cast<uint32_t*>(p.state + 1);
    if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
      *ticket = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint64_t*>(p.state) = call;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Same all-reduce over plain peer memory (no multicast): two-shot, every transfer a PULL (16-byte loads from the
// peers' buffers over NVLink, many in flight per thread), the result written to a private tensor y.
//   barrier A | own slice: y = S_own = sum over ranks (rank order, fp32) of S_r | fence, barrier B |
//   other slices q: y = S_q (the owner's sum) | barrier C (nobody reads this rank's buffer any more)
// Block b works on share b of every slice, so block-to-block barriers are enough.  Per GPU (tp-1)/tp of a message
// arrives in each of the two phases.  Same bits on every rank: each slice is summed once, by its owner.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ld_peer_16(const void* p) {
  uint4 v;
  // A weak load is enough: nothing in this launch has read these lines before (L1 holds no stale copy; it is
  // invalidated between launches), and the data is complete before the barrier that precedes the load.
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
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

template <int TP>
__global__ void __launch_bounds__(kMcThreads) row_reduce_pull_kernel(const McReduceParams p) {
  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = 0;
  __syncthreads();
  const uint64_t call = *reinterpret_cast<volatile uint64_t*>(p.state) + 1ull;
  const uint32_t tag = static_cast<uint32_t>(call % 0xFFFFFFFFull) + 1u;

  mc_barrier(p, 0, tag, kSiteMcBarrierA, &s_abort);

  const int64_t per_rank = (p.n16 + TP - 1) / TP;
  const int64_t first = static_cast<int64_t>(blockIdx.x) * kMcThreads + threadIdx.x;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kMcThreads;
  uint4* own = reinterpret_cast<uint4*>(p.buf[p.rank]);
  if (!s_abort) {
    const int64_t lo = min(per_rank * p.rank, p.n16), hi = min(lo + per_rank, p.n16);
    constexpr int kElems = 8 / TP;                                              // 8 loads in flight per thread
    for (int64_t i = lo + first; i < hi; i += stride * kElems) {
      uint4 v[kElems][TP];
#pragma unroll
      for (int e = 0; e < kElems; ++e)
#pragma unroll
        for (int r = 0; r < TP; ++r)
          if (i + e * stride < hi) v[e][r] = ld_peer_16(p.buf[r] + (i + e * stride) * 16);
#pragma unroll
      for (int e = 0; e < kElems; ++e) {
        if (i + e * stride >= hi) break;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < TP; ++r) acc_bf16x8(acc, v[e][r]);                  // rank order
        const uint4 o = make_uint4(pack2(acc[0], acc[1]), pack2(acc[2], acc[3]), pack2(acc[4], acc[5]), pack2(acc[6], acc[7]));
        own[i + e * stride] = o;
        p.y[i + e * stride] = o;
      }
    }
  }
  __threadfence_system();
  __syncthreads();

  mc_barrier(p, 1, tag, kSiteMcBarrierB, &s_abort);

  if (!s_abort) {
    constexpr int kUnroll = 8;
#pragma unroll 1
    for (int d = 1; d < TP; ++d) {
      const int q = (p.rank + d) % TP;                                          // every rank starts with another owner
      const int64_t lo = min(per_rank * q, p.n16), hi = min(lo + per_rank, p.n16);
      const uint8_t* src = p.buf[q];
      for (int64_t i = lo + first; i < hi; i += stride * kUnroll) {
        uint4 v[kUnroll];
#pragma unroll
        for (int j = 0; j < kUnroll; ++j)
          if (i + j * stride < hi) v[j] = ld_peer_16(src + (i + j * stride) * 16);
#pragma unroll
        for (int j = 0; j < kUnroll; ++j)
          if (i + j * stride < hi) p.y[i + j * stride] = v[j];
      }
    }
  }
  __syncthreads();

  mc_barrier(p, 2, tag, kSiteMcBarrierC, &s_abort);

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
  p.mc = nullptr;
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
  if (tp == 2) row_reduce_pull_kernel<2><<<grid, kMcThreads, 0, s>>>(p);
  else if (tp == 4) row_reduce_pull_kernel<4><<<grid, kMcThreads, 0, s>>>(p);
  else row_reduce_pull_kernel<8><<<grid, kMcThreads, 0, s>>>(p);
  count_launch();
  return check_cuda(cudaGetLastError());
}

extern "C" int nq_row_reduce_mc(void* mc_ptr, int64_t count, void* const* pads, int rank, int tp, void* state,
                                int blocks, void* stream) {
  if (count < 0 || tp < 2 || tp > kMcMaxRanks || rank < 0 || rank >= tp) return NQ_ERR_BAD_ARGUMENT;
  if (count == 0) return NQ_OK;
  if (!mc_ptr || !pads || !state) return NQ_ERR_BAD_ARGUMENT;
  if (count % 8 != 0 || reinterpret_cast<uintptr_t>(mc_ptr) % 16) return NQ_ERR_BAD_ARGUMENT;
  if (blocks < 1 || blocks > kMcMaxBlocks) return NQ_ERR_BAD_ARGUMENT;
  DeviceCtx* ctx = nullptr;
  const int st = ensure_init(&ctx);
  if (st != NQ_OK) return st;
  McReduceParams p;
  p.mc = static_cast<uint8_t*>(mc_ptr);
  p.y = nullptr;
  for (int r = 0; r < kMcMaxRanks; ++r) p.buf[r] = nullptr;
  p.n16 = count / 8;
  for (int r = 0; r < kMcMaxRanks; ++r) {
    p.pad[r] = r < tp ? static_cast<uint32_t*>(pads[r]) : nullptr;
    if (r < tp && p.pad[r] == nullptr) return NQ_ERR_BAD_ARGUMENT;
  }
  p.rank = rank;
  p.tp = tp;
  p.state = static_cast<uint64_t*>(state);
  p.status = ctx->status_dev;
  p.limit_ns = wait_limit_ns();
  row_reduce_mc_kernel<<<static_cast<unsigned>(blocks), kMcThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  count_launch();
  return check_cuda(cudaGetLastError());
}
