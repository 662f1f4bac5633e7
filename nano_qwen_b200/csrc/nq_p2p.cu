// nq_row_reduce_p2p: the SUM all-reduce that ends a row-parallel linear, for decode-sized outputs, done by one
// kernel per rank over peer memory (plain NVLink stores and local loads; no multicast, no TMA).
//
// Stands in for `dist.all_reduce(y)` of RowParallelLinear.forward (nano_qwen, src/nano_qwen/layers/linear.py:154-155)
// when the output is small enough that the collective is bound by latency, not bandwidth.
//
// One-shot push protocol.  Every rank owns an inbox (2 parities x tp senders x slot_bytes) and a flag array
// (tp senders x kMaxBlocks words), both reachable by all peers.  Call number e (a counter kept in device memory,
// so that a CUDA graph replays correctly) works on parity e & 1:
//   1. block b copies its slice of this rank's partial into slot [e & 1][rank] of every peer's inbox,
//   2. fences system-wide and writes e into word [rank][b] of every peer's flag array,
//   3. waits (bounded) until its own words [r][b] hold e for every peer r,
//   4. adds the tp slices in rank order (its own from local memory, the others from its inbox) in fp32 and
//      writes bf16: every rank gets the same bits.
// A slot written for call e is written again for call e + 2, which a sender can reach only after it has seen the
// receiver's flag of call e + 1, i.e. after the receiver finished call e: two parities are enough and no barrier
// is needed at the end.  Block b depends on the blocks b of the peers only, and blocks start in index order on
// every GPU, so the wait cannot dead-lock even when not all blocks are resident.  A wait that runs out of time
// sets the device status block (NQ_ERR_DEVICE_TIMEOUT) and the kernel finishes with whatever it has.
#include <algorithm>
#include <cstring>

#include "nq_internal.cuh"

namespace nq {
namespace {

constexpr int kMaxRanks = NQ_P2P_MAX_RANKS;
constexpr int kMaxBlocks = NQ_P2P_MAX_BLOCKS;
constexpr int kThreads = 256;
constexpr int kSiteRowReduce = 64;

struct RowReduceParams {
  const uint4* src;             // this rank's partial, bf16, 16-byte chunks
  uint4* dst;                   // result (may be the same buffer)
  int64_t n16;                  // 16-byte chunks in the message
  uint8_t* inbox[kMaxRanks];    // inbox base of every rank (own entry: local address)
  uint32_t* flags[kMaxRanks];   // flag array base of every rank
  int rank, tp;
  int64_t slot_bytes;
  uint32_t* state;              // [0] calls completed so far, [1] block ticket of the call in flight
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
// Peers write the inbox behind this SM's back: read it from L2, never from a stale L1 line.
__device__ __forceinline__ uint4 ld_inbox(const uint4* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void add_bf16x8(float (&acc)[8], const uint4& v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[2 * i] += bf16_bits_to_float(w[i] & 0xFFFFu);
    acc[2 * i + 1] += bf16_bits_to_float(w[i] >> 16);
  }
}
__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

__global__ void __launch_bounds__(kThreads) row_reduce_p2p_kernel(const RowReduceParams p) {
  const int b = blockIdx.x, tid = threadIdx.x;
  const uint32_t e = *reinterpret_cast<volatile uint32_t*>(p.state) + 1u;   // number of this call, 1-based
  const int64_t par_off = static_cast<int64_t>(e & 1u) * p.tp;
  const int64_t per = (p.n16 + gridDim.x - 1) / gridDim.x;
  const int64_t lo = b * per, hi = min(lo + per, p.n16);

  // 1. push this block's slice to every peer
  for (int d = 1; d < p.tp; ++d) {
    const int peer = (p.rank + d) % p.tp;                    // start with a different peer on every rank
    uint4* out = reinterpret_cast<uint4*>(p.inbox[peer] + (par_off + p.rank) * p.slot_bytes);
    for (int64_t i = lo + tid; i < hi; i += kThreads) out[i] = p.src[i];
  }
  // 2. make the slice visible system-wide, then tell the peers
  __threadfence_system();
  __syncthreads();
  if (tid < p.tp && tid != p.rank) st_release_sys(p.flags[tid] + p.rank * kMaxBlocks + b, e);
  // 3. wait for the peers' slices of the same block
  if (tid < p.tp && tid != p.rank) {
    const uint32_t* f = p.flags[p.rank] + tid * kMaxBlocks + b;
    const long long t0 = clock64();
    const long long limit_cycles = static_cast<long long>(p.limit_ns) * 2;   // ~2 GHz: a generous conversion
    while (static_cast<int32_t>(ld_acquire_sys(f) - e) < 0) {
      if (clock64() - t0 > limit_cycles) {
        if (p.status != nullptr && atomicCAS(&p.status->code, 0, kErrDeviceTimeout) == 0) {
          p.status->where = kSiteRowReduce;
          p.status->block = b;
          p.status->aux = tid;
          __threadfence_system();
        }
        break;
      }
    }
  }
  __syncthreads();
  // 4. sum in rank order (an aborted call still writes its slice: garbage in, status says so)
  const uint8_t* mine = p.inbox[p.rank];
  for (int64_t i = lo + tid; i < hi; i += kThreads) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < p.tp; ++r) {
      const uint4 v = (r == p.rank) ? p.src[i]
                                    : ld_inbox(reinterpret_cast<const uint4*>(mine + (par_off + r) * p.slot_bytes) + i);
      add_bf16x8(acc, v);
    }
    p.dst[i] = make_uint4(pack2_bf16(acc[0], acc[1]), pack2_bf16(acc[2], acc[3]), pack2_bf16(acc[4], acc[5]),
                          pack2_bf16(acc[6], acc[7]));
  }
  // the last block to finish closes the call
  __syncthreads();
  if (tid == 0) {
    const uint32_t t = atomicAdd(p.state + 1, 1u);
    if (t == gridDim.x - 1) {
      p.state[1] = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(p.state) = e;
    }
  }
}

}  // namespace
}  // namespace nq

using namespace nq;

extern "C" {

int nq_p2p_alloc(size_t bytes, void** dev_ptr) {
  if (dev_ptr == nullptr || bytes == 0) return NQ_ERR_BAD_ARGUMENT;
  DeviceCtx* ctx = nullptr;
  const int st = ensure_init(&ctx);
  if (st != NQ_OK) return st;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return check_cuda(e);
  e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) { cudaFree(p); return check_cuda(e); }
  *dev_ptr = p;
  return NQ_OK;
}

int nq_p2p_free(void* dev_ptr) {
  if (dev_ptr == nullptr) return NQ_OK;
  return check_cuda(cudaFree(dev_ptr));
}

int nq_p2p_export(void* dev_ptr, unsigned char* handle) {
  if (dev_ptr == nullptr || handle == nullptr) return NQ_ERR_BAD_ARGUMENT;
  static_assert(sizeof(cudaIpcMemHandle_t) == NQ_P2P_HANDLE_BYTES, "handle size");
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, dev_ptr);
  if (e != cudaSuccess) return check_cuda(e);
  memcpy(handle, &h, sizeof(h));
  return NQ_OK;
}

int nq_p2p_import(const unsigned char* handle, void** dev_ptr) {
  if (dev_ptr == nullptr || handle == nullptr) return NQ_ERR_BAD_ARGUMENT;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return check_cuda(e);
  *dev_ptr = p;
  return NQ_OK;
}

int nq_p2p_release(void* dev_ptr) {
  if (dev_ptr == nullptr) return NQ_OK;
  return check_cuda(cudaIpcCloseMemHandle(dev_ptr));
}

int nq_row_reduce_p2p(const void* partial, void* y, int64_t count, void* const* inbox, void* const* flags, int rank,
                      int tp, int64_t slot_bytes, void* state, void* stream) {
  if (count < 0 || tp < 1 || tp > kMaxRanks || rank < 0 || rank >= tp) return NQ_ERR_BAD_ARGUMENT;
  if (count == 0) return NQ_OK;
  if (!partial || !y || !inbox || !flags || !state) return NQ_ERR_BAD_ARGUMENT;
  if (count % 8 != 0 || reinterpret_cast<uintptr_t>(partial) % 16 || reinterpret_cast<uintptr_t>(y) % 16)
    return NQ_ERR_BAD_ARGUMENT;
  if (slot_bytes % 16 != 0 || count * 2 > slot_bytes) return NQ_ERR_WORKSPACE;
  DeviceCtx* ctx = nullptr;
  const int st = ensure_init(&ctx);
  if (st != NQ_OK) return st;
  RowReduceParams p;
  p.src = static_cast<const uint4*>(partial);
  p.dst = static_cast<uint4*>(y);
  p.n16 = count / 8;
  for (int r = 0; r < kMaxRanks; ++r) {
    p.inbox[r] = r < tp ? static_cast<uint8_t*>(inbox[r]) : nullptr;
    p.flags[r] = r < tp ? static_cast<uint32_t*>(flags[r]) : nullptr;
    if (r < tp && (p.inbox[r] == nullptr || p.flags[r] == nullptr)) return NQ_ERR_BAD_ARGUMENT;
  }
  p.rank = rank;
  p.tp = tp;
  p.slot_bytes = slot_bytes;
  p.state = static_cast<uint32_t*>(state);
  p.status = ctx->status_dev;
  p.limit_ns = wait_limit_ns();
  // 4 KiB of the message per block and pass; never more blocks than flag words, and few enough that they are
  // all resident at once on an idle GPU
  int64_t blocks = (p.n16 + kThreads - 1) / kThreads;
  const int64_t cap = std::min<int64_t>(kMaxBlocks, 2 * ctx->sm_count);
  if (blocks > cap) blocks = cap;
  row_reduce_p2p_kernel<<<static_cast<unsigned>(blocks), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  count_launch();
  return check_cuda(cudaGetLastError());
}

}  // extern "C"
