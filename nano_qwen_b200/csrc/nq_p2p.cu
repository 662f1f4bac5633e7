// nq_row_reduce_p2p: the SUM all-reduce that ends a row-parallel linear, for decode-sized outputs, done by one
// kernel per rank over peer memory (plain NVLink stores and local loads; no multicast, no TMA).
//
// Stands in for `dist.all_reduce(y)` of RowParallelLinear.forward (nano_qwen, src/nano_qwen/layers/linear.py:154-155)
// when the output is small enough that the collective is bound by latency, not bandwidth.
//
// One-shot push protocol with the flag inside the data (no fence, no second trip over the link).  Every rank owns an
// inbox of 2 parities x tp senders x (2 x slot_bytes), reachable by all peers.  The calls are counted by a 64-bit
// number n kept in device memory (so that a CUDA graph replays correctly); call n works on parity n & 1 and tags
// its words with e = n mod (2^32 - 1) + 1, which is never 0, the value of a word that was never written:
//   1. each thread turns 16 bytes of this rank's partial into four 8-byte words {4 bytes of data, e} and stores
//      them into slot [e & 1][rank] of every peer's inbox (8-byte stores are atomic: a word is either old or new),
//   2. then polls (bounded) the same positions of its own inbox until every word carries e, and adds the tp
//      contributions in rank order (its own from local memory) in fp32 and writes bf16: every rank gets the same bits.
// A slot written for call e is written again for call e + 2, which a sender can reach only after it has received
// the receiver's data of call e + 1, i.e. after the receiver finished call e: two parities are enough and no barrier
// is needed at the end.  No thread waits for anything but data that a peer sends unconditionally at the start of
// its kernel, so the wait cannot dead-lock.  A wait that runs out of time sets the device status block
// (NQ_ERR_DEVICE_TIMEOUT) and the kernel finishes with whatever it has.
#include <algorithm>
#include <cstring>

#include "nq_internal.cuh"

namespace nq {
namespace {

constexpr int kMaxRanks = NQ_P2P_MAX_RANKS;
constexpr int kThreads = 256;
constexpr int kSiteRowReduce = 64;

struct RowReduceParams {
  const uint4* src;             // this rank's partial, bf16, 16-byte chunks
  uint4* dst;                   // result (may be the same buffer)
  int64_t n16;                  // 16-byte chunks in the message
  uint8_t* inbox[kMaxRanks];    // inbox base of every rank (own entry: local address)
  int rank, tp;
  int64_t slot_bytes;           // payload capacity of a slot (it occupies twice that)
  uint64_t* state;              // [0] calls completed so far (64 bits), [1] low half: block ticket of the call in flight
  DeviceStatus* status;
  uint64_t limit_ns;
};

// Peers write the inbox behind this SM's back: read it from L2, never from a stale L1 line.
__device__ __forceinline__ uint4 ld_inbox(const uint4* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_inbox(uint4* p, const uint4& v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
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
  __shared__ int s_abort;
  const int b = blockIdx.x, tid = threadIdx.x;
  if (tid == 0) s_abort = 0;
  // Programmatic dependent launch: the kernel behind this one may start its set-up now; this one waits for the GEMM
  // that produces `src` before it reads anything.
  pdl_launch_next();
  pdl_wait_prior();
  __syncthreads();
  const uint64_t call = *reinterpret_cast<volatile uint64_t*>(p.state) + 1ull;   // number of this call, 1-based
  const uint32_t e = static_cast<uint32_t>(call % 0xFFFFFFFFull) + 1u;           // tag in the words: 1 .. 2^32 - 1
  const int64_t slot2 = 2 * p.slot_bytes;
  const int64_t par_off = static_cast<int64_t>(call & 1ull) * p.tp;
  const int64_t per = (p.n16 + gridDim.x - 1) / gridDim.x;
  const int64_t lo = b * per, hi = min(lo + per, p.n16);

  // 1. push: data and call number travel in the same 8-byte words
  for (int64_t i = lo + tid; i < hi; i += kThreads) {
    const uint4 v = p.src[i];
    const uint4 w0 = make_uint4(v.x, e, v.y, e), w1 = make_uint4(v.z, e, v.w, e);
    for (int d = 1; d < p.tp; ++d) {
      const int peer = (p.rank + d) % p.tp;                  // start with a different peer on every rank
      uint4* out = reinterpret_cast<uint4*>(p.inbox[peer] + (par_off + p.rank) * slot2) + 2 * i;
      st_inbox(out, w0);
      st_inbox(out + 1, w1);
    }
  }
  // 2. collect and sum in rank order
  const uint8_t* mine = p.inbox[p.rank];
  const long long t0 = clock64();
  const long long limit_cycles = static_cast<long long>(p.limit_ns) * 2;     // ~2 GHz: a generous conversion
  for (int64_t i = lo + tid; i < hi; i += kThreads) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < p.tp; ++r) {
      uint4 v;
      if (r == p.rank) {
        v = p.src[i];
      } else {
        const uint4* in = reinterpret_cast<const uint4*>(mine + (par_off + r) * slot2) + 2 * i;
        uint4 a = ld_inbox(in), c = ld_inbox(in + 1);
        for (uint32_t spin = 1; a.y != e || a.w != e || c.y != e || c.w != e; ++spin) {
          if ((spin & 63u) == 0u) {
            if (*reinterpret_cast<volatile int*>(&s_abort)) break;
            if (clock64() - t0 > limit_cycles) {
              s_abort = 1;
              if (p.status != nullptr && atomicCAS(&p.status->code, 0, kErrDeviceTimeout) == 0) {
                p.status->where = kSiteRowReduce;
                p.status->block = b;
                p.status->aux = r;
                __threadfence_system();
              }
              break;
            }
          }
          a = ld_inbox(in);
          c = ld_inbox(in + 1);
        }
        v = make_uint4(a.x, a.z, c.x, c.z);                  // after a time-out: whatever is there; the status says so
      }
      add_bf16x8(acc, v);
    }
    p.dst[i] = make_uint4(pack2_bf16(acc[0], acc[1]), pack2_bf16(acc[2], acc[3]), pack2_bf16(acc[4], acc[5]),
                          pack2_bf16(acc[6], acc[7]));
  }
  // the last block to finish closes the call
  __syncthreads();
  if (tid == 0) {
    uint32_t* ticket = reinterpret_cast<uint32_t*>(p.state + 1);
    const uint32_t t = atomicAdd(ticket, 1u);
    if (t == gridDim.x - 1) {
      *ticket = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint64_t*>(p.state) = call;
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

int nq_row_reduce_p2p(const void* partial, void* y, int64_t count, void* const* inbox, int rank, int tp,
                      int64_t slot_bytes, void* state, void* stream) {
  if (count < 0 || tp < 1 || tp > kMaxRanks || rank < 0 || rank >= tp) return NQ_ERR_BAD_ARGUMENT;
  if (count == 0) return NQ_OK;
  if (!partial || !y || !inbox || !state) return NQ_ERR_BAD_ARGUMENT;
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
    if (r < tp && p.inbox[r] == nullptr) return NQ_ERR_BAD_ARGUMENT;
  }
  p.rank = rank;
  p.tp = tp;
  p.slot_bytes = slot_bytes;
  p.state = static_cast<uint64_t*>(state);
  p.status = ctx->status_dev;
  p.limit_ns = wait_limit_ns();
  // 4 KiB of the message per block and pass
  int64_t blocks = (p.n16 + kThreads - 1) / kThreads;
  const int64_t cap = 2 * ctx->sm_count;
  if (blocks > cap) blocks = cap;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(blocks));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, row_reduce_p2p_kernel, p);
  count_launch();
  return check_cuda(e);
}

}  // extern "C"
