// nq_fp8_linear_noalloc: the quantise-then-GEMM linear for callers that cannot allocate device memory.
//
// nq_fp8_linear needs two scratch buffers for the quantised activations (e4m3 bytes and fp32 group
// scales) and leaves their allocation to the caller.  Some hosts have no allocator to offer: a runtime
// that hands a plugin only the tensors it registered up front, a real-time loop with a frozen memory
// budget, code that runs while a stream is being captured (cudaMalloc is not legal there).  For them
// the scratch lives in this library's own image: a fixed-size array in device memory that exists on
// every GPU that loads the library, from load until the process exits.
#include <mutex>

#include "nq_internal.cuh"

namespace {

// 8 MiB of e4m3 activations followed by 256 KiB of fp32 group scales: enough for 64 tokens at any K of the
// Qwen3 shapes, or 512 tokens at K = 12288.  Held on each GPU for the life of the process.
constexpr size_t kXqBytes = NQ_NOALLOC_MAX_XQ_BYTES;
constexpr size_t kSxFloats = NQ_NOALLOC_MAX_SX_FLOATS;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kXqBytes + kSxFloats * sizeof(float)];

constexpr int kMaxDevices = 64;
void* g_scratch_ptr[kMaxDevices] = {};   // device address of the array above, per device
std::mutex g_scratch_mu;

// The array's name is only a host-side handle; the address a kernel can use has to be asked for, once per
// device, with that device current.
int scratch_address(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return nq::check_cuda(e);
  if (dev < 0 || dev >= kMaxDevices) return NQ_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return nq::check_cuda(e);
    if (p == nullptr) return NQ_ERR_CUDA;
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return NQ_OK;
}

}  // namespace

extern "C" int nq_fp8_linear_noalloc(const void* x, int64_t ldx, const void* wq, int64_t ld_wq, const float* sw,
                                     int64_t ld_sw, const void* bias, void* y, int64_t ldy, int64_t M, int64_t N,
                                     int64_t K, int algo, int split_k, void* stream) {
  if (M < 0 || N < 0 || K < 0) return NQ_ERR_BAD_ARGUMENT;
  if (M == 0 || N == 0) return NQ_OK;
  // sizes the GEMM would refuse anyway; checked first so that the products below cannot wrap around
  if (M > (1ll << 30) || N > (1ll << 30) || K > (1ll << 30)) return NQ_ERR_UNSUPPORTED;
  const int64_t ld_xq = (K + 15) / 16 * 16;
  const int64_t ld_sx = (M + 3) / 4 * 4;
  const int64_t groups = (K + 127) / 128;
  // refuse what does not fit instead of touching memory past the array
  if (static_cast<uint64_t>(M) * static_cast<uint64_t>(ld_xq) > kXqBytes) return NQ_ERR_WORKSPACE;
  if (static_cast<uint64_t>(groups) * static_cast<uint64_t>(ld_sx) > kSxFloats) return NQ_ERR_WORKSPACE;
  nq::DeviceCtx* ctx = nullptr;
  int st = nq::ensure_init(&ctx);
  if (st != NQ_OK) return st;
  void* base = nullptr;
  st = scratch_address(&base);
  if (st != NQ_OK) return st;
  void* xq = base;
  float* sx = reinterpret_cast<float*>(static_cast<unsigned char*>(base) + kXqBytes);
  // Same two launches as nq_fp8_linear; the quantiser rewrites every byte the GEMM reads, so nothing has to be
  // cleared between calls.
  return nq_fp8_linear(x, ldx, wq, ld_wq, sw, ld_sw, bias, y, ldy, M, N, K, xq, sx, nullptr, 0, algo, split_k, stream);
}
