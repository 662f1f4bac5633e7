// extern "C" entry points of libnq_fp8.so and the per-device set-up behind them.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "nq_internal.cuh"

namespace nq {

namespace {
constexpr int kMaxDevices = 64;
DeviceCtx g_ctx[kMaxDevices];
std::mutex g_mu;
std::atomic<int64_t> g_launches{0};
std::atomic<uint64_t> g_wait_limit_ns{2000000000ull};
std::atomic<int> g_sm_reserve{0};
thread_local char t_cuda_err[256] = "";

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
}  // namespace

int check_cuda(cudaError_t e) {
  if (e == cudaSuccess) return NQ_OK;
  snprintf(t_cuda_err, sizeof(t_cuda_err), "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
  cudaGetLastError();   // clear the sticky-less error state
  return NQ_ERR_CUDA;
}
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
uint64_t wait_limit_ns() { return g_wait_limit_ns.load(std::memory_order_relaxed); }
int sm_reserve() { return g_sm_reserve.load(std::memory_order_relaxed); }

int ensure_init(DeviceCtx** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return check_cuda(e);
  if (dev < 0 || dev >= kMaxDevices) return NQ_ERR_UNSUPPORTED;
  DeviceCtx* c = &g_ctx[dev];
  if (!c->ready.load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lock(g_mu);
    if (!c->ready.load(std::memory_order_relaxed)) {
      int major = 0;
      e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
      if (e != cudaSuccess) return check_cuda(e);
      if (major != 10) return NQ_ERR_NOT_SM100;
      e = cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, dev);
      if (e != cudaSuccess) return check_cuda(e);
      if (g_encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess) return check_cuda(e);
        if (fn == nullptr || qres != cudaDriverEntryPointSuccess) {
          snprintf(t_cuda_err, sizeof(t_cuda_err), "cuTensorMapEncodeTiled not available from the driver");
          return NQ_ERR_CUDA;
        }
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
      }
      void* host = nullptr;
      e = cudaHostAlloc(&host, sizeof(DeviceStatus), cudaHostAllocMapped | cudaHostAllocPortable);
      if (e != cudaSuccess) return check_cuda(e);
      memset(host, 0, sizeof(DeviceStatus));
      void* devp = nullptr;
      e = cudaHostGetDevicePointer(&devp, host, 0);
      if (e != cudaSuccess) return check_cuda(e);
      c->status_host = static_cast<DeviceStatus*>(host);
      c->status_dev = static_cast<DeviceStatus*>(devp);
      int st = setup_gemm_kernels();
      if (st != NQ_OK) return st;
      st = setup_sym_kernels();
      if (st != NQ_OK) return st;
      c->ready.store(true, std::memory_order_release);
    }
  }
  *out = c;
  return NQ_OK;
}

namespace {
// Tensor maps are pure functions of (base, extents, stride, box, type): the weights of a layer and the static
// buffers of a CUDA-graph runner come back with the same arguments on every call, so the driver's encoder
// (1-2 us per map) is asked once per distinct argument set.  Small direct-mapped cache, one per thread.
struct TmapKey {
  const void* base; int64_t rows, cols, ld; int box_rows, box_cols, kind;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows &&
           box_cols == o.box_cols && kind == o.kind;
  }
};
struct TmapSlot { TmapKey key; CUtensorMap map; bool valid; };
constexpr int kTmapSlots = 1024;
thread_local TmapSlot t_tmap_cache[kTmapSlots];

int cached_encode(CUtensorMap* out, const TmapKey& k) {
  uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
  h ^= static_cast<uint64_t>(k.rows) * 0xC2B2AE3D27D4EB4Full + static_cast<uint64_t>(k.cols) * 0x165667B19E3779F9ull;
  h ^= static_cast<uint64_t>(k.ld) * 0x27D4EB2F165667C5ull + static_cast<uint64_t>(k.box_rows * 4 + k.box_cols * 4096 + k.kind);
  TmapSlot& slot = t_tmap_cache[(h >> 32) % kTmapSlots];
  if (slot.valid && slot.key == k) { *out = slot.map; return NQ_OK; }
  const bool u8 = (k.kind == 0);
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k.cols), static_cast<cuuint64_t>(k.rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k.ld) * (u8 ? 1 : 2)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(k.box_cols), static_cast<cuuint32_t>(k.box_rows)};
  const cuuint32_t elem[2] = {1u, 1u};
  const CUresult r = g_encode(out, u8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                              const_cast<void*>(k.base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              u8 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                              u8 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_NONE,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(t_cuda_err, sizeof(t_cuda_err), "cuTensorMapEncodeTiled (%s) failed with CUresult %d", u8 ? "u8" : "bf16",
             static_cast<int>(r));
    return NQ_ERR_CUDA;
  }
  slot.key = k;
  slot.map = *out;
  slot.valid = true;
  return NQ_OK;
}
}  // namespace

int make_tmap_u8_2d(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
  return cached_encode(out, TmapKey{base, rows, cols, ld, box_rows, 128, 0});
}

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows,
                      int box_cols) {
  return cached_encode(out, TmapKey{base, rows, cols, ld, box_rows, box_cols, 1});
}

namespace {

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int validate_gemm(const GemmArgs& a) {
  if (a.M < 0 || a.N < 0 || a.K < 0) return NQ_ERR_BAD_ARGUMENT;
  if (a.M == 0 || a.N == 0) return NQ_OK;
  if (a.K == 0) return NQ_ERR_UNSUPPORTED;
  if (!a.xq || !a.sx || !a.wq || !a.sw || !a.y) return NQ_ERR_BAD_ARGUMENT;
  if (!aligned16(a.xq) || !aligned16(a.wq)) return NQ_ERR_BAD_ARGUMENT;
  if (a.ld_xq % 16 || a.ld_wq % 16 || a.ld_xq < a.K || a.ld_wq < a.K) return NQ_ERR_BAD_ARGUMENT;
  if (a.ld_sx < a.M || a.ld_sw < (a.K + 127) / 128 || a.ldy < a.N) return NQ_ERR_BAD_ARGUMENT;
  if (a.M > (1ll << 30) || a.N > (1ll << 30) || a.K > (1ll << 30)) return NQ_ERR_UNSUPPORTED;
  return NQ_OK;
}

int gemm_dispatch(const GemmArgs& a, int algo) {
  int st = validate_gemm(a);
  if (st != NQ_OK) return st;
  if (a.M == 0 || a.N == 0) return NQ_OK;
  DeviceCtx* ctx = nullptr;
  st = ensure_init(&ctx);
  if (st != NQ_OK) return st;
  // Measured crossover on B200 (CUDA graph, 8B layer shapes): weight rows on the lanes up to 64 tokens; at 128 tokens
  // the token-lane kernel with 128-wide tiles is ahead (71 us against 76 us for the four linears of a layer).
  // Prefill-sized launches with at least two rounds of 256 x 256 tiles go to the CTA-pair kernel: alone it runs
  // level with the single-CTA kernel (2.0-2.1 PFLOP/s), inside a long power-capped step it is 1-2 % ahead
  // (a third fewer operand bytes cross the L2 -> SM path; three interleaved runs of the 36-layer step each).
  if (algo == NQ_ALGO_AUTO) {
    algo = (a.M <= 64) ? NQ_ALGO_WEIGHT_LANE : NQ_ALGO_TOKEN_LANE;
    if (a.M >= 2048 && ((a.M + 255) / 256) * ((a.N + 255) / 256) >= ctx->sm_count) algo = NQ_ALGO_TOKEN_PAIR;
  }
  if (algo == NQ_ALGO_TOKEN_LANE) return launch_gemm_token_lane(a, ctx, 0);
  if (algo == NQ_ALGO_TOKEN_LANE_128) return launch_gemm_token_lane(a, ctx, 128);
  if (algo == NQ_ALGO_TOKEN_LANE_192) return launch_gemm_token_lane(a, ctx, 192);
  if (algo == NQ_ALGO_TOKEN_LANE_256) return launch_gemm_token_lane(a, ctx, 256);
  if (algo == NQ_ALGO_WEIGHT_LANE) return launch_gemm_weight_lane(a, ctx);
  if (algo == NQ_ALGO_TOKEN_PAIR) return launch_gemm_token_pair(a, ctx, 256);
  return NQ_ERR_BAD_ARGUMENT;
}

}  // namespace
}  // namespace nq

using namespace nq;

extern "C" {

int nq_version(void) { return 100; }

#ifndef NQ_SOURCE_HASH
#define NQ_SOURCE_HASH "unknown"
#endif
const char* nq_source_hash(void) { return NQ_SOURCE_HASH; }

const char* nq_status_string(int status) {
  switch (status) {
    case NQ_OK: return "ok";
    case NQ_ERR_BAD_ARGUMENT: return "bad argument (null pointer, negative size, misaligned pointer or stride)";
    case NQ_ERR_UNSUPPORTED: return "unsupported shape";
    case NQ_ERR_WORKSPACE: return "workspace missing or too small";
    case NQ_ERR_CUDA: return "CUDA call failed";
    case NQ_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait expired";
    case NQ_ERR_NOT_SM100: return "current device is not compute capability 10.x";
    default: return "unknown status";
  }
}

const char* nq_last_cuda_error(void) { return t_cuda_err; }

int nq_init(void) {
  DeviceCtx* ctx = nullptr;
  return ensure_init(&ctx);
}

int nq_act_quant_e4m3_g128(const void* x, int64_t M, int64_t K, int64_t ldx, void* xq, int64_t ld_xq, float* sx,
                           int64_t ld_sx, void* stream) {
  if (M < 0 || K < 0) return NQ_ERR_BAD_ARGUMENT;
  if (M == 0 || K == 0) return NQ_OK;
  if (!x || !xq || !sx || ldx < K || ld_xq < K || ld_sx < M) return NQ_ERR_BAD_ARGUMENT;
  DeviceCtx* ctx = nullptr;
  const int st = ensure_init(&ctx);
  if (st != NQ_OK) return st;
  return launch_act_quant(x, M, K, ldx, xq, ld_xq, sx, ld_sx, static_cast<cudaStream_t>(stream), true);
}

int nq_weight_quant_e4m3_b128(const void* w, int64_t N, int64_t K, int64_t ldw, void* wq, int64_t ld_wq, float* sw,
                              int64_t ld_sw, void* stream) {
  if (N < 0 || K < 0) return NQ_ERR_BAD_ARGUMENT;
  if (N == 0 || K == 0) return NQ_OK;
  if (!w || !wq || !sw || ldw < K || ld_wq < K || ld_sw < (K + 127) / 128) return NQ_ERR_BAD_ARGUMENT;
  if ((N + 127) / 128 > 65535) return NQ_ERR_UNSUPPORTED;
  DeviceCtx* ctx = nullptr;
  const int st = ensure_init(&ctx);
  if (st != NQ_OK) return st;
  return launch_weight_quant(w, N, K, ldw, wq, ld_wq, sw, ld_sw, static_cast<cudaStream_t>(stream));
}

size_t nq_fp8_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K) { return weight_lane_workspace_bytes(M, N, K); }

int nq_fp8_gemm_bs128(const void* xq, int64_t ld_xq, const float* sx, int64_t ld_sx, const void* wq, int64_t ld_wq,
                      const float* sw, int64_t ld_sw, const void* bias, void* y, int64_t ldy, int64_t M, int64_t N,
                      int64_t K, void* workspace, size_t workspace_bytes, int algo, int split_k, void* stream) {
  GemmArgs a;
  a.xq = xq; a.ld_xq = ld_xq; a.sx = sx; a.ld_sx = ld_sx;
  a.wq = wq; a.ld_wq = ld_wq; a.sw = sw; a.ld_sw = ld_sw;
  a.bias = bias; a.y = y; a.ldy = ldy; a.M = M; a.N = N; a.K = K;
  a.workspace = workspace; a.workspace_bytes = workspace_bytes;
  a.split_k = split_k;
  a.stream = static_cast<cudaStream_t>(stream);
  a.pdl = true;
  return gemm_dispatch(a, algo);
}

int nq_fp8_linear(const void* x, int64_t ldx, const void* wq, int64_t ld_wq, const float* sw, int64_t ld_sw,
                  const void* bias, void* y, int64_t ldy, int64_t M, int64_t N, int64_t K, void* xq_scratch,
                  float* sx_scratch, void* workspace, size_t workspace_bytes, int algo, int split_k, void* stream) {
  if (M < 0 || N < 0 || K < 0) return NQ_ERR_BAD_ARGUMENT;
  if (M == 0 || N == 0) return NQ_OK;
  if (M > (1ll << 30) || N > (1ll << 30) || K > (1ll << 30)) return NQ_ERR_UNSUPPORTED;   // before the quantiser runs
  const int64_t ld_xq = (K + 15) / 16 * 16;
  const int64_t ld_sx = (M + 3) / 4 * 4;
  // A handful of tokens: quantise inside the weight-lane GEMM (one launch, no xq / sx round trip) when the rows
  // of x can be read 16 bytes at a time.  Bit-identical to the two-launch path.  Every CTA of that kernel
  // converts the activations it needs itself, which beats the separate quantiser launch up to about 8 tokens
  // (measured on B200 with the four layer shapes of an 8B model); on request it runs up to 32.
  const bool fusable = M <= NQ_FUSED_MAX_TOKENS && K > 0 && K % 8 == 0 && ldx % 8 == 0 && aligned16(x);
  if (algo == NQ_ALGO_WEIGHT_LANE_FUSED && !fusable) return NQ_ERR_UNSUPPORTED;
  if (algo == NQ_ALGO_WEIGHT_LANE_FUSED || (algo == NQ_ALGO_AUTO && fusable && M <= NQ_FUSED_AUTO_TOKENS)) {
    if (!x || !wq || !sw || !y || ldx < K) return NQ_ERR_BAD_ARGUMENT;
    if (!aligned16(wq) || ld_wq % 16 || ld_wq < K || ld_sw < (K + 127) / 128 || ldy < N) return NQ_ERR_BAD_ARGUMENT;
    if (N > (1ll << 30) || K > (1ll << 30)) return NQ_ERR_UNSUPPORTED;
    {
      DeviceCtx* ctx = nullptr;
      const int st0 = ensure_init(&ctx);
      if (st0 != NQ_OK) return st0;
      GemmArgs a;
      a.x = x; a.ldx = ldx; a.xq = nullptr; a.ld_xq = 0; a.sx = nullptr; a.ld_sx = 0;
      a.wq = wq; a.ld_wq = ld_wq; a.sw = sw; a.ld_sw = ld_sw;
      a.bias = bias; a.y = y; a.ldy = ldy; a.M = M; a.N = N; a.K = K;
      a.workspace = workspace; a.workspace_bytes = workspace_bytes;
      a.split_k = split_k;
      a.stream = static_cast<cudaStream_t>(stream);
      a.pdl = true;
      return launch_gemm_weight_lane(a, ctx);
    }
  }
  int st = nq_act_quant_e4m3_g128(x, M, K, ldx, xq_scratch, ld_xq, sx_scratch, ld_sx, stream);
  if (st != NQ_OK) return st;
  return nq_fp8_gemm_bs128(xq_scratch, ld_xq, sx_scratch, ld_sx, wq, ld_wq, sw, ld_sw, bias, y, ldy, M, N, K,
                           workspace, workspace_bytes, algo, split_k, stream);
}

int nq_device_status(int* code, int* where, int* block, int* aux, int reset) {
  DeviceCtx* ctx = nullptr;
  const int st = ensure_init(&ctx);
  if (st != NQ_OK) return st;
  volatile DeviceStatus* s = ctx->status_host;
  if (code) *code = s->code;
  if (where) *where = s->where;
  if (block) *block = s->block;
  if (aux) *aux = s->aux;
  if (reset) { s->code = 0; s->where = 0; s->block = 0; s->aux = 0; }
  return NQ_OK;
}

int nq_set_wait_limit_ns(uint64_t ns) {
  if (ns == 0) return NQ_ERR_BAD_ARGUMENT;
  g_wait_limit_ns.store(ns);
  return NQ_OK;
}

int nq_set_sm_reserve(int n) {
  if (n < 0) return NQ_ERR_BAD_ARGUMENT;
  return g_sm_reserve.exchange(n);
}

int64_t nq_launch_count(void) { return g_launches.load(); }

}  // extern "C"
