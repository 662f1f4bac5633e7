// Declarations shared by the translation units of libnq_fp8.so.
#pragma once
#include "../../include/nq_fp8.h"
#include "nq_ptx.cuh"
#include <atomic>

namespace nq {

// Per-device state created by ensure_init().
struct DeviceCtx {
  std::atomic<bool> ready{false};   // set last, with release order; read with acquire before the other fields
  int sm_count = 0;
  DeviceStatus* status_host = nullptr;  // mapped pinned host memory
  DeviceStatus* status_dev = nullptr;   // device alias of the same block
};

int ensure_init(DeviceCtx** out);             // NQ_* status; *out valid on NQ_OK
int check_cuda(cudaError_t e);                // records the message, returns NQ_OK / NQ_ERR_CUDA
void count_launch();
uint64_t wait_limit_ns();
int sm_reserve();

// 2-D row-major uint8 tensor [rows, cols] with row stride `ld` bytes, tiled
// into boxes of [box_rows, 128] bytes, 128-byte swizzle, zero fill out of range.
int make_tmap_u8_2d(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows);
// 2-D row-major bf16 tensor [rows, cols] with row stride `ld` elements, boxes of [box_rows, box_cols], no swizzle (stores).
int make_tmap_bf16_2d(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows, int box_cols);

int launch_act_quant(const void* x, int64_t M, int64_t K, int64_t ldx, void* xq, int64_t ld_xq, float* sx,
                     int64_t ld_sx, cudaStream_t stream, bool pdl);
int launch_weight_quant(const void* w, int64_t N, int64_t K, int64_t ldw, void* wq, int64_t ld_wq, float* sw,
                        int64_t ld_sw, cudaStream_t stream);

struct GemmArgs {
  const void* x = nullptr; int64_t ldx = 0;   // unquantised bf16 activations: set only for the fused decode path
  const void* xq; int64_t ld_xq;
  const float* sx; int64_t ld_sx;
  const void* wq; int64_t ld_wq;
  const float* sw; int64_t ld_sw;
  const void* bias;
  void* y; int64_t ldy;
  int64_t M, N, K;
  void* workspace; size_t workspace_bytes;
  int split_k;
  cudaStream_t stream;
  bool pdl;
};
int launch_gemm_token_lane(const GemmArgs& a, DeviceCtx* ctx, int tile_n);   // tile_n: 0 = choose, else 128/192/256
int launch_gemm_weight_lane(const GemmArgs& a, DeviceCtx* ctx);
int launch_gemm_token_pair(const GemmArgs& a, DeviceCtx* ctx, int tile_n);   // 256 x tile_n tiles on CTA pairs (cta_group::2)
size_t weight_lane_workspace_bytes(int64_t M, int64_t N, int64_t K);
int weight_lane_pick_split(int64_t M, int64_t N, int64_t K, int sm_count);
int setup_gemm_kernels();   // cudaFuncSetAttribute for the large dynamic shared memory
int setup_sym_kernels();    // the same for the peer-memory reduction

}  // namespace nq
