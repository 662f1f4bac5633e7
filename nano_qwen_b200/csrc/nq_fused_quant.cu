// Producers of linear-layer inputs that emit FP8 directly: the activation quantiser fused into the op in front of it.
//
//   silu_mul_quant_kernel   h = silu(gate) * up      (nano_qwen, src/nano_qwen/layers/activation.py:6-11)
//                           -> e4m3 [M, I] + fp32 1x128 group scales: the input of down_proj
//   rmsnorm_quant_kernel    (x [+ residual]) -> RMS norm -> * weight  or  * (1 + weight)
//                           (src/nano_qwen/layers/layernorm.py:16-40 RMSNorm, :79-105 GemmaRMSNorm)
//                           -> e4m3 [M, H] + group scales (+ the new residual, + the bf16 result when asked for):
//                           the input of qkv_proj / gate_up_proj
//
// Both round to bf16 exactly where the reference's eager code produces a bf16 tensor, and then apply the
// rule of act_quant_kernel (scale = max(amax, 1e-10) / 448, q = RNE_e4m3(h / scale), IEEE divides), so that the
// bytes equal "reference op, then activation quantiser" whenever the fp32 intermediates agree.
// Layout: 8 lanes per 128-wide group, 16 consecutive elements per lane, like act_quant_kernel.
#include "nq_internal.cuh"

namespace nq {
namespace {

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ void unpack16(const uint4& a, const uint4& b, float (&v)[16]) {
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

// 16 bf16-valued floats of one lane -> group amax over the lane's 8-lane sub-warp -> scale -> 16 e4m3 bytes.
__device__ __forceinline__ uint4 quantise16(const float (&h)[16], uint32_t mask8, float& scale) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(h[i]));
  amax = fmaxf(amax, __shfl_xor_sync(mask8, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(mask8, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(mask8, amax, 4));
  scale = __fdiv_rn(fmaxf(amax, 1e-10f), 448.0f);
  const ExactDivider div(scale);
  uint32_t q[4];
  if (!div.slow) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 a = div.fast2(make_float2(h[4 * i], h[4 * i + 1]));
      const float2 b = div.fast2(make_float2(h[4 * i + 2], h[4 * i + 3]));
      q[i] = pack4_e4m3(a.x, a.y, b.x, b.y);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      q[i] = pack4_e4m3(__fdiv_rn(h[4 * i], scale), __fdiv_rn(h[4 * i + 1], scale), __fdiv_rn(h[4 * i + 2], scale),
                        __fdiv_rn(h[4 * i + 3], scale));
  }
  return make_uint4(q[0], q[1], q[2], q[3]);
}

__device__ __forceinline__ uint4 pack8_bf16(const float* v) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// gate_up [M, 2*I] bf16 (gate = columns [0, I), up = columns [I, 2I)), row stride ld elements.
__global__ void __launch_bounds__(256) silu_mul_quant_kernel(const __nv_bfloat16* __restrict__ gu, int64_t M, int64_t I,
                                                             int64_t ld, uint8_t* __restrict__ xq, int64_t ld_xq,
                                                             float* __restrict__ sx, int64_t ld_sx) {
  pdl_launch_next();   // the consumer GEMM sets up and prefetches weights meanwhile; it waits for this grid itself
  pdl_wait_prior();
  const int64_t G = (I + 127) >> 7;
  const int64_t items = M * G;
  const int sub = threadIdx.x >> 3, l8 = threadIdx.x & 7;
  const uint32_t mask8 = 0xFFu << (threadIdx.x & 24);
  for (int64_t item = static_cast<int64_t>(blockIdx.x) * 32 + sub; item < items;
       item += static_cast<int64_t>(gridDim.x) * 32) {
    const int64_t m = item / G, g = item - m * G;
    const int64_t k0 = (g << 7) + (l8 << 4);
    float a[16], b[16], h[16];
    if (k0 < I) {                                            // I is a multiple of 16: a lane is all in or all out
      const uint4* pg = reinterpret_cast<const uint4*>(gu + m * ld + k0);
      const uint4* pu = reinterpret_cast<const uint4*>(gu + m * ld + I + k0);
      unpack16(__ldg(pg), __ldg(pg + 1), a);
      unpack16(__ldg(pu), __ldg(pu + 1), b);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        // silu in fp32 with the hardware exponential and reciprocal: a few fp32 ulp, far below the bf16 rounding
        // that follows (F.silu returns bf16; bf16 * bf16 rounds once more)
        const float s = __fdividef(a[i], 1.0f + __expf(-a[i]));
        h[i] = bf16_round(bf16_round(s) * b[i]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) h[i] = 0.0f;
    }
    float scale;
    const uint4 q = quantise16(h, mask8, scale);
    if (l8 == 0) sx[g * ld_sx + m] = scale;
    if (k0 < I) *reinterpret_cast<uint4*>(xq + m * ld_xq + k0) = q;
  }
}

// One CTA of 256 threads per token row.  Pass 1: x (+ residual) in fp32, sum of squares.  Pass 2 reads the row again
// (from L1/L2), writes the new residual, normalises, rounds to bf16, multiplies by the weight in bf16 and quantises.
// (Keeping the row in registers between the passes was measured slower: 80 registers halve the CTAs per SM.)
__global__ void __launch_bounds__(256) rmsnorm_quant_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* res_in,
                                                            const __nv_bfloat16* __restrict__ weight, float eps, int gemma,
                                                            int64_t H, int64_t ldx, int64_t ld_res, __nv_bfloat16* res_out,
                                                            __nv_bfloat16* y_out, int64_t ldy, uint8_t* __restrict__ xq,
                                                            int64_t ld_xq, float* __restrict__ sx, int64_t ld_sx) {
  __shared__ float warp_sum[8];
  __shared__ float s_rstd;
  pdl_launch_next();   // the consumer GEMM sets up and prefetches weights meanwhile; it waits for this grid itself
  pdl_wait_prior();
  const int64_t m = blockIdx.x;
  const int64_t G = (H + 127) >> 7;
  const int sub = threadIdx.x >> 3, l8 = threadIdx.x & 7;
  const uint32_t mask8 = 0xFFu << (threadIdx.x & 24);
  const __nv_bfloat16* xr = x + m * ldx;
  const __nv_bfloat16* rr = res_in != nullptr ? res_in + m * ld_res : nullptr;

  auto load_row16 = [&](int64_t k0, float (&v)[16]) {
    const uint4* px = reinterpret_cast<const uint4*>(xr + k0);
    unpack16(__ldg(px), __ldg(px + 1), v);
    if (rr != nullptr) {
      float r[16];
      // the residual may be updated in place (res_out == res_in): plain loads, each lane reads before it writes
      const uint4* pr = reinterpret_cast<const uint4*>(rr + k0);
      unpack16(pr[0], pr[1], r);
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = v[i] + r[i];
    }
  };

  float ss = 0.0f;
  for (int64_t g = sub; g < G; g += 32) {
    const int64_t k0 = (g << 7) + (l8 << 4);
    if (k0 >= H) continue;
    float v[16];
    load_row16(k0, v);
#pragma unroll
    for (int i = 0; i < 16; ++i) ss = fmaf(v[i], v[i], ss);
  }
  // (The new residual is written in pass 2, by the lane that has just re-read the old values of the same 16
  //  elements, so updating it in place is safe.)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
  if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += warp_sum[i];
    const float var = __fdiv_rn(t, static_cast<float>(H));
    s_rstd = __fdiv_rn(1.0f, __fsqrt_rn(var + eps));
  }
  __syncthreads();
  const float rstd = s_rstd;

  for (int64_t g = sub; g < G; g += 32) {
    const int64_t k0 = (g << 7) + (l8 << 4);
    const bool in = k0 < H;                                  // H is a multiple of 16
    float h[16];
    if (in) {
      float v[16], w[16];
      load_row16(k0, v);
      if (res_out != nullptr) {
        uint4* po = reinterpret_cast<uint4*>(res_out + m * ld_res + k0);
        po[0] = pack8_bf16(v);
        po[1] = pack8_bf16(v + 8);
      }
      const uint4* pw = reinterpret_cast<const uint4*>(weight + k0);
      unpack16(__ldg(pw), __ldg(pw + 1), w);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float n = bf16_round(v[i] * rstd);             // x.to(orig_dtype)
        const float wm = gemma ? bf16_round(1.0f + w[i]) : w[i];
        h[i] = bf16_round(n * wm);                           // bf16 tensor * bf16 tensor
      }
      if (y_out != nullptr) {
        uint4* py = reinterpret_cast<uint4*>(y_out + m * ldy + k0);
        py[0] = pack8_bf16(h);
        py[1] = pack8_bf16(h + 8);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) h[i] = 0.0f;
    }
    float scale;
    const uint4 q = quantise16(h, mask8, scale);
    if (l8 == 0 && (g << 7) < H) sx[g * ld_sx + m] = scale;
    if (in) *reinterpret_cast<uint4*>(xq + m * ld_xq + k0) = q;
  }
}

bool aligned16p(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace
}  // namespace nq

using namespace nq;

extern "C" {

int nq_silu_mul_quant_e4m3_g128(const void* gate_up, int64_t M, int64_t I, int64_t ld, void* xq, int64_t ld_xq,
                                float* sx, int64_t ld_sx, void* stream) {
  if (M < 0 || I < 0) return NQ_ERR_BAD_ARGUMENT;
  if (M == 0 || I == 0) return NQ_OK;
  if (!gate_up || !xq || !sx || ld < 2 * I || ld_xq < I || ld_sx < M) return NQ_ERR_BAD_ARGUMENT;
  if (I % 16 || ld % 8 || ld_xq % 16 || !aligned16p(gate_up) || !aligned16p(xq)) return NQ_ERR_UNSUPPORTED;
  DeviceCtx* ctx = nullptr;
  const int st = ensure_init(&ctx);
  if (st != NQ_OK) return st;
  const int64_t items = M * ((I + 127) / 128);
  int64_t blocks = (items + 31) / 32;
  const int64_t cap = static_cast<int64_t>(ctx->sm_count) * 16;
  if (blocks > cap) blocks = cap;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(blocks));
  cfg.blockDim = dim3(256);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, silu_mul_quant_kernel, static_cast<const __nv_bfloat16*>(gate_up), M, I,
                                           ld, static_cast<uint8_t*>(xq), ld_xq, sx, ld_sx);
  count_launch();
  return check_cuda(e);
}

int nq_rmsnorm_quant_e4m3_g128(const void* x, const void* residual_in, const void* weight, float eps, int gemma,
                               int64_t M, int64_t H, int64_t ldx, int64_t ld_res, void* residual_out, void* y_out,
                               int64_t ldy, void* xq, int64_t ld_xq, float* sx, int64_t ld_sx, void* stream) {
  if (M < 0 || H < 0) return NQ_ERR_BAD_ARGUMENT;
  if (M == 0 || H == 0) return NQ_OK;
  if (!x || !weight || !xq || !sx || ldx < H || ld_xq < H || ld_sx < M) return NQ_ERR_BAD_ARGUMENT;
  if ((residual_in || residual_out) && ld_res < H) return NQ_ERR_BAD_ARGUMENT;
  if (residual_out && !residual_in) return NQ_ERR_BAD_ARGUMENT;
  if (y_out && ldy < H) return NQ_ERR_BAD_ARGUMENT;
  if (H % 16 || ldx % 8 || ld_xq % 16 || !aligned16p(x) || !aligned16p(xq) || !aligned16p(weight))
    return NQ_ERR_UNSUPPORTED;
  if ((residual_in && (!aligned16p(residual_in) || ld_res % 8)) || (residual_out && !aligned16p(residual_out)) ||
      (y_out && (!aligned16p(y_out) || ldy % 8)))
    return NQ_ERR_UNSUPPORTED;
  if (M > 2147483647ll) return NQ_ERR_UNSUPPORTED;
  DeviceCtx* ctx = nullptr;
  const int st = ensure_init(&ctx);
  if (st != NQ_OK) return st;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(M));
  cfg.blockDim = dim3(256);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(
      &cfg, rmsnorm_quant_kernel, static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual_in),
      static_cast<const __nv_bfloat16*>(weight), eps, gemma, H, ldx, ld_res, static_cast<__nv_bfloat16*>(residual_out),
      static_cast<__nv_bfloat16*>(y_out), ldy, static_cast<uint8_t*>(xq), ld_xq, sx, ld_sx);
  count_launch();
  return check_cuda(e);
}

}  // extern "C"
