// Quantisers of the FP8 linear path (HBM-bound streaming kernels).
//
//   act_quant_kernel     bf16 [M,K] -> e4m3 [M,K] + fp32 scale per (token, 128-wide K-group)
//   weight_quant_kernel  bf16 [N,K] -> e4m3 [N,K] + fp32 scale per 128x128 block
//
// Rule (both): scale = max(amax, 1e-10) / 448 with an IEEE fp32 divide,
// q = RNE_e4m3(float(v) / scale) with an IEEE fp32 divide, so the bytes equal a
// plain fp32 CPU evaluation of the same formulas.
#include "nq_internal.cuh"

namespace nq {

// ------------------------------------------------------------------------- //
// Activation quantiser.  One 8-lane sub-warp per (token, group); each lane owns
// 16 consecutive elements: two 128-bit loads, one 128-bit store.  A warp covers
// four consecutive groups = 1 KiB of contiguous input when the groups share a row.
// amax over the sub-warp by three xor-shuffles.
// VEC=false is the ragged/unaligned variant (element-wise guarded accesses).
// ------------------------------------------------------------------------- //
template <bool VEC>
__global__ void __launch_bounds__(256) act_quant_kernel(const __nv_bfloat16* __restrict__ x, int64_t M, int64_t K,
                                                        int64_t ldx, uint8_t* __restrict__ xq, int64_t ld_xq,
                                                        float* __restrict__ sx, int64_t ld_sx) {
  // Let the GEMM that follows start at once: its set-up and its first weight tiles do not depend on this kernel (it
  // waits for this grid's completion itself, with griddepcontrol.wait, before it touches xq / sx).
  pdl_launch_next();
  pdl_wait_prior();
  const int64_t G = (K + 127) >> 7;
  const int64_t items = M * G;
  const int sub = threadIdx.x >> 3;   // 0..31 sub-warp within the block
  const int l8 = threadIdx.x & 7;     // lane within the sub-warp
  // Grid-stride loop; the aligned variant requests the next item's 32 bytes before it converts the current one.
  const int64_t stride = static_cast<int64_t>(gridDim.x) * 32;
  int64_t item = static_cast<int64_t>(blockIdx.x) * 32 + sub;
  uint4 na = make_uint4(0u, 0u, 0u, 0u), nb = na;
  if (VEC && item < items) {
    const int64_t m = item / G, g = item - m * G;
    const uint4* src = reinterpret_cast<const uint4*>(x + m * ldx + (g << 7) + (l8 << 4));
    na = __ldg(src);
    nb = __ldg(src + 1);
  }
  for (; item < items; item += stride) {
    const int64_t m = item / G;
    const int64_t g = item - m * G;
    const int64_t k0 = (g << 7) + (l8 << 4);
    // the 16 elements as 8 words of two bf16 each (element 2i in the low half of word i)
    uint32_t w[8];
    if (VEC) {
      w[0] = na.x; w[1] = na.y; w[2] = na.z; w[3] = na.w; w[4] = nb.x; w[5] = nb.y; w[6] = nb.z; w[7] = nb.w;
      const int64_t nxt = item + stride;
      if (nxt < items) {
        const int64_t m1 = nxt / G, g1 = nxt - m1 * G;
        const uint4* src = reinterpret_cast<const uint4*>(x + m1 * ldx + (g1 << 7) + (l8 << 4));
        na = __ldg(src);
        nb = __ldg(src + 1);
      }
    } else {
      const unsigned short* src = reinterpret_cast<const unsigned short*>(x + m * ldx);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t lo = (k0 + 2 * i < K) ? src[k0 + 2 * i] : 0u;
        const uint32_t hi = (k0 + 2 * i + 1 < K) ? src[k0 + 2 * i + 1] : 0u;
        w[i] = lo | (hi << 16);
      }
    }
    // amax on the packed pairs (a maximum of bf16 values is exact), then across the pair and the sub-warp
    uint32_t m2 = bf16x2_absmax(w[0], w[1]);
#pragma unroll
    for (int i = 2; i < 8; i += 2) m2 = bf16x2_absmax(m2, bf16x2_absmax(w[i], w[i + 1]));
    float amax = fmaxf(bf16_bits_to_float(m2 & 0xFFFFu), bf16_bits_to_float(m2 >> 16));
    // sub-warps of one warp may leave the loop at different items: mask = own 8 lanes
    const uint32_t mask8 = 0xFFu << (threadIdx.x & 24);
    amax = fmaxf(amax, __shfl_xor_sync(mask8, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(mask8, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(mask8, amax, 4));
    const float scale = __fdiv_rn(fmaxf(amax, 1e-10f), 448.0f);
    if (l8 == 0) sx[g * ld_sx + m] = scale;
    const ExactDivider div(scale);
    uint32_t qw[4];
    if (!div.slow) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 a = div.fast2(make_float2(__uint_as_float(w[2 * i] << 16), __uint_as_float(w[2 * i] & 0xFFFF0000u)));
        const float2 b = div.fast2(make_float2(__uint_as_float(w[2 * i + 1] << 16), __uint_as_float(w[2 * i + 1] & 0xFFFF0000u)));
        qw[i] = pack4_e4m3(a.x, a.y, b.x, b.y);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        qw[i] = pack4_e4m3(__fdiv_rn(__uint_as_float(w[2 * i] << 16), scale), __fdiv_rn(__uint_as_float(w[2 * i] & 0xFFFF0000u), scale),
                           __fdiv_rn(__uint_as_float(w[2 * i + 1] << 16), scale), __fdiv_rn(__uint_as_float(w[2 * i + 1] & 0xFFFF0000u), scale));
      }
    }
    const uint4 q = make_uint4(qw[0], qw[1], qw[2], qw[3]);
    if (VEC) {
      *reinterpret_cast<uint4*>(xq + m * ld_xq + k0) = q;
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if (k0 + i < K) xq[m * ld_xq + k0 + i] = static_cast<uint8_t>(qw[i >> 2] >> ((i & 3) * 8));
    }
  }
}

// ------------------------------------------------------------------------- //
// Weight quantiser.  One CTA of 256 threads per 128x128 block; thread t owns
// row t/2, 64 consecutive elements (columns (t&1)*64 ...).  Offline work.
// ------------------------------------------------------------------------- //
__global__ void __launch_bounds__(256) weight_quant_kernel(const __nv_bfloat16* __restrict__ w, int64_t N, int64_t K,
                                                           int64_t ldw, uint8_t* __restrict__ wq, int64_t ld_wq,
                                                           float* __restrict__ sw, int64_t ld_sw, int vec) {
  __shared__ float warp_max[8];
  const int64_t bk = blockIdx.x, bn = blockIdx.y;
  const int64_t n = bn * 128 + (threadIdx.x >> 1);
  const int64_t k0 = bk * 128 + (threadIdx.x & 1) * 64;
  float amax = 0.0f;
  const bool row_ok = n < N;
  if (row_ok) {
    if (vec) {
      const uint4* src = reinterpret_cast<const uint4*>(w + n * ldw + k0);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint4 a = __ldg(src + i);
        const uint32_t u[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          amax = fmaxf(amax, fabsf(bf16_bits_to_float(u[j] & 0xFFFFu)));
          amax = fmaxf(amax, fabsf(bf16_bits_to_float(u[j] >> 16)));
        }
      }
    } else {
      const unsigned short* src = reinterpret_cast<const unsigned short*>(w + n * ldw);
      for (int i = 0; i < 64; ++i)
        if (k0 + i < K) amax = fmaxf(amax, fabsf(bf16_bits_to_float(src[k0 + i])));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = warp_max[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, warp_max[i]);
  const float scale = __fdiv_rn(fmaxf(amax, 1e-10f), 448.0f);
  if (threadIdx.x == 0) sw[bn * ld_sw + bk] = scale;
  if (!row_ok) return;
  const unsigned short* src = reinterpret_cast<const unsigned short*>(w + n * ldw);
  uint8_t* dst = wq + n * ld_wq;
  if (vec) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float v[16];
      const uint4 a = __ldg(reinterpret_cast<const uint4*>(src + k0) + 2 * i);
      const uint4 b = __ldg(reinterpret_cast<const uint4*>(src + k0) + 2 * i + 1);
      const uint32_t u[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[2 * j] = __fdiv_rn(bf16_bits_to_float(u[j] & 0xFFFFu), scale);
        v[2 * j + 1] = __fdiv_rn(bf16_bits_to_float(u[j] >> 16), scale);
      }
      uint4 q;
      q.x = pack4_e4m3(v[0], v[1], v[2], v[3]);
      q.y = pack4_e4m3(v[4], v[5], v[6], v[7]);
      q.z = pack4_e4m3(v[8], v[9], v[10], v[11]);
      q.w = pack4_e4m3(v[12], v[13], v[14], v[15]);
      *reinterpret_cast<uint4*>(dst + k0 + 16 * i) = q;
    }
  } else {
    for (int i = 0; i < 64; ++i) {
      if (k0 + i < K) {
        const float q = __fdiv_rn(bf16_bits_to_float(src[k0 + i]), scale);
        dst[k0 + i] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3));
      }
    }
  }
}

// ------------------------------- launchers -------------------------------- //
int launch_act_quant(const void* x, int64_t M, int64_t K, int64_t ldx, void* xq, int64_t ld_xq, float* sx,
                     int64_t ld_sx, cudaStream_t stream, bool pdl) {
  const int64_t G = (K + 127) / 128;
  const int64_t items = M * G;
  if (items == 0) return NQ_OK;
  const bool vec = (K % 128 == 0) && (ldx % 8 == 0) && (ld_xq % 16 == 0) &&
                   (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (reinterpret_cast<uintptr_t>(xq) % 16 == 0);
  int64_t blocks = (items + 31) / 32;
  DeviceCtx* ctx = nullptr;
  const int st = ensure_init(&ctx);
  if (st != NQ_OK) return st;
  // grid-stride loop over at most 32 CTAs per SM (several waves smooth the tail; measured equal from 10 to 64)
  const int64_t cap = static_cast<int64_t>(ctx->sm_count) * 32;
  if (blocks > cap) blocks = cap;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(blocks));
  cfg.blockDim = dim3(256);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  auto* xp = static_cast<const __nv_bfloat16*>(x);
  auto* qp = static_cast<uint8_t*>(xq);
  cudaError_t e = vec ? cudaLaunchKernelEx(&cfg, act_quant_kernel<true>, xp, M, K, ldx, qp, ld_xq, sx, ld_sx)
                      : cudaLaunchKernelEx(&cfg, act_quant_kernel<false>, xp, M, K, ldx, qp, ld_xq, sx, ld_sx);
  count_launch();
  return check_cuda(e);
}

int launch_weight_quant(const void* w, int64_t N, int64_t K, int64_t ldw, void* wq, int64_t ld_wq, float* sw,
                        int64_t ld_sw, cudaStream_t stream) {
  if (N == 0 || K == 0) return NQ_OK;
  const int vec = (K % 128 == 0) && (ldw % 8 == 0) && (ld_wq % 16 == 0) &&
                  (reinterpret_cast<uintptr_t>(w) % 16 == 0) && (reinterpret_cast<uintptr_t>(wq) % 16 == 0);
  dim3 grid(static_cast<unsigned>((K + 127) / 128), static_cast<unsigned>((N + 127) / 128));
  weight_quant_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(w), N, K, ldw,
                                                static_cast<uint8_t*>(wq), ld_wq, sw, ld_sw, vec);
  count_launch();
  return check_cuda(cudaGetLastError());
}

}  // namespace nq
