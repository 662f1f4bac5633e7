// Block-scaled FP8 GEMM kernels for sm_100a.
//
//   y[m,n] = bf16( sum_t sx[t,m] * sw[n/128,t] * ( xq[m, tile t] . wq[n, tile t] ) + bias[n] )
//
// Both kernels share one structure: a TMA producer warp fills a ring of
// shared-memory stages (one 128-byte-swizzled K-tile of each operand per
// stage), one thread issues tcgen05.mma (kind::f8f6f4, e4m3 x e4m3 -> fp32)
// into a ring of TMEM accumulators, ONE K-TILE PER ACCUMULATOR, and the
// epilogue warps drain each accumulator with tcgen05.ld, multiply by the fp32
// scale product of that K-tile and add into fp32 registers ("promotion").  The
// fp32 scales cannot ride inside the MMA, hence one drain per 128-wide K-tile;
// the TMEM ring lets the drain of tile t overlap the MMAs of tile t+1.
//
//   token_lane_kernel   tokens on the 128 TMEM lanes, BN weight rows on the
//                       columns; persistent over output tiles.  One scale per
//                       thread and K-tile.  For prefill-sized M (tensor bound).
//   weight_lane_kernel  swap-AB: 128 weight rows on the lanes, the (few) tokens
//                       on the columns; split-K over a thread-block cluster,
//                       partial sums exchanged through distributed shared
//                       memory and summed in a fixed order (deterministic, no
//                       global scratch).  For decode-sized M (HBM bound).
//
// No TMA multicast anywhere (these kernels also run in multi-GPU jobs).
#include <cstdlib>
#include "nq_internal.cuh"
#include <type_traits>


namespace nq {

namespace {

constexpr int kTileK = 128;          // bytes == elements per K-tile row; one swizzle atom
constexpr int kLaneTileBytes = 128 * kTileK;
constexpr int kXchStride = 260;      // floats per row of a token-lane partial tile in shared memory (256 + pad)

// wait-site ids reported in DeviceStatus::where
enum : int {
  kSiteProdEmpty = 1, kSiteMmaFull = 2, kSiteMmaTmemEmpty = 3, kSiteEpiTmemFull = 4, kSiteTeardown = 5, kSiteScaleEmpty = 6,
  kSiteWeightLane = 16  // added to the above for the weight-lane kernel
};

struct __align__(8) PipeBars {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[8];
  uint64_t tmem_empty[8];
  uint64_t teardown;
  uint64_t teardown2;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint8_t* align_1024(uint8_t* p) {
  return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~static_cast<uintptr_t>(1023));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ float bf16_to_float(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// After an abort: give copies and MMAs still in flight a bounded time to land
// before shared memory and TMEM are released.
__device__ __noinline__ void drain_after_abort(PipeBars* bars, int stages, uint32_t issued) {
  const uint64_t t0 = globaltimer_ns();
  const uint32_t first = issued > static_cast<uint32_t>(stages) ? issued - stages : 0;
  for (uint32_t i = first; i < issued; ++i) {
    const int s = i % stages;
    const uint32_t ph = (i / stages) & 1;
    while (!mbar_try_wait(&bars->full[s], ph)) {
      if (globaltimer_ns() - t0 > 20000000ull) return;   // 20 ms in total
    }
  }
}

}  // namespace

// =========================================================================== //
//                            token-lane kernel                                //
// =========================================================================== //
template <int BN>
struct TokenLane {
  // BN = 192 is the balanced shape: 64 accumulator columns per epilogue thread leave room
  // for 64 staging registers, so a whole accumulator is drained in one burst and handed
  // back to the tensor core before any FMA is issued.  BN = 256 moves fewer operand bytes
  // per flop but needs 128 accumulator registers per thread (drain in two halves).
  static constexpr int kCols = (BN == 256) ? 128 : 64;        // accumulator columns per epilogue thread
  static constexpr int kEpiGroups = BN / kCols;                // column groups: 2 (BN 128/256) or 3 (BN 192)
  static constexpr int kEpiWarps = 4 * kEpiGroups;
  static constexpr int kFirstEpiWarp = 4;           // warps 0..3: producer, MMA issuer, scale loader, idle
  static constexpr int kThreads = 32 * (kFirstEpiWarp + kEpiWarps);
  static constexpr int kAccStride = (BN == 128) ? 128 : 256;   // TMEM columns between accumulators
  static constexpr int kNumAcc = 512 / kAccStride;             // accumulator ring: 4 x 128 or 2 x 192/256 columns
  static constexpr int kTmemCols = 512;
  static constexpr int kStageBytes = kLaneTileBytes + BN * kTileK;
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 192) ? 5 : 6;
  static constexpr int kScaleBytes = kNumAcc * kEpiGroups * 128 * 4;   // scale product per accumulator, column group, row
  // Output staging for TMA stores: per epilogue warp two buffers of 32 rows x 16 bf16 columns (BN 192 has
  // no shared memory left for them and stores from registers).
  static constexpr bool kTmaStore = (BN != 192);
  static constexpr int kStoreBytes = kTmaStore ? kEpiWarps * 2048 : 0;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kScaleBytes + kStoreBytes + 1024;
  static constexpr int kGroupM = 16;                // M-tiles per rasterisation group
  static constexpr int kScalePrefetch = 4;          // K-tiles of scale factors in flight in the loader warp
  // register split between the first warpgroup and the epilogue warpgroups (setmaxnreg)
  // (a warpgroup that asks for more registers than the CTA's pool holds would wait for ever: the sum over the
  //  warpgroups must not exceed what the kernel is launched with - checked here against the launch-bounds figure
  //  and again on the host, against the compiled kernel, before the first launch)
  static constexpr int kRegsLow = (kThreads == 512) ? 56 : 64;
  static constexpr int kRegsHigh = (kThreads == 512) ? 152 : 216;
  static constexpr int kRegsNeeded = kRegsLow + (kThreads / 128 - 1) * kRegsHigh;
  static_assert(kRegsNeeded <= (65536 / kThreads / 8 * 8) * (kThreads / 128), "setmaxnreg split exceeds the register pool");
};

struct TokenLaneParams {
  const float* sx; int64_t ld_sx;
  const float* sw; int64_t ld_sw;
  const __nv_bfloat16* bias;
  __nv_bfloat16* y; int64_t ldy;
  int M, N, K;
  int splits;                 // K split over a cluster (1, splits, 1); > 1 means one tile per CTA
  int y_vec;                  // 1: 16-byte stores are legal for y
  int y_tma;                  // 1: the output tensor map is valid (y 16-byte aligned, row stride a multiple of 16 bytes)
  int sx_vec;                 // 1: 16-byte loads of sx rows are legal
  uint32_t wait_mode;         // 0 try_wait, 1 test_wait spin, >1 try_wait with that suspend hint (ns)
  DeviceStatus* status;
  uint64_t wait_limit_ns;
};

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t local_smem_addr, uint32_t cta_rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(cta_rank));
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(remote)
               : "memory");
  return v;
}

template <int BN>
__device__ __forceinline__ void token_lane_tile_coords(int tile, int num_m, int num_n, int& m_t, int& n_t) {
  constexpr int G = TokenLane<BN>::kGroupM;
  const int per_group = G * num_n;
  const int group = tile / per_group;
  const int first_m = group * G;
  const int gsize = min(num_m - first_m, G);
  const int r = tile - group * per_group;
  m_t = first_m + r % gsize;
  n_t = r / gsize;
}

// acc[0..32) += r[0..32) * s with packed two-wide FMAs (half the issue slots of scalar FMAs).
__device__ __forceinline__ void promote32(float* acc, const uint32_t (&r)[32], float s) {
  const float2 s2 = make_float2(s, s);
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    const float2 v = __ffma2_rn(make_float2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), s2,
                                make_float2(acc[i], acc[i + 1]));
    acc[i] = v.x;
    acc[i + 1] = v.y;
  }
}

// Position of the scale loader in the (tile, K-tile) iteration space of one CTA.
struct ScaleCursor {
  int tile, kt, m0, n0;
};

template <int BN>
__global__ void __launch_bounds__(TokenLane<BN>::kThreads, 1)
token_lane_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                  const __grid_constant__ CUtensorMap tm_y, const TokenLaneParams p) {
  using C = TokenLane<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align_1024(smem_raw);
  float* scale_ring = reinterpret_cast<float*>(smem + C::kStages * C::kStageBytes);   // [kNumAcc][groups][128]
  uint8_t* store_ring = smem + C::kStages * C::kStageBytes + C::kScaleBytes;            // [epilogue warp][2][32 rows x 32 B]
  PipeBars* bars = reinterpret_cast<PipeBars*>(smem + C::kStages * C::kStageBytes + C::kScaleBytes + C::kStoreBytes);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) { mbar_init(&bars->full[s], 1); mbar_init(&bars->empty[s], 1); }
    for (int b = 0; b < C::kNumAcc; ++b) {
      mbar_init(&bars->tmem_full[b], 2);            // UMMA commit + scale loader
      mbar_init(&bars->tmem_empty[b], C::kEpiWarps);
    }
    mbar_init(&bars->teardown, 1);
    mbar_init(&bars->teardown2, 1);
    bars->abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_w);
    if (p.y_tma) tma_prefetch_desc(&tm_y);
  }
  if (warp == 1) { tmem_alloc(&bars->tmem_base, C::kTmemCols); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  const AbortCtl ac{&bars->abort_flag, p.status, p.wait_limit_ns, p.wait_mode};

  pdl_launch_next();
  pdl_wait_prior();   // xq / sx come from the preceding quantiser launch

  const int num_m = (p.M + 127) / 128;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int KT_all = (p.K + kTileK - 1) / kTileK;
  // K split: CTA z of a cluster owns K-tiles [kt0, kt1) of its tile; unsplit launches own all of them.
  const int z = (p.splits > 1) ? static_cast<int>(blockIdx.y) : 0;
  const int kt0 = static_cast<int>((static_cast<int64_t>(z) * KT_all) / p.splits);
  const int kt1 = static_cast<int>((static_cast<int64_t>(z + 1) * KT_all) / p.splits);

  // The epilogue holds BN/2 fp32 accumulators per thread: move registers from
  // the first warpgroup to the two epilogue warpgroups.
  if (warp < C::kFirstEpiWarp) {
   setmaxnreg_dec<C::kRegsLow>();
   if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        int m_t, n_t;
        token_lane_tile_coords<BN>(tile, num_m, num_n, m_t, n_t);
        for (int kt = kt0; kt < kt1; ++kt, ++it) {
          const int s = it % C::kStages;
          const uint32_t ph = (it / C::kStages) & 1;
          if (!mbar_wait(&bars->empty[s], ph ^ 1, ac, kSiteProdEmpty, kt)) { ok = false; break; }
          uint8_t* a = smem + s * C::kStageBytes;
          mbar_arrive_expect_tx(&bars->full[s], C::kStageBytes);
          tma_load_2d(a, &tm_x, &bars->full[s], kt * kTileK, m_t * 128);
          tma_load_2d(a + kLaneTileBytes, &tm_w, &bars->full[s], kt * kTileK, n_t * BN);
        }
      }
      if (!ok) drain_after_abort(bars, C::kStages, it);
    }
   } else if (warp == 1 || warp == 3) {
    // ------------------------------ MMA issuers -------------------------------
    // Two issuing threads, one for the even and one for the odd K-tiles of this CTA's sequence.  A thread
    // spends several hundred cycles per K-tile on things that are not UMMA issue (two barrier waits, two
    // commits); with a single issuer the tensor pipe sat idle for that time after every K-tile.  With two,
    // one thread's waits overlap the other's UMMAs.  Consecutive K-tiles use different accumulators and
    // different stages, so the two instruction streams are independent.
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_e4m3_f32(128, BN);
      const uint32_t mine = (warp == 1) ? 0u : 1u;
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        for (int kt = kt0; kt < kt1; ++kt, ++it) {
          if ((it & 1u) != mine) continue;
          const int b = it % C::kNumAcc;
          const uint32_t aph = (it / C::kNumAcc) & 1;
          const int s = it % C::kStages;
          const uint32_t ph = (it / C::kStages) & 1;
          const uint32_t a_addr = smem_u32(smem + s * C::kStageBytes);
          const uint64_t a_desc = umma_smem_desc_sw128(a_addr);
          const uint64_t b_desc = umma_smem_desc_sw128(a_addr + kLaneTileBytes);
          const uint32_t d = tmem_base + b * C::kAccStride;
          if (!mbar_wait(&bars->tmem_empty[b], aph ^ 1, ac, kSiteMmaTmemEmpty, kt)) { ok = false; break; }
          if (!mbar_wait(&bars->full[s], ph, ac, kSiteMmaFull, kt)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll
          for (int k = 0; k < kTileK / 32; ++k)   // 32 bytes of K per UMMA: +2 in the (addr >> 4) field
            umma_f8(d, a_desc + 2 * k, b_desc + 2 * k, idesc, k > 0 ? 1u : 0u);
          umma_commit(&bars->empty[s]);
          umma_commit(&bars->tmem_full[b]);
        }
      }
      if (!ok) {   // let MMAs already issued finish before TMEM is freed
        uint64_t* td = (warp == 1) ? &bars->teardown : &bars->teardown2;
        umma_commit(td);
        const long long t0 = clock64();
        while (!mbar_try_wait(td, 0) && clock64() - t0 < 40000000ll) {}
      }
    }
   } else if (warp == 2) {
    // ------------------------------ scale loader ------------------------------
    // Keeps the per-row scale products of the next K-tiles ready in shared memory so
    // that the epilogue threads never wait on a global load between two drains:
    //   ring[b][h][row] = sx[kt, m0+row] * sw[block of column half h, kt]
    // The ring slot is the accumulator slot; this warp is the second arrival on the
    // accumulator's "full" barrier.
    {
      const int nblk = (p.N + 127) >> 7;
      auto place = [&](ScaleCursor& c) {
        int m_t, n_t;
        token_lane_tile_coords<BN>(c.tile, num_m, num_n, m_t, n_t);
        c.m0 = m_t * 128;
        c.n0 = n_t * BN;
      };
      auto advance = [&](ScaleCursor& c) {
        if (++c.kt == kt1) {
          c.kt = kt0;
          c.tile += gridDim.x;
          if (c.tile < num_tiles) place(c);
        }
      };
      auto fetch = [&](const ScaleCursor& c, float4& v, float (&w)[C::kEpiGroups]) {
        const int m = c.m0 + 4 * lane;
        const float* src = p.sx + static_cast<int64_t>(c.kt) * p.ld_sx + m;
        if (p.sx_vec && m + 3 < p.M) {
          v = __ldg(reinterpret_cast<const float4*>(src));
        } else {
          v.x = (m < p.M) ? __ldg(src) : 0.f;
          v.y = (m + 1 < p.M) ? __ldg(src + 1) : 0.f;
          v.z = (m + 2 < p.M) ? __ldg(src + 2) : 0.f;
          v.w = (m + 3 < p.M) ? __ldg(src + 3) : 0.f;
        }
#pragma unroll
        for (int g = 0; g < C::kEpiGroups; ++g) {
          const int nb = (c.n0 + g * C::kCols) >> 7;      // a column group never straddles a 128-block
          w[g] = (nb < nblk) ? __ldg(p.sw + static_cast<int64_t>(nb) * p.ld_sw + c.kt) : 0.f;
        }
      };
      constexpr int P = C::kScalePrefetch;
      float4 v[P];
      float w[P][C::kEpiGroups];
      ScaleCursor pf{static_cast<int>(blockIdx.x), kt0, 0, 0}, cs = pf;
      if (pf.tile < num_tiles) place(pf);
#pragma unroll
      for (int j = 0; j < P; ++j) {
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int g = 0; g < C::kEpiGroups; ++g) w[j][g] = 0.f;
        if (pf.tile < num_tiles) { fetch(pf, v[j], w[j]); advance(pf); }
      }
      uint32_t it = 0;
      bool ok = true;
      while (ok && cs.tile < num_tiles) {
#pragma unroll
        for (int j = 0; j < P; ++j) {
          if (cs.tile >= num_tiles) break;
          const int b = it % C::kNumAcc;
          const uint32_t aph = (it / C::kNumAcc) & 1;
          if (!mbar_wait(&bars->tmem_empty[b], aph ^ 1, ac, kSiteScaleEmpty, cs.kt)) { ok = false; break; }
          float4* dst = reinterpret_cast<float4*>(scale_ring + b * (C::kEpiGroups * 128)) + lane;
#pragma unroll
          for (int g = 0; g < C::kEpiGroups; ++g)
            dst[32 * g] = make_float4(v[j].x * w[j][g], v[j].y * w[j][g], v[j].z * w[j][g], v[j].w * w[j][g]);
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->tmem_full[b]);
          advance(cs);
          ++it;
          if (pf.tile < num_tiles) { fetch(pf, v[j], w[j]); advance(pf); }
        }
      }
    }
   }
  } else {
    setmaxnreg_inc<C::kRegsHigh>();
    // ------------------------------ epilogue ----------------------------------
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int h = (warp - C::kFirstEpiWarp) >> 2;   // which column group of the tile
    const int row = q * 32 + lane;
    float acc[C::kCols];
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      int m_t, n_t;
      token_lane_tile_coords<BN>(tile, num_m, num_n, m_t, n_t);
      const int m = m_t * 128 + row;
      const int n_base = n_t * BN + h * C::kCols;
#pragma unroll
      for (int i = 0; i < C::kCols; ++i) acc[i] = 0.0f;
      for (int kt = kt0; kt < kt1; ++kt, ++it) {
        const int b = it % C::kNumAcc;
        const uint32_t aph = (it / C::kNumAcc) & 1;
        if (!mbar_wait(&bars->tmem_full[b], aph, ac, kSiteEpiTmemFull, kt)) { ok = false; break; }
        tc_fence_after_sync();
        const float s = scale_ring[(b * C::kEpiGroups + h) * 128 + row];
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + b * C::kAccStride + h * C::kCols;
        uint32_t ra[32], rb[32];
        // Two TMEM loads in flight; the accumulator is handed back as soon as the
        // last load has landed, the remaining FMAs run while the next UMMAs execute.
        tmem_ld_32x32(taddr, ra);
        tmem_ld_32x32(taddr + 32, rb);
        tmem_ld_wait_on(ra);
        tmem_ld_wait_on(rb);
        if constexpr (C::kCols == 128) {
          promote32(acc, ra, s);
          tmem_ld_32x32(taddr + 64, ra);
          promote32(acc + 32, rb, s);
          tmem_ld_32x32(taddr + 96, rb);
          tmem_ld_wait_on(ra);
          tmem_ld_wait_on(rb);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->tmem_empty[b]);
        promote32(acc + C::kCols - 64, ra, s);
        promote32(acc + C::kCols - 32, rb, s);
      }
      if (!ok) break;
      if (p.splits > 1) {
        // K-split launch: the partial tile goes to shared memory (the drained pipeline stages) for the
        // cluster-wide sum below.  Row stride 260 floats keeps 16-byte stores of a quarter-warp apart.
        float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(smem) + row * kXchStride + h * C::kCols);
#pragma unroll
        for (int j = 0; j < C::kCols / 4; ++j) dst[j] = make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
        break;
      }
      // ---- write the tile: this thread owns row m, kCols consecutive columns ----
      if (C::kTmaStore && p.y_tma) {
        // Through shared memory and TMA: the warp packs 32 rows x 16 columns into one of its two staging
        // buffers and one lane issues a bulk tensor store (rows / columns past the edge are clipped by the
        // hardware), so the warp is back at the next tile's accumulators while the stores drain.
        uint8_t* stg = store_ring + (warp - C::kFirstEpiWarp) * 2048;
#pragma unroll
        for (int j = 0; j < C::kCols; j += 16) {
          const int n = n_base + j;
          if (n >= p.N) break;                                  // warp-uniform
          uint8_t* buf = stg + ((j >> 4) & 1) * 1024;
          if (lane == 0) tma_store_wait_read<1>();              // the store that last read this buffer is done with it
          __syncwarp();
          float v[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = acc[j + i];
          if (p.bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (n + i < p.N) v[i] += bf16_to_float(p.bias + n + i);
          }
          uint4 o0, o1;
          o0.x = pack_bf16x2(v[0], v[1]);   o0.y = pack_bf16x2(v[2], v[3]);
          o0.z = pack_bf16x2(v[4], v[5]);   o0.w = pack_bf16x2(v[6], v[7]);
          o1.x = pack_bf16x2(v[8], v[9]);   o1.y = pack_bf16x2(v[10], v[11]);
          o1.z = pack_bf16x2(v[12], v[13]); o1.w = pack_bf16x2(v[14], v[15]);
          uint4* dst = reinterpret_cast<uint4*>(buf + lane * 32);
          dst[0] = o0;
          dst[1] = o1;
          fence_proxy_async_smem();                             // make the generic-proxy writes visible to the TMA engine
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tm_y, buf, n, m_t * 128 + q * 32);
            tma_store_commit();
          }
        }
      } else if (m < p.M) {
        __nv_bfloat16* yrow = p.y + static_cast<int64_t>(m) * p.ldy;
#pragma unroll
        for (int j = 0; j < C::kCols; j += 8) {
          const int n = n_base + j;
          if (n >= p.N) break;
          float v[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = acc[j + i];
          if (p.bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (n + i < p.N) v[i] += bf16_to_float(p.bias + n + i);
          }
          if (p.y_vec && n + 8 <= p.N) {
            uint4 o;
            o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
            o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
            *reinterpret_cast<uint4*>(yrow + n) = o;
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (n + i < p.N) yrow[n + i] = __float2bfloat16_rn(v[i]);
          }
        }
      }
    }
    // shared memory must stay valid until the last bulk stores have read it (and y must be complete)
    if (C::kTmaStore && p.y_tma && lane == 0) tma_store_wait_all<0>();
  }

  if (p.splits > 1) {
    // ---- K-split launches: sum the partial tiles of the cluster in rank order (deterministic) ----
    __syncthreads();
    cluster_sync_all();                                  // every split's partial tile is in its shared memory
    if (warp >= C::kFirstEpiWarp && bars->abort_flag == 0) {
      int m_t, n_t;
      token_lane_tile_coords<BN>(blockIdx.x, num_m, num_n, m_t, n_t);
      const int ew = warp - C::kFirstEpiWarp;
      constexpr int kLanesPerRow = BN / 8;               // each lane owns 8 consecutive columns
      const int sub = lane / kLanesPerRow;               // BN 128: two rows per warp pass; BN 192: lanes >= 24 idle
      const int cl = lane % kLanesPerRow;
      constexpr int kRowsPerPass = (32 / kLanesPerRow) > 0 ? (32 / kLanesPerRow) : 1;
      for (int r = z + p.splits * (ew * kRowsPerPass + sub); r < 128; r += p.splits * C::kEpiWarps * kRowsPerPass) {
        const int m = m_t * 128 + r;
        if (sub >= kRowsPerPass || m >= p.M) continue;
        const uint32_t local = smem_u32(reinterpret_cast<float*>(smem) + r * kXchStride + cl * 8);
        float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int c = 0; c < p.splits; ++c) {             // summed in rank order
          const float4 a0 = ld_dsmem_f4(local, static_cast<uint32_t>(c));
          const float4 a1 = ld_dsmem_f4(local + 16, static_cast<uint32_t>(c));
          v[0] += a0.x; v[1] += a0.y; v[2] += a0.z; v[3] += a0.w;
          v[4] += a1.x; v[5] += a1.y; v[6] += a1.z; v[7] += a1.w;
        }
        const int n = n_t * BN + cl * 8;
        if (n >= p.N) continue;
        if (p.bias != nullptr) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (n + i < p.N) v[i] += bf16_to_float(p.bias + n + i);
        }
        __nv_bfloat16* yrow = p.y + static_cast<int64_t>(m) * p.ldy;
        if (p.y_vec && n + 8 <= p.N) {
          uint4 o;
          o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
          o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
          *reinterpret_cast<uint4*>(yrow + n) = o;
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (n + i < p.N) yrow[n + i] = __float2bfloat16_rn(v[i]);
        }
      }
    }
    cluster_sync_all();                                  // nobody leaves while a peer may still read its shared memory
  }

  // ------------------------------ teardown ------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// =========================================================================== //
//                        token-lane kernel, CTA pairs                          //
// =========================================================================== //
// Same computation as token_lane_kernel<256>, but two CTAs of a cluster share one 256 x BN output tile:
// each owns 128 token rows (its own A tile and TMEM accumulators) and loads only HALF of the weight
// rows of a K-tile; one tcgen05.mma.cta_group::2 (issued by the leader CTA) multiplies 256 x BN x 32 on
// both SMs, reading the other half of B from the peer's shared memory.  Operand traffic per SM drops from
// 48 KB to 32 KB per K-tile (BN = 256) - the L2 -> SM path, not the tensor pipe, is what bounds the
// single-CTA kernel - and the ring holds 6 stages.  Everything else is the single-CTA kernel's design: two
// issuing threads (in the leader) taking alternate K-tiles, a scale-loader warp per CTA, eight epilogue
// warps per CTA with the 64 / 216 register split and TMA stores from shared memory.
// No multicast is used anywhere: both CTAs issue plain TMA loads whose completion bytes are counted on the
// leader's barrier, UMMA completion is signalled to each CTA's barriers by separate commits, and the
// follower's epilogue warps hand accumulators back with remote mbarrier arrivals (plain arrivals: an arrival with
// cluster-scope release semantics measured twice as slow for the whole kernel, 1000 against 2000 TFLOP/s).
template <int BN>
struct TokenPair {
  static constexpr int kHalfRows = BN / 2;                      // weight rows of a K-tile that one CTA loads
  static constexpr int kStageBytes = kLaneTileBytes + kHalfRows * kTileK;   // A: 128 tokens, B: half of the BN rows
  static constexpr int kStages = (BN == 256) ? 6 : 8;
  static constexpr int kEpiWarps = 8;
  static constexpr int kFirstEpiWarp = 4;
  static constexpr int kThreads = 32 * (kFirstEpiWarp + kEpiWarps);
  static constexpr int kCols = BN / 2;                          // accumulator columns per epilogue thread
  static constexpr int kNumAcc = 512 / BN;                      // 2 x 256 or 4 x 128 TMEM columns
  static constexpr int kTmemCols = 512;
  static constexpr int kScaleBytes = kNumAcc * 2 * 128 * 4;
  static constexpr int kStoreBytes = kEpiWarps * 2048;          // per epilogue warp two 32 x 16 bf16 staging tiles
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kScaleBytes + kStoreBytes + 1024;
  static constexpr int kGroupM = 8;                             // pair-tiles (256 rows) per rasterisation group
  static constexpr int kScalePrefetch = 4;
  static constexpr int kRegsLow = 64;
  static constexpr int kRegsHigh = 216;
  static constexpr int kRegsNeeded = kRegsLow + (kThreads / 128 - 1) * kRegsHigh;
  static_assert(kRegsNeeded <= (65536 / kThreads / 8 * 8) * (kThreads / 128), "setmaxnreg split exceeds the register pool");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

struct __align__(8) PairBars {
  uint64_t full[8];          // used in the leader: both CTAs' loads of a stage have landed
  uint64_t empty[8];         // per CTA: the UMMAs that read the stage are complete
  uint64_t tmem_full[4];     // per CTA: UMMAs of the K-tile complete + local scale loader
  uint64_t tmem_empty[4];    // used in the leader: all 16 epilogue warps of the pair have drained
  uint64_t slot_free[4];     // per CTA: the 8 local epilogue warps have read scale slot and accumulator
  uint64_t teardown;
  uint64_t teardown2;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void pair_tile_coords(int tile, int num_m2, int num_n, int& m2, int& n_t) {
  constexpr int G = 8;
  const int per_group = G * num_n;
  const int group = tile / per_group;
  const int first_m = group * G;
  const int gsize = min(num_m2 - first_m, G);
  const int r = tile - group * per_group;
  m2 = first_m + r % gsize;
  n_t = r / gsize;
}

template <int BN>
__global__ void __launch_bounds__(TokenPair<BN>::kThreads, 1)
token_pair_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                  const __grid_constant__ CUtensorMap tm_y, const TokenLaneParams p) {
  using C = TokenPair<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align_1024(smem_raw);
  float* scale_ring = reinterpret_cast<float*>(smem + C::kStages * C::kStageBytes);   // [kNumAcc][2][128]
  uint8_t* store_ring = smem + C::kStages * C::kStageBytes + C::kScaleBytes;            // [epilogue warp][2][32 rows x 32 B]
  PairBars* bars = reinterpret_cast<PairBars*>(smem + C::kStages * C::kStageBytes + C::kScaleBytes + C::kStoreBytes);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();              // 0 = leader (issues the UMMAs)
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) { mbar_init(&bars->full[s], 1); mbar_init(&bars->empty[s], 1); }
    for (int b = 0; b < C::kNumAcc; ++b) {
      mbar_init(&bars->tmem_full[b], 2);                // pair-wide UMMA commit + local scale loader
      mbar_init(&bars->tmem_empty[b], 2 * C::kEpiWarps);
      mbar_init(&bars->slot_free[b], C::kEpiWarps);
    }
    mbar_init(&bars->teardown, 1);
    mbar_init(&bars->teardown2, 1);
    bars->abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_w);
    if (p.y_tma) tma_prefetch_desc(&tm_y);
  }
  if (warp == 1) { tmem_alloc_pair(&bars->tmem_base, C::kTmemCols); tmem_relinquish_pair(); }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                                   // both CTAs' barriers and TMEM exist before anything crosses
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  const AbortCtl ac{&bars->abort_flag, p.status, p.wait_limit_ns, p.wait_mode};

  pdl_launch_next();
  pdl_wait_prior();

  const int num_m2 = (p.M + 255) / 256;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m2 * num_n;
  const int KT = (p.K + kTileK - 1) / kTileK;

  if (warp < C::kFirstEpiWarp) {
   setmaxnreg_dec<C::kRegsLow>();
   if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
        int m2, n_t;
        pair_tile_coords(tile, num_m2, num_n, m2, n_t);
        const int m_row = m2 * 256 + static_cast<int>(rank) * 128;
        const int n_row = n_t * BN + static_cast<int>(rank) * C::kHalfRows;
        for (int kt = 0; kt < KT; ++kt, ++it) {
          const int s = it % C::kStages;
          const uint32_t ph = (it / C::kStages) & 1;
          if (!mbar_wait(&bars->empty[s], ph ^ 1, ac, kSiteProdEmpty, kt)) { ok = false; break; }
          uint8_t* a = smem + s * C::kStageBytes;
          const uint32_t full_leader = mapa_shared(smem_u32(&bars->full[s]), 0);
          if (rank == 0) mbar_arrive_expect_tx(&bars->full[s], 2 * C::kStageBytes);   // both CTAs' bytes
          tma_load_2d_pair(a, &tm_x, full_leader, kt * kTileK, m_row);
          tma_load_2d_pair(a + kLaneTileBytes, &tm_w, full_leader, kt * kTileK, n_row);
        }
      }
    }
   } else if (warp == 1 || warp == 3) {
    // ------------------------------ MMA issuers (leader only) ------------------------------
    // Two issuing threads take alternate K-tiles (different stages, different accumulators), so that the barrier
    // waits and commits of one overlap the UMMAs of the other.
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_idesc_e4m3_f32(256, BN);
      const uint32_t mine = (warp == 1) ? 0u : 1u;
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
        for (int kt = 0; kt < KT; ++kt, ++it) {
          if ((it & 1u) != mine) continue;
          const int b = it % C::kNumAcc;
          const uint32_t aph = (it / C::kNumAcc) & 1;
          const int s = it % C::kStages;
          const uint32_t ph = (it / C::kStages) & 1;
          const uint32_t a_addr = smem_u32(smem + s * C::kStageBytes);
          const uint64_t a_desc = umma_smem_desc_sw128(a_addr);
          const uint64_t b_desc = umma_smem_desc_sw128(a_addr + kLaneTileBytes);
          const uint32_t d = tmem_base + b * BN;
          if (!mbar_wait(&bars->tmem_empty[b], aph ^ 1, ac, kSiteMmaTmemEmpty, kt)) { ok = false; break; }
          if (!mbar_wait(&bars->full[s], ph, ac, kSiteMmaFull, kt)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll
          for (int k = 0; k < kTileK / 32; ++k)
            umma_f8_pair(d, a_desc + 2 * k, b_desc + 2 * k, idesc, k > 0 ? 1u : 0u);
          // completion goes to this stage's "empty" and this accumulator's "full" barrier of BOTH CTAs
          umma_commit_pair(smem_u32(&bars->tmem_full[b]));
          umma_commit_pair(mapa_shared(smem_u32(&bars->tmem_full[b]), 1));
          umma_commit_pair(smem_u32(&bars->empty[s]));
          umma_commit_pair(mapa_shared(smem_u32(&bars->empty[s]), 1));
        }
      }
      if (!ok) {   // let MMAs already issued finish before TMEM is freed
        uint64_t* td = (warp == 1) ? &bars->teardown : &bars->teardown2;
        umma_commit_pair(smem_u32(td));
        const long long t0 = clock64();
        while (!mbar_try_wait(td, 0) && clock64() - t0 < 40000000ll) {}
      }
    }
   } else if (warp == 2) {
    // ------------------------------ scale loader (both CTAs) ------------------------------
    const int nblk = (p.N + 127) >> 7;
    auto place = [&](ScaleCursor& c) {
      int m2, n_t;
      pair_tile_coords(c.tile, num_m2, num_n, m2, n_t);
      c.m0 = m2 * 256 + static_cast<int>(rank) * 128;
      c.n0 = n_t * BN;
    };
    auto advance = [&](ScaleCursor& c) {
      if (++c.kt == KT) {
        c.kt = 0;
        c.tile += num_pairs;
        if (c.tile < num_tiles) place(c);
      }
    };
    auto fetch = [&](const ScaleCursor& c, float4& v, float (&w)[2]) {
      const int m = c.m0 + 4 * lane;
      const float* src = p.sx + static_cast<int64_t>(c.kt) * p.ld_sx + m;
      if (p.sx_vec && m + 3 < p.M) {
        v = __ldg(reinterpret_cast<const float4*>(src));
      } else {
        v.x = (m < p.M) ? __ldg(src) : 0.f;
        v.y = (m + 1 < p.M) ? __ldg(src + 1) : 0.f;
        v.z = (m + 2 < p.M) ? __ldg(src + 2) : 0.f;
        v.w = (m + 3 < p.M) ? __ldg(src + 3) : 0.f;
      }
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        const int nb = (c.n0 + g * C::kCols) >> 7;
        w[g] = (nb < nblk) ? __ldg(p.sw + static_cast<int64_t>(nb) * p.ld_sw + c.kt) : 0.f;
      }
    };
    constexpr int P = C::kScalePrefetch;
    float4 v[P];
    float w[P][2];
    ScaleCursor pf{pair, 0, 0, 0}, cs = pf;
    if (pf.tile < num_tiles) place(pf);
#pragma unroll
    for (int j = 0; j < P; ++j) {
      v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      w[j][0] = 0.f; w[j][1] = 0.f;
      if (pf.tile < num_tiles) { fetch(pf, v[j], w[j]); advance(pf); }
    }
    uint32_t it = 0;
    bool ok = true;
    while (ok && cs.tile < num_tiles) {
#pragma unroll
      for (int j = 0; j < P; ++j) {
        if (cs.tile >= num_tiles) break;
        const int b = it % C::kNumAcc;
        const uint32_t aph = (it / C::kNumAcc) & 1;
        if (!mbar_wait(&bars->slot_free[b], aph ^ 1, ac, kSiteScaleEmpty, cs.kt)) { ok = false; break; }
        float4* dst = reinterpret_cast<float4*>(scale_ring + b * 256) + lane;
#pragma unroll
        for (int g = 0; g < 2; ++g)
          dst[32 * g] = make_float4(v[j].x * w[j][g], v[j].y * w[j][g], v[j].z * w[j][g], v[j].w * w[j][g]);
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->tmem_full[b]);
        advance(cs);
        ++it;
        if (pf.tile < num_tiles) { fetch(pf, v[j], w[j]); advance(pf); }
      }
    }
   }
  } else {
    setmaxnreg_inc<C::kRegsHigh>();
    // ------------------------------ epilogue (both CTAs) ------------------------------
    const int q = warp & 3;
    const int h = (warp - C::kFirstEpiWarp) >> 2;
    const int row = q * 32 + lane;
    const uint32_t leader_tmem_empty0 = mapa_shared(smem_u32(&bars->tmem_empty[0]), 0);
    float acc[C::kCols];
    uint32_t it = 0;
    bool ok = true;
    for (int tile = pair; ok && tile < num_tiles; tile += num_pairs) {
      int m2, n_t;
      pair_tile_coords(tile, num_m2, num_n, m2, n_t);
      const int m0 = m2 * 256 + static_cast<int>(rank) * 128;
      const int m = m0 + row;
      const int n_base = n_t * BN + h * C::kCols;
#pragma unroll
      for (int i = 0; i < C::kCols; ++i) acc[i] = 0.0f;
      for (int kt = 0; kt < KT; ++kt, ++it) {
        const int b = it % C::kNumAcc;
        const uint32_t aph = (it / C::kNumAcc) & 1;
        if (!mbar_wait(&bars->tmem_full[b], aph, ac, kSiteEpiTmemFull, kt)) { ok = false; break; }
        tc_fence_after_sync();
        const float s = scale_ring[(b * 2 + h) * 128 + row];
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + b * BN + h * C::kCols;
        uint32_t ra[32], rb[32];
        tmem_ld_32x32(taddr, ra);
        tmem_ld_32x32(taddr + 32, rb);
        tmem_ld_wait_on(ra);
        tmem_ld_wait_on(rb);
        if constexpr (C::kCols == 128) {
          promote32(acc, ra, s);
          tmem_ld_32x32(taddr + 64, ra);
          promote32(acc + 32, rb, s);
          tmem_ld_32x32(taddr + 96, rb);
          tmem_ld_wait_on(ra);
          tmem_ld_wait_on(rb);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive_remote(leader_tmem_empty0 + b * 8);                              // the leader's UMMA issuers
          mbar_arrive(&bars->slot_free[b]);                                            // local scale loader
        }
        promote32(acc + C::kCols - 64, ra, s);
        promote32(acc + C::kCols - 32, rb, s);
      }
      if (!ok) break;
      if (p.y_tma) {
        // through shared memory and TMA, as in the single-CTA kernel
        uint8_t* stg = store_ring + (warp - C::kFirstEpiWarp) * 2048;
#pragma unroll
        for (int j = 0; j < C::kCols; j += 16) {
          const int n = n_base + j;
          if (n >= p.N) break;                                  // warp-uniform
          uint8_t* buf = stg + ((j >> 4) & 1) * 1024;
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
          float v[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = acc[j + i];
          if (p.bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (n + i < p.N) v[i] += bf16_to_float(p.bias + n + i);
          }
          uint4 o0, o1;
          o0.x = pack_bf16x2(v[0], v[1]);   o0.y = pack_bf16x2(v[2], v[3]);
          o0.z = pack_bf16x2(v[4], v[5]);   o0.w = pack_bf16x2(v[6], v[7]);
          o1.x = pack_bf16x2(v[8], v[9]);   o1.y = pack_bf16x2(v[10], v[11]);
          o1.z = pack_bf16x2(v[12], v[13]); o1.w = pack_bf16x2(v[14], v[15]);
          uint4* dst = reinterpret_cast<uint4*>(buf + lane * 32);
          dst[0] = o0;
          dst[1] = o1;
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tm_y, buf, n, m0 + q * 32);
            tma_store_commit();
          }
        }
      } else if (m < p.M) {
        __nv_bfloat16* yrow = p.y + static_cast<int64_t>(m) * p.ldy;
#pragma unroll
        for (int j = 0; j < C::kCols; j += 8) {
          const int n = n_base + j;
          if (n >= p.N) break;
          float v[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = acc[j + i];
          if (p.bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (n + i < p.N) v[i] += bf16_to_float(p.bias + n + i);
          }
          if (p.y_vec && n + 8 <= p.N) {
            uint4 o;
            o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
            o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
            *reinterpret_cast<uint4*>(yrow + n) = o;
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (n + i < p.N) yrow[n + i] = __float2bfloat16_rn(v[i]);
          }
        }
      }
    }
    if (p.y_tma && lane == 0) tma_store_wait_all<0>();   // shared memory stays valid until the last stores have read it
  }

  // ------------------------------ teardown ------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();          // the peer's UMMAs read this CTA's shared memory; its arrivals target this CTA's barriers
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc_pair(tmem_base, C::kTmemCols);
  }
}

// =========================================================================== //
//                            weight-lane kernel                               //
// =========================================================================== //
template <int TOK, bool FUSED = false>
struct WeightLane {
  // as many stages as two CTAs per SM allow (decode tiles); the 16-token tile spends what it saves on the
  // activation tile on a sixth stage: 96 KB of weights in flight per CTA against 80 KB with the 32-token tile
  static constexpr int kStages = (TOK == 16) ? 6 : (TOK == 32) ? 5 : (TOK == 64) ? 4 : (TOK == 128) ? 6 : 4;
  static constexpr int kStageBytes = kLaneTileBytes + TOK * kTileK;
  static constexpr int kEpiWarps = (TOK == 256) ? 8 : 4;
  static constexpr int kFirstEpiWarp = 4;                 // warps 0..3: producer, MMA issuer, scale loader, second issuer / idle
  // FUSED (small decode batches, 32-token tile): the activations are quantised inside the GEMM by a third
  // warpgroup straight into the shared-memory operand tiles; no quantiser launch, no xq / sx round trip.  Every
  // CTA converts the activations of its own K-range again, so the work grows with tokens x weight tiles and
  // pays off only for a handful of tokens.  Two CTAs share an SM, so the kernel starts at 80 registers per
  // thread and the warpgroups trade them (setmaxnreg): 40 for the producer / issuer group, 96 for the
  // epilogue, 104 for the quantisers.
  static constexpr int kQuantWarps = FUSED ? 4 : 0;
  static constexpr int kFirstQuantWarp = kFirstEpiWarp + kEpiWarps;
  static constexpr int kThreads = 32 * (kFirstEpiWarp + kEpiWarps + kQuantWarps);
  static constexpr int kMinCtas = (TOK <= 64) ? 2 : 1;      // decode tiles: two CTAs per SM keep more loads in flight
  // Issuing a K-tile costs one thread about 450 cycles (each tcgen05.mma about 60, each commit about 55, measured
  // in place).  Next to the weight stream of a long K range that is nothing, but a CTA whose whole K range landed
  // before the activations arrive (short K ranges after the dependency wait) is through in half the time with two
  // issuing threads on alternate K-tiles.  Measured per decoder layer: 3-5 % faster up to 32 tokens, 1 % slower at 64.
  static constexpr int kIssuers = (TOK <= 32) ? 2 : 1;
  static constexpr bool kTradeRegs = FUSED;
  static constexpr int kRegsLow = 40;
  static constexpr int kRegsHigh = 96;
  static constexpr int kRegsQuant = 104;
  static_assert(!FUSED || TOK == 32, "the fused quantiser is built for the 32-token tile only");
  static constexpr int kRegsNeeded = kRegsLow + kRegsHigh + kRegsQuant;    // the three warpgroups of the fused kernel
  static_assert(!FUSED || kRegsNeeded <= (65536 / (kThreads * kMinCtas) / 8 * 8) * 3, "setmaxnreg split exceeds the register pool");
  static constexpr int kCols = TOK / (kEpiWarps / 4);     // accumulator columns per epilogue thread
  static constexpr int kNumAcc = (TOK == 256) ? 2 : 4;
  static constexpr int kTmemCols = (kNumAcc * TOK) < 32 ? 32 : (kNumAcc * TOK);
  static constexpr int kExchangeBytes = 128 * TOK * 4;    // fp32 partial tile, [token][weight row]
  static constexpr int kPipeBytes = kStages * kStageBytes;
  static_assert(kExchangeBytes <= kPipeBytes, "partial tile must fit in the drained pipeline stages");
  static constexpr int kScaleBytes = kNumAcc * TOK * 4;   // per accumulator: scale product per token column
  static constexpr int kSmemBytes = 1024 + kPipeBytes + kScaleBytes + 1024;
  static constexpr int kScalePrefetch = 4;
};

struct WeightLaneParams {
  const float* sx; int64_t ld_sx;
  const float* sw; int64_t ld_sw;
  const __nv_bfloat16* bias;
  __nv_bfloat16* y; int64_t ldy;
  int M, N, K;
  uint32_t wait_mode;         // 0 try_wait, 1 test_wait spin, >1 try_wait with that suspend hint (ns)
  int splits;                 // == cluster size along grid y
  int tok_box;                // token rows per TMA box of xq (what one stage receives)
  int y_vec;                  // 1: 8-byte stores are legal for y
  const __nv_bfloat16* x;     // FUSED kernels: unquantised activations [M, K], row stride ldx (16-byte aligned rows)
  int64_t ldx;
  DeviceStatus* status;
  uint64_t wait_limit_ns;
};


// acc[0..16) += r[0..16) * sc[0..16)   (sc in shared memory, read as four broadcast float4; packed two-wide FMAs)
__device__ __forceinline__ void promote16_cols(float* acc, const uint32_t* r, const float* sc) {
  const float4* s4 = reinterpret_cast<const float4*>(sc);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float4 sv = s4[j];
    const float2 lo = __ffma2_rn(make_float2(__uint_as_float(r[4 * j + 0]), __uint_as_float(r[4 * j + 1])),
                                 make_float2(sv.x, sv.y), make_float2(acc[4 * j + 0], acc[4 * j + 1]));
    const float2 hi = __ffma2_rn(make_float2(__uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])),
                                 make_float2(sv.z, sv.w), make_float2(acc[4 * j + 2], acc[4 * j + 3]));
    acc[4 * j + 0] = lo.x; acc[4 * j + 1] = lo.y;
    acc[4 * j + 2] = hi.x; acc[4 * j + 3] = hi.y;
  }
}

// Rare path of quantise_rows_e4m3: a scale whose reciprocal trick is not exact; plain IEEE divisions.
__device__ __noinline__ uint2 quantise8_e4m3_ieee(uint4 raw, float scale) {
  const uint32_t w4[4] = {raw.x, raw.y, raw.z, raw.w};
  float v[8];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    v[2 * e] = __fdiv_rn(bf16_bits_to_float(w4[e] & 0xFFFFu), scale);
    v[2 * e + 1] = __fdiv_rn(bf16_bits_to_float(w4[e] >> 16), scale);
  }
  return make_uint2(pack4_e4m3(v[0], v[1], v[2], v[3]), pack4_e4m3(v[4], v[5], v[6], v[7]));
}

// Dynamic 1x128 quantisation of NR token rows at once, 16 lanes per row (8 consecutive bf16 per lane, given as
// raw bits), both 16-lane halves of the warp busy on different rows: per row amax -> scale = max(amax, 1e-10) /
// 448 -> q = RNE_e4m3(x / scale), the arithmetic of act_quant_kernel.  The whole warp must call it together.
template <int NR>
__device__ __forceinline__ void quantise_rows_e4m3(const uint4 (&raw)[NR], uint32_t mask16, uint2 (&q)[NR],
                                                   float (&scale)[NR]) {
  float y[NR];
  bool slow = false;
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    const uint32_t m2 = bf16x2_absmax(bf16x2_absmax(raw[r].x, raw[r].y), bf16x2_absmax(raw[r].z, raw[r].w));
    float amax = fmaxf(bf16_bits_to_float(m2 & 0xFFFFu), bf16_bits_to_float(m2 >> 16));
    amax = fmaxf(amax, __shfl_xor_sync(mask16, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(mask16, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(mask16, amax, 4));
    amax = fmaxf(amax, __shfl_xor_sync(mask16, amax, 8));
    scale[r] = __fdiv_rn(fmaxf(amax, 1e-10f), 448.0f);
    const ExactDivider div(scale[r]);
    y[r] = div.y;
    slow |= div.slow;
  }
  if (__any_sync(0xFFFFFFFFu, slow)) {
#pragma unroll
    for (int r = 0; r < NR; ++r) q[r] = quantise8_e4m3_ieee(raw[r], scale[r]);
    return;
  }
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    ExactDivider div(scale[r]);
    div.y = y[r];
    const uint32_t w[4] = {raw[r].x, raw[r].y, raw[r].z, raw[r].w};
    float2 v[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
      v[e] = div.fast2(make_float2(__uint_as_float(w[e] << 16), __uint_as_float(w[e] & 0xFFFF0000u)));
    q[r] = make_uint2(pack4_e4m3(v[0].x, v[0].y, v[1].x, v[1].y), pack4_e4m3(v[2].x, v[2].y, v[3].x, v[3].y));
  }
}

// The exchange at the end of the weight-lane kernel is the epilogue warps' business (it needs their registers);
// every other warp only takes part in its CTA-wide and cluster-wide barriers, in the same order.
__device__ __forceinline__ void weight_lane_keep_barriers() {
  __syncthreads();      // main loop over: the epilogue may overwrite the pipeline stages
  cluster_sync_all();   // partial tiles visible cluster-wide
  cluster_sync_all();   // all peers have read them
}

// Scale loader of the unfused weight-lane kernel (one warp).
template <int TOK, bool FUSED>
__device__ __forceinline__ void weight_lane_scale_loader(const WeightLaneParams& p, PipeBars* bars, float* sc,
                                                         const AbortCtl& ac, int lane, int n_t, int m0, int m_count,
                                                         int kt0, int nkt) {
  using C = WeightLane<TOK, FUSED>;
    // ------------------------------ scale loader ------------------------------
    // sc[b][c] = sx[kt, m0+c] * sw[n_t, kt] for the K-tile that accumulator b will hold; second
    // arrival on the accumulator's "full" barrier.  Factors are fetched kScalePrefetch K-tiles ahead.
    pdl_wait_prior();                                       // sx comes from the quantiser launch
    constexpr int P = C::kScalePrefetch;
    constexpr int V = (TOK + 31) / 32;                      // token columns per lane
    float fx[P][V], fw[P];
    const float* sw_row = p.sw + static_cast<int64_t>(n_t) * p.ld_sw;
    auto fetch = [&](int i, float (&x)[V], float& w) {
      const float* src = p.sx + static_cast<int64_t>(kt0 + i) * p.ld_sx + m0;
#pragma unroll
      for (int v = 0; v < V; ++v) {
        const int c = lane + 32 * v;
        x[v] = (c < m_count) ? __ldg(src + c) : 0.f;
      }
      w = __ldg(sw_row + kt0 + i);
    };
#pragma unroll
    for (int j = 0; j < P; ++j) {
#pragma unroll
      for (int v = 0; v < V; ++v) fx[j][v] = 0.f;
      fw[j] = 0.f;
      if (j < nkt) fetch(j, fx[j], fw[j]);
    }
    bool ok = true;
    for (int i0 = 0; ok && i0 < nkt; i0 += P) {
#pragma unroll
      for (int j = 0; j < P; ++j) {
        const int i = i0 + j;
        if (i >= nkt) break;
        const int b = i % C::kNumAcc;
        const uint32_t aph = (i / C::kNumAcc) & 1;
        if (!mbar_wait(&bars->tmem_empty[b], aph ^ 1, ac, kSiteWeightLane + kSiteScaleEmpty, i)) { ok = false; break; }
#pragma unroll
        for (int v = 0; v < V; ++v)
          if (lane + 32 * v < TOK) sc[b * TOK + lane + 32 * v] = fx[j][v] * fw[j];
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->tmem_full[b]);
        if (i + P < nkt) fetch(i + P, fx[j], fw[j]);
      }
    }
}

// grid = (ceil(N/128), splits, ceil(M/TOK)), cluster = (1, splits, 1).
template <int TOK, bool FUSED>
__global__ void __launch_bounds__(WeightLane<TOK, FUSED>::kThreads, WeightLane<TOK, FUSED>::kMinCtas)
weight_lane_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                   const WeightLaneParams p) {
  using C = WeightLane<TOK, FUSED>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align_1024(smem_raw);
  float* sc = reinterpret_cast<float*>(smem + C::kPipeBytes);             // [kNumAcc][TOK] scale products
  PipeBars* bars = reinterpret_cast<PipeBars*>(smem + C::kPipeBytes + C::kScaleBytes);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int n_t = blockIdx.x;
  const int z = blockIdx.y;
  const int m0 = blockIdx.z * TOK;
  const int m_count = min(p.M - m0, TOK);
  const int n_umma = (m_count + 15) & ~15;                // tokens padded to the UMMA N granularity
  const int KT = (p.K + kTileK - 1) / kTileK;
  const int kt0 = static_cast<int>((static_cast<int64_t>(z) * KT) / p.splits);
  const int kt1 = static_cast<int>((static_cast<int64_t>(z + 1) * KT) / p.splits);
  const int nkt = kt1 - kt0;
  const uint32_t stage_tx = FUSED ? kLaneTileBytes : kLaneTileBytes + p.tok_box * kTileK;
  const int pre = min(nkt, C::kStages);                   // weight tiles requested before anything else

  if (threadIdx.x == 0) {
    // a stage is full when the weight tile has landed (and, fused, its quantiser warp has written the activations);
    // an accumulator is full when its UMMAs are complete and its scale products are in shared memory
    for (int s = 0; s < C::kStages; ++s) { mbar_init(&bars->full[s], FUSED ? 2 : 1); mbar_init(&bars->empty[s], 1); }
    for (int b = 0; b < C::kNumAcc; ++b) {
      mbar_init(&bars->tmem_full[b], 2);
      mbar_init(&bars->tmem_empty[b], C::kEpiWarps);
    }
    mbar_init(&bars->teardown, 1);
    mbar_init(&bars->teardown2, 1);
    bars->abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tm_w);
    if (!FUSED) tma_prefetch_desc(&tm_x);
    // This thread is also the TMA producer.  Weights never depend on the preceding launch, so the first
    // ring of weight tiles is requested right here - before the CTA-wide barrier, the TMEM allocation and
    // the dependency wait - to shorten the time from launch to the first byte.
    const uint64_t stream_once = l2_policy_evict_first();
    for (int i = 0; i < pre; ++i) {
      mbar_arrive_expect_tx(&bars->full[i], stage_tx);
      tma_load_2d_hint(smem + i * C::kStageBytes, &tm_w, &bars->full[i], (kt0 + i) * kTileK, n_t * 128, stream_once);
    }
  }
  if (warp == 1) { tmem_alloc(&bars->tmem_base, C::kTmemCols); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  const AbortCtl ac{&bars->abort_flag, p.status, p.wait_limit_ns, p.wait_mode};
  pdl_launch_next();

  float acc[C::kCols];
  const int q = warp & 3;
  const int h = (warp >= C::kFirstEpiWarp && warp < C::kFirstEpiWarp + C::kEpiWarps) ? ((warp - C::kFirstEpiWarp) >> 2) : 0;   // column half (TOK == 256 only)
  const int col0 = h * C::kCols;
  bool epi_ok = true;

  if (warp < C::kFirstEpiWarp) {
   if (C::kTradeRegs) setmaxnreg_dec<C::kRegsLow>();
   if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    // The first ring of weight tiles is already in flight (requested during set-up); the activation
    // tiles of those stages follow after the dependency wait.
    if (lane == 0) {
      const uint64_t stream_once = l2_policy_evict_first();
      if (!FUSED) {
        pdl_wait_prior();
        for (int i = 0; i < pre; ++i)
          tma_load_2d(smem + i * C::kStageBytes + kLaneTileBytes, &tm_x, &bars->full[i], (kt0 + i) * kTileK, m0);
      }
      bool ok = true;
      int i = pre;
      for (; i < nkt; ++i) {
        const int s = i % C::kStages;
        const uint32_t ph = (i / C::kStages) & 1;
        if (!mbar_wait(&bars->empty[s], ph ^ 1, ac, kSiteWeightLane + kSiteProdEmpty, i)) { ok = false; break; }
        uint8_t* a = smem + s * C::kStageBytes;
        mbar_arrive_expect_tx(&bars->full[s], stage_tx);
        tma_load_2d_hint(a, &tm_w, &bars->full[s], (kt0 + i) * kTileK, n_t * 128, stream_once);
        if (!FUSED) tma_load_2d(a + kLaneTileBytes, &tm_x, &bars->full[s], (kt0 + i) * kTileK, m0);
      }
      if (!ok) drain_after_abort(bars, C::kStages, static_cast<uint32_t>(i));
    }
   } else if (warp == 1 || (C::kIssuers == 2 && warp == 3)) {
    // ------------------------------ MMA issuer(s) -----------------------------
    // with two issuers: alternate K-tiles (different stages, different accumulators)
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_e4m3_f32(128, n_umma);
      bool ok = true;
      for (int i = (warp == 1) ? 0 : 1; i < nkt; i += C::kIssuers) {
        const int b = i % C::kNumAcc;
        const uint32_t aph = (i / C::kNumAcc) & 1;
        if (!mbar_wait(&bars->tmem_empty[b], aph ^ 1, ac, kSiteWeightLane + kSiteMmaTmemEmpty, i)) { ok = false; break; }
        const int s = i % C::kStages;
        const uint32_t ph = (i / C::kStages) & 1;
        if (!mbar_wait(&bars->full[s], ph, ac, kSiteWeightLane + kSiteMmaFull, i)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t a_addr = smem_u32(smem + s * C::kStageBytes);
        const uint64_t a_desc = umma_smem_desc_sw128(a_addr);
        const uint64_t b_desc = umma_smem_desc_sw128(a_addr + kLaneTileBytes);
        const uint32_t d = tmem_base + b * TOK;
#pragma unroll
        for (int k = 0; k < kTileK / 32; ++k)
          umma_f8(d, a_desc + 2 * k, b_desc + 2 * k, idesc, k > 0 ? 1u : 0u);
        umma_commit(&bars->empty[s]);
        umma_commit(&bars->tmem_full[b]);
      }
      if (!ok) {
        uint64_t* td = (warp == 1) ? &bars->teardown : &bars->teardown2;
        umma_commit(td);
        const long long t0 = clock64();
        while (!mbar_try_wait(td, 0) && clock64() - t0 < 40000000ll) {}
      }
    }
   } else if (!FUSED && warp == 2) {
    weight_lane_scale_loader<TOK, FUSED>(p, bars, sc, ac, lane, n_t, m0, m_count, kt0, nkt);
   }
   __syncwarp();
   weight_lane_keep_barriers();
  } else if (FUSED && warp >= C::kFirstQuantWarp) {
    // ------------------------------ activation quantisers ---------------------
    // Four warps turn the bf16 activations into the e4m3 operand tiles in shared memory (same arithmetic as
    // act_quant_kernel, so the bytes are identical) and into the scale products of the accumulators.  Warp w
    // owns K-tiles w, w + 4, ...: a conversion is one long dependency chain (amax -> scale -> reciprocal ->
    // quotients -> pack), so four tiles in flight matter more than four warps on one tile.  Inside a tile, 16
    // lanes serve a token row (8 elements each), two rows per warp instruction, up to four row pairs (a unit)
    // converted together; two units are held in registers and the loads of the unit after next are issued as
    // soon as a unit has been converted.
    setmaxnreg_inc<C::kRegsQuant>();
    const int qw = warp - C::kFirstQuantWarp;              // 0..3
    const int sub = lane >> 4, j = lane & 15;
    const uint32_t mask16 = 0xFFFFu << (lane & 16);
    const float* sw_row = p.sw + static_cast<int64_t>(n_t) * p.ld_sw;
    const int npairs = (m_count + 1) >> 1;                 // row pairs that hold a token
    const int upt = (npairs + 3) >> 2;                     // units per tile
    struct Cursor { int i, hh; };                          // K-tile (relative to kt0) and unit inside it
    auto advance = [&](Cursor& c) { if (++c.hh == upt) { c.hh = 0; c.i += C::kQuantWarps; } };
    auto pairs_in = [&](int hh) { const int c = min(4, npairs - 4 * hh); return c == 3 ? 4 : c; };   // 1, 2 or 4
    auto row_of = [&](int hh, int r) { return (hh * 4 + r) * 2 + sub; };
    pdl_wait_prior();                                       // x comes from the preceding launch
    uint4 raw[2][4];
    auto fetch = [&](const Cursor& c, uint4 (&dst)[4]) {
      // addresses are clamped into the matrix and the surplus is masked when the values are used: an
      // unconditional load does not have to be waited for before the next instruction
      const int k = min((kt0 + c.i) * kTileK + j * 8, p.K - 8);
      const int n = pairs_in(c.hh);
#pragma unroll
      for (int r = 0; r < 4; ++r)
        if (r < n)
          dst[r] = ld_global_v4_pinned(p.x + static_cast<int64_t>(m0 + min(row_of(c.hh, r), m_count - 1)) * p.ldx + k);
    };
    Cursor cur{qw, 0}, pf{qw, 0};
    if (pf.i < nkt) { fetch(pf, raw[0]); advance(pf); }
    if (pf.i < nkt) { fetch(pf, raw[1]); advance(pf); }
    bool ok = true;
    float sw_tile = 0.0f;
    while (ok && cur.i < nkt) {
#pragma unroll
      for (int ub = 0; ub < 2; ++ub) {
        if (cur.i >= nkt) break;
        const int i = cur.i, hh = cur.hh;
        const int s = i % C::kStages;
        const int b = i % C::kNumAcc;
        uint8_t* tile = smem + s * C::kStageBytes + kLaneTileBytes;
        if (hh == 0) {
          sw_tile = ld_global_f32_pinned(sw_row + kt0 + i);
          const uint32_t ph = (i / C::kStages) & 1;
          const uint32_t aph = (i / C::kNumAcc) & 1;
          if (!mbar_wait(&bars->empty[s], ph ^ 1, ac, kSiteWeightLane + kSiteProdEmpty, i) ||
              !mbar_wait(&bars->tmem_empty[b], aph ^ 1, ac, kSiteWeightLane + kSiteScaleEmpty, i)) { ok = false; break; }
          if (i < (C::kStages > C::kNumAcc ? C::kStages : C::kNumAcc)) {
            // rows between the last token pair and the UMMA's N extent: zeros, written on the first pass over the rings
            for (int pz = npairs; pz * 2 < n_umma; ++pz) {
              const int row = pz * 2 + sub;
              *reinterpret_cast<uint2*>(tile + row * 128 + (((j >> 1) ^ (row & 7)) << 4) + (j & 1) * 8) = make_uint2(0u, 0u);
              if (j == 0) sc[b * TOK + row] = 0.0f;
            }
          }
        }
        const bool k_in = (kt0 + i) * kTileK + j * 8 < p.K;
        auto convert = [&](auto nr_tag) {
          constexpr int NR = decltype(nr_tag)::value;
          uint4 in[NR];
          uint2 out[NR];
          float scale[NR];
#pragma unroll
          for (int r = 0; r < NR; ++r) {
            const uint32_t keep = (k_in && row_of(hh, r) < m_count) ? 0xFFFFFFFFu : 0u;
            in[r] = make_uint4(raw[ub][r].x & keep, raw[ub][r].y & keep, raw[ub][r].z & keep, raw[ub][r].w & keep);
          }
          quantise_rows_e4m3<NR>(in, mask16, out, scale);
#pragma unroll
          for (int r = 0; r < NR; ++r) {
            const int row = row_of(hh, r);
            // K-major tile with 128-byte swizzle: 16-byte chunk c of row r lives at chunk c ^ (r & 7)
            *reinterpret_cast<uint2*>(tile + row * 128 + (((j >> 1) ^ (row & 7)) << 4) + (j & 1) * 8) = out[r];
            if (j == 0) sc[b * TOK + row] = scale[r] * sw_tile;
          }
        };
        const int n = pairs_in(hh);
        if (n == 4) convert(std::integral_constant<int, 4>{});
        else if (n == 2) convert(std::integral_constant<int, 2>{});
        else convert(std::integral_constant<int, 1>{});
        if (hh == upt - 1) {
          fence_proxy_async_smem();                         // generic-proxy writes -> visible to the tensor core
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(&bars->full[s]);
            mbar_arrive(&bars->tmem_full[b]);
          }
        }
        advance(cur);
        if (pf.i < nkt) { fetch(pf, raw[ub]); advance(pf); }
      }
    }
    __syncwarp();
    weight_lane_keep_barriers();
  } else if (warp >= C::kFirstEpiWarp && warp < C::kFirstEpiWarp + C::kEpiWarps) {
    // ------------------------------ epilogue ----------------------------------
    if (C::kTradeRegs) setmaxnreg_inc<C::kRegsHigh>();
#pragma unroll
    for (int i = 0; i < C::kCols; ++i) acc[i] = 0.0f;
    for (int i = 0; i < nkt; ++i) {
      const int b = i % C::kNumAcc;
      const uint32_t aph = (i / C::kNumAcc) & 1;
      if (!mbar_wait(&bars->tmem_full[b], aph, ac, kSiteWeightLane + kSiteEpiTmemFull, i)) { epi_ok = false; break; }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + b * TOK + col0;
      const float* scb = sc + b * TOK + col0;
      if constexpr (C::kCols == 16) {
        uint32_t r[16];
        tmem_ld_32x16(taddr, r);
        tmem_ld_wait_on(r);
        promote16_cols(acc, r, scb);
      }
#pragma unroll
      for (int c = 0; c < C::kCols / 32; ++c) {
        if (col0 + c * 32 + 16 < n_umma) {                  // both 16-column halves hold tokens
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait_on(r);
          promote16_cols(acc + c * 32, r, scb + c * 32);
          promote16_cols(acc + c * 32 + 16, r + 16, scb + c * 32 + 16);
        } else if (col0 + c * 32 < n_umma) {
          uint32_t r[16];
          tmem_ld_32x16(taddr + c * 32, r);
          tmem_ld_wait_on(r);
          promote16_cols(acc + c * 32, r, scb + c * 32);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->tmem_empty[b]);
    }

    // All MMAs of this CTA have completed (the epilogue waited for the last
    // accumulator), so the pipeline stages are free: reuse them for the exchange.
    __syncthreads();
    float* xch = reinterpret_cast<float*>(smem);              // [TOK][128] fp32, weight row fastest
    {
      const int nrow = q * 32 + lane;
  #pragma unroll
      for (int c = 0; c < C::kCols; ++c)
        if (col0 + c < n_umma) xch[(col0 + c) * 128 + nrow] = epi_ok ? acc[c] : 0.0f;
    }
    cluster_sync_all();   // partial tiles of all splits are visible cluster-wide

    if (bars->abort_flag == 0) {
      // This CTA sums tokens z, z+splits, ... over all splits in rank order (fixed
      // order => bit-identical results run to run), adds the bias and writes y.
      const uint32_t my_rank = cluster_ctarank();
      const int et = threadIdx.x - 32 * C::kFirstEpiWarp;
      const int nq4 = et & 31;                               // which 4 weight rows
      const int n = n_t * 128 + nq4 * 4;
      auto finish_row = [&](int mi, float4 sum) {
        if (n >= p.N) return;
        float v[4] = {sum.x, sum.y, sum.z, sum.w};
        if (p.bias != nullptr) {
  #pragma unroll
          for (int i = 0; i < 4; ++i)
            if (n + i < p.N) v[i] += bf16_to_float(p.bias + n + i);
        }
        __nv_bfloat16* yp = p.y + static_cast<int64_t>(m0 + mi) * p.ldy + n;
        if (p.y_vec && n + 4 <= p.N) {
          uint2 o;
          o.x = pack_bf16x2(v[0], v[1]);
          o.y = pack_bf16x2(v[2], v[3]);
          *reinterpret_cast<uint2*>(yp) = o;
        } else {
  #pragma unroll
          for (int i = 0; i < 4; ++i)
            if (n + i < p.N) yp[i] = __float2bfloat16_rn(v[i]);
        }
      };
      const int tok_stride = p.splits * C::kEpiWarps;
      const int mi_first = static_cast<int>(my_rank) + (et >> 5) * p.splits;
      if (p.splits == 1) {
        // no peers: plain reads of this CTA's own tile (the compiler pipelines them)
  #pragma unroll 4
        for (int mi = mi_first; mi < m_count; mi += tok_stride)
          finish_row(mi, *reinterpret_cast<const float4*>(xch + mi * 128 + nq4 * 4));
      } else {
        // Remote loads are slow one at a time: keep eight in flight (8 / splits token rows per pass),
        // then add them up in rank order.
        const int rows_per_pass = p.splits >= 8 ? 1 : 8 / p.splits;
        for (int mi = mi_first; mi < m_count; mi += tok_stride * rows_per_pass) {
          float4 part[8];
  #pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int t = j / p.splits, r = j - t * p.splits;
            const int row = mi + t * tok_stride;
            if (t < rows_per_pass && row < m_count)
              part[j] = ld_dsmem_f4(smem_u32(xch + row * 128 + nq4 * 4), static_cast<uint32_t>(r));
          }
          for (int t = 0; t < rows_per_pass; ++t) {
            const int row = mi + t * tok_stride;
            if (row >= m_count) break;
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
  #pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int tj = j / p.splits;
              if (tj == t) { sum.x += part[j].x; sum.y += part[j].y; sum.z += part[j].z; sum.w += part[j].w; }
            }
            finish_row(row, sum);
          }
        }
      }
    }
    cluster_sync_all();   // nobody leaves while a peer may still read its shared memory
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// =========================================================================== //
//                                launchers                                     //
// =========================================================================== //
namespace {

template <typename Kern, typename... Args>
cudaError_t launch_ex(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster_y, bool pdl,
                      Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (cluster_y > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = static_cast<unsigned>(cluster_y);
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

template <int BN>
int run_token_lane(const GemmArgs& a, DeviceCtx* ctx) {
  using C = TokenLane<BN>;
  static_assert(128 * kXchStride * 4 <= C::kStages * C::kStageBytes, "partial tile must fit in the pipeline stages");
  CUtensorMap tm_x, tm_w;
  int st = make_tmap_u8_2d(&tm_x, a.xq, a.M, a.K, a.ld_xq, 128);
  if (st != NQ_OK) return st;
  st = make_tmap_u8_2d(&tm_w, a.wq, a.N, a.K, a.ld_wq, BN);
  if (st != NQ_OK) return st;
  const int64_t tiles = ((a.M + 127) / 128) * ((a.N + BN - 1) / BN);
  const int64_t KT = (a.K + 127) / 128;
  // Few tiles: split K over a cluster of 2 or 4 CTAs (larger clusters measured slower: they cannot all be
  // placed at once), keeping the launch within one wave and at least 4 K-tiles per CTA.
  int splits = 1;
  if (a.split_k > 0) {
    splits = a.split_k > 8 ? 8 : a.split_k;
  } else {
    while (splits < 4 && tiles * splits * 2 <= 128) splits *= 2;
  }
  while (splits > 1 && KT / splits < 4) --splits;
  if (splits > KT) splits = static_cast<int>(KT);
  if (splits < 1) splits = 1;
  TokenLaneParams p;
  p.sx = a.sx; p.ld_sx = a.ld_sx; p.sw = a.sw; p.ld_sw = a.ld_sw;
  p.bias = static_cast<const __nv_bfloat16*>(a.bias);
  p.y = static_cast<__nv_bfloat16*>(a.y); p.ldy = a.ldy;
  p.M = static_cast<int>(a.M); p.N = static_cast<int>(a.N); p.K = static_cast<int>(a.K);
  p.splits = splits;
  p.y_vec = (a.ldy % 8 == 0) && (reinterpret_cast<uintptr_t>(a.y) % 16 == 0);
  p.y_tma = 0;
  CUtensorMap tm_y = tm_x;                                     // placeholder when TMA stores are not possible
  if (C::kTmaStore && p.y_vec && splits == 1) {
    st = make_tmap_bf16_2d(&tm_y, a.y, a.M, a.N, a.ldy, 32, 16);
    if (st != NQ_OK) return st;
    p.y_tma = 1;
  }
  p.sx_vec = (a.ld_sx % 4 == 0) && (reinterpret_cast<uintptr_t>(a.sx) % 16 == 0);
  p.wait_mode = 0;
  p.status = ctx->status_dev;
  p.wait_limit_ns = wait_limit_ns();
  dim3 grid;
  if (splits > 1) grid = dim3(static_cast<unsigned>(tiles), static_cast<unsigned>(splits));
  else {
    int ctas = ctx->sm_count - sm_reserve();
    if (ctas < ctx->sm_count / 2) ctas = ctx->sm_count / 2;
    grid = dim3(static_cast<unsigned>(tiles < ctas ? tiles : ctas));
  }
  cudaError_t e = launch_ex(token_lane_kernel<BN>, grid, dim3(C::kThreads), C::kSmemBytes, a.stream, splits, a.pdl,
                            tm_x, tm_w, tm_y, p);
  count_launch();
  return check_cuda(e);
}

template <int BN>
int run_token_pair(const GemmArgs& a, DeviceCtx* ctx) {
  using C = TokenPair<BN>;
  CUtensorMap tm_x, tm_w;
  int st = make_tmap_u8_2d(&tm_x, a.xq, a.M, a.K, a.ld_xq, 128);
  if (st != NQ_OK) return st;
  st = make_tmap_u8_2d(&tm_w, a.wq, a.N, a.K, a.ld_wq, BN / 2);   // each CTA of a pair loads half of the BN rows
  if (st != NQ_OK) return st;
  TokenLaneParams p;
  p.sx = a.sx; p.ld_sx = a.ld_sx; p.sw = a.sw; p.ld_sw = a.ld_sw;
  p.bias = static_cast<const __nv_bfloat16*>(a.bias);
  p.y = static_cast<__nv_bfloat16*>(a.y); p.ldy = a.ldy;
  p.M = static_cast<int>(a.M); p.N = static_cast<int>(a.N); p.K = static_cast<int>(a.K);
  p.splits = 1;
  p.y_vec = (a.ldy % 8 == 0) && (reinterpret_cast<uintptr_t>(a.y) % 16 == 0);
  p.y_tma = 0;
  CUtensorMap tm_y = tm_x;                                     // placeholder when TMA stores are not possible
  if (p.y_vec) {
    st = make_tmap_bf16_2d(&tm_y, a.y, a.M, a.N, a.ldy, 32, 16);
    if (st != NQ_OK) return st;
    p.y_tma = 1;
  }
  p.sx_vec = (a.ld_sx % 4 == 0) && (reinterpret_cast<uintptr_t>(a.sx) % 16 == 0);
  p.wait_mode = 0;
  p.status = ctx->status_dev;
  p.wait_limit_ns = wait_limit_ns();
  const int64_t tiles = ((a.M + 255) / 256) * ((a.N + BN - 1) / BN);
  int pairs = (ctx->sm_count - sm_reserve()) / 2;
  if (pairs < 1) pairs = 1;
  if (tiles < pairs) pairs = static_cast<int>(tiles);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
  cfg.blockDim = dim3(C::kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = a.stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = a.pdl ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, token_pair_kernel<BN>, tm_x, tm_w, tm_y, p);
  count_launch();
  return check_cuda(e);
}

template <int TOK, bool FUSED = false>
int run_weight_lane(const GemmArgs& a, DeviceCtx* ctx, int splits) {
  using C = WeightLane<TOK, FUSED>;
  const int tokens_box = static_cast<int>(a.M >= TOK ? TOK : ((a.M + 15) / 16) * 16);
  CUtensorMap tm_x, tm_w;
  int st = make_tmap_u8_2d(&tm_w, a.wq, a.N, a.K, a.ld_wq, 128);
  if (st != NQ_OK) return st;
  if (FUSED) tm_x = tm_w;                                   // unused by the fused kernel
  else st = make_tmap_u8_2d(&tm_x, a.xq, a.M, a.K, a.ld_xq, tokens_box);
  if (st != NQ_OK) return st;
  WeightLaneParams p;
  p.x = static_cast<const __nv_bfloat16*>(a.x); p.ldx = a.ldx;
  p.sx = a.sx; p.ld_sx = a.ld_sx; p.sw = a.sw; p.ld_sw = a.ld_sw;
  p.bias = static_cast<const __nv_bfloat16*>(a.bias);
  p.y = static_cast<__nv_bfloat16*>(a.y); p.ldy = a.ldy;
  p.M = static_cast<int>(a.M); p.N = static_cast<int>(a.N); p.K = static_cast<int>(a.K);
  p.splits = splits;
  p.wait_mode = 0;
  p.tok_box = tokens_box;
  p.y_vec = (a.ldy % 4 == 0) && (reinterpret_cast<uintptr_t>(a.y) % 8 == 0);
  p.status = ctx->status_dev;
  p.wait_limit_ns = wait_limit_ns();
  dim3 grid(static_cast<unsigned>((a.N + 127) / 128), static_cast<unsigned>(splits),
            static_cast<unsigned>((a.M + TOK - 1) / TOK));
  cudaError_t e = launch_ex(weight_lane_kernel<TOK, FUSED>, grid, dim3(C::kThreads), C::kSmemBytes, a.stream, splits, a.pdl,
                            tm_w, tm_x, p);
  count_launch();
  return check_cuda(e);
}

}  // namespace

int launch_gemm_token_pair(const GemmArgs& a, DeviceCtx* ctx, int tile_n) {
  (void)tile_n;
  return run_token_pair<256>(a, ctx);
}

int launch_gemm_token_lane(const GemmArgs& a, DeviceCtx* ctx, int tile_n) {
  if (tile_n == 128) return run_token_lane<128>(a, ctx);
  if (tile_n == 192) return run_token_lane<192>(a, ctx);
  if (tile_n == 256) return run_token_lane<256>(a, ctx);
  // Measured on B200 (8B-shaped layers): 256-wide tiles are fastest when there is work for every SM (fewest
  // operand bytes per flop).  128-wide tiles win when twice as many tiles still fit in one round of the SMs
  // (256-384 tokens of qkv, 256-512 of o_proj and down: 13-23 us against 18-26 us), and when the 256-wide tiles
  // fill between one and one and a half rounds, where half-size tiles cut the idle tail of the last round
  // (256 tokens of gate_up: 192 tiles on 148 SMs, 40 us against 43 us).
  if (a.N <= 128) return run_token_lane<128>(a, ctx);
  const int64_t tiles256 = ((a.M + 127) / 128) * ((a.N + 255) / 256);
  const int64_t sm = ctx->sm_count;
  if (2 * tiles256 <= sm || (tiles256 > sm && 2 * tiles256 <= 3 * sm)) return run_token_lane<128>(a, ctx);
  return run_token_lane<256>(a, ctx);
}

int weight_lane_pick_split(int64_t M, int64_t N, int64_t K, int sm_count) {
  // Measured on B200 (8B-shaped layers): the best K split is the largest power of two (cluster size <= 8)
  // that still lets every CTA of the launch be resident at once - two CTAs per SM for <= 64 tokens, one
  // per SM above (the ring of 128/256-token stages fills the shared memory) - with >= 2 K-tiles per CTA.
  const int64_t KT = (K + 127) / 128;
  const int64_t tiles = ((N + 127) / 128) * (M <= 256 ? 1 : (M + 255) / 256);
  const int64_t slots = static_cast<int64_t>(sm_count) * (M <= 64 ? 2 : 1);
  int best = 1;
  for (int s = 2; s <= 8; s *= 2) {
    if (KT / s < 2 || tiles * s > slots) break;
    best = s;
  }
  return best;
}

size_t weight_lane_workspace_bytes(int64_t, int64_t, int64_t) { return 0; }

int launch_gemm_weight_lane(const GemmArgs& a, DeviceCtx* ctx) {
  int splits = a.split_k;
  if (splits <= 0) splits = weight_lane_pick_split(a.M, a.N, a.K, ctx->sm_count);
  const int64_t KT = (a.K + 127) / 128;
  if (splits > 8) splits = 8;
  while (splits > 1 && splits > KT) splits >>= 1;
  if (splits & (splits - 1)) {   // round down to a power of two (cluster shapes 1,2,4,8)
    int s = 1;
    while (s * 2 <= splits) s *= 2;
    splits = s;
  }
  if (a.x != nullptr) {                                      // quantise inside the GEMM (decode batches)
    if (a.M <= 32) return run_weight_lane<32, true>(a, ctx, splits);
    return NQ_ERR_UNSUPPORTED;
  }
  if (a.M <= 16) return run_weight_lane<16>(a, ctx, splits);
  if (a.M <= 32) return run_weight_lane<32>(a, ctx, splits);
  if (a.M <= 64) return run_weight_lane<64>(a, ctx, splits);
  if (a.M <= 128) return run_weight_lane<128>(a, ctx, splits);
  return run_weight_lane<256>(a, ctx, splits);
}

int setup_gemm_kernels() {
  cudaError_t e;
#define NQ_SET_SMEM(kern, bytes)                                                                  \
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);             \
  if (e != cudaSuccess) return check_cuda(e);
  NQ_SET_SMEM(token_pair_kernel<256>, TokenPair<256>::kSmemBytes)
  NQ_SET_SMEM(token_lane_kernel<128>, TokenLane<128>::kSmemBytes)
  NQ_SET_SMEM(token_lane_kernel<192>, TokenLane<192>::kSmemBytes)
  NQ_SET_SMEM(token_lane_kernel<256>, TokenLane<256>::kSmemBytes)
  NQ_SET_SMEM((weight_lane_kernel<16, false>), (WeightLane<16>::kSmemBytes))
  NQ_SET_SMEM((weight_lane_kernel<32, false>), (WeightLane<32>::kSmemBytes))
  NQ_SET_SMEM((weight_lane_kernel<64, false>), (WeightLane<64>::kSmemBytes))
  NQ_SET_SMEM((weight_lane_kernel<128, false>), (WeightLane<128>::kSmemBytes))
  NQ_SET_SMEM((weight_lane_kernel<256, false>), (WeightLane<256>::kSmemBytes))
  NQ_SET_SMEM((weight_lane_kernel<32, true>), (WeightLane<32, true>::kSmemBytes))
#undef NQ_SET_SMEM
  // Kernels whose warpgroups trade registers: the compiled kernel must be launched with at least the registers
  // the warpgroups will ask for in total, or a setmaxnreg.inc would wait for ever.  Refuse to run instead.
  cudaFuncAttributes fa;
#define NQ_CHECK_REGS(kern, threads, needed)                                                      \
  e = cudaFuncGetAttributes(&fa, kern);                                                           \
  if (e != cudaSuccess) return check_cuda(e);                                                     \
  if (fa.numRegs * ((threads) / 128) < (needed)) return NQ_ERR_UNSUPPORTED;
  NQ_CHECK_REGS(token_pair_kernel<256>, TokenPair<256>::kThreads, TokenPair<256>::kRegsNeeded)
  NQ_CHECK_REGS(token_lane_kernel<128>, TokenLane<128>::kThreads, TokenLane<128>::kRegsNeeded)
  NQ_CHECK_REGS(token_lane_kernel<192>, TokenLane<192>::kThreads, TokenLane<192>::kRegsNeeded)
  NQ_CHECK_REGS(token_lane_kernel<256>, TokenLane<256>::kThreads, TokenLane<256>::kRegsNeeded)
  NQ_CHECK_REGS((weight_lane_kernel<32, true>), (WeightLane<32, true>::kThreads), (WeightLane<32, true>::kRegsNeeded))
#undef NQ_CHECK_REGS
  return NQ_OK;
}

}  // namespace nq
