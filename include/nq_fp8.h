/*
 * nq_fp8.h — C ABI of libnq_fp8.so: the FP8 (e4m3) W8A8 block-scaled linear
 * path for NVIDIA B200 (sm_100a).
 *
 * This is the native boundary behind the drop-in replacements for nano_qwen's
 * tensor-parallel linear layers.  Plain pointers and sizes only: no torch
 * types, no C++ types.  All pointers are DEVICE pointers unless said
 * otherwise; `stream` is a `cudaStream_t` passed as `void*` (NULL = the legacy
 * default stream).  Every function returns an NQ_* status: 0 on success,
 * negative on a rejected call; nothing throws, aborts or traps.  Calls only
 * enqueue work (no host synchronisation), so they are legal inside CUDA-graph
 * stream capture once the library has been initialised on the device
 * (nq_init, or any earlier call).
 *
 * Layouts
 *   x    [M, K]  bf16, row-major, row stride `ldx` elements
 *   xq   [M, K]  e4m3, row-major, row stride `ld_xq` BYTES (multiple of 16)
 *   sx   [ceil(K/128), ld_sx] fp32, K-group major: sx[g*ld_sx + m] is the
 *        dequantisation multiplier of token m, K-group g   (ld_sx >= M)
 *   wq   [N, K]  e4m3, row-major, row stride `ld_wq` bytes (multiple of 16)
 *   sw   [ceil(N/128), ld_sw] fp32, row-major: sw[bn*ld_sw + bk]
 *        (what FP8 checkpoints call `weight_scale_inv`)        (ld_sw >= ceil(K/128))
 *   bias [N] bf16 or NULL
 *   y    [M, N]  bf16, row-major, row stride `ldy` elements
 *
 * What each entry point stands in for in the reference (nano_qwen,
 * src/nano_qwen/layers/linear.py):
 *   nq_fp8_linear / nq_fp8_gemm_bs128   the `F.linear(x, W, b)` call of
 *       ReplicatedLinear.forward (:50-51), ColumnParallelLinear.forward
 *       (:72-73; inherited by MergedColumnParallelLinear and
 *       QKVParallelLinear) and RowParallelLinear.forward (:152-153).
 *   nq_act_quant_e4m3_g128              no counterpart: the reference keeps
 *       activations in bf16; this is the dynamic per-token 1x128 quantiser
 *       that feeds the FP8 GEMM.
 *   nq_weight_quant_e4m3_b128           no counterpart: offline 128x128 block
 *       quantiser used for random-init weights and bf16 checkpoints.
 * The row-parallel all-reduce (linear.py:154-155) stays in the host layer
 * (torch.distributed / NCCL).
 */
#ifndef NQ_FP8_H_
#define NQ_FP8_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NQ_OK 0
#define NQ_ERR_BAD_ARGUMENT (-1)   /* null pointer, negative size, misaligned pointer or stride */
#define NQ_ERR_UNSUPPORTED (-2)    /* shape outside what the kernels cover */
#define NQ_ERR_WORKSPACE (-3)      /* a size limit of a fixed buffer is exceeded (noalloc scratch, p2p slot) */
#define NQ_ERR_CUDA (-4)           /* a CUDA runtime/driver call failed (see nq_last_cuda_error) */
#define NQ_ERR_DEVICE_TIMEOUT (-5) /* a bounded device-side wait expired (reported by nq_device_status) */
#define NQ_ERR_NOT_SM100 (-6)      /* the current device is not compute capability 10.x */

/* Algorithm selector for the GEMM (`algo` argument). */
#define NQ_ALGO_AUTO 0
#define NQ_ALGO_TOKEN_LANE 1  /* tokens on the 128 UMMA lanes; 128 x {128,192,256} tiles; prefill-sized M */
#define NQ_ALGO_WEIGHT_LANE 2 /* weight rows on the lanes (swap-AB), split-K; decode-sized M */
#define NQ_ALGO_TOKEN_LANE_128 3 /* token-lane with a fixed tile width of 128 / 192 / 256 weight rows */
#define NQ_ALGO_TOKEN_LANE_192 4 /* (NQ_ALGO_TOKEN_LANE picks the width itself)                        */
#define NQ_ALGO_TOKEN_LANE_256 5
#define NQ_ALGO_TOKEN_PAIR 6 /* token-lane on CTA pairs: one 256x256 tile per two SMs (tcgen05 cta_group::2) */
#define NQ_ALGO_WEIGHT_LANE_FUSED 8 /* nq_fp8_linear only: weight-lane with the activation quantiser inside the GEMM
                                       kernel (M <= NQ_FUSED_MAX_TOKENS, K and ldx multiples of 8, x 16-byte aligned) */
#define NQ_FUSED_MAX_TOKENS 32  /* most tokens NQ_ALGO_WEIGHT_LANE_FUSED accepts */
#define NQ_FUSED_AUTO_TOKENS 0  /* most tokens for which NQ_ALGO_AUTO picks it: none (see nq_fp8_linear) */

/* ABI version of this header (major*100 + minor). */
int nq_version(void);

/* Hash of the CUDA sources and headers this binary was compiled from (set by the build script; "unknown" for a
 * hand-made build).  Lets a host check that a shipped binary matches the source tree it sits in. */
const char* nq_source_hash(void);

/* Human-readable name of a status code (static storage, never NULL). */
const char* nq_status_string(int status);

/* Text of the last CUDA error seen by this library on the calling thread. */
const char* nq_last_cuda_error(void);

/* One-time per-device set-up (driver entry points, status block, kernel
 * attributes) for the CURRENT device.  Implicit in every other call; call it
 * explicitly before starting a stream capture. */
int nq_init(void);

/* Dynamic activation quantiser: bf16 [M,K] -> e4m3 [M,K] + fp32 group scales.
 * scale = max(amax, 1e-10) / 448 (IEEE fp32 divide), q = RNE_e4m3(x / scale).
 * A ragged last group (K % 128 != 0) takes its amax over the elements present. */
int nq_act_quant_e4m3_g128(const void* x, int64_t M, int64_t K, int64_t ldx,
                           void* xq, int64_t ld_xq, float* sx, int64_t ld_sx, void* stream);

/* Offline weight quantiser: bf16 [N,K] -> e4m3 [N,K] + fp32 128x128 block scales,
 * same scale/rounding rule as above. */
int nq_weight_quant_e4m3_b128(const void* w, int64_t N, int64_t K, int64_t ldw,
                              void* wq, int64_t ld_wq, float* sw, int64_t ld_sw, void* stream);

/* ---- Producers that emit FP8 directly (the quantiser fused into the op in front of a linear layer) --------
 * Same output contract as nq_act_quant_e4m3_g128 (xq / sx layouts, scale rule); the value that is quantised is
 * the bf16 tensor the reference's eager code would have produced.  Vector path only: the feature size must be
 * a multiple of 16, row strides multiples of 8 elements (16 bytes for xq), pointers 16-byte aligned; anything
 * else returns NQ_ERR_UNSUPPORTED (run the reference op and nq_act_quant_e4m3_g128 instead).
 *
 * nq_silu_mul_quant_e4m3_g128: gate_up [M, 2*I] bf16 (gate = columns [0, I), up = [I, 2I)), row stride `ld`;
 *   h = bf16(bf16(silu(gate)) * up), silu evaluated in fp32 — SiluAndMul.forward, layers/activation.py:8-11;
 *   xq [M, I], sx [ceil(I/128), ld_sx]: the input of down_proj. */
int nq_silu_mul_quant_e4m3_g128(const void* gate_up, int64_t M, int64_t I, int64_t ld,
                                void* xq, int64_t ld_xq, float* sx, int64_t ld_sx, void* stream);

/* nq_rmsnorm_quant_e4m3_g128: RMSNorm.forward / GemmaRMSNorm.forward (layers/layernorm.py:16-56, :79-120).
 *   v = float(x) [+ float(residual_in)];  residual_out = bf16(v) (only with residual_in; may be the same buffer);
 *   n = bf16(v * rsqrt(mean(v^2) + eps));  h = bf16(n * weight)  or, gemma != 0,  bf16(n * bf16(1 + weight));
 *   xq / sx = quantised h; y_out (optional, may be NULL) receives h in bf16 for consumers that are not FP8 linears.
 *   weight [H] bf16; x, residual, y_out [M, H] bf16 with row strides ldx, ld_res, ldy. */
int nq_rmsnorm_quant_e4m3_g128(const void* x, const void* residual_in, const void* weight, float eps, int gemma,
                               int64_t M, int64_t H, int64_t ldx, int64_t ld_res, void* residual_out,
                               void* y_out, int64_t ldy,
                               void* xq, int64_t ld_xq, float* sx, int64_t ld_sx, void* stream);

/* Bytes of global scratch the GEMM needs for this problem: always 0.  Every kernel of this library keeps its
 * split-K partial sums in shared memory (exchanged across a thread-block cluster), so the `workspace` /
 * `workspace_bytes` arguments below are accepted and ignored (pass NULL, 0).  The query stays in the ABI so that a
 * caller written against it keeps working if a later kernel does need scratch. */
size_t nq_fp8_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K);

/* y = bf16( sum_t sx[t,m] * sw[n/128,t] * (xq[m, tile t] . wq[n, tile t]) + bias[n] ),
 * tile = 128 consecutive k; inner products accumulate in fp32 on the tensor
 * cores, the scaled sum over tiles in fp32 registers.
 * `split_k` = 0 lets the library choose; otherwise it is a hint for
 * NQ_ALGO_WEIGHT_LANE. */
int nq_fp8_gemm_bs128(const void* xq, int64_t ld_xq, const float* sx, int64_t ld_sx,
                      const void* wq, int64_t ld_wq, const float* sw, int64_t ld_sw,
                      const void* bias, void* y, int64_t ldy,
                      int64_t M, int64_t N, int64_t K,
                      void* workspace, size_t workspace_bytes,
                      int algo, int split_k, void* stream);

/* Convenience: activation quantiser + GEMM in one call.  `xq_scratch`
 * (M*ld_xq bytes, ld_xq = K rounded up to 16) and `sx_scratch`
 * (ceil(K/128)*ld_sx floats, ld_sx = M rounded up to 4) are caller-owned.
 * NQ_ALGO_WEIGHT_LANE_FUSED (M <= NQ_FUSED_MAX_TOKENS, x readable 16 bytes at a
 * time) runs the quantiser inside the GEMM kernel: one launch, scratch untouched
 * and allowed to be NULL, result bit-identical to the two-launch path.
 * NQ_ALGO_AUTO does not pick it any more: since the quantiser kernel releases its
 * dependents at its start (programmatic dependent launch), the GEMM's set-up and
 * first weight tiles overlap the quantiser, and two launches measured faster at
 * every batch size (8 tokens: 47.9 us per 8B-shaped layer against 58.0 us). */
int nq_fp8_linear(const void* x, int64_t ldx,
                  const void* wq, int64_t ld_wq, const float* sw, int64_t ld_sw,
                  const void* bias, void* y, int64_t ldy,
                  int64_t M, int64_t N, int64_t K,
                  void* xq_scratch, float* sx_scratch,
                  void* workspace, size_t workspace_bytes,
                  int algo, int split_k, void* stream);

/* Capacity of the built-in scratch of nq_fp8_linear_noalloc. */
#define NQ_NOALLOC_MAX_XQ_BYTES (8u << 20)   /* M * (K rounded up to 16)            must not exceed this */
#define NQ_NOALLOC_MAX_SX_FLOATS (64u << 10) /* ceil(K/128) * (M rounded up to 4)   must not exceed this */

/* nq_fp8_linear without any scratch argument, for callers that cannot allocate device memory (a host that
 * only passes pre-registered tensors, a fixed memory budget, a call made while a stream is being captured).
 * No counterpart in the reference: nano_qwen allocates freely through torch.
 * The quantised activations go to a fixed array inside the library image (8.25 MiB, present on every GPU
 * that loads the library until the process exits), so:
 *   - M * roundup(K,16) <= NQ_NOALLOC_MAX_XQ_BYTES and ceil(K/128) * roundup(M,4) <= NQ_NOALLOC_MAX_SX_FLOATS,
 *     otherwise NQ_ERR_WORKSPACE is returned and nothing is launched;
 *   - all calls on one GPU share that array: two calls that may run at the same time on the GPU (different
 *     streams) corrupt each other; calls on one stream are safe;
 *   - the first call on each device looks up the array's device address (a host-side CUDA call); make that
 *     first call, or nq_init plus one call, before starting a stream capture.
 * It calls no cudaMalloc / cudaFree and no allocating library routine.  Inputs, outputs and all other
 * arguments are those of nq_fp8_linear. */
int nq_fp8_linear_noalloc(const void* x, int64_t ldx,
                          const void* wq, int64_t ld_wq, const float* sw, int64_t ld_sw,
                          const void* bias, void* y, int64_t ldy,
                          int64_t M, int64_t N, int64_t K,
                          int algo, int split_k, void* stream);

/* ---- Row-parallel reduction over peer memory (one process per GPU, all GPUs of one node) ------------------
 * Stands in for the `dist.all_reduce(y)` that ends RowParallelLinear.forward (linear.py:154-155) when y is
 * small (decode batches): one kernel per rank pushes its partial into every peer's inbox over NVLink (each
 * 8-byte word carries 4 bytes of data and the call number, so no fence and no second trip are needed), polls
 * (bounded) its own inbox for the peers' partials and adds them in rank order in fp32, so every rank ends
 * with the same bf16 bits.  Legal inside CUDA-graph capture: the call number lives in device memory.
 *
 * Set-up, once per process (host side; the caller moves the 64-byte handles between processes itself):
 *   inbox : nq_p2p_alloc(4 * tp * slot_bytes)    zero-filled device memory of the current device
 *   state : nq_p2p_alloc(256)                     private to the rank, never exported
 *   nq_p2p_export(inbox, handle) on the owner, nq_p2p_import(handle, &ptr) on every peer, then a barrier
 *   between the processes before the first reduction.
 * All ranks must make the same sequence of nq_row_reduce_p2p calls (same count, same slot_bytes). */
#define NQ_P2P_MAX_RANKS 8
#define NQ_P2P_HANDLE_BYTES 64
int nq_p2p_alloc(size_t bytes, void** dev_ptr);
int nq_p2p_free(void* dev_ptr);                                   /* memory from nq_p2p_alloc */
int nq_p2p_export(void* dev_ptr, unsigned char* handle);          /* handle: NQ_P2P_HANDLE_BYTES bytes, host */
int nq_p2p_import(const unsigned char* handle, void** dev_ptr);   /* maps a peer's allocation, enables peer access */
int nq_p2p_release(void* dev_ptr);                                /* unmaps a pointer from nq_p2p_import */

/* y[i] = bf16( sum over ranks r = 0..tp-1 of partial_r[i] ), i < count (bf16 elements; count % 8 == 0,
 * count * 2 <= slot_bytes, slot_bytes % 16 == 0, both pointers 16-byte aligned; y may be the same buffer as
 * partial).  inbox: HOST array of tp device pointers, entry r = rank r's inbox as mapped in this process
 * (entry `rank` is the local allocation).  A peer that never arrives makes the bounded wait expire: the call
 * still completes and nq_device_status reports NQ_ERR_DEVICE_TIMEOUT. */
int nq_row_reduce_p2p(const void* partial, void* y, int64_t count,
                      void* const* inbox, int rank, int tp,
                      int64_t slot_bytes, void* state, void* stream);

/* ---- Row-parallel reduction over peer-mapped buffers, for prefill-sized outputs ----------------------------
 * Stands in for the same `dist.all_reduce(y)` (linear.py:154-155) when y is large.  The partial outputs of all
 * ranks live at the same offset of a buffer that every GPU of the group has mapped (the host obtains the
 * mappings from its symmetric-memory allocator; this library only needs the pointers).  One kernel per rank, a
 * two-shot exchange in which every transfer is a pull (bulk asynchronous copies from the peers' buffers into
 * shared memory; no multicast, no tensor map): rank r adds slice r
 * of all ranks' partials in rank order in fp32, writes the sum to y and back into its own buffer, and after a
 * barrier fetches the other slices' sums from their owners into y; a last barrier keeps every buffer intact until
 * all peers have read it.  All ranks end with the same bits.
 *   bufs   : HOST array of tp device pointers, entry r = the message in rank r's buffer as mapped in this process
 *   y      : private result, count bf16 elements (count % 8 == 0), 16-byte aligned
 *   pads   : HOST array of tp device pointers, entry r = rank r's signal pad (NQ_SYM_PAD_BYTES, zero-filled once,
 *            peer-mapped) as mapped in this process
 *   state  : 16 bytes of zero-filled device memory private to the rank (call counter; graph-replay safe)
 *   blocks : thread blocks to use, 1..NQ_SYM_MAX_BLOCKS, THE SAME ON EVERY RANK (block b pairs with block b);
 *            measured on B200s for 64 MiB: 32 blocks reach the rate of any larger count (219 us on 8 ranks, 140 us
 *            on 2), 16 blocks 240 / 195 us
 * tp must be 2, 4 or 8.  All ranks must make the same sequence of calls.  Waits are bounded
 * (nq_set_wait_limit_ns); a peer that never arrives yields NQ_ERR_DEVICE_TIMEOUT in nq_device_status (site 80..82,
 * aux = the peer) and a wrong result. */
#define NQ_SYM_MAX_BLOCKS 160
#define NQ_SYM_PAD_BYTES (3 * NQ_SYM_MAX_BLOCKS * NQ_P2P_MAX_RANKS * 4)
int nq_row_reduce_pull(void* const* bufs, void* y, int64_t count, void* const* pads, int rank, int tp,
                       void* state, int blocks, void* stream);

/* Reads the device-side status block of the current device (mapped host
 * memory; call after synchronising the stream).  code = 0 or
 * NQ_ERR_DEVICE_TIMEOUT, where/block/aux say which wait expired.  `reset`
 * non-zero clears it. */
int nq_device_status(int* code, int* where, int* block, int* aux, int reset);

/* Wall-clock limit (nanoseconds) of one device-side wait; default 2e9. */
int nq_set_wait_limit_ns(uint64_t ns);

/* Number of SMs the persistent GEMM (token-lane, unsplit) leaves without a CTA, so that a kernel running
 * next to it on another stream (a collective) can be scheduled at once.  Process-wide, default 0;
 * read at launch time.  Returns the previous value, or a negative status for n < 0. */
int nq_set_sm_reserve(int n);

/* Number of kernels this library has launched on the calling process so far. */
int64_t nq_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* NQ_FP8_H_ */
