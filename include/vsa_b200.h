/*
 * vsa_b200.h -- C ABI of the B200 Video Sparse Attention kernels.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (passed as void*, i.e. a cudaStream_t), launches on that stream without
 * synchronising the host, and returns 0 on success or a negative vsa_status.
 * Nothing is allocated by the library: outputs and scratch buffers are the
 * caller's.  Nothing throws across the boundary; vsa_last_error_string()
 * returns the text of the calling thread's most recent failure.
 *
 * Layouts (all contiguous, row-major):
 *   q, out, dout, dq, gate, dgate   [BH, Lq,  D]     BH = batch * heads
 *   k, v, dk, dv                    [BH, Lkv, D]
 *   pooled q / k / v and their grads [BH, Qb | Kb, D], Qb = Lq/be, Kb = Lkv/be
 *   scores, probs                   [BH, Qb, Kb]
 *   selected                        [BH, Qb, topk]   int32 key-block ids
 *   kv_sizes [Kb], q_sizes [Qb]     int32 valid tokens per block (shared by all BH)
 *   lse2, delta                     [BH, Lq]         fp32
 *   counts, offsets                 [BH, Kb]         int32 (CSR of key block -> query blocks)
 *   inverse                         [BH, Qb*topk]    int32 query-block ids grouped by key block
 *
 * dtype: VSA_BF16 or VSA_F16 (tcgen05 kernels for D = 128 and be = 64, 128 or 256, warp-level
 * tensor-core kernels for D = 64 at those block volumes, scalar kernels otherwise; the reference
 * accepts both) or VSA_F32 (scalar kernels, the fp32
 * validation mode).
 *
 * Each comment names the function of the reference project (path inside that
 * project : lines) whose work the entry point replaces.
 */
#ifndef VSA_B200_H_
#define VSA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum vsa_status {
  VSA_OK = 0,
  VSA_ERR_BAD_ARGUMENT = -1,   /* null pointer, non-positive size, topk out of range ... */
  VSA_ERR_UNSUPPORTED = -2,    /* shape or dtype outside what the kernels cover */
  VSA_ERR_LAUNCH = -3,         /* the CUDA runtime refused the launch */
  VSA_ERR_DEVICE_TIMEOUT = -4  /* a bounded device-side wait ran out */
} vsa_status;

typedef enum vsa_dtype { VSA_BF16 = 0, VSA_F32 = 1, VSA_F16 = 2 } vsa_dtype;

/* Text of the last error on the calling thread ("" if none). */
const char* vsa_last_error_string(void);

/* Library version as major*10000 + minor*100 + patch. */
int vsa_version(void);

/* Number of kernels this library has launched in the process so far (all threads). */
int64_t vsa_launch_count(void);

/* Device-side status word: 0, or the code of the first bounded wait (mbarrier) that ran out in a
 * tcgen05 kernel since the last call.  Synchronises the device; clears the word.
 *
 * Every wait inside the tcgen05 kernels is bounded (250 ms).  When one runs out the CTA records a code
 * here, stops issuing work, frees its tensor memory and returns; from then on every tcgen05 kernel of this
 * library returns at its first instruction WITHOUT writing its outputs, until this call has cleared the
 * word.  The launching entry points cannot see that (they do not synchronise), so a caller that consumes
 * results must call this after it has synchronised: non-zero means the outputs since the last clear are
 * not valid.  (The Python layer does so wherever it synchronises anyway and raises VsaError.)
 * The entry points use the CALLER'S CURRENT DEVICE: set it (cudaSetDevice) to the device that owns the
 * pointers and the stream before calling; the status word is per device.  No reference counterpart. */
int vsa_device_status(int* status);

/* Size in bytes of a scratch or intermediate buffer the caller must provide (nothing is allocated by the
 * library): which = one of vsa_scratch.  -1 for an unknown buffer, dtype or a negative extent.
 * No reference counterpart (it allocates with torch inside its launchers). */
typedef enum vsa_scratch {
  VSA_SCRATCH_SCORES = 0,    /* scores, probs, dscores_ws: [BH, Qb, Kb] of dtype                    */
  VSA_SCRATCH_ROWDOT = 1,    /* rowdot_ws: [BH, Qb] fp32                                             */
  VSA_SCRATCH_ROW_STATS = 2, /* lse2, delta: [BH, Lq] fp32                                           */
  VSA_SCRATCH_CSR_ROWS = 3,  /* counts, offsets, cursor_ws: [BH, Kb] int32                           */
  VSA_SCRATCH_CSR_EDGES = 4, /* inverse / inverse_edges: [BH, Qb*topk] int32                         */
  VSA_SCRATCH_POOLED = 5,    /* q_mean and its gradient: [BH, Qb, D] of dtype (Kb for k_mean, v_mean) */
  VSA_SCRATCH_DS_TILES = 6   /* ds_ws of the stored-dS backward (= vsa_sparse_bwd_ds_workspace_bytes) */
} vsa_scratch;
int64_t vsa_workspace_bytes(int which, int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk, int dtype);

/* Exercises the time-out path without making anything fail: one warp waits up to limit_ns
 * (1 us .. 100 ms) on a barrier nothing arrives at, gives up, records code 201 in the status word, writes
 * 1 to *gave_up (a device pointer) and returns.  For tests of the reporting path. */
int vsa_selftest_wait_timeout(int64_t limit_ns, int* gave_up, void* stream);

/* Unit check of the tcgen05 building blocks (TMA boxes, shared-memory operand descriptors, tensor
 * memory read-out): out[128x64] fp32 = A * B for bf16 operands.  mode 0: a is [128 x 128] with the
 * reduction dim contiguous, b is [64 x 128] likewise (out = a b^T).  mode 1: a is [128 k x 128 m], b is
 * [128 k x 64 n] (out = a^T b).  No counterpart in the reference; used by the GPU tests. */
int vsa_selftest_umma(const void* a, const void* b, float* out, int mode, void* stream);

/* Padding-aware block means of q, k and v in ONE pass: fp32 sum of the first
 * sizes[b] tokens / max(sizes[b],1), rounded to dtype.
 * Replaces block_mean / fused_block_mean x3: vsa/common.py:55-82,
 * vsa/fused_common.py:20-59,106-144. */
int vsa_block_mean3_fwd(const void* q, const void* k, const void* v,
                        const int32_t* q_sizes, const int32_t* kv_sizes,
                        void* q_mean, void* k_mean, void* v_mean,
                        int64_t BH, int64_t Lq, int64_t Lkv, int D, int be,
                        int dtype, void* stream);

/* Single-tensor form of the above (x [BH,L,D] -> mean [BH,L/be,D]). */
int vsa_block_mean_fwd(const void* x, const int32_t* sizes, void* mean,
                       int64_t BH, int64_t L, int D, int be, int dtype, void* stream);

/* Block-mean backward folded into the accumulation autograd would do:
 * dx[t] += dmean[block]/max(size,1) for t < size (padding rows untouched).
 * Replaces _block_mean_backward_kernel + AccumulateGrad add:
 * vsa/fused_common.py:62-103,146-172. */
int vsa_block_mean_bwd_accumulate(void* dx, const void* dmean, const int32_t* sizes,
                                  int64_t BH, int64_t L, int D, int be,
                                  int dtype, void* stream);

/* Stand-alone block-mean backward: dx[t] = dmean[block]/max(size,1) for t < size, else 0. */
int vsa_block_mean_bwd(void* dx, const void* dmean, const int32_t* sizes,
                       int64_t BH, int64_t L, int D, int be, int dtype, void* stream);

/* Pooled attention: scores = round(round(q_mean k_mean^T) * scale), probs =
 * round(softmax(scores)), out_c = round(probs v_mean); every rounding to dtype.
 * Replaces coarse_branch_compact's matmul/softmax/matmul: vsa/common.py:164-166. */
int vsa_coarse_fwd(const void* q_mean, const void* k_mean, const void* v_mean,
                   void* scores, void* probs, void* out_c,
                   int64_t BH, int Qb, int Kb, int D, float scale,
                   int dtype, void* stream);

/* Top-K key blocks per query block from the pooled scores; ids are written in
 * ascending order, ties broken towards the lower id.
 * Replaces scores.topk(...).indices: vsa/torch_impl.py:85, vsa/triton_impl.py:1710. */
int vsa_topk(const void* scores, int32_t* selected,
             int64_t rows, int Kb, int topk, int dtype, void* stream);

/* Backward of the pooled attention.  dscores_ws is scratch [BH,Qb,Kb] of dtype,
 * rowdot_ws is fp32 scratch [BH,Qb].
 * Replaces autograd of vsa/common.py:164-166. */
int vsa_coarse_bwd(const void* d_out_c, const void* out_c,
                   const void* q_mean, const void* k_mean, const void* v_mean,
                   const void* probs, void* dscores_ws, float* rowdot_ws,
                   void* dq_mean, void* dk_mean, void* dv_mean,
                   int64_t BH, int Qb, int Kb, int D, float scale,
                   int dtype, void* stream);

/* Fine attention of each query block over the valid tokens of its selected key
 * blocks; lse2 (may be NULL, which selects the warp-level kernel instead of the tcgen05 one)
 * receives row_max + log2(row_sum) of the scores times scale*log2(e).
 * Replaces _triton_sparse_attention_forward and both forward kernels:
 * vsa/triton_impl.py:39-355,358-473 (oracle form: vsa/torch_impl.py:86-106). */
int vsa_sparse_fwd(const void* q, const void* k, const void* v,
                   const int32_t* selected, const int32_t* kv_sizes,
                   void* out, float* lse2,
                   int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk,
                   float scale, int dtype, void* stream);

/* vsa_sparse_fwd with the gated combine folded into the store of the fine output: out_s (kept: the
 * backward's delta needs it) and out = out_s + out_c[block] * gate (gate may be NULL) leave the kernel
 * together, bit-identical to vsa_sparse_fwd followed by vsa_combine_fwd, one pass over out_s fewer.
 * Replaces the forward kernels PLUS _combine_forward_kernel: vsa/triton_impl.py:358-473,1720-1726,
 * vsa/fused_common.py:175-199,259-295. */
int vsa_sparse_fwd_combine(const void* q, const void* k, const void* v,
                           const int32_t* selected, const int32_t* kv_sizes,
                           void* out_s, float* lse2, const void* out_c, const void* gate, void* out,
                           int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk,
                           float scale, int dtype, void* stream);

/* CSR of key block -> query blocks from the routing table, built on the device
 * by count / scan / scatter with exactly Qb*topk stored edges per BH slice.
 * cursor_ws is int32 scratch [BH,Kb].  Order inside a key row is unspecified.
 * Replaces _invert_indices and its two kernels: vsa/triton_impl.py:476-595. */
int vsa_route_invert(const int32_t* selected, int32_t* counts, int32_t* offsets,
                     int32_t* inverse, int32_t* cursor_ws,
                     int64_t BH, int Qb, int Kb, int topk, void* stream);

/* Same result as vsa_route_invert, for callers that cannot provide the cursor scratch: a host whose
 * own pool owns all device memory (cudaMalloc fails there) or a loop where allocation is banned
 * because it synchronises the device.  The cursor lives in a 1 MiB array built into the library
 * (held by every GPU that loads it, until exit); BH*Kb must not exceed 262,144 or the call is
 * refused with VSA_ERR_UNSUPPORTED.  The call allocates nothing.  Its first use on a device looks up
 * the array's device address (cudaGetSymbolAddress), so make that first call before any stream
 * capture.  All calls share the one array: calls that overlap on the same GPU race and must be
 * serialised by the caller; no state carries over between calls (every entry used is rewritten).
 * The looked-up address is kept per device ordinal (ordinals 0..63) for the life of the process: after a
 * cudaDeviceReset, or any other re-creation of the device's primary context, reload the library.
 * No counterpart in the reference (it always allocates with torch). */
int vsa_route_invert_static(const int32_t* selected, int32_t* counts, int32_t* offsets,
                            int32_t* inverse, int64_t BH, int Qb, int Kb, int topk, void* stream);

/* Query-owned backward: delta = rowsum(out_s * dout) (written to delta, which
 * vsa_sparse_bwd_dkdv reads) and dq = scale * sum_edges dS K.
 * Replaces _delta_kernel/_delta_256_kernel + _vsa_dq_kernel/_vsa_dq_256_kernel:
 * vsa/triton_impl.py:598-700,703-969. */
int vsa_sparse_bwd_dq(const void* dout, const void* q, const void* k, const void* v,
                      const void* out_s, const float* lse2,
                      const int32_t* selected, const int32_t* kv_sizes,
                      float* delta, void* dq,
                      int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk,
                      float scale, int dtype, void* stream);

/* Key-owned backward over the CSR in-edges: dk = scale * sum dS^T Q, dv = sum P^T dO;
 * rows beyond a ragged block's size get zero.
 * Replaces _vsa_dkdv_kernel/_vsa_dkdv_256_kernel: vsa/triton_impl.py:972-1318. */
int vsa_sparse_bwd_dkdv(const void* dout, const void* q, const void* k, const void* v,
                        const float* lse2, const float* delta,
                        const int32_t* counts, const int32_t* offsets, const int32_t* inverse,
                        const int32_t* kv_sizes, void* dk, void* dv,
                        int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk,
                        float scale, int dtype, void* stream);

/* vsa_sparse_bwd_dq / vsa_sparse_bwd_dkdv with the block-mean backward folded into their stores:
 * dq[t] = fine gradient + dq_mean[block] / max(q_sizes[block], 1) for t < q_sizes[block] (and likewise dk, dv
 * with kv_sizes), rounded once.  dq_mean, dk_mean, dv_mean are the pooled gradients [BH, Qb | Kb, D] that
 * vsa_coarse_bwd produced.  Replaces the fine backward kernels PLUS _block_mean_backward_kernel and the
 * AccumulateGrad adds that follow it: vsa/triton_impl.py:703-1318 + vsa/fused_common.py:62-103,146-172. */
int vsa_sparse_bwd_dq_fused(const void* dout, const void* q, const void* k, const void* v,
                            const void* out_s, const float* lse2,
                            const int32_t* selected, const int32_t* kv_sizes,
                            float* delta, void* dq, const void* dq_mean, const int32_t* q_sizes,
                            int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk,
                            float scale, int dtype, void* stream);
int vsa_sparse_bwd_dkdv_fused(const void* dout, const void* q, const void* k, const void* v,
                              const float* lse2, const float* delta,
                              const int32_t* counts, const int32_t* offsets, const int32_t* inverse,
                              const int32_t* kv_sizes, void* dk, void* dv,
                              const void* dk_mean, const void* dv_mean,
                              int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk,
                              float scale, int dtype, void* stream);

/* ---- the backward that forms dS once ---------------------------------------------------------------
 * The two passes above (like _vsa_dq_kernel and _vsa_dkdv_kernel of the reference,
 * vsa/triton_impl.py:838-1126) each recompute the scores and dP.  The entry points below compute them
 * once: vsa_sparse_bwd_delta, then vsa_sparse_bwd_dkdv_ds (key-owned; also writes every dS tile), then
 * vsa_sparse_bwd_dq_from_ds (query-owned; only multiplies the stored tiles by K).  Same results within
 * rounding, deterministic, 16 of 56 tensor-core products per pair of edges fewer -- paid for with 8 KB per
 * edge written and read back, which on a B200 costs the key-owned pass about what the dQ pass gains; the
 * Python operator therefore uses it only on request.  Tensor path only: vsa_sparse_bwd_ds_supported() says
 * whether a shape qualifies (bf16 or fp16, D = 128, be = 64, 128 or 256).
 *
 * ds_ws holds one 16-bit tile (the dtype of the call) of 64 query rows x 64 key tokens (8 KB, stored as 8 chunks of 8 key tokens, each
 * chunk [64 rows][16 bytes]) per (query tile, selected key tile):
 * vsa_sparse_bwd_ds_workspace_bytes(BH, Lq, be, topk) bytes in all, BH*Qb*topk*(be/64)^2 tiles, tile index
 * ((edge * be/64 + query sub-tile) * be/64 + key sub-tile) with edge = (bh*Qb + query block)*topk + slot.
 * At 2.1 GB per slice for 92,160 tokens x topk 180, callers with many slices run the two passes over groups
 * of slices (every pointer advanced to the group's first slice, BH = slices in the group). */

/* vsa_route_invert with each in-edge recorded as (query block << 11) | slot, slot = position of the key
 * block in that query block's row of `selected` (so the entry names the edge).  Needs topk <= 2048 and
 * Qb < 2^20.  Extends _invert_indices: vsa/triton_impl.py:544-595. */
int vsa_route_invert_edges(const int32_t* selected, int32_t* counts, int32_t* offsets,
                           int32_t* inverse_edges, int32_t* cursor_ws,
                           int64_t BH, int Qb, int Kb, int topk, void* stream);

/* delta[row] = sum_d out_s[row, d] * dout[row, d] in fp32.
 * Replaces _delta_kernel / _delta_256_kernel: vsa/triton_impl.py:598-700. */
int vsa_sparse_bwd_delta(const void* out_s, const void* dout, float* delta,
                         int64_t BH, int64_t Lq, int D, int dtype, void* stream);

/* 1 if the two entry points below cover (D, be, topk, dtype) in this process, else 0. */
int vsa_sparse_bwd_ds_supported(int D, int be, int topk, int dtype);

/* Size of ds_ws in bytes (see above); -1 for a block volume that is not a multiple of 64. */
int64_t vsa_sparse_bwd_ds_workspace_bytes(int64_t BH, int64_t Lq, int be, int topk);

/* vsa_sparse_bwd_dkdv_fused over packed edges, also writing dS = P * (dP - delta) (not yet times scale) of
 * every edge tile to ds_ws.  dk_mean and dv_mean may both be NULL (no pooled gradients folded in).
 * Replaces _vsa_dkdv_kernel / _vsa_dkdv_256_kernel: vsa/triton_impl.py:972-1318. */
int vsa_sparse_bwd_dkdv_ds(const void* dout, const void* q, const void* k, const void* v,
                           const float* lse2, const float* delta,
                           const int32_t* counts, const int32_t* offsets, const int32_t* inverse_edges,
                           const int32_t* kv_sizes, void* dk, void* dv,
                           const void* dk_mean, const void* dv_mean, void* ds_ws,
                           int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk,
                           float scale, int dtype, void* stream);

/* dq = scale * sum over the selected key tiles of dS K (+ dq_mean[block] / max(q_sizes[block], 1) on the
 * block's valid rows when dq_mean and q_sizes are given; both may be NULL).  Ids in `selected` outside
 * [0, Kb) count as empty blocks.  Replaces _vsa_dq_kernel / _vsa_dq_256_kernel: vsa/triton_impl.py:703-969. */
int vsa_sparse_bwd_dq_from_ds(const void* k, const int32_t* selected, const int32_t* kv_sizes,
                              const void* ds_ws, void* dq, const void* dq_mean, const int32_t* q_sizes,
                              int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk,
                              float scale, int dtype, void* stream);

/* ---- shard-major K/V: the fine kernels of the sequence-parallel mode ----------------------------------
 * (No counterpart in the reference, whose kernels index every (batch, head) slice of one GPU's tensors:
 * vsa/triton_impl.py:83-86.)  After an all-gather over W ranks the K/V shards lie one after another,
 * [W][BH][Lkv/W][D].  These entry points read k_sh, v_sh -- and write dk_sh, dv_sh -- in that layout in
 * place: row of (slice bh, token t) = ((t / kv_shard) * BH + bh) * kv_shard + t % kv_shard, kv_shard = Lkv/W
 * tokens (a multiple of be).  So no re-layout copy follows the gather, and the partial dK/dV are contiguous
 * per owner rank, ready for the reduce-scatter.  q, out, dq ... are this rank's [BH, Lq, D] as usual;
 * selected holds GLOBAL key-block ids; kv_sizes lists all Kb = Lkv/be blocks.  Tensor path only (bf16 or
 * fp16, D = 128, be = 64, 128 or 256), VSA_ERR_UNSUPPORTED otherwise.  kv_shard = Lkv is the ordinary layout. */

/* 1 if the three entry points below cover (D, be, topk, dtype) in this process, else 0. */
int vsa_sparse_sharded_supported(int D, int be, int topk, int dtype);

/* vsa_sparse_fwd_combine on shard-major K/V; out_c, gate and out may all be NULL (fine output only). */
int vsa_sparse_fwd_combine_sharded(const void* q, const void* k_sh, const void* v_sh,
                                   const int32_t* selected, const int32_t* kv_sizes,
                                   void* out_s, float* lse2, const void* out_c, const void* gate, void* out,
                                   int64_t BH, int64_t Lq, int64_t Lkv, int64_t kv_shard, int D, int be, int topk,
                                   float scale, int dtype, void* stream);

/* vsa_sparse_bwd_dq_fused on shard-major K/V; dq_mean and q_sizes may both be NULL. */
int vsa_sparse_bwd_dq_sharded(const void* dout, const void* q, const void* k_sh, const void* v_sh,
                              const void* out_s, const float* lse2,
                              const int32_t* selected, const int32_t* kv_sizes,
                              float* delta, void* dq, const void* dq_mean, const int32_t* q_sizes,
                              int64_t BH, int64_t Lq, int64_t Lkv, int64_t kv_shard, int D, int be, int topk,
                              float scale, int dtype, void* stream);

/* vsa_sparse_bwd_dkdv_fused on shard-major K/V, writing shard-major dK/dV (this rank's partial sums over its
 * own query blocks, all Kb key blocks); dk_mean and dv_mean ([BH, Kb, D], global block order) may both be NULL. */
int vsa_sparse_bwd_dkdv_sharded(const void* dout, const void* q, const void* k_sh, const void* v_sh,
                                const float* lse2, const float* delta,
                                const int32_t* counts, const int32_t* offsets, const int32_t* inverse,
                                const int32_t* kv_sizes, void* dk_sh, void* dv_sh,
                                const void* dk_mean, const void* dv_mean,
                                int64_t BH, int64_t Lq, int64_t Lkv, int64_t kv_shard, int D, int be, int topk,
                                float scale, int dtype, void* stream);

/* dst[b, r, :] = map[r] >= 0 ? src[b, map[r], :] : 0 for rows of row_bytes bytes (even; 16-byte
 * multiples take the vector path).  With the maps of the tiling metadata this is the raster ->
 * zero-padded tile layout move and its inverse.
 * Replaces tile / untile: vsa/fastvideo_tiling.py:128-145. */
int vsa_gather_rows(const void* src, const int32_t* map, void* dst,
                    int64_t batch, int64_t src_rows, int64_t dst_rows, int64_t row_bytes, void* stream);

/* Which kernels the fine-attention entry points run for a shape in this process (environment switches included):
 * 2 = tcgen05/TMA (bf16 or fp16, D = 128, be = 64, 128 or 256, topk*ceil(be/64) <= 1024), 1 = warp-level mma.sync
 * (bf16 or fp16, D = 64 or 128, be = 64, 128 or 256), 0 = CUDA-core kernels (everything else the reference accepts,
 * and the fp32 validation mode).  No reference counterpart: its Triton launcher has one kernel family. */
int vsa_sparse_kernel_family(int D, int be, int topk, int dtype);

/* ---- raster-order activations: the tiling front end folded into the kernels --------------------------------
 * (No single reference counterpart: the reference tiles with index ops, vsa/fastvideo_tiling.py:128-145, and model
 * code transposes [B,S,H,D] to [B,H,L,D] around the operator.)  A model keeps q/k/v, the gate and the output as
 * [B, S, H, D] in raster (t, h, w) token order; the kernels read tile-order [B*H, L, D] operands.
 * vsa_gather_rows_heads builds an operand in one pass (row gather + head transpose + zero padding; to_tiled = 1:
 * dst [B,H,dst_rows,row] from src [B,src_rows,H,row] with dst row l = src row map[l] or zero where map[l] < 0;
 * to_tiled = 0: dst [B,dst_rows,H,row] from src [B,H,src_rows,row]; rows are multiples of 16 bytes).
 * The three *_raster entry points are vsa_sparse_fwd_combine / vsa_sparse_bwd_dq_fused / vsa_sparse_bwd_dkdv_fused
 * with one difference: the gate is read, and out / dq / dk / dv are written, at the token's raster row
 * (b*raster_rows + map[token])*heads + h of a [B, raster_rows, heads, D] tensor (BH = B*heads; map[token] < 0 is a
 * padding row: nothing is read or written for it).  q, k, v, dout, out_s stay tile-order.  Tensor path only
 * (vsa_sparse_raster_supported), VSA_ERR_UNSUPPORTED otherwise. */
int vsa_sparse_raster_supported(int D, int be, int topk, int dtype);

int vsa_gather_rows_heads(const void* src, const int32_t* map, void* dst,
                          int64_t batch, int heads, int64_t src_rows, int64_t dst_rows, int64_t row_bytes,
                          int to_tiled, void* stream);

int vsa_sparse_fwd_combine_raster(const void* q, const void* k, const void* v,
                                  const int32_t* selected, const int32_t* kv_sizes,
                                  void* out_s, float* lse2, const void* out_c,
                                  const void* gate_raster, void* out_raster,
                                  const int32_t* q_map, int64_t raster_rows, int heads,
                                  int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk,
                                  float scale, int dtype, void* stream);

/* vsa_combine_bwd for raster-order activations: dout_raster and gate_raster are [B, raster_rows, heads, D]; dgate is
 * written in that layout; dout_tiled [BH, Lq, D] receives dout in tile order (zeros in padding rows) for the two
 * entry points below.  gate_raster and dgate_raster may both be NULL.  Any dtype and head dim the plain form takes. */
int vsa_combine_bwd_raster(const void* dout_raster, const void* gate_raster, const void* out_c,
                           void* d_out_c, void* dgate_raster, void* dout_tiled,
                           const int32_t* q_map, int64_t raster_rows, int heads,
                           int64_t BH, int64_t Lq, int D, int be, int dtype, void* stream);

int vsa_sparse_bwd_dq_raster(const void* dout, const void* q, const void* k, const void* v,
                             const void* out_s, const float* lse2,
                             const int32_t* selected, const int32_t* kv_sizes,
                             float* delta, void* dq_raster, const void* dq_mean, const int32_t* q_sizes,
                             const int32_t* q_map, int64_t raster_rows, int heads,
                             int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk,
                             float scale, int dtype, void* stream);

int vsa_sparse_bwd_dkdv_raster(const void* dout, const void* q, const void* k, const void* v,
                               const float* lse2, const float* delta,
                               const int32_t* counts, const int32_t* offsets, const int32_t* inverse,
                               const int32_t* kv_sizes, void* dk_raster, void* dv_raster,
                               const void* dk_mean, const void* dv_mean,
                               const int32_t* kv_map, int64_t raster_rows, int heads,
                               int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk,
                               float scale, int dtype, void* stream);

/* out = out_s + out_c[block] * gate (gate may be NULL) in fp32, one rounding.
 * Replaces _combine_forward_kernel: vsa/fused_common.py:175-199,259-295. */
int vsa_combine_fwd(const void* out_s, const void* out_c, const void* gate, void* out,
                    int64_t BH, int64_t Lq, int D, int be, int dtype, void* stream);

/* Combine backward in one pass over dout: d_out_c[block] = sum over all be
 * rows of dout*gate, dgate = dout * out_c[block] (dgate/gate may be NULL).
 * Replaces _combine_coarse_backward_kernel + _combine_gate_backward_kernel:
 * vsa/fused_common.py:202-256,297-337. */
int vsa_combine_bwd(const void* dout, const void* gate, const void* out_c,
                    void* d_out_c, void* dgate,
                    int64_t BH, int64_t Lq, int D, int be, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* VSA_B200_H_ */
