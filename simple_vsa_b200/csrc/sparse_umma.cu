// Fine (block-sparse) attention forward on the Blackwell tensor path: TMA tile gathers by
// block id, tcgen05.mma with accumulators in tensor memory, warp-specialised softmax.
//
// Formulation.  A 64-row query tile gives only M = 64 for the usual S = Q K^T product, which
// runs tcgen05 at half rate.  The kernel therefore computes the TRANSPOSED products on PAIRS of
// selected key tiles:
//     S^T [128 key tokens x 64 query rows] = K2 [128 x 128] * Q^T          (M 128, N 64, K 128)
//     O^T [128 dims       x 64 query rows] += V2^T [128 x 128] * P^T       (M 128, N 64, K 128)
// K2/V2 are two 64-token tiles stacked in shared memory by four TMA boxes each.  In tensor
// memory a lane is then a key token and a column a query row, so the softmax statistics run
// ACROSS lanes.  They are handled without per-tile cross-lane traffic:
//   * the shift m[q] is the exact column maximum of the FIRST live pair only (one cross-lane
//     reduction per CTA); softmax is shift-invariant, so any later score simply gives
//     P = 2^(s-m) > 1, which bf16 and fp32 hold up to 2^127;
//   * every thread keeps its own partial row sums (64 registers) and they are reduced across
//     lanes once at the end;
//   * if a sum or an output leaves the finite range (scores more than ~2^7 apart in log2
//     units from the first pair's maximum) the tile writes NaN into its log-sum-exp rows and
//     the exact warp-level kernel recomputes just those tiles in a follow-up launch.
// P^T is written by its owner thread as one swizzled 128-byte row of shared memory (N-major B
// operand), so no transposition is ever needed.
//
// Roles: warp 0 = K producer, warp 1 = V producer (four lanes, one TMA box each; warp 1 also owns the
// tensor memory), warp 2 = issuer of the S^T MMAs, warp 3 = issuer of the O^T MMAs, warps 4-19 = softmax (a TMEM lane quarter and half of the
// query-row columns each).  Every mbarrier wait is bounded; on a time-out the CTA records an error code in a
// device status word, stops issuing work, frees its tensor memory and returns.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "kernels.h"
#include "umma.cuh"

namespace vsa {

__device__ int g_device_status = 0;

namespace {

using bf16 = __nv_bfloat16;
using namespace umma;

constexpr int kD = 128;
constexpr int kTile = 64;
constexpr int kMaxTiles = 1024;        // live 64-token key tiles per query tile the list can hold
constexpr int kSlab = 64 * 128;        // one TMA box: 64 rows x 128 bytes
constexpr int kPairHalf = 2 * kSlab;   // 128 rows x 128 bytes (one head-dim half of a stacked pair)
constexpr int kPairBytes = 2 * kPairHalf;
constexpr uint32_t kTmemCols = 512;
// K pairs in flight: a reload from L2 takes ~2000 cycles, two stages left the S^T issuer waiting for it
constexpr int kFwdKStages = 2;
constexpr int kSBufs = 4;              // S^T accumulators in flight (64 columns each); O^T sits behind them

// ---- host: tensor maps ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// [rows, cols] row-major of a 16-bit element type (cols = 128: q/k/v-like tensors; cols = 64: stored dS tiles), boxes of 64 rows x 64
// columns, 128-byte swizzle.
int make_map_of(CUtensorMap* map, CUtensorMapDataType elem, const void* ptr, int64_t rows, const char* what, int cols = kD) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(VSA_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled is not available from the driver", what);
  if (reinterpret_cast<uintptr_t>(ptr) % 16) return fail(VSA_ERR_BAD_ARGUMENT, "%s: pointer is not 16-byte aligned", what);
  if (rows > 0x7fffffffLL) return fail(VSA_ERR_UNSUPPORTED, "%s: %lld rows exceed the TMA coordinate range", what, (long long)rows);
  const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {64, 64};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, elem, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(VSA_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled failed with code %d", what, (int)r);
  return VSA_OK;
}

__device__ __forceinline__ void report_timeout(int code) { atomicCAS(&g_device_status, 0, code); }
// all waits of this file poll the status word so that a failure anywhere drains the grid quickly
#define VSA_WAIT(bar_, parity_) mbar_wait((bar_), (parity_), &g_device_status)
#define VSA_WARP_WAIT(bar_, parity_) warp_wait((bar_), (parity_), &g_device_status, lane)
#define VSA_WARP_WAIT2(a_, pa_, b_, pb_) warp_wait2((a_), (pa_), (b_), (pb_), &g_device_status, lane)
#define VSA_WARP_WAIT_TEST(a_, pa_, b_, pb_, done_) warp_wait_and_test((a_), (pa_), (b_), (pb_), &g_device_status, lane, (done_))

// One 64x128 tile = two boxes (head-dim halves); `dst` is the row offset inside a stacked pair.
__device__ __forceinline__ void load_tile(uint32_t pair_base, int half_rows_off, const CUtensorMap* map, int row,
                                          uint32_t bar) {
  tma_load_2d(pair_base + half_rows_off, map, 0, row, bar);
  tma_load_2d(pair_base + kPairHalf + half_rows_off, map, 64, row, bar);
}

// ---- descriptor / TMEM self-test ---------------------------------------------------------------------
// mode 0: D[128x64] = A[128 x 128 (k contiguous)] * B[64 x 128 (k contiguous)]^T
// mode 1: D[128x64] = A[128 k x 128 m (m contiguous)]^T * B[128 k x 64 n (n contiguous)], B written by threads
__global__ void __launch_bounds__(128) umma_selftest_kernel(const __grid_constant__ CUtensorMap map_a,
                                                            const __grid_constant__ CUtensorMap map_b,
                                                            const bf16* __restrict__ b_raw, float* __restrict__ out,
                                                            int mode) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sA = base, sB = base + kPairBytes;
  const uint32_t bar_load = base + kPairBytes + 16384, bar_mma = bar_load + 8, tmem_slot = bar_load + 16;
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    mbar_init(bar_load, 1);
    mbar_init(bar_mma, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 64);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(base_ptr + kPairBytes + 16384 + 16);
  bool ok = true;
  if (mode == 1) {   // B rows written by their owner thread as swizzled 128-byte rows
    const uint4* src = reinterpret_cast<const uint4*>(b_raw + tid * 64);
#pragma unroll
    for (int c = 0; c < 8; ++c)
      *reinterpret_cast<uint4*>(base_ptr + kPairBytes + tid * 128 + ((c ^ (tid & 7)) << 4)) = src[c];
    fence_proxy_async_smem();
  }
  __syncthreads();
  if (tid == 0) {
    const uint32_t bytes = kPairBytes + (mode == 0 ? 2 * kSlab : 0);
    mbar_arrive_expect_tx(bar_load, bytes);
    load_tile(sA, 0, &map_a, 0, bar_load);
    load_tile(sA, kSlab, &map_a, 64, bar_load);
    if (mode == 0) {
      tma_load_2d(sB, &map_b, 0, 0, bar_load);
      tma_load_2d(sB + kSlab, &map_b, 64, 0, bar_load);
    }
    ok = VSA_WAIT(bar_load, 0);
    if (ok) {
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        if (mode == 0) {
          const uint32_t off = (ks >> 2) * kPairHalf + (ks & 3) * 32;
          const uint32_t offb = (ks >> 2) * kSlab + (ks & 3) * 32;
          mma_ss(tmem, smem_desc(sA + off, 16, 1024), smem_desc(sB + offb, 16, 1024), instr_desc(128, 64, 0, 0), ks > 0);
        } else {
          mma_ss(tmem, smem_desc(sA + ks * 2048, kPairHalf, 1024), smem_desc(sB + ks * 2048, 16, 1024),
                 instr_desc(128, 64, 1, 1), ks > 0);
        }
      }
      mma_commit(bar_mma);
    } else {
      report_timeout(101);
    }
  }
  __syncthreads();
  if (VSA_WAIT(bar_mma, 0)) {
    tc_fence_after();
    uint32_t r[32];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + half * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) out[tid * 64 + half * 32 + j] = __uint_as_float(r[j]);
    }
  } else {
    report_timeout(102);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 64);
}

// ---- bounded-wait self-test ---------------------------------------------------------------------------
// One warp waits, with a caller-chosen limit, on a barrier that nothing will ever arrive at.  The wait must give
// up, the code must land in the device status word, and the kernel must return normally: the path every product
// kernel takes when a producer or a tensor-core commit fails to show up, exercised without making anything fail.
constexpr int kSelftestTimeoutCode = 201;
__global__ void __launch_bounds__(32) wait_timeout_selftest_kernel(unsigned long long limit_ns, int* __restrict__ gave_up) {
  __shared__ __align__(8) unsigned long long bar_storage;
  const uint32_t bar = smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    fence_barrier_init();
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    const bool ok = mbar_wait(bar, 0, &g_device_status, limit_ns);
    if (!ok) report_timeout(kSelftestTimeoutCode);
    *gave_up = ok ? 0 : 1;
  }
}

// [batch, rows, cols] row-major of a 16-bit element type; boxes of 64 columns x box_rows rows of one batch slice, 128-byte swizzle.
int make_map3d_of(CUtensorMap* map, CUtensorMapDataType elem, const void* ptr, int64_t batch, int64_t rows, int64_t cols, int box_rows,
               const char* what) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(VSA_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled is not available from the driver", what);
  if (reinterpret_cast<uintptr_t>(ptr) % 16 || (cols * 2) % 16)
    return fail(VSA_ERR_BAD_ARGUMENT, "%s: pointer or row pitch is not 16-byte aligned", what);
  const cuuint64_t gdim[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  const cuuint64_t gstride[2] = {(cuuint64_t)cols * 2, (cuuint64_t)rows * cols * 2};
  const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(map, elem, 3, const_cast<void*>(ptr), gdim, gstride, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(VSA_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled failed with code %d", what, (int)r);
  return VSA_OK;
}

template <typename Kern>
int reserve_smem(Kern kern, int bytes, const char* what) {
  const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return fail(VSA_ERR_LAUNCH, "%s: shared memory: %s", what, cudaGetErrorString(e));
  return VSA_OK;
}

int check_kv_shard(int64_t Lkv, int be, int64_t* kv_shard, const char* what) {
  if (*kv_shard <= 0) *kv_shard = Lkv;
  if (Lkv % *kv_shard || *kv_shard % be)
    return fail(VSA_ERR_BAD_ARGUMENT, "%s: the K/V shard length %lld must divide Lkv = %lld and be a multiple of the block volume %d",
                what, (long long)*kv_shard, (long long)Lkv, be);
  return VSA_OK;
}

}  // namespace

// A logical block of 64, 128 or 256 tokens is walked as 1, 2 or 4 tiles of 64 tokens (the kernels' SUB parameter).
#define VSA_BY_BLOCK_VOLUME(be_, launch_, kernel_) \
  return (be_) == 64 ? launch_(kernel_<1>) : (be_) == 128 ? launch_(kernel_<2>) : launch_(kernel_<4>)

// The kernels exist once per 16-bit element type: same code, other input format in the instruction descriptor and
// the tensor maps, other conversions in the epilogues.
namespace tc_bf16 {
using elem_t = __nv_bfloat16;
constexpr uint32_t kInFmt = 1u;
constexpr CUtensorMapDataType kTmaElem = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
constexpr int kDtypeCode = VSA_BF16;
constexpr float kShiftBias = 0.f;
#include "sparse_umma_typed.inl"
}  // namespace tc_bf16
namespace tc_f16 {
using elem_t = __half;
constexpr uint32_t kInFmt = 0u;
constexpr CUtensorMapDataType kTmaElem = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
constexpr int kDtypeCode = VSA_F16;
// The forward's fixed softmax shift is the first pair's column maximum plus this many binades, so that P = 2^(s - shift)
// of the first pair tops out at 2^-4: fp16 then holds later scores up to 20 binades (13.9 nats) above the first pair's
// maximum before P overflows (and the tile goes to the exact kernel) and keeps scores down to 20 binades below it --
// the middle of fp16's 2^-24 .. 2^16 instead of its top.  The row sum uses the same shift, so O/l and the saved
// statistic are unchanged.  bf16 has 2^127 above the first pair's maximum and needs no bias.
constexpr float kShiftBias = 4.f;
#include "sparse_umma_typed.inl"
}  // namespace tc_f16

#define VSA_BY_DTYPE(dtype_, call_) ((dtype_) == VSA_F16 ? tc_f16::call_ : tc_bf16::call_)

// ---- host entry points ---------------------------------------------------------------------------------------
bool sparse_umma_eligible(int D, int be, int dtype, int topk) {
  if ((dtype != VSA_BF16 && dtype != VSA_F16) || D != 128) return false;
  if (be == 64 || be == 128 || be == 256) return topk * (be / kTile) <= kMaxTiles;
  return false;
}

int64_t sparse_ds_workspace_bytes(int64_t BH, int64_t Lq, int be, int topk) {
  const int64_t sub = be / kTile;
  return BH * (Lq / be) * topk * sub * sub * (int64_t)(kTile * kTile * 2);
}

int sparse_fwd_umma(const void* q, const void* k, const void* v, const int32_t* selected, const int32_t* kv_sizes,
                    void* out, float* lse2, int64_t BH, int64_t Lq, int64_t Lkv, int be, int topk, float scale,
                    int dtype, cudaStream_t st, const void* out_c, const void* gate, void* out_comb, int64_t kv_shard,
                    const int32_t* comb_map, int64_t comb_rows, int comb_heads) {
  const RasterMap rm{comb_map, (long long)comb_rows, comb_heads > 0 ? comb_heads : 1};
  return VSA_BY_DTYPE(dtype, sparse_fwd_umma(q, k, v, selected, kv_sizes, out, lse2, BH, Lq, Lkv, be, topk, scale, st,
                                             out_c, gate, out_comb, kv_shard, rm));
}

int sparse_dq_umma(const void* dout, const void* q, const void* k, const void* v, const void* out_s,
                   const float* lse2, const int32_t* selected, const int32_t* kv_sizes, float* delta, void* dq,
                   int64_t BH, int64_t Lq, int64_t Lkv, int be, int topk, float scale, int dtype, cudaStream_t st,
                   const void* dq_mean, const int32_t* q_sizes, int64_t kv_shard, const int32_t* out_map,
                   int64_t out_rows, int out_heads) {
  const RasterMap rm{out_map, (long long)out_rows, out_heads > 0 ? out_heads : 1};
  return VSA_BY_DTYPE(dtype, sparse_dq_umma(dout, q, k, v, out_s, lse2, selected, kv_sizes, delta, dq, BH, Lq, Lkv, be,
                                            topk, scale, st, dq_mean, q_sizes, kv_shard, rm));
}

int sparse_dkdv_umma(const void* dout, const void* q, const void* k, const void* v, const float* lse2,
                     const float* delta, const int32_t* counts, const int32_t* offsets, const int32_t* inverse,
                     const int32_t* kv_sizes, void* dk, void* dv, int64_t BH, int64_t Lq, int64_t Lkv, int be, int topk,
                     float scale, int dtype, cudaStream_t st, const void* dk_mean, const void* dv_mean, void* ds_ws,
                     int64_t kv_shard, const int32_t* out_map, int64_t out_rows, int out_heads) {
  const RasterMap rm{out_map, (long long)out_rows, out_heads > 0 ? out_heads : 1};
  return VSA_BY_DTYPE(dtype, sparse_dkdv_umma(dout, q, k, v, lse2, delta, counts, offsets, inverse, kv_sizes, dk, dv, BH,
                                              Lq, Lkv, be, topk, scale, st, dk_mean, dv_mean, ds_ws, kv_shard, rm));
}

int sparse_dq_from_ds_umma(const void* k, const int32_t* selected, const int32_t* kv_sizes, const void* ds_ws, void* dq,
                           int64_t BH, int64_t Lq, int64_t Lkv, int be, int topk, float scale, int dtype,
                           cudaStream_t st, const void* dq_mean, const int32_t* q_sizes) {
  return VSA_BY_DTYPE(dtype, sparse_dq_from_ds_umma(k, selected, kv_sizes, ds_ws, dq, BH, Lq, Lkv, be, topk, scale, st,
                                                    dq_mean, q_sizes));
}

// ---- pooled attention on tcgen05 ---------------------------------------------------------------------------
bool coarse_umma_eligible(int Qb, int Kb, int D, int dtype) {
  // head dim 64: the same kernel, the second 64-column box of a 128-wide tile lies outside the tensor and is zero-filled
  return (dtype == VSA_BF16 || dtype == VSA_F16) && (D == 128 || D == 64) && Qb % 8 == 0 && Kb % 8 == 0;
}

int coarse_fwd_umma(const void* qc, const void* kc, const void* vc, void* scores, void* probs, void* out_c, int64_t BH,
                    int Qb, int Kb, int D, float scale, int dtype, cudaStream_t st) {
  return VSA_BY_DTYPE(dtype, coarse_fwd_umma(qc, kc, vc, scores, probs, out_c, BH, Qb, Kb, D, scale, st));
}

int coarse_bwd_umma(const void* d_out_c, const void* out_c, const void* qc, const void* kc, const void* vc,
                    const void* probs, void* ds, float* rowdot, void* dqc, void* dkc, void* dvc, int64_t BH, int Qb,
                    int Kb, int D, float scale, int dtype, cudaStream_t st) {
  return VSA_BY_DTYPE(dtype, coarse_bwd_umma(d_out_c, out_c, qc, kc, vc, probs, ds, rowdot, dqc, dkc, dvc, BH, Qb, Kb, D,
                                             scale, st));
}

int umma_selftest(const void* a, const void* b, float* out, int mode, cudaStream_t st) {
  CUtensorMap ma, mb;
  int rc;
  if ((rc = make_map_of(&ma, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a, 128, "selftest (a)"))) return rc;
  if ((rc = make_map_of(&mb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, mode == 0 ? b : a, mode == 0 ? 64 : 128, "selftest (b)"))) return rc;
  const int smem = kPairBytes + 16384 + 64 + 1024;
  const cudaError_t e = cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return fail(VSA_ERR_LAUNCH, "selftest: shared memory: %s", cudaGetErrorString(e));
  umma_selftest_kernel<<<1, 128, smem, st>>>(ma, mb, (const bf16*)b, out, mode);
  return check_launch("umma_selftest_kernel");
}

int wait_timeout_selftest(unsigned long long limit_ns, int* gave_up, cudaStream_t st) {
  wait_timeout_selftest_kernel<<<1, 32, 0, st>>>(limit_ns, gave_up);
  return check_launch("wait_timeout_selftest_kernel");
}

int device_status_fetch_and_clear(int* status) {
  int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(status, g_device_status, sizeof(int));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
  if (e != cudaSuccess) return fail(VSA_ERR_LAUNCH, "device status: %s", cudaGetErrorString(e));
  return VSA_OK;
}

}  // namespace vsa
