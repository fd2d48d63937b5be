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

// [rows, cols] bf16 row-major (cols = 128: q/k/v-like tensors; cols = 64: stored dS tiles), boxes of 64 rows x 64
// columns, 128-byte swizzle.
int make_map(CUtensorMap* map, const void* ptr, int64_t rows, const char* what, int cols = kD) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(VSA_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled is not available from the driver", what);
  if (reinterpret_cast<uintptr_t>(ptr) % 16) return fail(VSA_ERR_BAD_ARGUMENT, "%s: pointer is not 16-byte aligned", what);
  if (rows > 0x7fffffffLL) return fail(VSA_ERR_UNSUPPORTED, "%s: %lld rows exceed the TMA coordinate range", what, (long long)rows);
  const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t gstride[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {64, 64};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
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

// 8 MMAs over the 128-wide reduction, both operands reduction-contiguous ("K-major").
// a_pair: a stacked pair [2 halves][128 rows][128 B]; b_tile: one tile [2 halves][64 rows][128 B].
// Descriptors are advanced with one 32-bit add each (offsets in 16-byte units are compile-time constants).
__device__ __forceinline__ void issue_kmajor(uint32_t d_tmem, uint32_t a_pair, uint32_t b_tile) {
  constexpr uint32_t idesc = instr_desc(128, 64, 0, 0);
  constexpr uint32_t hi = desc_hi(1024);
  const uint32_t a0 = desc_lo(a_pair, 16), b0 = desc_lo(b_tile, 16);
#pragma unroll
  for (int ks = 0; ks < 8; ++ks)
    mma_ss(d_tmem, desc_pack(a0 + (uint32_t)(((ks >> 2) * kPairHalf + (ks & 3) * 32) >> 4), hi),
           desc_pack(b0 + (uint32_t)(((ks >> 2) * kSlab + (ks & 3) * 32) >> 4), hi), idesc, ks > 0 ? 1u : 0u);
}
// 8 MMAs over 128 rows of reduction, both operands output-contiguous ("MN-major"):
// D[128 dims x 64] (+)= a_pair^T [128 dims x 128 rows] * b_rows [128 rows x 64].
__device__ __forceinline__ void issue_mnmajor(uint32_t d_tmem, uint32_t a_pair, uint32_t b_rows, bool accumulate) {
  constexpr uint32_t idesc = instr_desc(128, 64, 1, 1);
  constexpr uint32_t hi = desc_hi(1024);
  const uint32_t a0 = desc_lo(a_pair, kPairHalf), b0 = desc_lo(b_rows, 16);
  const uint32_t acc0 = accumulate ? 1u : 0u;
#pragma unroll
  for (int ks = 0; ks < 8; ++ks)
    mma_ss(d_tmem, desc_pack(a0 + (uint32_t)(ks * 128), hi), desc_pack(b0 + (uint32_t)(ks * 128), hi), idesc,
           ks > 0 ? 1u : acc0);
}

// ---- forward -------------------------------------------------------------------------------------------
struct FwdSmem {
  static constexpr uint32_t q = 0;                               // 16 KB
  static constexpr uint32_t k = q + 2 * kSlab;                   // 2 stages x 32 KB
  static constexpr uint32_t v = k + kFwdKStages * kPairBytes;    // 2 stages x 32 KB (K above: 3 stages)
  static constexpr uint32_t p = v + 2 * kPairBytes;              // 2 buffers x 16 KB
  static constexpr uint32_t tile_row = p + 2 * kPairHalf;        // int32 [kMaxTiles]
  static constexpr uint32_t tile_valid = tile_row + 4 * kMaxTiles;   // uint8 [kMaxTiles]
  static constexpr uint32_t m_warp = tile_valid + kMaxTiles;     // float [4 lane quarters][64]
  static constexpr uint32_t m_col = m_warp + 4 * 64 * 4;         // float [64]
  static constexpr uint32_t l_col = m_col + 64 * 4;              // float [64]
  static constexpr uint32_t bars = l_col + 64 * 4;               // 8-byte mbarriers
  static constexpr uint32_t misc = bars + 32 * 8;                // tmem base, n_live, flags
  static constexpr uint32_t total = misc + 64;
};
constexpr int kEwCols = 16;          // columns of a TMEM tile one elementwise thread owns
constexpr int kEwWarps = 4 * (64 / kEwCols);   // lane quarters x column groups = 16 warps
constexpr int kEwThreads = 32 * kEwWarps;
constexpr int kFwdThreads = 128 + kEwThreads;   // K producer, V producer, two MMA issuers, elementwise warps
enum FwdBar { Q_FULL = 0, K_FULL = 1, K_EMPTY = 4, V_FULL = 7, V_EMPTY = 9, P_FULL = 11, P_EMPTY = 13, O_FULL = 15,
              S_FULL = 16, S_EMPTY = 16 + kSBufs };

template <int SUB>
__global__ void __launch_bounds__(kFwdThreads, 1)
sparse_fwd_umma_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const int32_t* __restrict__ selected,
                       const int32_t* __restrict__ kv_sizes, bf16* __restrict__ out, float* __restrict__ lse2,
                       const bf16* __restrict__ out_c, const bf16* __restrict__ gate, bf16* __restrict__ out_comb,
                       long long Lq, long long Lkv, long long kv_shard, int topk, float scale) {
  extern __shared__ uint8_t smem_raw[];
  if (*(volatile int*)&g_device_status != 0) return;   // an earlier wait ran out: drain without touching anything
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qtile = blockIdx.x;
  const long long bh = blockIdx.y;
  const int Qb = (int)(Lq / (kTile * SUB));
  const int qb = qtile / SUB;
  const int32_t* sel = selected + (bh * Qb + qb) * (long long)topk;
  const int n_iter = topk * SUB;
  const float c = scale * kLog2e;

  int32_t* tile_row = reinterpret_cast<int32_t*>(sm + FwdSmem::tile_row);
  uint8_t* tile_valid = sm + FwdSmem::tile_valid;
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(sm + FwdSmem::misc);
  auto bar = [&](int i) -> uint32_t { return base + FwdSmem::bars + 8u * i; };

  // ---- set-up: barriers, tensor memory, the list of live key tiles ----
  if (tid == 0) {
    mbar_init(bar(Q_FULL), 1);
    for (int i = 0; i < kFwdKStages; ++i) {
      mbar_init(bar(K_FULL + i), 4);      // four producer lanes, one TMA box each
      mbar_init(bar(K_EMPTY + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(V_FULL + i), 4);
      mbar_init(bar(V_EMPTY + i), 1);
      mbar_init(bar(P_FULL + i), kEwWarps);      // one elected lane per softmax warp
      mbar_init(bar(P_EMPTY + i), 1);
    }
    for (int i = 0; i < kSBufs; ++i) {
      mbar_init(bar(S_FULL + i), 1);
      mbar_init(bar(S_EMPTY + i), kEwWarps);
    }
    mbar_init(bar(O_FULL), 1);
    misc[2] = 0u;
    fence_barrier_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
  }
  // every thread looks up some of the routed tiles (two dependent global loads, all in flight at once) ...
  for (int it = tid; it < n_iter; it += kFwdThreads) {
    const int kvb = sel[it / SUB];
    // an id outside the table is an empty tile, as route inversion treats it
    const int left = (unsigned)kvb < (unsigned)(Lkv / (kTile * SUB)) ? kv_sizes[kvb] - (it % SUB) * kTile : 0;
    tile_valid[it] = (uint8_t)(left < 0 ? 0 : (left > kTile ? kTile : left));
    tile_row[it] = left > 0 ? (int)kv_tensor_row(bh, gridDim.y, (long long)kvb * (kTile * SUB) + (it % SUB) * kTile, kv_shard) : 0;
  }
  __syncthreads();
  if (warp == 2) {   // ... then one warp squeezes out the empty ones in place, keeping the routing order
    int n_live = 0;
    for (int it0 = 0; it0 < n_iter; it0 += 32) {
      const int it = it0 + lane;
      const int valid = it < n_iter ? (int)tile_valid[it] : 0;
      const int row = it < n_iter ? tile_row[it] : 0;
      const unsigned live = __ballot_sync(0xffffffffu, valid > 0);
      __syncwarp();
      if (valid > 0) {
        const int pos = n_live + __popc(live & ((1u << lane) - 1u));
        tile_row[pos] = row;
        tile_valid[pos] = (uint8_t)valid;
      }
      n_live += __popc(live);
      __syncwarp();
    }
    if (lane == 0) misc[1] = (uint32_t)n_live;
  }
  if (warp == 1) {
    tmem_alloc(base + FwdSmem::misc, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = misc[0];
  const int n_live = (int)misc[1];
  const int n_pairs = (n_live + 1) >> 1;
  const uint32_t tmem_s0 = tmem, tmem_o = tmem + 64 * kSBufs;   // S^T buffers first, then O^T
  bool ok = true;

  if (warp == 0 || warp == 1) {
    // ================= TMA producers: warp 0 streams K pairs, warp 1 streams V pairs =================
    // Four lanes issue one 64-row x 128-byte box each (tile a/b x head-dim half 0/1), in lock step:
    // a single thread issuing all the boxes of a pair was the slowest stage of the pipeline.
    const bool is_k = warp == 0;
    if (is_k && lane == 0) {
      mbar_arrive_expect_tx(bar(Q_FULL), 2 * kSlab);
      const int qrow = (int)(bh * Lq + (long long)qtile * kTile);
      tma_load_2d(base + FwdSmem::q, &map_q, 0, qrow, bar(Q_FULL));
      tma_load_2d(base + FwdSmem::q + kSlab, &map_q, 64, qrow, bar(Q_FULL));
    }
    {
      const int which = lane & 1, dhalf = (lane >> 1) & 1;  // tile a or b of the pair; head-dim half
      const CUtensorMap* map = is_k ? &map_k : &map_v;
      const int full0 = is_k ? K_FULL : V_FULL, empty0 = is_k ? K_EMPTY : V_EMPTY;
      const uint32_t ring = base + (is_k ? FwdSmem::k : FwdSmem::v);
      const int depth = is_k ? kFwdKStages : 2;
      for (int p = 0; p < n_pairs; ++p) {
        const int s = p % depth;
        const uint32_t ph = (p / depth) & 1;
        int idx = 2 * p + which;
        if (idx >= n_live) idx = 2 * p;                     // odd tail: repeat the first tile (masked later)
        const int row = tile_row[idx];                        // row of the tile in the K/V tensors
        ok = VSA_WARP_WAIT(bar(empty0 + s), ph ^ 1);
        if (!ok) break;
        if (lane < 4) {
          mbar_arrive_expect_tx(bar(full0 + s), kSlab);
          tma_load_2d(ring + s * kPairBytes + dhalf * kPairHalf + which * kSlab, map, dhalf * 64, row, bar(full0 + s));
        }
      }
      if (!ok && lane == 0) report_timeout(1);
    }
  } else if (warp == 2) {
    // ================= MMA issuer 1: S^T = K2 Q^T, as far ahead as operands and accumulators allow =================
    if (lane == 0) {
      ok = VSA_WAIT(bar(Q_FULL), 0);
      for (int p = 0; p < n_pairs && ok; ++p) {
        const int s = p % kFwdKStages, b = p % kSBufs;
        ok = VSA_WAIT(bar(K_FULL + s), (p / kFwdKStages) & 1) && VSA_WAIT(bar(S_EMPTY + b), ((p / kSBufs) & 1) ^ 1);
        if (!ok) break;
        tc_fence_after();
        issue_kmajor(tmem_s0 + b * 64, base + FwdSmem::k + s * kPairBytes, base + FwdSmem::q);
        mma_commit(bar(K_EMPTY + s));
        mma_commit(bar(S_FULL + b));
      }
      if (!ok) report_timeout(2);
    }
  } else if (warp == 3) {
    // ================= MMA issuer 2: O^T += V2^T P^T =================
    if (lane == 0) {
      for (int j = 0; j < n_pairs && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        ok = VSA_WAIT(bar(V_FULL + s), ph);
        ok = ok && VSA_WAIT(bar(P_FULL + s), ph);
        if (!ok) break;
        tc_fence_after();
        issue_mnmajor(tmem_o, base + FwdSmem::v + s * kPairBytes, base + FwdSmem::p + s * kPairHalf, j > 0);
        mma_commit(bar(V_EMPTY + s));
        mma_commit(bar(P_EMPTY + s));
      }
      if (ok) mma_commit(bar(O_FULL));
      if (!ok) report_timeout(5);
    }
  } else if (warp >= 4) {
    // ================= softmax warps =================
    // warp -> (TMEM lane quarter = warp & 3, column group = (warp-4) >> 2): a thread owns one key token of
    // the stacked pair (lane t) and kEwCols of the 64 query rows (columns c0..c0+kEwCols-1).
    const int quarter = warp & 3;
    const int cg = (warp - 4) >> 2;
    const int c0 = cg * kEwCols;
    const int t = quarter * 32 + lane;
    const int half = t >> 6, r = t & 63;
    const int st = tid - 128;                     // index among the softmax threads
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    float* m_warp = reinterpret_cast<float*>(sm + FwdSmem::m_warp);
    float* m_col = reinterpret_cast<float*>(sm + FwdSmem::m_col);
    float* l_col = reinterpret_cast<float*>(sm + FwdSmem::l_col);
    float lsum[kEwCols];
#pragma unroll
    for (int j = 0; j < kEwCols; ++j) lsum[j] = 0.f;

    for (int p = 0; p < n_pairs && ok; ++p) {
      const int s = p & 1;
      const uint32_t ph = (p >> 1) & 1;
      const int idx = 2 * p + half;
      const int valid = idx < n_live ? (int)tile_valid[idx] : 0;
      const bool live = r < valid;
      const int sb = p % kSBufs;
      // the score accumulator and the free P buffer (released by the O^T MMA two pairs back) in one round trip
      ok = VSA_WARP_WAIT2(bar(S_FULL + sb), (p / kSBufs) & 1, bar(P_EMPTY + s), ph ^ 1);
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[kEwCols];
      tmem_ld(tmem_s0 + sb * 64 + lane_addr + c0, sv);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(S_EMPTY + sb));

      if (p == 0) {   // exact column maxima of the first live pair: warp shuffle, then across the lane quarters
#pragma unroll
        for (int j = 0; j < kEwCols; ++j) {
          const float x = warp_max(live ? __uint_as_float(sv[j]) * c : -INFINITY);
          if (lane == 0) m_warp[quarter * 64 + c0 + j] = x;
        }
        named_barrier(1, kEwThreads);
        if (st < 64) m_col[st] = fmaxf(fmaxf(m_warp[st], m_warp[64 + st]), fmaxf(m_warp[128 + st], m_warp[192 + st]));
        named_barrier(1, kEwThreads);
      }
      // padding rows of a ragged tile (and the repeated tile of an odd tail): whatever sits in V there
      // must not reach the tensor core, where 0 * NaN would poison the sum
      if (!live && cg == 0) {
        ok = VSA_WAIT(bar(V_FULL + s), ph);
        uint8_t* vrow = sm + FwdSmem::v + s * kPairBytes + t * 128;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          *reinterpret_cast<uint4*>(vrow + ch * 16) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(vrow + kPairHalf + ch * 16) = make_uint4(0, 0, 0, 0);
        }
      }
      ok = __all_sync(0xffffffffu, ok);     // keep the warp's control flow uniform
      if (!ok) break;
      uint32_t packed[kEwCols / 2];
#pragma unroll
      for (int j4 = 0; j4 < kEwCols / 4; ++j4) {
        const float4 m4 = *reinterpret_cast<const float4*>(m_col + c0 + 4 * j4);
        const float p0 = live ? fast_exp2(fmaf(__uint_as_float(sv[4 * j4 + 0]), c, -m4.x)) : 0.f;
        const float p1 = live ? fast_exp2(fmaf(__uint_as_float(sv[4 * j4 + 1]), c, -m4.y)) : 0.f;
        const float p2 = live ? fast_exp2(fmaf(__uint_as_float(sv[4 * j4 + 2]), c, -m4.z)) : 0.f;
        const float p3 = live ? fast_exp2(fmaf(__uint_as_float(sv[4 * j4 + 3]), c, -m4.w)) : 0.f;
        lsum[4 * j4 + 0] += p0; lsum[4 * j4 + 1] += p1; lsum[4 * j4 + 2] += p2; lsum[4 * j4 + 3] += p3;
        packed[2 * j4] = pack_bf16(p0, p1);
        packed[2 * j4 + 1] = pack_bf16(p2, p3);
      }
      uint8_t* prow = sm + FwdSmem::p + s * kPairHalf + t * 128;
#pragma unroll
      for (int ch = 0; ch < kEwCols / 8; ++ch)     // this thread's query rows are 16-byte chunks of row t
        *reinterpret_cast<uint4*>(prow + ((((kEwCols / 8) * cg + ch) ^ (t & 7)) << 4)) =
            make_uint4(packed[4 * ch], packed[4 * ch + 1], packed[4 * ch + 2], packed[4 * ch + 3]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(P_FULL + s));
    }
    if (!ok) report_timeout(3);

    // ---- epilogue: reduce the row sums across lanes (fixed order), normalise O^T, transpose via shared memory ----
#pragma unroll
    for (int j = 0; j < kEwCols; ++j) {
      const float x = warp_sum(lsum[j]);
      if (lane == 0) m_warp[quarter * 64 + c0 + j] = x;       // the maxima scratch is free by now
    }
    named_barrier(1, kEwThreads);
    if (st < 64) l_col[st] = (m_warp[st] + m_warp[64 + st]) + (m_warp[128 + st] + m_warp[192 + st]);
    named_barrier(1, kEwThreads);
    if (ok && n_pairs > 0) ok = VSA_WARP_WAIT(bar(O_FULL), 0);
    if (!ok) report_timeout(4);
    tc_fence_after();
    bool finite = true;
    bf16* stage = reinterpret_cast<bf16*>(sm + FwdSmem::k);     // [64 query rows][128 dims], all MMAs are done
    if (ok && n_pairs > 0) {
      uint32_t ov[kEwCols];
      tmem_ld(tmem_o + lane_addr + c0, ov);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < kEwCols; ++j) {
        const int qi = c0 + j;
        const float l = l_col[qi];
        const float o = __uint_as_float(ov[j]) / l;
        finite = finite && (fabsf(o) <= 3.0e38f) && (l <= 3.0e38f);
        stage[qi * kD + t] = __float2bfloat16_rn(o);
      }
    } else {
      for (int j = 0; j < kEwCols; ++j) stage[(c0 + j) * kD + t] = __float2bfloat16_rn(n_pairs == 0 ? NAN : 0.f);
    }
    // vote across the softmax threads through shared memory
    volatile uint32_t* flag = misc + 2;
    if (!finite) *flag = 1u;
    named_barrier(1, kEwThreads);
    const bool redo = (*flag != 0u) && ok;
    const long long row0 = bh * Lq + (long long)qtile * kTile;
    bf16* og = out + row0 * kD;
#pragma unroll
    for (int i = 0; i < 1024 / kEwThreads; ++i) {
      const int cidx = st + kEwThreads * i;         // 1024 chunks of 16 bytes
      const int row = cidx >> 4, ch = cidx & 15;
      const uint4 sv = *reinterpret_cast<const uint4*>(stage + row * kD + ch * 8);
      *reinterpret_cast<uint4*>(og + row * kD + ch * 8) = sv;
      if (out_comb != nullptr) {   // gated combine with the pooled branch on the way out (the fine output is kept: delta needs it)
        const uint4 cv = *reinterpret_cast<const uint4*>(out_c + (bh * Qb + qb) * (long long)kD + ch * 8);
        uint4 gv = make_uint4(0, 0, 0, 0);
        if (gate != nullptr) gv = *reinterpret_cast<const uint4*>(gate + (row0 + row) * kD + ch * 8);
        *reinterpret_cast<uint4*>(out_comb + (row0 + row) * kD + ch * 8) = combine_bf16x8(sv, cv, gv, gate != nullptr);
      }
    }
    if (st < 64) {
      const float l = l_col[st];
      lse2[bh * Lq + (long long)qtile * kTile + st] = (redo || n_pairs == 0) ? NAN : m_col[st] + log2f(l);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

#include "sparse_umma_fwd_persistent.inl"
#include "sparse_umma_bwd.inl"
#include "coarse_umma.inl"

}  // namespace

// ---- host entry points ---------------------------------------------------------------------------------------
bool sparse_umma_eligible(int D, int be, int dtype, int topk) {
  if (dtype != VSA_BF16 || D != 128) return false;
  if (be == 64) return topk <= kMaxTiles;
  if (be == 256) return topk * 4 <= kMaxTiles;
  return false;
}

template <typename Kern>
static int reserve_smem(Kern kern, int bytes, const char* what) {
  const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return fail(VSA_ERR_LAUNCH, "%s: shared memory: %s", what, cudaGetErrorString(e));
  return VSA_OK;
}

static int check_kv_shard(int64_t Lkv, int be, int64_t* kv_shard, const char* what) {
  if (*kv_shard <= 0) *kv_shard = Lkv;
  if (Lkv % *kv_shard || *kv_shard % be)
    return fail(VSA_ERR_BAD_ARGUMENT, "%s: the K/V shard length %lld must divide Lkv = %lld and be a multiple of the block volume %d",
                what, (long long)*kv_shard, (long long)Lkv, be);
  return VSA_OK;
}

int sparse_fwd_umma(const void* q, const void* k, const void* v, const int32_t* selected, const int32_t* kv_sizes,
                    void* out, float* lse2, int64_t BH, int64_t Lq, int64_t Lkv, int be, int topk, float scale,
                    cudaStream_t st, const void* out_c, const void* gate, void* out_comb, int64_t kv_shard) {
  if (BH == 0 || Lq == 0) return VSA_OK;
  { const int rc0 = check_kv_shard(Lkv, be, &kv_shard, "sparse forward"); if (rc0) return rc0; }
  if (BH > 65535) return fail(VSA_ERR_UNSUPPORTED, "sparse forward: batch*heads %lld exceeds 65535", (long long)BH);
  CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = make_map(&mq, q, BH * Lq, "sparse forward (q)"))) return rc;
  if ((rc = make_map(&mk, k, BH * Lkv, "sparse forward (k)"))) return rc;
  if ((rc = make_map(&mv, v, BH * Lkv, "sparse forward (v)"))) return rc;
  // Two schedules of the same arithmetic.  One CTA per query tile is faster when a tile walks many pairs (the
  // headline shape: 90); with short routes the per-CTA set-up and drain are a large share of a CTA's life and the
  // persistent form (one CTA per SM, next tile's list, loads and first S^T MMAs under the current tile's epilogue)
  // wins: measured -7 % at 16 pairs per tile, -9 % at 8, +1 % at 40, +4 % at 90.  VSA_B200_FWD=classic|persistent
  // overrides the choice.
  const char* fwd_env = std::getenv("VSA_B200_FWD");
  bool persistent = topk * (be / kTile) <= 48;
  if (fwd_env && std::strcmp(fwd_env, "persistent") == 0) persistent = true;
  if (fwd_env && std::strcmp(fwd_env, "classic") == 0) persistent = false;
  if (persistent) {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      return fail(VSA_ERR_LAUNCH, "sparse forward: cannot read the SM count of the current device");
    const long long items = (Lq / kTile) * BH;
    const unsigned ctas = (unsigned)std::min<long long>(items, sms);
    const int psmem = FwdPSmem::total + 1024;
    auto launch = [&](auto kern) -> int {
      if ((rc = reserve_smem(kern, psmem, "sparse forward"))) return rc;
      kern<<<ctas, kFwdPThreads, psmem, st>>>(mq, mk, mv, selected, kv_sizes, (bf16*)out, lse2, (const bf16*)out_c,
                                              (const bf16*)gate, (bf16*)out_comb, (long long)BH, Lq, Lkv, kv_shard, topk, scale);
      return check_launch("sparse_fwd_umma_persistent_kernel");
    };
    return be == 64 ? launch(sparse_fwd_umma_persistent_kernel<1>) : launch(sparse_fwd_umma_persistent_kernel<4>);
  }
  const int smem = FwdSmem::total + 1024;
  dim3 grid((unsigned)(Lq / kTile), (unsigned)BH);
  cudaError_t e;
  if (be == 64) {
    e = cudaFuncSetAttribute(sparse_fwd_umma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail(VSA_ERR_LAUNCH, "sparse forward: shared memory: %s", cudaGetErrorString(e));
    sparse_fwd_umma_kernel<1><<<grid, kFwdThreads, smem, st>>>(mq, mk, mv, selected, kv_sizes, (bf16*)out, lse2, (const bf16*)out_c,
                                                               (const bf16*)gate, (bf16*)out_comb, Lq, Lkv, kv_shard, topk, scale);
  } else {
    e = cudaFuncSetAttribute(sparse_fwd_umma_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail(VSA_ERR_LAUNCH, "sparse forward: shared memory: %s", cudaGetErrorString(e));
    sparse_fwd_umma_kernel<4><<<grid, kFwdThreads, smem, st>>>(mq, mk, mv, selected, kv_sizes, (bf16*)out, lse2, (const bf16*)out_c,
                                                               (const bf16*)gate, (bf16*)out_comb, Lq, Lkv, kv_shard, topk, scale);
  }
  return check_launch("sparse_fwd_umma_kernel");
}

int sparse_dq_umma(const void* dout, const void* q, const void* k, const void* v, const void* out_s,
                   const float* lse2, const int32_t* selected, const int32_t* kv_sizes, float* delta, void* dq,
                   int64_t BH, int64_t Lq, int64_t Lkv, int be, int topk, float scale, cudaStream_t st,
                   const void* dq_mean, const int32_t* q_sizes, int64_t kv_shard) {
  if (BH == 0 || Lq == 0) return VSA_OK;
  if (BH > 65535) return fail(VSA_ERR_UNSUPPORTED, "sparse dQ: batch*heads %lld exceeds 65535", (long long)BH);
  { const int rc0 = check_kv_shard(Lkv, be, &kv_shard, "sparse dQ"); if (rc0) return rc0; }
  CUtensorMap mq, mdo, mk, mv;
  int rc;
  if ((rc = make_map(&mq, q, BH * Lq, "sparse dQ (q)"))) return rc;
  if ((rc = make_map(&mdo, dout, BH * Lq, "sparse dQ (dout)"))) return rc;
  if ((rc = make_map(&mk, k, BH * Lkv, "sparse dQ (k)"))) return rc;
  if ((rc = make_map(&mv, v, BH * Lkv, "sparse dQ (v)"))) return rc;
  const int smem = DqSmem::total + 1024;
  dim3 grid((unsigned)(Lq / kTile), (unsigned)BH);
  if (be == 64) {
    if ((rc = reserve_smem(sparse_dq_umma_kernel<1>, smem, "sparse dQ"))) return rc;
    sparse_dq_umma_kernel<1><<<grid, kBwdThreads, smem, st>>>(mq, mdo, mk, mv, (const bf16*)dout, (const bf16*)out_s, lse2,
                                                              selected, kv_sizes, delta, (bf16*)dq, (const bf16*)dq_mean, q_sizes, Lq, Lkv,
                                                              kv_shard, topk, scale);
  } else {
    if ((rc = reserve_smem(sparse_dq_umma_kernel<4>, smem, "sparse dQ"))) return rc;
    sparse_dq_umma_kernel<4><<<grid, kBwdThreads, smem, st>>>(mq, mdo, mk, mv, (const bf16*)dout, (const bf16*)out_s, lse2,
                                                              selected, kv_sizes, delta, (bf16*)dq, (const bf16*)dq_mean, q_sizes, Lq, Lkv,
                                                              kv_shard, topk, scale);
  }
  return check_launch("sparse_dq_umma_kernel");
}

int64_t sparse_ds_workspace_bytes(int64_t BH, int64_t Lq, int be, int topk) {
  const int64_t sub = be / kTile;
  return BH * (Lq / be) * topk * sub * sub * (int64_t)(kTile * kTile * 2);
}

int sparse_dkdv_umma(const void* dout, const void* q, const void* k, const void* v, const float* lse2,
                     const float* delta, const int32_t* counts, const int32_t* offsets, const int32_t* inverse,
                     const int32_t* kv_sizes, void* dk, void* dv, int64_t BH, int64_t Lq, int64_t Lkv, int be, int topk,
                     float scale, cudaStream_t st, const void* dk_mean, const void* dv_mean, void* ds_ws,
                     int64_t kv_shard) {
  if (BH == 0 || Lkv == 0) return VSA_OK;
  if (BH > 65535) return fail(VSA_ERR_UNSUPPORTED, "sparse dK/dV: batch*heads %lld exceeds 65535", (long long)BH);
  { const int rc0 = check_kv_shard(Lkv, be, &kv_shard, "sparse dK/dV"); if (rc0) return rc0; }
  if (ds_ws && topk > (1 << kEdgeSlotBits))
    return fail(VSA_ERR_UNSUPPORTED, "sparse dK/dV: packed edges hold at most %d routes per query block", 1 << kEdgeSlotBits);
  CUtensorMap mq, mdo, mk, mv;
  int rc;
  if ((rc = make_map(&mq, q, BH * Lq, "sparse dK/dV (q)"))) return rc;
  if ((rc = make_map(&mdo, dout, BH * Lq, "sparse dK/dV (dout)"))) return rc;
  if ((rc = make_map(&mk, k, BH * Lkv, "sparse dK/dV (k)"))) return rc;
  if ((rc = make_map(&mv, v, BH * Lkv, "sparse dK/dV (v)"))) return rc;
  if (ds_ws && reinterpret_cast<uintptr_t>(ds_ws) % 16)
    return fail(VSA_ERR_BAD_ARGUMENT, "sparse dK/dV: the dS workspace is not 16-byte aligned");
  const int smem = DkSmem::total + 1024;
  dim3 grid((unsigned)(Lkv / kTile), (unsigned)BH);
  auto launch = [&](auto kern) -> int {
    if ((rc = reserve_smem(kern, smem, "sparse dK/dV"))) return rc;
    kern<<<grid, kBwdThreads, smem, st>>>(mq, mdo, mk, mv, lse2, delta, counts, offsets, inverse, kv_sizes, (bf16*)dk,
                                          (bf16*)dv, (const bf16*)dk_mean, (const bf16*)dv_mean, (bf16*)ds_ws, Lq, Lkv,
                                          kv_shard, topk, scale);
    return check_launch("sparse_dkdv_umma_kernel");
  };
  if (be == 64) return ds_ws ? launch(sparse_dkdv_umma_kernel<1, true>) : launch(sparse_dkdv_umma_kernel<1, false>);
  return ds_ws ? launch(sparse_dkdv_umma_kernel<4, true>) : launch(sparse_dkdv_umma_kernel<4, false>);
}

int sparse_dq_from_ds_umma(const void* k, const int32_t* selected, const int32_t* kv_sizes, const void* ds_ws, void* dq,
                           int64_t BH, int64_t Lq, int64_t Lkv, int be, int topk, float scale, cudaStream_t st,
                           const void* dq_mean, const int32_t* q_sizes) {
  if (BH == 0 || Lq == 0) return VSA_OK;
  if (BH > 65535) return fail(VSA_ERR_UNSUPPORTED, "sparse dQ: batch*heads %lld exceeds 65535", (long long)BH);
  if (reinterpret_cast<uintptr_t>(ds_ws) % 16)
    return fail(VSA_ERR_BAD_ARGUMENT, "sparse dQ: the dS workspace is not 16-byte aligned");
  CUtensorMap mk;
  int rc;
  if ((rc = make_map(&mk, k, BH * Lkv, "sparse dQ (k)"))) return rc;
  const int smem = DqdsSmem::total + 1024;
  dim3 grid((unsigned)(Lq / kTile), (unsigned)BH);
  auto launch = [&](auto kern) -> int {
    if ((rc = reserve_smem(kern, smem, "sparse dQ"))) return rc;
    kern<<<grid, kDsThreads, smem, st>>>(mk, (const bf16*)ds_ws, selected, kv_sizes, (bf16*)dq, (const bf16*)dq_mean,
                                         q_sizes, Lq, Lkv, topk, scale);
    return check_launch("sparse_dq_from_ds_kernel");
  };
  return be == 64 ? launch(sparse_dq_from_ds_kernel<1>) : launch(sparse_dq_from_ds_kernel<4>);
}

// ---- pooled attention on tcgen05 ---------------------------------------------------------------------------
namespace {
// [batch, rows, cols] bf16 row-major; boxes of 64 columns x box_rows rows of one batch slice, 128-byte swizzle.
int make_map3d(CUtensorMap* map, const void* ptr, int64_t batch, int64_t rows, int64_t cols, int box_rows,
               const char* what) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(VSA_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled is not available from the driver", what);
  if (reinterpret_cast<uintptr_t>(ptr) % 16 || (cols * 2) % 16)
    return fail(VSA_ERR_BAD_ARGUMENT, "%s: pointer or row pitch is not 16-byte aligned", what);
  const cuuint64_t gdim[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  const cuuint64_t gstride[2] = {(cuuint64_t)cols * 2, (cuuint64_t)rows * cols * 2};
  const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), gdim, gstride, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(VSA_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled failed with code %d", what, (int)r);
  return VSA_OK;
}

// C[batch, M, N] = A * B.  a_rows/a_cols and b_rows/b_cols describe the operands as stored in memory.
template <int A_MN, int B_MN, int EPI>
int launch_gemm(const void* A, int64_t a_rows, int64_t a_cols, const void* B, int64_t b_rows, int64_t b_cols, void* C,
                int64_t batch, int M, int N, int K, float scale, const void* probs, const float* rowdot,
                cudaStream_t st, const char* what) {
  if (batch == 0 || M == 0 || N == 0) return VSA_OK;
  if (batch > 65535) return fail(VSA_ERR_UNSUPPORTED, "%s: batch*heads %lld exceeds 65535", what, (long long)batch);
  CUtensorMap ma, mb;
  int rc;
  if ((rc = make_map3d(&ma, A, batch, a_rows, a_cols, A_MN ? 64 : 128, what))) return rc;
  if ((rc = make_map3d(&mb, B, batch, b_rows, b_cols, B_MN ? 64 : 128, what))) return rc;
  const int smem = GemmSmem::total + 1024;
  auto kern = coarse_gemm_umma_kernel<A_MN, B_MN, EPI>;
  if ((rc = reserve_smem(kern, smem, what))) return rc;
  dim3 grid((unsigned)((N + 127) / 128), (unsigned)((M + 127) / 128), (unsigned)batch);
  kern<<<grid, 192, smem, st>>>(ma, mb, (bf16*)C, M, N, K, scale, (const bf16*)probs, rowdot);
  return check_launch(what);
}
}  // namespace

bool coarse_umma_eligible(int Qb, int Kb, int D, int dtype) {
  return dtype == VSA_BF16 && D == 128 && Qb % 8 == 0 && Kb % 8 == 0;
}

int coarse_fwd_umma(const void* qc, const void* kc, const void* vc, void* scores, void* probs, void* out_c, int64_t BH,
                    int Qb, int Kb, int D, float scale, cudaStream_t st) {
  int rc = launch_gemm<0, 0, kEpiScores>(qc, Qb, D, kc, Kb, D, scores, BH, Qb, Kb, D, scale, nullptr, nullptr, st,
                                         "pooled scores");
  if (rc) return rc;
  if ((rc = softmax_rows(scores, probs, BH * Qb, Kb, VSA_BF16, st))) return rc;
  return launch_gemm<0, 1, kEpiStore>(probs, Qb, Kb, vc, Kb, D, out_c, BH, Qb, D, Kb, 1.f, nullptr, nullptr, st,
                                      "pooled output");
}

int coarse_bwd_umma(const void* d_out_c, const void* out_c, const void* qc, const void* kc, const void* vc,
                    const void* probs, void* ds, float* rowdot, void* dqc, void* dkc, void* dvc, int64_t BH, int Qb,
                    int Kb, int D, float scale, cudaStream_t st) {
  int rc = rowdot_rows(d_out_c, out_c, rowdot, BH * Qb, D, VSA_BF16, st);
  if (rc) return rc;
  // dV_c[Kb,D] = P^T dO_c : A = P stored [Qb rows (reduction), Kb cols (M)], B = dO_c stored [Qb rows, D cols]
  if ((rc = launch_gemm<1, 1, kEpiStore>(probs, Qb, Kb, d_out_c, Qb, D, dvc, BH, Kb, D, Qb, 1.f, nullptr, nullptr, st,
                                         "pooled dV")))
    return rc;
  // dS[Qb,Kb] = P * (dO_c v_c^T - rowdot) * scale
  if ((rc = launch_gemm<0, 0, kEpiSoftmaxBwd>(d_out_c, Qb, D, vc, Kb, D, ds, BH, Qb, Kb, D, scale, probs, rowdot, st,
                                              "pooled dS")))
    return rc;
  // dQ_c[Qb,D] = dS k_c
  if ((rc = launch_gemm<0, 1, kEpiStore>(ds, Qb, Kb, kc, Kb, D, dqc, BH, Qb, D, Kb, 1.f, nullptr, nullptr, st,
                                         "pooled dQ")))
    return rc;
  // dK_c[Kb,D] = dS^T q_c
  return launch_gemm<1, 1, kEpiStore>(ds, Qb, Kb, qc, Qb, D, dkc, BH, Kb, D, Qb, 1.f, nullptr, nullptr, st, "pooled dK");
}

int umma_selftest(const void* a, const void* b, float* out, int mode, cudaStream_t st) {
  CUtensorMap ma, mb;
  int rc;
  if ((rc = make_map(&ma, a, 128, "selftest (a)"))) return rc;
  if ((rc = make_map(&mb, mode == 0 ? b : a, mode == 0 ? 64 : 128, "selftest (b)"))) return rc;
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
