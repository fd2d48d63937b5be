// Tensor-path kernels and their launchers for ONE 16-bit element type.  The including file opens a namespace,
// defines there
//     elem_t      the element type (__nv_bfloat16 or __half),
//     kInFmt      its code in the tcgen05 instruction descriptor (1 = bf16, 0 = fp16),
//     kTmaElem    its CUtensorMapDataType,
//     kDtypeCode  its VSA_* dtype code,
//     kShiftBias  binades added to the forward's fixed softmax shift (centres P in the type's exponent range),
// and includes this file; everything else (tiling, barriers, pipelines, tensor-memory use) is the same for both.
int make_map(CUtensorMap* map, const void* ptr, int64_t rows, const char* what, int cols = kD) {
  return make_map_of(map, kTmaElem, ptr, rows, what, cols);
}
int make_map3d(CUtensorMap* map, const void* ptr, int64_t batch, int64_t rows, int64_t cols, int box_rows, const char* what) {
  return make_map3d_of(map, kTmaElem, ptr, batch, rows, cols, box_rows, what);
}

// 8 MMAs over the 128-wide reduction, both operands reduction-contiguous ("K-major").
// a_pair: a stacked pair [2 halves][128 rows][128 B]; b_tile: one tile [2 halves][64 rows][128 B].
// Descriptors are advanced with one 32-bit add each (offsets in 16-byte units are compile-time constants).
__device__ __forceinline__ void issue_kmajor(uint32_t d_tmem, uint32_t a_pair, uint32_t b_tile) {
  constexpr uint32_t idesc = instr_desc(128, 64, 0, 0, kInFmt);
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
  constexpr uint32_t idesc = instr_desc(128, 64, 1, 1, kInFmt);
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
                       const int32_t* __restrict__ kv_sizes, elem_t* __restrict__ out, float* __restrict__ lse2,
                       const elem_t* __restrict__ out_c, const elem_t* __restrict__ gate, elem_t* __restrict__ out_comb,
                       long long Lq, long long Lkv, long long kv_shard, int topk, float scale, RasterMap comb_map) {
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
        if (st < 64) m_col[st] = fmaxf(fmaxf(m_warp[st], m_warp[64 + st]), fmaxf(m_warp[128 + st], m_warp[192 + st])) + kShiftBias;
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
        packed[2 * j4] = Elem<elem_t>::pack(p0, p1);
        packed[2 * j4 + 1] = Elem<elem_t>::pack(p2, p3);
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
    elem_t* stage = reinterpret_cast<elem_t*>(sm + FwdSmem::k);     // [64 query rows][128 dims], all MMAs are done
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
        stage[qi * kD + t] = Elem<elem_t>::from(o);
      }
    } else {
      for (int j = 0; j < kEwCols; ++j) stage[(c0 + j) * kD + t] = Elem<elem_t>::from(n_pairs == 0 ? NAN : 0.f);
    }
    // vote across the softmax threads through shared memory
    volatile uint32_t* flag = misc + 2;
    if (!finite) *flag = 1u;
    named_barrier(1, kEwThreads);
    const bool redo = (*flag != 0u) && ok;
    const long long row0 = bh * Lq + (long long)qtile * kTile;
    elem_t* og = out + row0 * kD;
#pragma unroll
    for (int i = 0; i < 1024 / kEwThreads; ++i) {
      const int cidx = st + kEwThreads * i;         // 1024 chunks of 16 bytes
      const int row = cidx >> 4, ch = cidx & 15;
      const uint4 sv = *reinterpret_cast<const uint4*>(stage + row * kD + ch * 8);
      *reinterpret_cast<uint4*>(og + row * kD + ch * 8) = sv;
      if (out_comb != nullptr) {   // gated combine with the pooled branch on the way out (the fine output is kept: delta needs it)
        const uint4 cv = *reinterpret_cast<const uint4*>(out_c + (bh * Qb + qb) * (long long)kD + ch * 8);
        uint4 gv = make_uint4(0, 0, 0, 0);
        // with a raster map the gate is read, and the combined output written, at the token's raster row
        const long long crow = comb_map.map == nullptr ? row0 + row : raster_row(comb_map, bh, (long long)qtile * kTile + row);
        if (crow >= 0) {
          if (gate != nullptr) gv = *reinterpret_cast<const uint4*>(gate + crow * kD + ch * 8);
          *reinterpret_cast<uint4*>(out_comb + crow * kD + ch * 8) = combine_x8<elem_t>(sv, cv, gv, gate != nullptr);
        }
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

// ---- host launchers of this element type ----------------------------------------------------------------------
int sparse_fwd_umma(const void* q, const void* k, const void* v, const int32_t* selected, const int32_t* kv_sizes,
                    void* out, float* lse2, int64_t BH, int64_t Lq, int64_t Lkv, int be, int topk, float scale,
                    cudaStream_t st, const void* out_c, const void* gate, void* out_comb, int64_t kv_shard,
                    RasterMap comb_map) {
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
      kern<<<ctas, kFwdPThreads, psmem, st>>>(mq, mk, mv, selected, kv_sizes, (elem_t*)out, lse2, (const elem_t*)out_c,
                                              (const elem_t*)gate, (elem_t*)out_comb, (long long)BH, Lq, Lkv, kv_shard, topk, scale,
                                              comb_map);
      return check_launch("sparse_fwd_umma_persistent_kernel");
    };
    VSA_BY_BLOCK_VOLUME(be, launch, sparse_fwd_umma_persistent_kernel);
  }
  const int smem = FwdSmem::total + 1024;
  dim3 grid((unsigned)(Lq / kTile), (unsigned)BH);
  auto launch = [&](auto kern) -> int {
    if ((rc = reserve_smem(kern, smem, "sparse forward"))) return rc;
    kern<<<grid, kFwdThreads, smem, st>>>(mq, mk, mv, selected, kv_sizes, (elem_t*)out, lse2, (const elem_t*)out_c,
                                          (const elem_t*)gate, (elem_t*)out_comb, Lq, Lkv, kv_shard, topk, scale, comb_map);
    return check_launch("sparse_fwd_umma_kernel");
  };
  VSA_BY_BLOCK_VOLUME(be, launch, sparse_fwd_umma_kernel);
}

int sparse_dq_umma(const void* dout, const void* q, const void* k, const void* v, const void* out_s,
                   const float* lse2, const int32_t* selected, const int32_t* kv_sizes, float* delta, void* dq,
                   int64_t BH, int64_t Lq, int64_t Lkv, int be, int topk, float scale, cudaStream_t st,
                   const void* dq_mean, const int32_t* q_sizes, int64_t kv_shard, RasterMap out_map) {
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
  auto launch = [&](auto kern) -> int {
    if ((rc = reserve_smem(kern, smem, "sparse dQ"))) return rc;
    kern<<<grid, kBwdThreads, smem, st>>>(mq, mdo, mk, mv, (const elem_t*)dout, (const elem_t*)out_s, lse2, selected, kv_sizes,
                                          delta, (elem_t*)dq, (const elem_t*)dq_mean, q_sizes, Lq, Lkv, kv_shard, topk, scale,
                                          out_map);
    return check_launch("sparse_dq_umma_kernel");
  };
  VSA_BY_BLOCK_VOLUME(be, launch, sparse_dq_umma_kernel);
}

int sparse_dkdv_umma(const void* dout, const void* q, const void* k, const void* v, const float* lse2,
                     const float* delta, const int32_t* counts, const int32_t* offsets, const int32_t* inverse,
                     const int32_t* kv_sizes, void* dk, void* dv, int64_t BH, int64_t Lq, int64_t Lkv, int be, int topk,
                     float scale, cudaStream_t st, const void* dk_mean, const void* dv_mean, void* ds_ws,
                     int64_t kv_shard, RasterMap out_map) {
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
    kern<<<grid, kBwdThreads, smem, st>>>(mq, mdo, mk, mv, lse2, delta, counts, offsets, inverse, kv_sizes, (elem_t*)dk,
                                          (elem_t*)dv, (const elem_t*)dk_mean, (const elem_t*)dv_mean, (elem_t*)ds_ws, Lq, Lkv,
                                          kv_shard, topk, scale, out_map);
    return check_launch("sparse_dkdv_umma_kernel");
  };
  if (be == 64) return ds_ws ? launch(sparse_dkdv_umma_kernel<1, true>) : launch(sparse_dkdv_umma_kernel<1, false>);
  if (be == 128) return ds_ws ? launch(sparse_dkdv_umma_kernel<2, true>) : launch(sparse_dkdv_umma_kernel<2, false>);
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
    kern<<<grid, kDsThreads, smem, st>>>(mk, (const elem_t*)ds_ws, selected, kv_sizes, (elem_t*)dq, (const elem_t*)dq_mean,
                                         q_sizes, Lq, Lkv, topk, scale);
    return check_launch("sparse_dq_from_ds_kernel");
  };
  VSA_BY_BLOCK_VOLUME(be, launch, sparse_dq_from_ds_kernel);
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
  kern<<<grid, 192, smem, st>>>(ma, mb, (elem_t*)C, M, N, K, scale, (const elem_t*)probs, rowdot);
  return check_launch(what);
}

int coarse_fwd_umma(const void* qc, const void* kc, const void* vc, void* scores, void* probs, void* out_c, int64_t BH,
                    int Qb, int Kb, int D, float scale, cudaStream_t st) {
  int rc = launch_gemm<0, 0, kEpiScores>(qc, Qb, D, kc, Kb, D, scores, BH, Qb, Kb, D, scale, nullptr, nullptr, st,
                                         "pooled scores");
  if (rc) return rc;
  if ((rc = softmax_rows(scores, probs, BH * Qb, Kb, kDtypeCode, st))) return rc;
  return launch_gemm<0, 1, kEpiStore>(probs, Qb, Kb, vc, Kb, D, out_c, BH, Qb, D, Kb, 1.f, nullptr, nullptr, st,
                                      "pooled output");
}

int coarse_bwd_umma(const void* d_out_c, const void* out_c, const void* qc, const void* kc, const void* vc,
                    const void* probs, void* ds, float* rowdot, void* dqc, void* dkc, void* dvc, int64_t BH, int Qb,
                    int Kb, int D, float scale, cudaStream_t st) {
  int rc = rowdot_rows(d_out_c, out_c, rowdot, BH * Qb, D, kDtypeCode, st);
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
