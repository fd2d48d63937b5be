// Backward of the fine attention on the Blackwell tensor path.  Included by sparse_umma.cu (same
// translation unit: the kernels share its device status word, tensor-map helper and constants).
//
// Both passes use the transposed, 128-row formulation of the forward so that every tcgen05.mma has
// M = 128 although a block holds only 64 tokens, and so that P / dS are produced by the thread that
// owns their row and are written once, as a swizzled 128-byte shared-memory row (N-major B operand):
//
//  query-owned dQ pass, per PAIR of selected key tiles (lanes = 128 key tokens, columns = 64 query rows)
//      S^T  = K2 Q^T                 dP^T = V2 dO^T
//      dS^T = 2^(S^T c - lse[q]) * (dP^T - delta[q]) * scale      (elementwise, statistics per COLUMN)
//      dQ^T [128 dims x 64 rows] += K2^T dS^T
//
//  key-owned dK/dV pass, per PAIR of query tiles that selected this key tile (lanes = 128 query rows,
//  columns = 64 key tokens)
//      S  = Q2 K^T                   dP = dO2 V^T
//      P  = 2^(S c - lse[row]),      dS = P * (dP - delta[row])   (elementwise, statistics per LANE)
//      dV^T [128 dims x 64 keys] += dO2^T P          dK^T += Q2^T dS          (dK^T * scale at the end)
//
// Nothing here needs a running maximum (the forward saved the log-sum-exp), so there is no
// cross-lane traffic at all.  Roles per CTA: warp 0 and 1 = TMA producers (four lanes, one box each),
// warp 2 = issuer of the S MMAs, warp 3 = issuer of the gradient MMAs, warps 4-11 = elementwise (a TMEM
// lane quarter x 32 of the 64 columns each), warp 12 = issuer of the dP MMAs (the three issuers wait on
// different operands and must not hold one another back).

// The backward passes are closest to the shared-memory bandwidth limit (every operand byte is read by an
// MMA once or twice per pair); eight wider elementwise warps disturb that pipe less than sixteen narrow ones.
constexpr int kBwCols = 32;
constexpr int kBwWarps = 4 * (64 / kBwCols);
constexpr int kBwEwThreads = 32 * kBwWarps;
constexpr int kBwdThreads = 128 + kBwEwThreads + 32;   // ... plus the dP issuer, the last warp
constexpr int kDpWarp = 4 + kBwWarps;

// ------------------------------------------------------------------------------------------------------
// dQ
// ------------------------------------------------------------------------------------------------------
constexpr int kDqBufs = 3;     // (S^T, dP^T) accumulator pairs in flight: 3 x 128 columns, dQ^T behind them
// A K pair stays in shared memory from its score MMA until its dQ MMA, i.e. across the whole elementwise
// stage plus a ~2000-cycle reload; with two stages that chain was the throughput limit, so K gets three
// (V is released right after dP^T and keeps two; dS^T makes do with one buffer to pay for it).
constexpr int kDqKStages = 3;
struct DqSmem {
  static constexpr uint32_t q = 0;                                // 16 KB
  static constexpr uint32_t d_o = q + 2 * kSlab;                  // 16 KB
  static constexpr uint32_t k = d_o + 2 * kSlab;                  // 3 x 32 KB
  static constexpr uint32_t v = k + kDqKStages * kPairBytes;      // 2 x 32 KB
  static constexpr uint32_t ds = v + 2 * kPairBytes;              // 1 x 16 KB
  static constexpr uint32_t tile_row = ds + kPairHalf;            // int32 [kMaxTiles]
  static constexpr uint32_t tile_valid = tile_row + 4 * kMaxTiles;
  static constexpr uint32_t lse = tile_valid + kMaxTiles;         // float [64]
  static constexpr uint32_t delta = lse + 256;                    // float [64]
  static constexpr uint32_t bars = delta + 256;
  static constexpr uint32_t misc = bars + 32 * 8;
  static constexpr uint32_t total = misc + 64;
};
enum DqBar { DQ_QDO_FULL = 0, DQ_K_FULL = 1, DQ_K_EMPTY = 4, DQ_V_FULL = 7, DQ_V_EMPTY = 9, DQ_DS_FULL = 11,
             DQ_DS_EMPTY = 12, DQ_ACC_FULL = 13, DQ_S_FULL = 14, DQ_S_EMPTY = 14 + kDqBufs,
             DQ_DP_FULL = 14 + 2 * kDqBufs };

template <int SUB>
__global__ void __launch_bounds__(kBwdThreads, 1)
sparse_dq_umma_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                      const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                      const elem_t* __restrict__ dout, const elem_t* __restrict__ out_s, const float* __restrict__ lse2,
                      const int32_t* __restrict__ selected, const int32_t* __restrict__ kv_sizes,
                      float* __restrict__ delta, elem_t* __restrict__ dq, const elem_t* __restrict__ mean_grad,
                      const int32_t* __restrict__ q_sizes, long long Lq, long long Lkv, long long kv_shard, int topk,
                      float scale, RasterMap out_map) {
  extern __shared__ uint8_t smem_raw[];
  if (*(volatile int*)&g_device_status != 0) return;
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
  const long long qrow0 = bh * Lq + (long long)qtile * kTile;

  int32_t* tile_row = reinterpret_cast<int32_t*>(sm + DqSmem::tile_row);
  uint8_t* tile_valid = sm + DqSmem::tile_valid;
  float* s_lse = reinterpret_cast<float*>(sm + DqSmem::lse);
  float* s_delta = reinterpret_cast<float*>(sm + DqSmem::delta);
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(sm + DqSmem::misc);
  auto bar = [&](int i) -> uint32_t { return base + DqSmem::bars + 8u * i; };

  if (tid == 0) {
    mbar_init(bar(DQ_QDO_FULL), 1);
    for (int i = 0; i < kDqKStages; ++i) {
      mbar_init(bar(DQ_K_FULL + i), 4);
      mbar_init(bar(DQ_K_EMPTY + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(DQ_V_FULL + i), 4);
      mbar_init(bar(DQ_V_EMPTY + i), 1);
    }
    mbar_init(bar(DQ_DS_FULL), kBwWarps);
    mbar_init(bar(DQ_DS_EMPTY), 1);
    for (int i = 0; i < kDqBufs; ++i) {
      mbar_init(bar(DQ_S_FULL + i), 1);
      mbar_init(bar(DQ_DP_FULL + i), 1);
      mbar_init(bar(DQ_S_EMPTY + i), kBwWarps);
    }
    mbar_init(bar(DQ_ACC_FULL), 1);
    fence_barrier_init();
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
    // Q and dO of this tile depend on nothing the prologue computes: their loads fly under the tile-list build and delta
    mbar_arrive_expect_tx(bar(DQ_QDO_FULL), 4 * kSlab);
    tma_load_2d(base + DqSmem::q, &map_q, 0, (int)qrow0, bar(DQ_QDO_FULL));
    tma_load_2d(base + DqSmem::q + kSlab, &map_q, 64, (int)qrow0, bar(DQ_QDO_FULL));
    tma_load_2d(base + DqSmem::d_o, &map_do, 0, (int)qrow0, bar(DQ_QDO_FULL));
    tma_load_2d(base + DqSmem::d_o + kSlab, &map_do, 64, (int)qrow0, bar(DQ_QDO_FULL));
  }
  for (int it = tid; it < n_iter; it += kBwdThreads) {
    const int kvb = sel[it / SUB];
    // an id outside the table is an empty tile, as route inversion treats it
    const int left = (unsigned)kvb < (unsigned)(Lkv / (kTile * SUB)) ? kv_sizes[kvb] - (it % SUB) * kTile : 0;
    tile_valid[it] = (uint8_t)(left < 0 ? 0 : (left > kTile ? kTile : left));
    tile_row[it] = left > 0 ? (int)kv_tensor_row(bh, gridDim.y, (long long)kvb * (kTile * SUB) + (it % SUB) * kTile, kv_shard) : 0;
  }
  if (warp >= 4 && warp < kDpWarp) {   // delta = rowsum(out_s * dout) and the saved statistic, eight threads per query row
    constexpr int kPer = kBwEwThreads / 64;            // threads per row
    constexpr int kDims = kD / kPer;                 // dims per thread
    const int st = tid - 128;
    const int row = st / kPer, part = st % kPer;
    const uint4* po = reinterpret_cast<const uint4*>(out_s + (qrow0 + row) * kD + part * kDims);
    const uint4* pd = reinterpret_cast<const uint4*>(dout + (qrow0 + row) * kD + part * kDims);
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < kDims / 8; ++i) {
      const uint4 a = po[i], b = pd[i];
      const elem_t* ea = reinterpret_cast<const elem_t*>(&a);
      const elem_t* eb = reinterpret_cast<const elem_t*>(&b);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc = fmaf(Elem<elem_t>::to(ea[j]), Elem<elem_t>::to(eb[j]), acc);
    }
#pragma unroll
    for (int o = 1; o < kPer; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (part == 0) {
      s_delta[row] = acc;
      delta[qrow0 + row] = acc;
      s_lse[row] = lse2[qrow0 + row] - log2f(scale);   // 2^(s c - lse) * scale in one exponential
    }
  }
  __syncthreads();
  if (warp == 2) {
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
    tmem_alloc(base + DqSmem::misc, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = misc[0];
  const int n_live = (int)misc[1];
  const int n_pairs = (n_live + 1) >> 1;
  const uint32_t tmem_acc = tmem + 128 * kDqBufs;
  bool ok = true;

  if (warp == 0 || warp == 1) {
    const bool is_k = warp == 0;
    const int which = lane & 1, dhalf = (lane >> 1) & 1;
    const CUtensorMap* map = is_k ? &map_k : &map_v;
    const int full0 = is_k ? DQ_K_FULL : DQ_V_FULL, empty0 = is_k ? DQ_K_EMPTY : DQ_V_EMPTY;
    const uint32_t ring = base + (is_k ? DqSmem::k : DqSmem::v);
    const int depth = is_k ? kDqKStages : 2;
    for (int p = 0; p < n_pairs; ++p) {
      const int s = p % depth;
      const uint32_t ph = (p / depth) & 1;
      int idx = 2 * p + which;
      if (idx >= n_live) idx = 2 * p;
      const int row = tile_row[idx];                          // row of the tile in the K/V tensors
      ok = VSA_WARP_WAIT(bar(empty0 + s), ph ^ 1);
      if (!ok) break;
      if (lane < 4) {
        mbar_arrive_expect_tx(bar(full0 + s), kSlab);
        tma_load_2d(ring + s * kPairBytes + dhalf * kPairHalf + which * kSlab, map, dhalf * 64, row, bar(full0 + s));
      }
    }
    if (!ok && lane == 0) report_timeout(11);
  } else if (warp == 2) {
    if (lane == 0) {   // scores: S^T = K2 Q^T
      ok = VSA_WAIT(bar(DQ_QDO_FULL), 0);
      for (int p = 0; p < n_pairs && ok; ++p) {
        const int ks = p % kDqKStages, b = p % kDqBufs;
        ok = VSA_WAIT(bar(DQ_K_FULL + ks), (p / kDqKStages) & 1) &&
             VSA_WAIT(bar(DQ_S_EMPTY + b), ((p / kDqBufs) & 1) ^ 1);
        if (!ok) break;
        tc_fence_after();
        // S^T is signalled on its own: the elementwise warps turn it into 2^(S c - lse) while dP^T still runs
        issue_kmajor(tmem + b * 128, base + DqSmem::k + ks * kPairBytes, base + DqSmem::q);
        mma_commit(bar(DQ_S_FULL + b));
      }
      if (!ok) report_timeout(12);
    }
  } else if (warp == kDpWarp) {
    if (lane == 0) {   // dP^T = V2 dO^T from a thread of its own: a late V pair must not hold back the next S^T
      ok = VSA_WAIT(bar(DQ_QDO_FULL), 0);
      for (int p = 0; p < n_pairs && ok; ++p) {
        const int s = p & 1, b = p % kDqBufs;
        ok = VSA_WAIT(bar(DQ_V_FULL + s), (p >> 1) & 1) && VSA_WAIT(bar(DQ_S_EMPTY + b), ((p / kDqBufs) & 1) ^ 1);
        if (!ok) break;
        tc_fence_after();
        issue_kmajor(tmem + b * 128 + 64, base + DqSmem::v + s * kPairBytes, base + DqSmem::d_o);
        mma_commit(bar(DQ_V_EMPTY + s));
        mma_commit(bar(DQ_DP_FULL + b));
      }
      if (!ok) report_timeout(16);
    }
  } else if (warp == 3) {
    if (lane == 0) {   // dQ^T += K2^T dS^T
      for (int p = 0; p < n_pairs && ok; ++p) {
        const int ks = p % kDqKStages;
        ok = VSA_WAIT(bar(DQ_K_FULL + ks), (p / kDqKStages) & 1) && VSA_WAIT(bar(DQ_DS_FULL), p & 1);
        if (!ok) break;
        tc_fence_after();
        issue_mnmajor(tmem_acc, base + DqSmem::k + ks * kPairBytes, base + DqSmem::ds, p > 0);
        mma_commit(bar(DQ_K_EMPTY + ks));
        mma_commit(bar(DQ_DS_EMPTY));
      }
      if (ok) mma_commit(bar(DQ_ACC_FULL));
      if (!ok) report_timeout(13);
    }
  } else {
    // elementwise warps: lane t = key token of the pair, kBwCols of the 64 query rows (columns c0..)
    const int quarter = warp & 3;
    const int cg = (warp - 4) >> 2;
    const int c0 = cg * kBwCols;
    const int t = quarter * 32 + lane;
    const int half = t >> 6, r = t & 63;
    const int st = tid - 128;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    for (int p = 0; p < n_pairs && ok; ++p) {
      const int b = p % kDqBufs;
      const int idx = 2 * p + half;
      const int valid = idx < n_live ? (int)tile_valid[idx] : 0;
      const bool live = r < valid;
      ok = VSA_WARP_WAIT(bar(DQ_S_FULL + b), (p / kDqBufs) & 1);
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[kBwCols];
      tmem_ld(tmem + b * 128 + lane_addr + c0, sv);
      tmem_ld_wait();
      // rows of K beyond a ragged tile's size (and the repeated tile of an odd tail) must be finite zeros:
      // they meet dS = 0 in the dQ product, where 0 * NaN would poison the sum.  S(p) has completed.
      if (!live && cg == 0) {
        uint8_t* krow = sm + DqSmem::k + (p % kDqKStages) * kPairBytes + t * 128;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          *reinterpret_cast<uint4*>(krow + ch * 16) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(krow + kPairHalf + ch * 16) = make_uint4(0, 0, 0, 0);
        }
      }
      float pf[kBwCols];      // 2^(S c - lse) * scale
#pragma unroll
      for (int j4 = 0; j4 < kBwCols / 4; ++j4) {
        const float4 l4 = *reinterpret_cast<const float4*>(s_lse + c0 + 4 * j4);
        pf[4 * j4 + 0] = fast_exp2(fmaf(__uint_as_float(sv[4 * j4 + 0]), c, -l4.x));
        pf[4 * j4 + 1] = fast_exp2(fmaf(__uint_as_float(sv[4 * j4 + 1]), c, -l4.y));
        pf[4 * j4 + 2] = fast_exp2(fmaf(__uint_as_float(sv[4 * j4 + 2]), c, -l4.z));
        pf[4 * j4 + 3] = fast_exp2(fmaf(__uint_as_float(sv[4 * j4 + 3]), c, -l4.w));
      }
      bool ds_free;
      ok = VSA_WARP_WAIT_TEST(bar(DQ_DP_FULL + b), (p / kDqBufs) & 1, bar(DQ_DS_EMPTY), (p & 1) ^ 1, &ds_free);
      if (!ok) break;
      tc_fence_after();
      uint32_t dv[kBwCols];
      tmem_ld(tmem + b * 128 + 64 + lane_addr + c0, dv);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(DQ_S_EMPTY + b));      // both accumulators of this buffer have been read
      uint32_t packed[kBwCols / 2];
#pragma unroll
      for (int j4 = 0; j4 < kBwCols / 4; ++j4) {
        const float4 d4 = *reinterpret_cast<const float4*>(s_delta + c0 + 4 * j4);
        packed[2 * j4] = Elem<elem_t>::pack(pf[4 * j4 + 0] * (__uint_as_float(dv[4 * j4 + 0]) - d4.x),
                                   pf[4 * j4 + 1] * (__uint_as_float(dv[4 * j4 + 1]) - d4.y));
        packed[2 * j4 + 1] = Elem<elem_t>::pack(pf[4 * j4 + 2] * (__uint_as_float(dv[4 * j4 + 2]) - d4.z),
                                       pf[4 * j4 + 3] * (__uint_as_float(dv[4 * j4 + 3]) - d4.w));
      }
      if (!live) {   // a padding key row: its scores come from whatever sits in K and V there
#pragma unroll
        for (int j = 0; j < kBwCols / 2; ++j) packed[j] = 0u;
      }
      if (!ds_free) ok = VSA_WARP_WAIT(bar(DQ_DS_EMPTY), (p & 1) ^ 1);
      if (!ok) break;
      uint8_t* drow = sm + DqSmem::ds + t * 128;
#pragma unroll
      for (int ch = 0; ch < kBwCols / 8; ++ch)
        *reinterpret_cast<uint4*>(drow + ((((kBwCols / 8) * cg + ch) ^ (t & 7)) << 4)) =
            make_uint4(packed[4 * ch], packed[4 * ch + 1], packed[4 * ch + 2], packed[4 * ch + 3]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(DQ_DS_FULL));
    }
    if (!ok && lane == 0) report_timeout(14);
    if (ok && n_pairs > 0) ok = VSA_WARP_WAIT(bar(DQ_ACC_FULL), 0);
    if (!ok && lane == 0) report_timeout(15);
    tc_fence_after();
    elem_t* stage = reinterpret_cast<elem_t*>(sm + DqSmem::k);      // [64 query rows][128 dims]; every MMA is done
    // block-mean backward folded in (optional): query row r of the block also receives dmean[block] / max(size, 1)
    // while r < size (vsa/fused_common.py:62-103 of the reference); here lane t is the head dim, a column a row
    float gm = 0.f;
    int rows_live = 0;
    if (mean_grad != nullptr) {
      const int size = q_sizes[qb];
      gm = Elem<elem_t>::to(mean_grad[(bh * Qb + qb) * (long long)kD + t]) / (float)(size > 1 ? size : 1);
      rows_live = size - (qtile % SUB) * kTile;
    }
    if (ok && n_pairs > 0) {
      uint32_t av[kBwCols];
      tmem_ld(tmem_acc + lane_addr + c0, av);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < kBwCols; ++j)
        stage[(c0 + j) * kD + t] = Elem<elem_t>::from(__uint_as_float(av[j]) + ((c0 + j) < rows_live ? gm : 0.f));
    } else {
      for (int j = 0; j < kBwCols; ++j) stage[(c0 + j) * kD + t] = Elem<elem_t>::from((c0 + j) < rows_live ? gm : 0.f);
    }
    named_barrier(1, kBwEwThreads);
#pragma unroll
    for (int i = 0; i < 1024 / kBwEwThreads; ++i) {
      const int cidx = st + kBwEwThreads * i;
      const int row = cidx >> 4, ch = cidx & 15;
      // with a raster map the gradient row goes straight to the token's raster row (padding rows have none)
      const long long drow = out_map.map == nullptr ? qrow0 + row : raster_row(out_map, bh, (long long)qtile * kTile + row);
      if (drow >= 0)
        *reinterpret_cast<uint4*>(dq + drow * kD + ch * 8) = *reinterpret_cast<const uint4*>(stage + row * kD + ch * 8);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

// ------------------------------------------------------------------------------------------------------
// dK / dV
// ------------------------------------------------------------------------------------------------------
constexpr int kDkBufs = 2;     // (S, dP) accumulator pairs in flight: 2 x 128 columns, then dK^T and dV^T
// A Q2 pair stays in shared memory from its score MMA (the first of a pair) to its dK MMA (the last), across the
// whole elementwise stage, and a reload takes ~1500 cycles on top, so Q2 gets three stages; dO2 gets two and is
// released as early as the data flow allows: S and dP signal the elementwise warps separately, the warps turn S
// into P while the dP MMAs still run and publish P before they look at dP, and dV^T (which needs only P) is
// issued and committed on its own, ahead of dS and dK^T.  P and dS have one buffer each (written by pair p+1 only
// after the MMA of pair p that reads them has completed, checked right before the stores).
constexpr int kDkQStages = 3;
struct DkSmem {
  static constexpr uint32_t k = 0;                                // 16 KB
  static constexpr uint32_t v = k + 2 * kSlab;                    // 16 KB
  static constexpr uint32_t q = v + 2 * kSlab;                    // kDkQStages x 32 KB  (pairs of query tiles)
  static constexpr uint32_t d_o = q + kDkQStages * kPairBytes;    // 2 x 32 KB
  static constexpr uint32_t p = d_o + 2 * kPairBytes;             // 16 KB
  static constexpr uint32_t ds = p + kPairHalf;                   // 16 KB
  static constexpr uint32_t bars = ds + kPairHalf;
  static constexpr uint32_t misc = bars + 32 * 8;
  static constexpr uint32_t total = misc + 64;
};
enum DkBar { DK_KV_FULL = 0, DK_Q_FULL = 1, DK_DO_FULL = 4, DK_Q_EMPTY = 6, DK_DO_EMPTY = 9, DK_P_FULL = 11,
             DK_P_EMPTY = 12, DK_DS_FULL = 13, DK_DS_EMPTY = 14, DK_ACC_FULL = 15, DK_S_FULL = 16,
             DK_DP_FULL = 16 + kDkBufs, DK_S_EMPTY = 16 + 2 * kDkBufs };

// DS = true: the rows of `inverse` hold packed edges (query block << kEdgeSlotBits | slot in that block's route)
// and every dS tile (64 query rows x 64 key tokens, 8 KB) is also written to `ds_ws` at tile index
// ((edge * SUB + query sub-tile) * SUB + key sub-tile), edge = (slice * Qb + query block) * topk + slot, for the
// dQ pass that only multiplies it by K (sparse_dq_from_ds_kernel below) instead of recomputing S and dP.
// Layout of a stored tile: [8 chunks of 8 key tokens][64 query rows][16 bytes] -- the order in which the rows'
// owner threads hold it (a warp's 32 rows of one chunk are 512 contiguous bytes: fully coalesced stores straight
// from registers), and at the same time the un-swizzled K-major operand layout of tcgen05 (8 rows x 16 bytes per
// core matrix), so the dQ pass copies the 8 KB verbatim into shared memory and multiplies.
constexpr int kEdgeSlotBits = 11;
template <int SUB, bool DS>
__global__ void __launch_bounds__(kBwdThreads, 1)
sparse_dkdv_umma_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                        const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const float* __restrict__ lse2, const float* __restrict__ delta,
                        const int32_t* __restrict__ counts, const int32_t* __restrict__ offsets,
                        const int32_t* __restrict__ inverse, const int32_t* __restrict__ kv_sizes,
                        elem_t* __restrict__ dk, elem_t* __restrict__ dv, const elem_t* __restrict__ mean_grad_k,
                        const elem_t* __restrict__ mean_grad_v, elem_t* __restrict__ ds_ws, long long Lq, long long Lkv,
                        long long kv_shard, int topk, float scale, RasterMap out_map) {
  extern __shared__ uint8_t smem_raw[];
  if (*(volatile int*)&g_device_status != 0) return;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ktile = blockIdx.x;
  const long long bh = blockIdx.y;
  const int Kb = (int)(Lkv / (kTile * SUB)), Qb = (int)(Lq / (kTile * SUB));
  const int kvb = ktile / SUB, sub = ktile % SUB;
  int valid = kv_sizes[kvb] - sub * kTile;
  valid = valid < 0 ? 0 : (valid > kTile ? kTile : valid);
  const long long krow0 = kv_tensor_row(bh, gridDim.y, (long long)ktile * kTile, kv_shard);   // K, V, dK, dV rows of this tile
  const int cnt = counts[bh * Kb + kvb];
  const int32_t* inv = inverse + bh * (long long)Qb * topk + offsets[bh * Kb + kvb];
  const int n_tiles = valid > 0 ? cnt * SUB : 0;
  const int n_pairs = (n_tiles + 1) >> 1;
  const float c = scale * kLog2e;
  const long long q_row_base = bh * Lq;

  // block-mean backward folded in (optional): key row r of the block also receives dmean[block] / max(size, 1)
  // while r < size (vsa/fused_common.py:62-103 of the reference)
  const float mean_inv = 1.f / (float)(kv_sizes[kvb] > 1 ? kv_sizes[kvb] : 1);
  const long long mean_off = (bh * Kb + kvb) * (long long)kD;
  if (n_pairs == 0) {   // nobody selected this tile, or it is all padding: no fine gradient, no pipeline
    for (int i = tid; i < 1024; i += (int)blockDim.x) {
      const long long drow = out_map.map == nullptr ? krow0 + (i >> 4) : raster_row(out_map, bh, (long long)ktile * kTile + (i >> 4));
      if (drow < 0) continue;
      uint4 ok4 = make_uint4(0, 0, 0, 0), ov4 = make_uint4(0, 0, 0, 0);
      if (mean_grad_k != nullptr && (i >> 4) < valid) {     // 16 chunks of eight dims per row
        elem_t* ek = reinterpret_cast<elem_t*>(&ok4);
        elem_t* ev = reinterpret_cast<elem_t*>(&ov4);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          ek[e] = Elem<elem_t>::from(Elem<elem_t>::to(mean_grad_k[mean_off + (i & 15) * 8 + e]) * mean_inv);
          ev[e] = Elem<elem_t>::from(Elem<elem_t>::to(mean_grad_v[mean_off + (i & 15) * 8 + e]) * mean_inv);
        }
      }
      *reinterpret_cast<uint4*>(dk + drow * kD + (i & 15) * 8) = ok4;
      *reinterpret_cast<uint4*>(dv + drow * kD + (i & 15) * 8) = ov4;
    }
    return;
  }
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(sm + DkSmem::misc);
  auto bar = [&](int i) -> uint32_t { return base + DkSmem::bars + 8u * i; };
  // row (inside this batch-head slice) of the i-th query tile that selected this key block
  auto tile_row = [&](int i) -> int {
    const int e = inv[i / SUB];
    return (DS ? (e >> kEdgeSlotBits) : e) * (kTile * SUB) + (i % SUB) * kTile;
  };
  // index of the dS tile of the i-th in-edge query tile (DS only)
  auto ds_tile = [&](int i) -> long long {
    const int e = inv[i / SUB];
    const long long edge = (bh * Qb + (e >> kEdgeSlotBits)) * (long long)topk + (e & ((1 << kEdgeSlotBits) - 1));
    return (edge * SUB + (i % SUB)) * SUB + sub;
  };

  if (tid == 0) {
    mbar_init(bar(DK_KV_FULL), 1);
    for (int i = 0; i < kDkQStages; ++i) {
      mbar_init(bar(DK_Q_FULL + i), 4);
      mbar_init(bar(DK_Q_EMPTY + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(DK_DO_FULL + i), 4);
      mbar_init(bar(DK_DO_EMPTY + i), 2);    // read by the dP MMAs of one issuer and the dV^T MMAs of the other
    }
    mbar_init(bar(DK_P_FULL), kBwWarps);
    mbar_init(bar(DK_P_EMPTY), 1);
    mbar_init(bar(DK_DS_FULL), kBwWarps);
    mbar_init(bar(DK_DS_EMPTY), 1);
    for (int i = 0; i < kDkBufs; ++i) {
      mbar_init(bar(DK_S_FULL + i), 1);
      mbar_init(bar(DK_DP_FULL + i), 1);
      mbar_init(bar(DK_S_EMPTY + i), kBwWarps);
    }
    mbar_init(bar(DK_ACC_FULL), 1);
    fence_barrier_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_do);
    // the tile's own K and V, resident for the whole CTA: in flight before anything else
    mbar_arrive_expect_tx(bar(DK_KV_FULL), 4 * kSlab);
    tma_load_2d(base + DkSmem::k, &map_k, 0, (int)krow0, bar(DK_KV_FULL));
    tma_load_2d(base + DkSmem::k + kSlab, &map_k, 64, (int)krow0, bar(DK_KV_FULL));
    tma_load_2d(base + DkSmem::v, &map_v, 0, (int)krow0, bar(DK_KV_FULL));
    tma_load_2d(base + DkSmem::v + kSlab, &map_v, 64, (int)krow0, bar(DK_KV_FULL));
  }
  if (warp == 1) {
    tmem_alloc(base + DkSmem::misc, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = misc[0];
  const uint32_t tmem_dk = tmem + 128 * kDkBufs, tmem_dv = tmem_dk + 64;
  bool ok = true;

  if (warp == 0 || warp == 1) {
    const bool is_q = warp == 0;
    const int which = lane & 1, dhalf = (lane >> 1) & 1;
    const CUtensorMap* map = is_q ? &map_q : &map_do;
    const int full0 = is_q ? DK_Q_FULL : DK_DO_FULL, empty0 = is_q ? DK_Q_EMPTY : DK_DO_EMPTY;
    const uint32_t ring = base + (is_q ? DkSmem::q : DkSmem::d_o);
    const int depth = is_q ? kDkQStages : 2;
    for (int p = 0; p < n_pairs; ++p) {
      const int s = p % depth;
      const uint32_t ph = (p / depth) & 1;
      int idx = 2 * p + which;
      if (idx >= n_tiles) idx = 2 * p;                  // odd tail: repeat the tile (its rows are masked)
      const int row = (int)(q_row_base + tile_row(idx));
      ok = VSA_WARP_WAIT(bar(empty0 + s), ph ^ 1);
      if (!ok) break;
      if (lane < 4) {
        mbar_arrive_expect_tx(bar(full0 + s), kSlab);
        tma_load_2d(ring + s * kPairBytes + dhalf * kPairHalf + which * kSlab, map, dhalf * 64, row, bar(full0 + s));
      }
    }
    if (!ok && lane == 0) report_timeout(21);
  } else if (warp == 2) {
    if (lane == 0) {   // scores: S = Q2 K^T
      ok = VSA_WAIT(bar(DK_KV_FULL), 0);
      for (int p = 0; p < n_pairs && ok; ++p) {
        const int qs = p % kDkQStages, b = p % kDkBufs;
        ok = VSA_WAIT(bar(DK_Q_FULL + qs), (p / kDkQStages) & 1) &&
             VSA_WAIT(bar(DK_S_EMPTY + b), ((p / kDkBufs) & 1) ^ 1);
        if (!ok) break;
        tc_fence_after();
        issue_kmajor(tmem + b * 128, base + DkSmem::q + qs * kPairBytes, base + DkSmem::k);
        mma_commit(bar(DK_S_FULL + b));
      }
      if (!ok) report_timeout(22);
    }
  } else if (warp == kDpWarp) {
    if (lane == 0) {   // dP = dO2 V^T from a thread of its own: dO2 has two stages only and must not hold back the next S
      ok = VSA_WAIT(bar(DK_KV_FULL), 0);
      for (int p = 0; p < n_pairs && ok; ++p) {
        const int s = p & 1, b = p % kDkBufs;
        ok = VSA_WAIT(bar(DK_DO_FULL + s), (p >> 1) & 1) && VSA_WAIT(bar(DK_S_EMPTY + b), ((p / kDkBufs) & 1) ^ 1);
        if (!ok) break;
        tc_fence_after();
        issue_kmajor(tmem + b * 128 + 64, base + DkSmem::d_o + s * kPairBytes, base + DkSmem::v);
        mma_commit(bar(DK_DP_FULL + b));
        mma_commit(bar(DK_DO_EMPTY + s));      // a commit covers the MMAs of the committing thread only: dP here, dV^T there
      }
      if (!ok) report_timeout(26);
    }
  } else if (warp == 3) {
    if (lane == 0) {   // dV^T += dO2^T P and dK^T += Q2^T dS
      for (int p = 0; p < n_pairs && ok; ++p) {
        const int qs = p % kDkQStages, s = p & 1;
        const uint32_t ph = (p >> 1) & 1;
        ok = VSA_WAIT(bar(DK_DO_FULL + s), ph) && VSA_WAIT(bar(DK_P_FULL), p & 1);
        if (!ok) break;
        tc_fence_after();
        issue_mnmajor(tmem_dv, base + DkSmem::d_o + s * kPairBytes, base + DkSmem::p, p > 0);
        mma_commit(bar(DK_P_EMPTY));
        mma_commit(bar(DK_DO_EMPTY + s));      // second of two arrivals: the other issuer commits its dP reads of the stage
        ok = VSA_WAIT(bar(DK_Q_FULL + qs), (p / kDkQStages) & 1) && VSA_WAIT(bar(DK_DS_FULL), p & 1);
        if (!ok) break;
        tc_fence_after();
        issue_mnmajor(tmem_dk, base + DkSmem::q + qs * kPairBytes, base + DkSmem::ds, p > 0);
        mma_commit(bar(DK_Q_EMPTY + qs));
        mma_commit(bar(DK_DS_EMPTY));
      }
      if (ok) mma_commit(bar(DK_ACC_FULL));
      if (!ok) report_timeout(23);
    }
  } else {
    // elementwise warps: lane t = query row of the pair, kBwCols of the 64 key tokens (columns c0..)
    const int quarter = warp & 3;
    const int cg = (warp - 4) >> 2;
    const int c0 = cg * kBwCols;
    const int t = quarter * 32 + lane;
    const int half = t >> 6, r = t & 63;
    const int st = tid - 128;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const bool ragged = valid < kTile;      // same for the whole CTA: key columns >= valid are padding
    // statistics of this lane's query row, fetched one pair ahead of their use.  A row that does not exist (the
    // repeated tile of an odd tail) gets lse = +inf, i.e. P = 0 exactly, and delta = 0, so dS = 0 * finite = 0.
    float lse_n = INFINITY, dl_n = 0.f;
    long long dst_n = -1;                    // DS: tile index of this lane's dS row in the coming pair
    if (half < n_tiles) {
      const long long row = q_row_base + tile_row(half) + r;
      lse_n = lse2[row];
      dl_n = delta[row];
      if (DS) dst_n = ds_tile(half);
    }
    uint8_t* prow = sm + DkSmem::p + t * 128;
    uint8_t* grow = sm + DkSmem::ds + t * 128;
    for (int p = 0; p < n_pairs && ok; ++p) {
      const int b = p % kDkBufs;
      const float lse = lse_n, dl = dl_n;
      const long long dst = dst_n;
      {
        const int nidx = 2 * (p + 1) + half;
        lse_n = INFINITY;
        dl_n = 0.f;
        dst_n = -1;
        if (nidx < n_tiles) {
          const long long row = q_row_base + tile_row(nidx) + r;
          lse_n = lse2[row];
          dl_n = delta[row];
          if (DS) dst_n = ds_tile(nidx);
        }
      }
      // ---- P from S, published before dP is even looked at (the dP MMAs are still running)
      bool p_free, ds_free;       // looked at together with the blocking waits: usually already true
      ok = VSA_WARP_WAIT_TEST(bar(DK_S_FULL + b), (p / kDkBufs) & 1, bar(DK_P_EMPTY), (p & 1) ^ 1, &p_free);
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[kBwCols];
      tmem_ld(tmem + b * 128 + lane_addr + c0, sv);
      tmem_ld_wait();
      float pf[kBwCols];
      if (!ragged) {
#pragma unroll
        for (int j = 0; j < kBwCols; ++j) pf[j] = fast_exp2(fmaf(__uint_as_float(sv[j]), c, -lse));
      } else {   // scores of a padding column come from whatever sits in K there: select, do not multiply
#pragma unroll
        for (int j = 0; j < kBwCols; ++j)
          pf[j] = (c0 + j) < valid ? fast_exp2(fmaf(__uint_as_float(sv[j]), c, -lse)) : 0.f;
      }
      if (!p_free) ok = VSA_WARP_WAIT(bar(DK_P_EMPTY), (p & 1) ^ 1);      // dV^T of the previous pair has read the buffer
      if (!ok) break;
#pragma unroll
      for (int ch = 0; ch < kBwCols / 8; ++ch)
        *reinterpret_cast<uint4*>(prow + ((((kBwCols / 8) * cg + ch) ^ (t & 7)) << 4)) =
            make_uint4(Elem<elem_t>::pack(pf[8 * ch], pf[8 * ch + 1]), Elem<elem_t>::pack(pf[8 * ch + 2], pf[8 * ch + 3]),
                       Elem<elem_t>::pack(pf[8 * ch + 4], pf[8 * ch + 5]), Elem<elem_t>::pack(pf[8 * ch + 6], pf[8 * ch + 7]));
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(DK_P_FULL));
      // ---- dS = P * (dP - delta)
      ok = VSA_WARP_WAIT_TEST(bar(DK_DP_FULL + b), (p / kDkBufs) & 1, bar(DK_DS_EMPTY), (p & 1) ^ 1, &ds_free);
      if (!ok) break;
      tc_fence_after();
      uint32_t dvv[kBwCols];
      tmem_ld(tmem + b * 128 + 64 + lane_addr + c0, dvv);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(DK_S_EMPTY + b));       // both accumulators of this buffer have been read
      uint32_t pg[kBwCols / 2];
      if (!ragged) {
#pragma unroll
        for (int j2 = 0; j2 < kBwCols / 2; ++j2)
          pg[j2] = Elem<elem_t>::pack(pf[2 * j2] * (__uint_as_float(dvv[2 * j2]) - dl),
                             pf[2 * j2 + 1] * (__uint_as_float(dvv[2 * j2 + 1]) - dl));
      } else {   // dP of a padding column comes from whatever sits in V there
#pragma unroll
        for (int j2 = 0; j2 < kBwCols / 2; ++j2) {
          const float g0 = (c0 + 2 * j2) < valid ? pf[2 * j2] * (__uint_as_float(dvv[2 * j2]) - dl) : 0.f;
          const float g1 = (c0 + 2 * j2 + 1) < valid ? pf[2 * j2 + 1] * (__uint_as_float(dvv[2 * j2 + 1]) - dl) : 0.f;
          pg[j2] = Elem<elem_t>::pack(g0, g1);
        }
      }
      if (DS && dst >= 0) {   // chunk-major tile: chunk c of row r at c * 1024 + r * 16 bytes
        uint4* g = reinterpret_cast<uint4*>(ds_ws + dst * (kTile * kTile)) + ((kBwCols / 8) * cg) * kTile + r;
#pragma unroll
        for (int ch = 0; ch < kBwCols / 8; ++ch)
          __stcs(g + ch * kTile, make_uint4(pg[4 * ch], pg[4 * ch + 1], pg[4 * ch + 2], pg[4 * ch + 3]));
      }
      if (!ds_free) ok = VSA_WARP_WAIT(bar(DK_DS_EMPTY), (p & 1) ^ 1);     // dK^T of the previous pair has read the buffer
      if (!ok) break;
#pragma unroll
      for (int ch = 0; ch < kBwCols / 8; ++ch)
        *reinterpret_cast<uint4*>(grow + ((((kBwCols / 8) * cg + ch) ^ (t & 7)) << 4)) =
            make_uint4(pg[4 * ch], pg[4 * ch + 1], pg[4 * ch + 2], pg[4 * ch + 3]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(DK_DS_FULL));
    }
    if (!ok && lane == 0) report_timeout(24);
    if (ok) ok = VSA_WARP_WAIT(bar(DK_ACC_FULL), 0);
    if (!ok && lane == 0) report_timeout(25);
    tc_fence_after();
    elem_t* stage_k = reinterpret_cast<elem_t*>(sm + DkSmem::q);          // [64 key rows][128 dims] each; all MMAs done
    elem_t* stage_v = stage_k + kTile * kD;
    if (ok) {
      uint32_t ak[kBwCols], av[kBwCols];
      tmem_ld(tmem_dk + lane_addr + c0, ak);
      tmem_ld(tmem_dv + lane_addr + c0, av);
      tmem_ld_wait();
      float gmk = 0.f, gmv = 0.f;            // lane t is the head dim here, a column a key row
      if (mean_grad_k != nullptr) {
        gmk = Elem<elem_t>::to(mean_grad_k[mean_off + t]) * mean_inv;
        gmv = Elem<elem_t>::to(mean_grad_v[mean_off + t]) * mean_inv;
      }
#pragma unroll
      for (int j = 0; j < kBwCols; ++j) {
        const bool row_live = (c0 + j) < valid;
        stage_k[(c0 + j) * kD + t] = Elem<elem_t>::from(__uint_as_float(ak[j]) * scale + (row_live ? gmk : 0.f));
        stage_v[(c0 + j) * kD + t] = Elem<elem_t>::from(__uint_as_float(av[j]) + (row_live ? gmv : 0.f));
      }
    } else {
      for (int j = 0; j < kBwCols; ++j) {
        stage_k[(c0 + j) * kD + t] = Elem<elem_t>::from(0.f);
        stage_v[(c0 + j) * kD + t] = Elem<elem_t>::from(0.f);
      }
    }
    named_barrier(1, kBwEwThreads);
#pragma unroll
    for (int i = 0; i < 1024 / kBwEwThreads; ++i) {
      const int cidx = st + kBwEwThreads * i;
      const int row = cidx >> 4, ch = cidx & 15;
      const long long drow = out_map.map == nullptr ? krow0 + row : raster_row(out_map, bh, (long long)ktile * kTile + row);
      if (drow >= 0) {
        *reinterpret_cast<uint4*>(dk + drow * kD + ch * 8) = *reinterpret_cast<const uint4*>(stage_k + row * kD + ch * 8);
        *reinterpret_cast<uint4*>(dv + drow * kD + ch * 8) = *reinterpret_cast<const uint4*>(stage_v + row * kD + ch * 8);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

// ------------------------------------------------------------------------------------------------------
// dQ from stored dS:  dQ^T [128 dims x 64 query rows] = scale * sum over the selected key tiles of K^T dS^T
// ------------------------------------------------------------------------------------------------------
// The key-owned pass above has already formed every dS tile; this query-owned pass only streams, per selected
// key tile, the K tile (16 KB) and the dS tile (8 KB) and issues four M128 x N64 x K16 MMAs: no scores, no
// exponentials, no elementwise stage.  It is bound by how fast TMA brings the 24 KB in, so the ring is deep.
// Roles: warp 0 = TMA producer of the K tiles (two lanes, one box each), warp 1 = MMA issuer (owns the tensor
// memory; the whole warp zero-fills the padding rows of a ragged K tile first), warps 2-5 = epilogue, warps 6-7 =
// loaders of the dS tiles with plain asynchronous 16-byte copies: one SM's TMA unit moves ~50 bytes per clock in
// 8 KB boxes, the load/store path adds its own bandwidth beside it, and a dS tile is a verbatim 8 KB copy.
constexpr int kDsStages = 8;
constexpr int kDsStageBytes = 3 * kSlab;        // K head-dim half 0 | K head-dim half 1 | dS
constexpr int kDsLoaders = 64;                  // threads that copy dS tiles
constexpr int kDsThreads = 192 + kDsLoaders;
struct DqdsSmem {
  static constexpr uint32_t ring = 0;
  static constexpr uint32_t tile_row = ring + kDsStages * kDsStageBytes;   // int32 [kMaxTiles]
  static constexpr uint32_t tile_it = tile_row + 4 * kMaxTiles;            // uint16 [kMaxTiles]: position in the route
  static constexpr uint32_t tile_valid = tile_it + 2 * kMaxTiles;          // uint8 [kMaxTiles]
  static constexpr uint32_t bars = tile_valid + kMaxTiles;
  static constexpr uint32_t misc = bars + 32 * 8;
  static constexpr uint32_t total = misc + 64;
};
enum DqdsBar { DD_FULL = 0, DD_EMPTY = kDsStages, DD_ACC_FULL = 2 * kDsStages };

template <int SUB>
__global__ void __launch_bounds__(kDsThreads, 1)
sparse_dq_from_ds_kernel(const __grid_constant__ CUtensorMap map_k, const elem_t* __restrict__ ds_ws,
                         const int32_t* __restrict__ selected, const int32_t* __restrict__ kv_sizes,
                         elem_t* __restrict__ dq, const elem_t* __restrict__ mean_grad, const int32_t* __restrict__ q_sizes,
                         long long Lq, long long Lkv, int topk, float scale) {
  extern __shared__ uint8_t smem_raw[];
  if (*(volatile int*)&g_device_status != 0) return;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qtile = blockIdx.x;
  const long long bh = blockIdx.y;
  const int Qb = (int)(Lq / (kTile * SUB)), Kb = (int)(Lkv / (kTile * SUB));
  const int qb = qtile / SUB, qsub = qtile % SUB;
  const int32_t* sel = selected + (bh * Qb + qb) * (long long)topk;
  const int n_iter = topk * SUB;
  const long long qrow0 = bh * Lq + (long long)qtile * kTile;
  const long long edge0 = (bh * Qb + qb) * (long long)topk;

  int32_t* tile_row = reinterpret_cast<int32_t*>(sm + DqdsSmem::tile_row);
  uint16_t* tile_it = reinterpret_cast<uint16_t*>(sm + DqdsSmem::tile_it);
  uint8_t* tile_valid = sm + DqdsSmem::tile_valid;
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(sm + DqdsSmem::misc);
  auto bar = [&](int i) -> uint32_t { return base + DqdsSmem::bars + 8u * i; };

  if (tid == 0) {
    for (int i = 0; i < kDsStages; ++i) {
      mbar_init(bar(DD_FULL + i), 2 + kDsLoaders);     // two TMA lanes and every loader thread
      mbar_init(bar(DD_EMPTY + i), 1);
    }
    mbar_init(bar(DD_ACC_FULL), 1);
    fence_barrier_init();
    tma_prefetch_desc(&map_k);
  }
  for (int it = tid; it < n_iter; it += kDsThreads) {
    const int kvb = sel[it / SUB];
    const int left = (unsigned)kvb < (unsigned)Kb ? kv_sizes[kvb] - (it % SUB) * kTile : 0;   // an id outside the table is an empty tile
    tile_valid[it] = (uint8_t)(left < 0 ? 0 : (left > kTile ? kTile : left));
    tile_row[it] = kvb * (kTile * SUB) + (it % SUB) * kTile;
    tile_it[it] = (uint16_t)it;
  }
  __syncthreads();
  if (warp == 2) {   // squeeze out the empty tiles in place, keeping the routing order
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
        tile_it[pos] = (uint16_t)it;
      }
      n_live += __popc(live);
      __syncwarp();
    }
    if (lane == 0) misc[1] = (uint32_t)n_live;
  }
  if (warp == 1) {
    tmem_alloc(base + DqdsSmem::misc, 64);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = misc[0];
  const int n_live = (int)misc[1];
  const long long kv_row_base = bh * Lkv;
  bool ok = true;

  if (warp == 0) {
    for (int i = 0; i < n_live; ++i) {
      const int s = i % kDsStages;
      ok = VSA_WARP_WAIT(bar(DD_EMPTY + s), ((i / kDsStages) & 1) ^ 1);
      if (!ok) break;
      if (lane < 2) {
        const uint32_t dst = base + DqdsSmem::ring + s * kDsStageBytes + lane * kSlab;
        mbar_arrive_expect_tx(bar(DD_FULL + s), kSlab);
        tma_load_2d(dst, &map_k, lane * 64, (int)(kv_row_base + tile_row[i]), bar(DD_FULL + s));
      }
    }
    if (!ok && lane == 0) report_timeout(31);
  } else if (warp >= 6) {
    const int lt = tid - 192;                          // 64 threads x 8 copies of 16 bytes = one 8 KB tile
    for (int i = 0; i < n_live; ++i) {
      const int s = i % kDsStages;
      ok = VSA_WARP_WAIT(bar(DD_EMPTY + s), ((i / kDsStages) & 1) ^ 1);
      if (!ok) break;
      const int it = tile_it[i];
      const long long tile = ((edge0 + it / SUB) * SUB + qsub) * SUB + (it % SUB);
      const uint8_t* src = reinterpret_cast<const uint8_t*>(ds_ws + tile * (kTile * kTile)) + lt * 16;
      const uint32_t dst = base + DqdsSmem::ring + s * kDsStageBytes + 2 * kSlab + lt * 16;
#pragma unroll
      for (int j = 0; j < kSlab / (16 * kDsLoaders); ++j) cp_async16(dst + j * 16 * kDsLoaders, src + j * 16 * kDsLoaders);
      cp_async_arrive_noinc(bar(DD_FULL + s));
    }
    if (!ok && lane == 0) report_timeout(34);
  } else if (warp == 1) {
    constexpr uint32_t idesc = instr_desc(128, 64, 1, 0, kInFmt);     // A = K^T (dims contiguous), B = dS (keys contiguous)
    constexpr uint32_t hi = desc_hi(1024);
    // B: un-swizzled K-major, core matrices of 8 query rows x 16 bytes; the next 8 rows 128 bytes on, the next
    // 8 key tokens (chunk) 1024 bytes on; one MMA consumes two chunks
    constexpr uint32_t hi_b = desc_hi_noswizzle(128);
    // Two tiles per trip: a wait on an mbarrier costs a shared-memory round trip of a few hundred cycles however
    // long ago it flipped, more than the four MMAs of a tile; two lanes look at two stages at once.
    for (int i0 = 0; i0 < n_live; i0 += 2) {
      const int n_here = n_live - i0 >= 2 ? 2 : 1;
      const int s0 = i0 % kDsStages, s1 = (i0 + 1) % kDsStages;
      if (n_here == 2)
        ok = VSA_WARP_WAIT2(bar(DD_FULL + s0), (i0 / kDsStages) & 1, bar(DD_FULL + s1), ((i0 + 1) / kDsStages) & 1);
      else
        ok = VSA_WARP_WAIT(bar(DD_FULL + s0), (i0 / kDsStages) & 1);
      if (!ok) break;
      for (int h = 0; h < n_here; ++h) {
        const int valid = tile_valid[i0 + h];
        if (valid < kTile) {
          // rows of K beyond a ragged tile's size meet dS = 0 in the product; they must be finite zeros (0 * NaN)
          uint8_t* kst = sm + DqdsSmem::ring + (h ? s1 : s0) * kDsStageBytes;
          for (int r = valid + (lane >> 4); r < kTile; r += 2) {
            const int ch = lane & 15;                 // 16 chunks of 16 bytes: both head-dim halves of the row
            *reinterpret_cast<uint4*>(kst + (ch >> 3) * kSlab + r * 128 + (ch & 7) * 16) = make_uint4(0, 0, 0, 0);
          }
          __syncwarp();
        }
      }
      if (lane == 0) {
        // the dS tiles were written by ordinary asynchronous copies (and padding rows by this warp); the tensor
        // core reads through the async proxy
        fence_proxy_async_smem();
        tc_fence_after();
        for (int h = 0; h < n_here; ++h) {
          const int s = h ? s1 : s0;
          const uint32_t stage = base + DqdsSmem::ring + s * kDsStageBytes;
          const uint32_t a0 = desc_lo(stage, kSlab), b0 = desc_lo(stage + 2 * kSlab, 1024);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            mma_ss(tmem, desc_pack(a0 + (uint32_t)(ks * 128), hi), desc_pack(b0 + (uint32_t)(ks * 128), hi_b), idesc,
                   (i0 + h > 0 || ks > 0) ? 1u : 0u);
          mma_commit(bar(DD_EMPTY + s));
        }
      }
      __syncwarp();
    }
    if (lane == 0) {
      if (ok) mma_commit(bar(DD_ACC_FULL));
      else report_timeout(32);
    }
  } else {
    // epilogue: lane t = head dim, a column = a query row
    const int quarter = warp & 3;
    const int t = quarter * 32 + lane;
    const int st = tid - 64;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    float gm = 0.f;
    int rows_live = 0;
    if (mean_grad != nullptr) {   // block-mean backward folded in, as in the recomputing dQ kernel
      const int size = q_sizes[qb];
      gm = Elem<elem_t>::to(mean_grad[(bh * Qb + qb) * (long long)kD + t]) / (float)(size > 1 ? size : 1);
      rows_live = size - qsub * kTile;
    }
    if (n_live > 0) ok = VSA_WARP_WAIT(bar(DD_ACC_FULL), 0);
    if (!ok && lane == 0) report_timeout(33);
    tc_fence_after();
    elem_t* stage = reinterpret_cast<elem_t*>(sm + DqdsSmem::ring);     // [64 query rows][128 dims]; every MMA is done
#pragma unroll
    for (int hcol = 0; hcol < 2; ++hcol) {
      uint32_t av[32];
      if (ok && n_live > 0) {
        tmem_ld(tmem + lane_addr + hcol * 32, av);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) av[j] = 0u;
      }
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int c = hcol * 32 + j;
        stage[c * kD + t] = Elem<elem_t>::from(__uint_as_float(av[j]) * scale + (c < rows_live ? gm : 0.f));
      }
    }
    named_barrier(1, 128);
    elem_t* og = dq + qrow0 * kD;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int cidx = st + 128 * i;
      const int row = cidx >> 4, ch = cidx & 15;
      *reinterpret_cast<uint4*>(og + row * kD + ch * 8) = *reinterpret_cast<const uint4*>(stage + row * kD + ch * 8);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 64);
}
