// Persistent form of the tcgen05 forward, used for short routes (at most 24 pairs of key tiles per query tile).
// Included by sparse_umma.cu after the per-tile kernel, whose formulation, operand layouts, softmax and epilogue
// arithmetic it shares line for line; what changes is the schedule.  A per-tile CTA spends a fixed ~10 us outside its
// steady state (7-12 % of its life at 90 pairs per tile, 40 % at 16): building the list of live key
// tiles (two dependent global loads), allocating tensor memory, filling the pipeline, and at the end draining it
// and writing the output while no MMA runs -- and with one 190 KB CTA per SM nothing else runs meanwhile.  Here
// one CTA per SM walks query tiles w = blockIdx.x, blockIdx.x + gridDim.x, ...:
//   * a scheduler warp builds the tile list of the NEXT query tile into the other half of a double buffer;
//   * Q has two buffers and O^T two accumulators in tensor memory, so the producers and the S^T issuer run ahead
//     into the next query tile (up to the four S^T accumulators) while the softmax warps are still in the
//     epilogue of the current one; the epilogue has a staging buffer of its own instead of borrowing the K ring;
//   * every ring keeps ONE running pair counter across query tiles, so stages and barrier phases simply continue.
// Roles: warp 0 = K producer (also loads Q), warp 1 = V producer (owns the tensor memory), warp 2 = issuer of the
// S^T MMAs, warp 3 = issuer of the O^T MMAs, warps 4-19 = softmax, warp 20 = scheduler.

struct FwdPSmem {
  static constexpr uint32_t q = 0;                                  // 2 x 16 KB
  static constexpr uint32_t k = q + 4 * kSlab;                      // 2 stages x 32 KB
  static constexpr uint32_t v = k + kFwdKStages * kPairBytes;       // 2 stages x 32 KB
  static constexpr uint32_t p = v + 2 * kPairBytes;                 // 2 buffers x 16 KB
  static constexpr uint32_t stage = p + 2 * kPairHalf;              // 16 KB: [64 query rows][128 dims] on the way out
  static constexpr uint32_t tile_row = stage + 2 * kSlab;           // int32 [2][kMaxTiles]
  static constexpr uint32_t tile_valid = tile_row + 2 * 4 * kMaxTiles;   // uint8 [2][kMaxTiles]
  static constexpr uint32_t m_warp = tile_valid + 2 * kMaxTiles;    // float [4 lane quarters][64]
  static constexpr uint32_t m_col = m_warp + 4 * 64 * 4;            // float [64]
  static constexpr uint32_t l_col = m_col + 64 * 4;                 // float [64]
  static constexpr uint32_t bars = l_col + 64 * 4;                  // 8-byte mbarriers
  static constexpr uint32_t misc = bars + 40 * 8;                   // tmem base, n_live[2], flag
  static constexpr uint32_t total = misc + 64;
};
constexpr int kFwdPThreads = kFwdThreads + 32;                      // ... plus the scheduler warp
constexpr int kSchedWarp = kFwdThreads / 32;
enum FwdPBar { PQ_FULL = 0, PQ_EMPTY = 2, PK_FULL = 4, PK_EMPTY = 6, PV_FULL = 8, PV_EMPTY = 10, PP_FULL = 12,
               PP_EMPTY = 14, PO_FULL = 16, PO_EMPTY = 18, PL_FULL = 20, PL_EMPTY = 22, PS_FULL = 24,
               PS_EMPTY = 24 + kSBufs };

template <int SUB>
__global__ void __launch_bounds__(kFwdPThreads, 1)
sparse_fwd_umma_persistent_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                  const __grid_constant__ CUtensorMap map_v, const int32_t* __restrict__ selected,
                                  const int32_t* __restrict__ kv_sizes, elem_t* __restrict__ out,
                                  float* __restrict__ lse2, const elem_t* __restrict__ out_c,
                                  const elem_t* __restrict__ gate, elem_t* __restrict__ out_comb, long long BH, long long Lq,
                                  long long Lkv, long long kv_shard, int topk, float scale, RasterMap comb_map) {
  extern __shared__ uint8_t smem_raw[];
  if (*(volatile int*)&g_device_status != 0) return;   // an earlier wait ran out: drain without touching anything
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q_tiles = (int)(Lq / kTile);
  const long long n_items = (long long)q_tiles * BH;
  const int Qb = (int)(Lq / (kTile * SUB));
  const int n_iter = topk * SUB;
  const float c = scale * kLog2e;

  int32_t* tile_row = reinterpret_cast<int32_t*>(sm + FwdPSmem::tile_row);
  uint8_t* tile_valid = sm + FwdPSmem::tile_valid;
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(sm + FwdPSmem::misc);   // [0] tmem, [1..2] n_live, [3] flag
  auto bar = [&](int i) -> uint32_t { return base + FwdPSmem::bars + 8u * i; };

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(PQ_FULL + i), 1);
      mbar_init(bar(PQ_EMPTY + i), 1);
      mbar_init(bar(PK_FULL + i), 4);      // four producer lanes, one TMA box each
      mbar_init(bar(PK_EMPTY + i), 1);
      mbar_init(bar(PV_FULL + i), 4);
      mbar_init(bar(PV_EMPTY + i), 1);
      mbar_init(bar(PP_FULL + i), kEwWarps);
      mbar_init(bar(PP_EMPTY + i), 1);
      mbar_init(bar(PO_FULL + i), 1);
      mbar_init(bar(PO_EMPTY + i), kEwWarps);
      mbar_init(bar(PL_FULL + i), 1);
      mbar_init(bar(PL_EMPTY + i), 4 + kEwWarps);   // every warp that reads a tile list gives it back
    }
    for (int i = 0; i < kSBufs; ++i) {
      mbar_init(bar(PS_FULL + i), 1);
      mbar_init(bar(PS_EMPTY + i), kEwWarps);
    }
    misc[3] = 0u;
    fence_barrier_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
  }
  if (warp == 1) {
    tmem_alloc(base + FwdPSmem::misc, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = misc[0];
  const uint32_t tmem_s0 = tmem, tmem_o0 = tmem + 64 * kSBufs;   // four S^T accumulators, then two O^T accumulators
  bool ok = true;

  if (warp == kSchedWarp) {
    // ================= scheduler: the list of live key tiles of each query tile, one item ahead =================
    int j = 0;
    for (long long w = blockIdx.x; w < n_items && ok; w += gridDim.x, ++j) {
      const int b = j & 1;
      ok = VSA_WARP_WAIT(bar(PL_EMPTY + b), ((j >> 1) & 1) ^ 1);
      if (!ok) break;
      const int qtile = (int)(w % q_tiles);
      const long long bh = w / q_tiles;
      const int32_t* sel = selected + (bh * Qb + qtile / SUB) * (long long)topk;
      int32_t* rows = tile_row + b * kMaxTiles;
      uint8_t* valids = tile_valid + b * kMaxTiles;
      int n_live = 0;
      for (int it0 = 0; it0 < n_iter; it0 += 32) {
        const int it = it0 + lane;
        int valid = 0, row = 0;
        if (it < n_iter) {
          const int kvb = sel[it / SUB];
          // an id outside the table is an empty tile, as route inversion treats it
          const int left = (unsigned)kvb < (unsigned)(Lkv / (kTile * SUB)) ? kv_sizes[kvb] - (it % SUB) * kTile : 0;
          valid = left < 0 ? 0 : (left > kTile ? kTile : left);
          if (valid > 0) row = (int)kv_tensor_row(bh, BH, (long long)kvb * (kTile * SUB) + (it % SUB) * kTile, kv_shard);
        }
        const unsigned live = __ballot_sync(0xffffffffu, valid > 0);
        if (valid > 0) {      // empty tiles are squeezed out, the routing order is kept
          const int pos = n_live + __popc(live & ((1u << lane) - 1u));
          rows[pos] = row;
          valids[pos] = (uint8_t)valid;
        }
        n_live += __popc(live);
      }
      if (lane == 0) misc[1 + b] = (uint32_t)n_live;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(PL_FULL + b));
    }
    if (!ok && lane == 0) report_timeout(41);
  } else if (warp == 0 || warp == 1) {
    // ================= TMA producers: warp 0 streams Q and K pairs, warp 1 streams V pairs =================
    const bool is_k = warp == 0;
    const int which = lane & 1, dhalf = (lane >> 1) & 1;  // tile a or b of the pair; head-dim half
    const CUtensorMap* map = is_k ? &map_k : &map_v;
    const int full0 = is_k ? PK_FULL : PV_FULL, empty0 = is_k ? PK_EMPTY : PV_EMPTY;
    const uint32_t ring = base + (is_k ? FwdPSmem::k : FwdPSmem::v);
    unsigned cnt = 0;                                      // pairs streamed so far, over all query tiles
    int j = 0;
    for (long long w = blockIdx.x; w < n_items && ok; w += gridDim.x, ++j) {
      const int b = j & 1;
      ok = VSA_WARP_WAIT(bar(PL_FULL + b), (j >> 1) & 1);
      if (!ok) break;
      const int n_live = (int)misc[1 + b];
      const int n_pairs = (n_live + 1) >> 1;
      const int32_t* rows = tile_row + b * kMaxTiles;
      if (is_k) {
        ok = VSA_WARP_WAIT(bar(PQ_EMPTY + b), ((j >> 1) & 1) ^ 1);
        if (!ok) break;
        if (lane == 0) {
          mbar_arrive_expect_tx(bar(PQ_FULL + b), 2 * kSlab);
          const int qrow = (int)((w / q_tiles) * Lq + (w % q_tiles) * kTile);
          tma_load_2d(base + FwdPSmem::q + b * 2 * kSlab, &map_q, 0, qrow, bar(PQ_FULL + b));
          tma_load_2d(base + FwdPSmem::q + b * 2 * kSlab + kSlab, &map_q, 64, qrow, bar(PQ_FULL + b));
        }
      }
      for (int p = 0; p < n_pairs; ++p, ++cnt) {
        const int s = cnt & 1;
        const uint32_t ph = (cnt >> 1) & 1;
        int idx = 2 * p + which;
        if (idx >= n_live) idx = 2 * p;                     // odd tail: repeat the first tile (masked later)
        const int row = rows[idx];
        ok = VSA_WARP_WAIT(bar(empty0 + s), ph ^ 1);
        if (!ok) break;
        if (lane < 4) {
          mbar_arrive_expect_tx(bar(full0 + s), kSlab);
          tma_load_2d(ring + s * kPairBytes + dhalf * kPairHalf + which * kSlab, map, dhalf * 64, row, bar(full0 + s));
        }
      }
      if (!ok) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(PL_EMPTY + b));
    }
    if (!ok && lane == 0) report_timeout(42);
  } else if (warp == 2) {
    // ================= MMA issuer 1: S^T = K2 Q^T, as far ahead as operands and accumulators allow =================
    if (lane == 0) {
      unsigned cnt = 0;
      int j = 0;
      for (long long w = blockIdx.x; w < n_items && ok; w += gridDim.x, ++j) {
        const int b = j & 1;
        ok = VSA_WAIT(bar(PL_FULL + b), (j >> 1) & 1) && VSA_WAIT(bar(PQ_FULL + b), (j >> 1) & 1);
        if (!ok) break;
        const int n_pairs = ((int)misc[1 + b] + 1) >> 1;
        for (int p = 0; p < n_pairs && ok; ++p, ++cnt) {
          const int s = cnt & 1, sb = cnt % kSBufs;
          ok = VSA_WAIT(bar(PK_FULL + s), (cnt >> 1) & 1) && VSA_WAIT(bar(PS_EMPTY + sb), ((cnt / kSBufs) & 1) ^ 1);
          if (!ok) break;
          tc_fence_after();
          issue_kmajor(tmem_s0 + sb * 64, base + FwdPSmem::k + s * kPairBytes, base + FwdPSmem::q + b * 2 * kSlab);
          mma_commit(bar(PK_EMPTY + s));
          mma_commit(bar(PS_FULL + sb));
        }
        if (!ok) break;
        mma_commit(bar(PQ_EMPTY + b));       // arrives once the last S^T MMA that reads this Q buffer has completed
        mbar_arrive(bar(PL_EMPTY + b));
      }
      if (!ok) report_timeout(43);
    }
  } else if (warp == 3) {
    // ================= MMA issuer 2: O^T += V2^T P^T =================
    if (lane == 0) {
      unsigned cnt = 0;
      int j = 0;
      for (long long w = blockIdx.x; w < n_items && ok; w += gridDim.x, ++j) {
        const int b = j & 1;
        ok = VSA_WAIT(bar(PL_FULL + b), (j >> 1) & 1) && VSA_WAIT(bar(PO_EMPTY + b), ((j >> 1) & 1) ^ 1);
        if (!ok) break;
        const int n_pairs = ((int)misc[1 + b] + 1) >> 1;
        for (int p = 0; p < n_pairs && ok; ++p, ++cnt) {
          const int s = cnt & 1;
          const uint32_t ph = (cnt >> 1) & 1;
          ok = VSA_WAIT(bar(PV_FULL + s), ph) && VSA_WAIT(bar(PP_FULL + s), ph);
          if (!ok) break;
          tc_fence_after();
          issue_mnmajor(tmem_o0 + b * 64, base + FwdPSmem::v + s * kPairBytes, base + FwdPSmem::p + s * kPairHalf, p > 0);
          mma_commit(bar(PV_EMPTY + s));
          mma_commit(bar(PP_EMPTY + s));
        }
        if (!ok) break;
        mma_commit(bar(PO_FULL + b));        // with no pair at all nothing is pending and the arrival is immediate
        mbar_arrive(bar(PL_EMPTY + b));
      }
      if (!ok) report_timeout(44);
    }
  } else {
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
    float* m_warp = reinterpret_cast<float*>(sm + FwdPSmem::m_warp);
    float* m_col = reinterpret_cast<float*>(sm + FwdPSmem::m_col);
    float* l_col = reinterpret_cast<float*>(sm + FwdPSmem::l_col);
    elem_t* stage = reinterpret_cast<elem_t*>(sm + FwdPSmem::stage);
    volatile uint32_t* flag = misc + 3;
    unsigned cnt = 0;
    int j = 0;
    for (long long w = blockIdx.x; w < n_items && ok; w += gridDim.x, ++j) {
      const int b = j & 1;
      ok = VSA_WARP_WAIT(bar(PL_FULL + b), (j >> 1) & 1);
      if (!ok) break;
      const int n_live = (int)misc[1 + b];
      const int n_pairs = (n_live + 1) >> 1;
      const uint8_t* valids = tile_valid + b * kMaxTiles;
      const int qtile = (int)(w % q_tiles);
      const long long bh = w / q_tiles;
      const int qb = qtile / SUB;
      float lsum[kEwCols];
#pragma unroll
      for (int i = 0; i < kEwCols; ++i) lsum[i] = 0.f;

      for (int p = 0; p < n_pairs && ok; ++p, ++cnt) {
        const int s = cnt & 1;
        const uint32_t ph = (cnt >> 1) & 1;
        const int idx = 2 * p + half;
        const int valid = idx < n_live ? (int)valids[idx] : 0;
        const bool live = r < valid;
        const int sb = cnt % kSBufs;
        // the score accumulator and the free P buffer (released by the O^T MMA two pairs back) in one round trip
        ok = VSA_WARP_WAIT2(bar(PS_FULL + sb), (cnt / kSBufs) & 1, bar(PP_EMPTY + s), ph ^ 1);
        if (!ok) break;
        tc_fence_after();
        uint32_t sv[kEwCols];
        tmem_ld(tmem_s0 + sb * 64 + lane_addr + c0, sv);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(PS_EMPTY + sb));

        if (p == 0) {   // exact column maxima of the first live pair: warp shuffle, then across the lane quarters
#pragma unroll
          for (int i = 0; i < kEwCols; ++i) {
            const float x = warp_max(live ? __uint_as_float(sv[i]) * c : -INFINITY);
            if (lane == 0) m_warp[quarter * 64 + c0 + i] = x;
          }
          named_barrier(1, kEwThreads);
          if (st < 64) m_col[st] = fmaxf(fmaxf(m_warp[st], m_warp[64 + st]), fmaxf(m_warp[128 + st], m_warp[192 + st])) + kShiftBias;
          named_barrier(1, kEwThreads);
        }
        // padding rows of a ragged tile (and the repeated tile of an odd tail): whatever sits in V there
        // must not reach the tensor core, where 0 * NaN would poison the sum
        if (!live && cg == 0) {
          ok = VSA_WAIT(bar(PV_FULL + s), ph);
          uint8_t* vrow = sm + FwdPSmem::v + s * kPairBytes + t * 128;
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
        uint8_t* prow = sm + FwdPSmem::p + s * kPairHalf + t * 128;
#pragma unroll
        for (int ch = 0; ch < kEwCols / 8; ++ch)     // this thread's query rows are 16-byte chunks of row t
          *reinterpret_cast<uint4*>(prow + ((((kEwCols / 8) * cg + ch) ^ (t & 7)) << 4)) =
              make_uint4(packed[4 * ch], packed[4 * ch + 1], packed[4 * ch + 2], packed[4 * ch + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(PP_FULL + s));
      }
      if (!ok) break;

      // ---- epilogue: reduce the row sums across lanes (fixed order), normalise O^T, transpose via shared memory ----
#pragma unroll
      for (int i = 0; i < kEwCols; ++i) {
        const float x = warp_sum(lsum[i]);
        if (lane == 0) m_warp[quarter * 64 + c0 + i] = x;       // the maxima scratch is free by now
      }
      named_barrier(1, kEwThreads);
      if (st < 64) l_col[st] = (m_warp[st] + m_warp[64 + st]) + (m_warp[128 + st] + m_warp[192 + st]);
      named_barrier(1, kEwThreads);
      ok = VSA_WARP_WAIT(bar(PO_FULL + b), (j >> 1) & 1);
      if (!ok) break;
      tc_fence_after();
      bool finite = true;
      if (n_pairs > 0) {
        uint32_t ov[kEwCols];
        tmem_ld(tmem_o0 + b * 64 + lane_addr + c0, ov);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(PO_EMPTY + b));         // the accumulator may be overwritten two query tiles on
#pragma unroll
        for (int i = 0; i < kEwCols; ++i) {
          const int qi = c0 + i;
          const float l = l_col[qi];
          const float o = __uint_as_float(ov[i]) / l;
          finite = finite && (fabsf(o) <= 3.0e38f) && (l <= 3.0e38f);
          stage[qi * kD + t] = Elem<elem_t>::from(o);
        }
      } else {
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(PO_EMPTY + b));
        for (int i = 0; i < kEwCols; ++i) stage[(c0 + i) * kD + t] = Elem<elem_t>::from(NAN);
      }
      // vote across the softmax threads through shared memory
      if (!finite) *flag = 1u;
      named_barrier(1, kEwThreads);
      const bool redo = (*flag != 0u);
      const long long row0 = bh * Lq + (long long)qtile * kTile;
      elem_t* og = out + row0 * kD;
#pragma unroll
      for (int i = 0; i < 1024 / kEwThreads; ++i) {
        const int cidx = st + kEwThreads * i;         // 1024 chunks of 16 bytes
        const int row = cidx >> 4, ch = cidx & 15;
        const uint4 sv4 = *reinterpret_cast<const uint4*>(stage + row * kD + ch * 8);
        *reinterpret_cast<uint4*>(og + row * kD + ch * 8) = sv4;
        if (out_comb != nullptr) {   // gated combine with the pooled branch on the way out (the fine output is kept: delta needs it)
          const uint4 cv = *reinterpret_cast<const uint4*>(out_c + (bh * Qb + qb) * (long long)kD + ch * 8);
          uint4 gv = make_uint4(0, 0, 0, 0);
          // with a raster map the gate is read, and the combined output written, at the token's raster row
          const long long crow = comb_map.map == nullptr ? row0 + row : raster_row(comb_map, bh, (long long)qtile * kTile + row);
          if (crow >= 0) {
            if (gate != nullptr) gv = *reinterpret_cast<const uint4*>(gate + crow * kD + ch * 8);
            *reinterpret_cast<uint4*>(out_comb + crow * kD + ch * 8) = combine_x8<elem_t>(sv4, cv, gv, gate != nullptr);
          }
        }
      }
      if (st < 64) {
        const float l = l_col[st];
        lse2[row0 + st] = (redo || n_pairs == 0) ? NAN : m_col[st] + log2f(l);
      }
      named_barrier(1, kEwThreads);             // everyone has read the flag, the statistics and the staging buffer
      if (st == 0) *flag = 0u;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(PL_EMPTY + b));
    }
    if (!ok) report_timeout(45);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}
