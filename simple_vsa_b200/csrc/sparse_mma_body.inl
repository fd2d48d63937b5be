// Warp-level kernels and their launchers for ONE head dim.  The including file opens a namespace, defines there
// `constexpr int kD` (64 or 128) and includes this file: tiles are 64 tokens x kD dims, rows of kD*2 bytes in
// kD/8 chunks of 16 bytes, swizzled chunk ^ (row & 7) (conflict-free for ldmatrix at both row pitches).
constexpr int kTileBytes = kTile * kD * 2;
constexpr int kChunks = kD / 8;               // 16-byte chunks per tile row
// resident CTAs per SM the register allocation aims for: the 64-wide kernels hold half the accumulators (four CTAs
// of the forward fit in 128 registers a thread without spilling, three of the backward passes in 168)
constexpr int kMinCtasFwd = kD == 64 ? 4 : 2;
constexpr int kMinCtasBwd = kD == 64 ? 3 : 2;

__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  return (uint32_t)(row * (kD * 2) + ((chunk ^ (row & 7)) << 4));
}

// Stage one 64 x kD tile of 16-bit elements; rows >= valid_rows are zero-filled instead of read.
template <typename T>
__device__ __forceinline__ void stage_tile(uint32_t smem_base, const T* __restrict__ g, int valid_rows, int tid) {
#pragma unroll
  for (int i = 0; i < kTile * kChunks / kThreads; ++i) {
    const int c = tid + i * kThreads;
    const int row = c / kChunks, ch = c % kChunks;
    const uint32_t dst = smem_base + tile_off(row, ch);
    if (row < valid_rows) {
      cp_async16(dst, g + row * kD + ch * 8);
    } else {
      asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(dst), "r"(0u));
    }
  }
}

// A fragment (16 rows x 16 k) of a row-major tile: rows row0.., k-chunk pair ks.
__device__ __forceinline__ void load_a(uint32_t base, int row0, int ks, int lane, uint32_t (&a)[4]) {
  const int row = row0 + (lane & 15);
  ldsm_x4(base + tile_off(row, ks * 2 + (lane >> 4)), a[0], a[1], a[2], a[3]);
}
// B fragments for two n-tiles (16 tile rows n0..n0+15 as N) with K along the tile's columns.
__device__ __forceinline__ void load_b_kcontig(uint32_t base, int n0, int ks, int lane, uint32_t (&b)[4]) {
  const int row = n0 + (lane & 7) + ((lane >> 4) << 3);
  ldsm_x4(base + tile_off(row, ks * 2 + ((lane >> 3) & 1)), b[0], b[1], b[2], b[3]);
}
// B fragments for two n-tiles (16 tile columns starting at chunk pair dp) with K along the tile's rows k0..k0+15.
__device__ __forceinline__ void load_b_ncontig(uint32_t base, int k0, int dp, int lane, uint32_t (&b)[4]) {
  const int row = k0 + (lane & 7) + (((lane >> 3) & 1) << 3);
  ldsm_x4_t(base + tile_off(row, dp * 2 + (lane >> 4)), b[0], b[1], b[2], b[3]);
}

__device__ __forceinline__ float quad_max(float x) {
  x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 1));
  return fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 2));
}
__device__ __forceinline__ float quad_sum(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  return x + __shfl_xor_sync(0xffffffffu, x, 2);
}

// Write a warp's 16 x kD fp32 accumulator (n-tiles of mma layout) as 16-bit elements into its
// rows of a swizzled tile, then copy those rows to global memory with 16-byte stores.
// With `comb` the gated combine with the pooled branch (pooled_row = the query block's pooled output row, gate_g
// optional) is written beside it.
template <typename T>
__device__ __forceinline__ void store_warp_rows(uint8_t* tile, uint32_t tile_u32, const float (&acc)[kD / 8][4], float mul0,
                                                float mul1, T* __restrict__ g, int warp, int lane,
                                                const T* __restrict__ pooled_row = nullptr,
                                                const T* __restrict__ gate_g = nullptr,
                                                T* __restrict__ comb = nullptr, long long comb_row0 = 0,
                                                RasterMap comb_map = RasterMap{nullptr, 0, 1}, long long bh = 0,
                                                long long token0 = 0) {
  const int gq = lane >> 2, t = lane & 3;
  const int r0 = warp * 16 + gq, r1 = r0 + 8;
#pragma unroll
  for (int nt = 0; nt < kD / 8; ++nt) {
    *reinterpret_cast<uint32_t*>(tile + tile_off(r0, nt) + 4 * t) = Elem<T>::pack(acc[nt][0] * mul0, acc[nt][1] * mul0);
    *reinterpret_cast<uint32_t*>(tile + tile_off(r1, nt) + 4 * t) = Elem<T>::pack(acc[nt][2] * mul1, acc[nt][3] * mul1);
  }
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 16 * kChunks / 32; ++i) {
    const int c = lane + 32 * i;
    const int row = warp * 16 + c / kChunks, ch = c % kChunks;
    const uint4 val = *reinterpret_cast<const uint4*>(tile + tile_off(row, ch));
    *reinterpret_cast<uint4*>(g + row * kD + ch * 8) = val;
    if (comb != nullptr) {   // gate and comb are whole-tensor pointers: tile order (comb_row0 + row) or raster rows
      const uint4 cv = *reinterpret_cast<const uint4*>(pooled_row + ch * 8);
      uint4 gv = make_uint4(0, 0, 0, 0);
      const long long crow = comb_map.map == nullptr ? comb_row0 + row : raster_row(comb_map, bh, token0 + row);
      if (crow >= 0) {
        if (gate_g != nullptr) gv = *reinterpret_cast<const uint4*>(gate_g + crow * kD + ch * 8);
        *reinterpret_cast<uint4*>(comb + crow * kD + ch * 8) = combine_x8<T>(val, cv, gv, gate_g != nullptr);
      }
    }
  }
  (void)tile_u32;
}

// ------------------------------------------------------------------------------------------
// Forward.  grid = (Lq/64, BH); one CTA = 64 query rows (4 warps x 16 rows).
// ------------------------------------------------------------------------------------------
template <typename T, int SUB>
__global__ void __launch_bounds__(kThreads, kMinCtasFwd)
sparse_fwd_mma_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                      const int32_t* __restrict__ selected, const int32_t* __restrict__ kv_sizes,
                      T* __restrict__ out, float* __restrict__ lse2, const T* __restrict__ out_c,
                      const T* __restrict__ gate, T* __restrict__ out_comb, long long Lq, long long Lkv,
                      long long kv_shard, int topk, float scale, int redo_only, RasterMap comb_map) {
  extern __shared__ __align__(128) uint8_t smem[];
  if (redo_only) {   // only tiles the tcgen05 forward marked with a NaN statistic are recomputed
    const float mark = lse2[(long long)blockIdx.y * Lq + (long long)blockIdx.x * kTile];
    if (mark == mark) return;
  }
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sK = sQ + kTileBytes;          // two stages
  const uint32_t sV = sK + 2 * kTileBytes;      // two stages
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, t = lane & 3;
  const int qtile = blockIdx.x;
  const long long bh = blockIdx.y;
  const int Qb = (int)(Lq / (kTile * SUB));
  const int qb = qtile / SUB;
  const int32_t* sel = selected + (bh * Qb + qb) * (long long)topk;
  // rows of a key tile in the K/V tensors (a sequence-parallel gather leaves them shard-major: see kv_tensor_row)
  auto kv_row = [&](long long token) -> long long { return kv_tensor_row(bh, gridDim.y, token, kv_shard); };
  const int n_iter = topk * SUB;
  const float c = scale * kLog2e;

  auto tile_valid = [&](int it, int& kvb) -> int {
    kvb = sel[it / SUB];
    // an id outside the table is an empty tile, as route inversion treats it
    const int left = (unsigned)kvb < (unsigned)(Lkv / (kTile * SUB)) ? kv_sizes[kvb] - (it % SUB) * kTile : 0;
    return left < 0 ? 0 : (left > kTile ? kTile : left);
  };
  auto next_live = [&](int it, int& kvb, int& valid) -> int {
    for (; it < n_iter; ++it) {
      valid = tile_valid(it, kvb);
      if (valid > 0) return it;
    }
    valid = 0;
    return n_iter;
  };

  stage_tile(sQ, q + (bh * Lq + (long long)qtile * kTile) * kD, kTile, tid);
  int kvb = 0, valid = 0;
  int it = next_live(0, kvb, valid);
  if (it < n_iter) {
    const long long row0 = kv_row((long long)kvb * (kTile * SUB) + (it % SUB) * kTile);
    stage_tile(sK, k + row0 * kD, kTile, tid);
    stage_tile(sV, v + row0 * kD, valid, tid);
  }
  cp_async_commit();

  float o[kD / 8][4];
#pragma unroll
  for (int i = 0; i < kD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.f, 0.f};
  uint32_t qf[kD / 16][4];
  bool q_loaded = false;
  int stage = 0;

  while (it < n_iter) {
    int nkvb = 0, nvalid = 0;
    const int nxt = next_live(it + 1, nkvb, nvalid);
    if (nxt < n_iter) {
      const long long row0 = kv_row((long long)nkvb * (kTile * SUB) + (nxt % SUB) * kTile);
      stage_tile(sK + (stage ^ 1) * kTileBytes, k + row0 * kD, kTile, tid);
      stage_tile(sV + (stage ^ 1) * kTileBytes, v + row0 * kD, nvalid, tid);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (!q_loaded) {
#pragma unroll
      for (int ks = 0; ks < kD / 16; ++ks) load_a(sQ, warp * 16, ks, lane, qf[ks]);
      q_loaded = true;
    }
    const uint32_t cK = sK + stage * kTileBytes, cV = sV + stage * kTileBytes;

    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < kD / 16; ++ks) {
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b[4];
        load_b_kcontig(cK, np * 16, ks, lane, b);
        mma_16816<T>(s[2 * np], qf[ks], b[0], b[1]);
        mma_16816<T>(s[2 * np + 1], qf[ks], b[2], b[3]);
      }
    }
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = nt * 8 + 2 * t + (j & 1);
        const float x = col < valid ? s[nt][j] * c : -INFINITY;
        s[nt][j] = x;
        tmax[j >> 1] = fmaxf(tmax[j >> 1], x);
      }
    }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const float nm = fmaxf(row_max[r], quad_max(tmax[r]));   // finite: the tile has a valid column
      alpha[r] = fast_exp2(row_max[r] - nm);
      row_max[r] = nm;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float p = fast_exp2(s[nt][j] - row_max[j >> 1]);
        s[nt][j] = p;
        psum[j >> 1] += p;
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) row_sum[r] = row_sum[r] * alpha[r] + psum[r];
#pragma unroll
    for (int nt = 0; nt < kD / 8; ++nt) {
      o[nt][0] *= alpha[0]; o[nt][1] *= alpha[0];
      o[nt][2] *= alpha[1]; o[nt][3] *= alpha[1];
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t pa[4];
      pa[0] = Elem<T>::pack(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = Elem<T>::pack(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = Elem<T>::pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = Elem<T>::pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int dp = 0; dp < kD / 16; ++dp) {
        uint32_t b[4];
        load_b_ncontig(cV, kk * 16, dp, lane, b);
        mma_16816<T>(o[2 * dp], pa, b[0], b[1]);
        mma_16816<T>(o[2 * dp + 1], pa, b[2], b[3]);
      }
    }
    __syncthreads();
    it = nxt; kvb = nkvb; valid = nvalid; stage ^= 1;
  }
  cp_async_wait<0>();
  __syncthreads();

  float inv[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    row_sum[r] = quad_sum(row_sum[r]);
    inv[r] = 1.f / row_sum[r];
  }
  const long long row0 = bh * Lq + (long long)qtile * kTile;
  T* og = out + row0 * kD;
  if (out_comb != nullptr)
    store_warp_rows(smem, sQ, o, inv[0], inv[1], og, warp, lane, out_c + (bh * Qb + qb) * (long long)kD, gate, out_comb, row0,
                    comb_map, bh, (long long)qtile * kTile);
  else
    store_warp_rows(smem, sQ, o, inv[0], inv[1], og, warp, lane);
  if (lse2 && t == 0) {
    float* lg = lse2 + bh * Lq + (long long)qtile * kTile + warp * 16 + gq;
    lg[0] = row_max[0] + log2f(row_sum[0]);
    lg[8] = row_max[1] + log2f(row_sum[1]);
  }
}

// ------------------------------------------------------------------------------------------
// dQ (query-owned).  grid = (Lq/64, BH).  Also writes delta = rowsum(out_s * dout).
// ------------------------------------------------------------------------------------------
template <typename T, int SUB>
__global__ void __launch_bounds__(kThreads, kMinCtasBwd)
sparse_dq_mma_kernel(const T* __restrict__ dout, const T* __restrict__ q, const T* __restrict__ k,
                     const T* __restrict__ v, const T* __restrict__ out_s, const float* __restrict__ lse2,
                     const int32_t* __restrict__ selected, const int32_t* __restrict__ kv_sizes,
                     float* __restrict__ delta, T* __restrict__ dq, long long Lq, long long Lkv, int topk,
                     float scale) {
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sdO = sQ + kTileBytes;
  const uint32_t sK = sdO + kTileBytes;
  const uint32_t sV = sK + 2 * kTileBytes;
  float* sStat = reinterpret_cast<float*>(smem + 6 * kTileBytes);   // [0..63] lse, [64..127] delta
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, t = lane & 3;
  const int qtile = blockIdx.x;
  const long long bh = blockIdx.y;
  const int Qb = (int)(Lq / (kTile * SUB));
  const int qb = qtile / SUB;
  const int32_t* sel = selected + (bh * Qb + qb) * (long long)topk;
  const T* kbase = k + bh * Lkv * kD;
  const T* vbase = v + bh * Lkv * kD;
  const long long qrow0 = bh * Lq + (long long)qtile * kTile;
  const int n_iter = topk * SUB;
  const float c = scale * kLog2e;

  auto tile_valid = [&](int it, int& kvb) -> int {
    kvb = sel[it / SUB];
    // an id outside the table is an empty tile, as route inversion treats it
    const int left = (unsigned)kvb < (unsigned)(Lkv / (kTile * SUB)) ? kv_sizes[kvb] - (it % SUB) * kTile : 0;
    return left < 0 ? 0 : (left > kTile ? kTile : left);
  };
  auto next_live = [&](int it, int& kvb, int& valid) -> int {
    for (; it < n_iter; ++it) {
      valid = tile_valid(it, kvb);
      if (valid > 0) return it;
    }
    valid = 0;
    return n_iter;
  };

  stage_tile(sQ, q + qrow0 * kD, kTile, tid);
  stage_tile(sdO, dout + qrow0 * kD, kTile, tid);
  int kvb = 0, valid = 0;
  int it = next_live(0, kvb, valid);
  if (it < n_iter) {
    const long long row0 = (long long)kvb * (kTile * SUB) + (it % SUB) * kTile;
    stage_tile(sK, kbase + row0 * kD, valid, tid);
    stage_tile(sV, vbase + row0 * kD, valid, tid);
  }
  cp_async_commit();

  {  // delta: two threads per row, half of the dims each, straight from global memory
    const int row = tid >> 1, half = tid & 1;
    const uint4* po = reinterpret_cast<const uint4*>(out_s + (qrow0 + row) * kD + half * (kD / 2));
    const uint4* pd = reinterpret_cast<const uint4*>(dout + (qrow0 + row) * kD + half * (kD / 2));
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < kD / 16; ++i) {
      const uint4 a = po[i], b = pd[i];
      const T* ea = reinterpret_cast<const T*>(&a);
      const T* eb = reinterpret_cast<const T*>(&b);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc = fmaf(Elem<T>::to(ea[j]), Elem<T>::to(eb[j]), acc);
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    if (half == 0) {
      sStat[64 + row] = acc;
      delta[qrow0 + row] = acc;
      sStat[row] = lse2[qrow0 + row];
    }
  }

  float acc_dq[kD / 8][4];
#pragma unroll
  for (int i = 0; i < kD / 8; ++i) acc_dq[i][0] = acc_dq[i][1] = acc_dq[i][2] = acc_dq[i][3] = 0.f;
  float lse_r[2] = {0.f, 0.f}, dl_r[2] = {0.f, 0.f};
  bool stats_loaded = false;
  int stage = 0;

  while (it < n_iter) {
    int nkvb = 0, nvalid = 0;
    const int nxt = next_live(it + 1, nkvb, nvalid);
    if (nxt < n_iter) {
      const long long row0 = (long long)nkvb * (kTile * SUB) + (nxt % SUB) * kTile;
      stage_tile(sK + (stage ^ 1) * kTileBytes, kbase + row0 * kD, nvalid, tid);
      stage_tile(sV + (stage ^ 1) * kTileBytes, vbase + row0 * kD, nvalid, tid);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (!stats_loaded) {
      lse_r[0] = sStat[warp * 16 + gq];      lse_r[1] = sStat[warp * 16 + gq + 8];
      dl_r[0] = sStat[64 + warp * 16 + gq];  dl_r[1] = sStat[64 + warp * 16 + gq + 8];
      stats_loaded = true;
    }
    const uint32_t cK = sK + stage * kTileBytes, cV = sV + stage * kTileBytes;

    float s[8][4], dp[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
      dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
    }
#pragma unroll
    for (int ks = 0; ks < kD / 16; ++ks) {
      uint32_t aq[4], ad[4];
      load_a(sQ, warp * 16, ks, lane, aq);
      load_a(sdO, warp * 16, ks, lane, ad);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b[4];
        load_b_kcontig(cK, np * 16, ks, lane, b);
        mma_16816<T>(s[2 * np], aq, b[0], b[1]);
        mma_16816<T>(s[2 * np + 1], aq, b[2], b[3]);
        load_b_kcontig(cV, np * 16, ks, lane, b);
        mma_16816<T>(dp[2 * np], ad, b[0], b[1]);
        mma_16816<T>(dp[2 * np + 1], ad, b[2], b[3]);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = nt * 8 + 2 * t + (j & 1);
        const float p = col < valid ? fast_exp2(s[nt][j] * c - lse_r[j >> 1]) : 0.f;
        s[nt][j] = col < valid ? p * (dp[nt][j] - dl_r[j >> 1]) * scale : 0.f;
      }
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t da[4];
      da[0] = Elem<T>::pack(s[2 * kk][0], s[2 * kk][1]);
      da[1] = Elem<T>::pack(s[2 * kk][2], s[2 * kk][3]);
      da[2] = Elem<T>::pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      da[3] = Elem<T>::pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int d2 = 0; d2 < kD / 16; ++d2) {
        uint32_t b[4];
        load_b_ncontig(cK, kk * 16, d2, lane, b);
        mma_16816<T>(acc_dq[2 * d2], da, b[0], b[1]);
        mma_16816<T>(acc_dq[2 * d2 + 1], da, b[2], b[3]);
      }
    }
    __syncthreads();
    it = nxt; kvb = nkvb; valid = nvalid; stage ^= 1;
  }
  cp_async_wait<0>();
  __syncthreads();
  store_warp_rows(smem, sQ, acc_dq, 1.f, 1.f, dq + qrow0 * kD, warp, lane);
}

// ------------------------------------------------------------------------------------------
// dK/dV (key-owned).  grid = (Lkv/64, BH); one CTA = one 64-row key tile, looping over the
// query blocks that selected its logical block (CSR in-edges), each SUB query tiles long.
// ------------------------------------------------------------------------------------------
template <typename T, int SUB>
__global__ void __launch_bounds__(kThreads, kMinCtasBwd)
sparse_dkdv_mma_kernel(const T* __restrict__ dout, const T* __restrict__ q, const T* __restrict__ k,
                       const T* __restrict__ v, const float* __restrict__ lse2, const float* __restrict__ delta,
                       const int32_t* __restrict__ counts, const int32_t* __restrict__ offsets,
                       const int32_t* __restrict__ inverse, const int32_t* __restrict__ kv_sizes,
                       T* __restrict__ dk, T* __restrict__ dv, long long Lq, long long Lkv, int topk,
                       float scale) {
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sK = smem_u32(smem);
  const uint32_t sV = sK + kTileBytes;
  const uint32_t sQ = sV + kTileBytes;            // two stages
  const uint32_t sdO = sQ + 2 * kTileBytes;       // two stages
  float* sStat = reinterpret_cast<float*>(smem + 6 * kTileBytes);   // [stage][lse 64 | delta 64]
  const uint32_t sStat_u32 = sK + 6 * kTileBytes;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, t = lane & 3;
  const int ktile = blockIdx.x;
  const long long bh = blockIdx.y;
  const int Kb = (int)(Lkv / (kTile * SUB));
  const int Qb = (int)(Lq / (kTile * SUB));
  const int kvb = ktile / SUB;
  const int sub = ktile % SUB;
  int valid = kv_sizes[kvb] - sub * kTile;
  valid = valid < 0 ? 0 : (valid > kTile ? kTile : valid);
  const long long krow0 = bh * Lkv + (long long)ktile * kTile;
  const int cnt = valid > 0 ? counts[bh * Kb + kvb] : 0;
  const int32_t* inv = inverse + bh * (long long)Qb * topk + offsets[bh * Kb + kvb];
  const int n_iter = cnt * SUB;
  const float c = scale * kLog2e;
  const T* qbase = q + bh * Lq * kD;
  const T* dobase = dout + bh * Lq * kD;

  auto stage_q = [&](int it, int stg) {
    const long long row0 = (long long)inv[it / SUB] * (kTile * SUB) + (it % SUB) * kTile;
    stage_tile(sQ + stg * kTileBytes, qbase + row0 * kD, kTile, tid);
    stage_tile(sdO + stg * kTileBytes, dobase + row0 * kD, kTile, tid);
    if (tid < 16) cp_async16(sStat_u32 + stg * 512 + tid * 16, lse2 + bh * Lq + row0 + tid * 4);
    else if (tid < 32) cp_async16(sStat_u32 + stg * 512 + 256 + (tid - 16) * 16, delta + bh * Lq + row0 + (tid - 16) * 4);
  };

  stage_tile(sK, k + krow0 * kD, valid, tid);
  stage_tile(sV, v + krow0 * kD, valid, tid);
  if (n_iter > 0) stage_q(0, 0);
  cp_async_commit();

  float acc_dk[kD / 8][4], acc_dv[kD / 8][4];
#pragma unroll
  for (int i = 0; i < kD / 8; ++i) {
    acc_dk[i][0] = acc_dk[i][1] = acc_dk[i][2] = acc_dk[i][3] = 0.f;
    acc_dv[i][0] = acc_dv[i][1] = acc_dv[i][2] = acc_dv[i][3] = 0.f;
  }
  const bool row_ok[2] = {warp * 16 + gq < valid, warp * 16 + gq + 8 < valid};

  for (int it = 0; it < n_iter; ++it) {
    const int stage = it & 1;
    if (it + 1 < n_iter) stage_q(it + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t cQ = sQ + stage * kTileBytes, cdO = sdO + stage * kTileBytes;
    const float* st_lse = sStat + stage * 128;
    const float* st_dl = st_lse + 64;

#pragma unroll 1
    for (int h = 0; h < 2; ++h) {
      float s[4][4], dp[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
        dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
      }
#pragma unroll
      for (int ks = 0; ks < kD / 16; ++ks) {
        uint32_t ak[4], av[4];
        load_a(sK, warp * 16, ks, lane, ak);
        load_a(sV, warp * 16, ks, lane, av);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          uint32_t b[4];
          load_b_kcontig(cQ, h * 32 + np * 16, ks, lane, b);
          mma_16816<T>(s[2 * np], ak, b[0], b[1]);
          mma_16816<T>(s[2 * np + 1], ak, b[2], b[3]);
          load_b_kcontig(cdO, h * 32 + np * 16, ks, lane, b);
          mma_16816<T>(dp[2 * np], av, b[0], b[1]);
          mma_16816<T>(dp[2 * np + 1], av, b[2], b[3]);
        }
      }
      // transposed tile: rows are key tokens, columns are query rows of this half
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int qi = h * 32 + nt * 8 + 2 * t + (j & 1);
          const bool ok = row_ok[j >> 1];
          const float p = ok ? fast_exp2(s[nt][j] * c - st_lse[qi]) : 0.f;
          s[nt][j] = p;
          dp[nt][j] = ok ? p * (dp[nt][j] - st_dl[qi]) : 0.f;
        }
      }
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        uint32_t pa[4], da[4];
        pa[0] = Elem<T>::pack(s[2 * kk][0], s[2 * kk][1]);
        pa[1] = Elem<T>::pack(s[2 * kk][2], s[2 * kk][3]);
        pa[2] = Elem<T>::pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pa[3] = Elem<T>::pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
        da[0] = Elem<T>::pack(dp[2 * kk][0], dp[2 * kk][1]);
        da[1] = Elem<T>::pack(dp[2 * kk][2], dp[2 * kk][3]);
        da[2] = Elem<T>::pack(dp[2 * kk + 1][0], dp[2 * kk + 1][1]);
        da[3] = Elem<T>::pack(dp[2 * kk + 1][2], dp[2 * kk + 1][3]);
#pragma unroll
        for (int d2 = 0; d2 < kD / 16; ++d2) {
          uint32_t b[4];
          load_b_ncontig(cdO, h * 32 + kk * 16, d2, lane, b);
          mma_16816<T>(acc_dv[2 * d2], pa, b[0], b[1]);
          mma_16816<T>(acc_dv[2 * d2 + 1], pa, b[2], b[3]);
          load_b_ncontig(cQ, h * 32 + kk * 16, d2, lane, b);
          mma_16816<T>(acc_dk[2 * d2], da, b[0], b[1]);
          mma_16816<T>(acc_dk[2 * d2 + 1], da, b[2], b[3]);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();
  store_warp_rows(smem, sK, acc_dk, scale, scale, dk + krow0 * kD, warp, lane);
  store_warp_rows(smem + kTileBytes, sV, acc_dv, 1.f, 1.f, dv + krow0 * kD, warp, lane);
}

constexpr int kFwdSmem = 5 * kTileBytes;
constexpr int kDqSmem = 6 * kTileBytes + 512;
constexpr int kDkdvSmem = 6 * kTileBytes + 1024;

template <typename T>
int launch_fwd(const void* q, const void* k, const void* v, const int32_t* selected, const int32_t* kv_sizes,
                      void* out, float* lse2, int64_t BH, int64_t Lq, int64_t Lkv, int be, int topk, float scale,
                      bool redo_only, cudaStream_t st, const void* out_c, const void* gate, void* out_comb, int64_t kv_shard,
                      RasterMap comb_map) {
  dim3 grid((unsigned)(Lq / kTile), (unsigned)BH);
  auto launch = [&](auto kern) -> int {
    const int rc = set_smem(kern, kFwdSmem, "sparse forward");
    if (rc) return rc;
    kern<<<grid, kThreads, kFwdSmem, st>>>((const T*)q, (const T*)k, (const T*)v, selected, kv_sizes, (T*)out, lse2,
                                           (const T*)out_c, (const T*)gate, (T*)out_comb, Lq, Lkv, kv_shard, topk, scale,
                                           redo_only ? 1 : 0, comb_map);
    return check_launch("sparse_fwd_mma_kernel");
  };
  return be == 64 ? launch(sparse_fwd_mma_kernel<T, 1>) : be == 128 ? launch(sparse_fwd_mma_kernel<T, 2>) : launch(sparse_fwd_mma_kernel<T, 4>);
}

template <typename T>
int launch_dq(const void* dout, const void* q, const void* k, const void* v, const void* out_s, const float* lse2,
                     const int32_t* selected, const int32_t* kv_sizes, float* delta, void* dq, int64_t BH, int64_t Lq,
                     int64_t Lkv, int be, int topk, float scale, cudaStream_t st) {
  dim3 grid((unsigned)(Lq / kTile), (unsigned)BH);
  auto launch = [&](auto kern) -> int {
    const int rc = set_smem(kern, kDqSmem, "sparse dQ");
    if (rc) return rc;
    kern<<<grid, kThreads, kDqSmem, st>>>((const T*)dout, (const T*)q, (const T*)k, (const T*)v, (const T*)out_s, lse2,
                                          selected, kv_sizes, delta, (T*)dq, Lq, Lkv, topk, scale);
    return check_launch("sparse_dq_mma_kernel");
  };
  return be == 64 ? launch(sparse_dq_mma_kernel<T, 1>) : be == 128 ? launch(sparse_dq_mma_kernel<T, 2>) : launch(sparse_dq_mma_kernel<T, 4>);
}

template <typename T>
int launch_dkdv(const void* dout, const void* q, const void* k, const void* v, const float* lse2,
                       const float* delta, const int32_t* counts, const int32_t* offsets, const int32_t* inverse,
                       const int32_t* kv_sizes, void* dk, void* dv, int64_t BH, int64_t Lq, int64_t Lkv, int be, int topk,
                       float scale, cudaStream_t st) {
  dim3 grid((unsigned)(Lkv / kTile), (unsigned)BH);
  auto launch = [&](auto kern) -> int {
    const int rc = set_smem(kern, kDkdvSmem, "sparse dK/dV");
    if (rc) return rc;
    kern<<<grid, kThreads, kDkdvSmem, st>>>((const T*)dout, (const T*)q, (const T*)k, (const T*)v, lse2, delta, counts,
                                            offsets, inverse, kv_sizes, (T*)dk, (T*)dv, Lq, Lkv, topk, scale);
    return check_launch("sparse_dkdv_mma_kernel");
  };
  return be == 64 ? launch(sparse_dkdv_mma_kernel<T, 1>) : be == 128 ? launch(sparse_dkdv_mma_kernel<T, 2>) : launch(sparse_dkdv_mma_kernel<T, 4>);
}

