// Pooled (block-vs-block) attention GEMMs on tcgen05.  Included by sparse_umma.cu.
//
// The six products of the pooled branch and its backward (vsa/common.py:164-166 of the reference and
// their autograd) are all C[b] = A[b] * B[b] with bf16 operands, fp32 accumulation and a 128-wide head
// dim on one side:
//     scores = q_c k_c^T          dP = dO_c v_c^T            (reduction over the head dim, K-major x K-major)
//     out_c  = P v_c              dQ_c = dS k_c               (reduction over key blocks,  K-major x N-major)
//     dV_c   = P^T dO_c           dK_c = dS^T q_c             (reduction over query blocks, M-major x N-major)
// One kernel covers them: a CTA owns a 128 x 128 output tile, streams 64-deep operand chunks through a
// three-stage TMA ring (3-D tensor maps over [batch, rows, cols]: whatever lies outside a batch slice is
// zero-filled by the TMA unit, so ragged M, N and K edges need no special code), issues four
// M128 x N128 x K16 MMAs per chunk into one TMEM accumulator, and finishes with an epilogue chosen at
// compile time: plain rounding store, the double rounding of the scores, or the softmax backward
// dS = P * (dP - rowdot) * scale.  Warp 0 = TMA producer, warp 1 = MMA issuer, warps 2-5 = epilogue.

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}

constexpr int kGemmStages = 3;
constexpr int kGemmChunk = 64;                 // reduction depth per stage
constexpr int kGemmOperandBytes = 128 * 128;   // 128 rows x 64 bf16, or 2 x (64 rows x 64 bf16): 16 KB either way
struct GemmSmem {
  static constexpr uint32_t a = 0;
  static constexpr uint32_t b = a + kGemmStages * kGemmOperandBytes;
  static constexpr uint32_t bars = b + kGemmStages * kGemmOperandBytes;
  static constexpr uint32_t misc = bars + 16 * 8;
  static constexpr uint32_t total = misc + 64;
};
enum GemmEpilogue { kEpiStore = 0, kEpiScores = 1, kEpiSoftmaxBwd = 2 };

// A_MN / B_MN: 0 = the operand's reduction dim is contiguous in memory ("K-major": rows are M or N),
//              1 = the operand's output dim is contiguous ("MN-major": rows are the reduction index).
template <int A_MN, int B_MN, int EPI>
__global__ void __launch_bounds__(192, 2)
coarse_gemm_umma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        elem_t* __restrict__ C, int M, int N, int K, float scale, const elem_t* __restrict__ probs,
                        const float* __restrict__ rowdot) {
  extern __shared__ uint8_t smem_raw[];
  if (*(volatile int*)&g_device_status != 0) return;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * 128, m0 = blockIdx.y * 128, batch = blockIdx.z;
  const int nk = (K + kGemmChunk - 1) / kGemmChunk;
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(sm + GemmSmem::misc);
  auto bar = [&](int i) -> uint32_t { return base + GemmSmem::bars + 8u * i; };   // full 0..2, empty 3..5, acc 6
  if (tid == 0) {
    for (int i = 0; i < kGemmStages; ++i) {
      mbar_init(bar(i), 1);
      mbar_init(bar(kGemmStages + i), 1);
    }
    mbar_init(bar(2 * kGemmStages), 1);
    fence_barrier_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(base + GemmSmem::misc, 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = misc[0];
  bool ok = true;

  if (warp == 0) {
    if (lane == 0) {
      for (int kc = 0; kc < nk && ok; ++kc) {
        const int s = kc % kGemmStages;
        ok = VSA_WAIT(bar(kGemmStages + s), ((kc / kGemmStages) & 1) ^ 1);
        if (!ok) break;
        const uint32_t a_dst = base + GemmSmem::a + s * kGemmOperandBytes;
        const uint32_t b_dst = base + GemmSmem::b + s * kGemmOperandBytes;
        mbar_arrive_expect_tx(bar(s), 2 * kGemmOperandBytes);
        if (A_MN) {          // source rows = reduction index, columns = M
          tma_load_3d(a_dst, &map_a, m0, kc * kGemmChunk, batch, bar(s));
          tma_load_3d(a_dst + 8192, &map_a, m0 + 64, kc * kGemmChunk, batch, bar(s));
        } else {             // source rows = M, columns = reduction index
          tma_load_3d(a_dst, &map_a, kc * kGemmChunk, m0, batch, bar(s));
        }
        if (B_MN) {
          tma_load_3d(b_dst, &map_b, n0, kc * kGemmChunk, batch, bar(s));
          tma_load_3d(b_dst + 8192, &map_b, n0 + 64, kc * kGemmChunk, batch, bar(s));
        } else {
          tma_load_3d(b_dst, &map_b, kc * kGemmChunk, n0, batch, bar(s));
        }
      }
      if (!ok) report_timeout(31);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(128, 128, A_MN, B_MN, kInFmt);
      constexpr uint32_t hi = desc_hi(1024);
      for (int kc = 0; kc < nk && ok; ++kc) {
        const int s = kc % kGemmStages;
        ok = VSA_WAIT(bar(s), (kc / kGemmStages) & 1);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_s = base + GemmSmem::a + s * kGemmOperandBytes;
        const uint32_t b_s = base + GemmSmem::b + s * kGemmOperandBytes;
        const uint32_t a0 = A_MN ? desc_lo(a_s, 8192) : desc_lo(a_s, 16);
        const uint32_t b0 = B_MN ? desc_lo(b_s, 8192) : desc_lo(b_s, 16);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)     // 16 reduction steps each: +32 bytes along a row, or +16 rows of 128 bytes
          mma_ss(tmem, desc_pack(a0 + (uint32_t)(A_MN ? ks * 128 : ks * 2), hi),
                 desc_pack(b0 + (uint32_t)(B_MN ? ks * 128 : ks * 2), hi), idesc, (kc > 0 || ks > 0) ? 1u : 0u);
        mma_commit(bar(kGemmStages + s));
      }
      if (ok) mma_commit(bar(2 * kGemmStages));
      if (!ok) report_timeout(32);
    }
  } else {
    const int quarter = warp & 3;
    const int m = m0 + quarter * 32 + lane;
    ok = VSA_WARP_WAIT(bar(2 * kGemmStages), 0);
    if (!ok && lane == 0) report_timeout(33);
    tc_fence_after();
    if (ok) {
      const long long row_off = ((long long)batch * M + m) * N;
      const float rd = (EPI == kEpiSoftmaxBwd && m < M) ? rowdot[(long long)batch * M + m] : 0.f;
#pragma unroll 1
      for (int c4 = 0; c4 < 4; ++c4) {
        uint32_t acc[32];
        tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + c4 * 32, acc);
        tmem_ld_wait();
        if (m >= M) continue;
        const int nb0 = n0 + c4 * 32;
#pragma unroll
        for (int j8 = 0; j8 < 4; ++j8) {
          const int n = nb0 + j8 * 8;
          if (n >= N) break;
          float v[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(acc[j8 * 8 + i]);
          if (EPI == kEpiScores) {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = Elem<elem_t>::to(Elem<elem_t>::from(v[i])) * scale;
          }
          if (EPI == kEpiSoftmaxBwd) {
            if (n + 8 <= N) {
              const uint4 praw = *reinterpret_cast<const uint4*>(probs + row_off + n);
              const elem_t* pe = reinterpret_cast<const elem_t*>(&praw);
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] = Elem<elem_t>::to(pe[i]) * (v[i] - rd) * scale;
            } else {
              for (int i = 0; i < 8 && n + i < N; ++i) v[i] = Elem<elem_t>::to(probs[row_off + n + i]) * (v[i] - rd) * scale;
            }
          }
          if (n + 8 <= N) {
            uint4 o;
            o.x = Elem<elem_t>::pack(v[0], v[1]); o.y = Elem<elem_t>::pack(v[2], v[3]);
            o.z = Elem<elem_t>::pack(v[4], v[5]); o.w = Elem<elem_t>::pack(v[6], v[7]);
            *reinterpret_cast<uint4*>(C + row_off + n) = o;
          } else {
            for (int i = 0; i < 8 && n + i < N; ++i) C[row_off + n + i] = Elem<elem_t>::from(v[i]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 128);
}
