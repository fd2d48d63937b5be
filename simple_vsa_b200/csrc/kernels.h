// Internal launchers shared between the translation units of the library.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace vsa {

// ---- scalar kernels (generic_kernels.cu) -------------------------------------------------
int block_mean_fwd(const void* const* x, void* const* out, const int32_t* const* sizes, const int64_t* L,
                   int ntensors, int64_t BH, int D, int be, int dtype, cudaStream_t st);
int block_mean_bwd(void* dx, const void* dmean, const int32_t* sizes, int64_t BH, int64_t L, int D, int be,
                   int dtype, bool accumulate, cudaStream_t st);
int coarse_fwd(const void* qc, const void* kc, const void* vc, void* scores, void* probs, void* out_c, int64_t BH,
               int Qb, int Kb, int D, float scale, int dtype, cudaStream_t st);
int coarse_bwd(const void* d_out_c, const void* out_c, const void* qc, const void* kc, const void* vc,
               const void* probs, void* ds, float* rowdot, void* dqc, void* dkc, void* dvc, int64_t BH, int Qb, int Kb,
               int D, float scale, int dtype, cudaStream_t st);
int softmax_rows(const void* scores, void* probs, int64_t rows, int n, int dtype, cudaStream_t st);
int rowdot_rows(const void* a, const void* b, float* out, int64_t rows, int D, int dtype, cudaStream_t st);
int topk_select(const void* scores, int32_t* selected, int64_t rows, int Kb, int topk, int dtype, cudaStream_t st);
// packed: rows hold (query block << 11) | slot of the key block in that query block's route, instead of query block ids
int route_invert(const int32_t* selected, int32_t* counts, int32_t* offsets, int32_t* inverse, int32_t* cursor,
                 int64_t BH, int Qb, int Kb, int topk, cudaStream_t st, bool packed = false);
int route_invert_static(const int32_t* selected, int32_t* counts, int32_t* offsets, int32_t* inverse, int64_t BH,
                        int Qb, int Kb, int topk, cudaStream_t st);
int gather_rows(const void* src, const int32_t* map, void* dst, int64_t batch, int64_t src_rows, int64_t dst_rows,
                int64_t row_bytes, cudaStream_t st);
// raster [B][S][H][row] <-> tile order [B][H][L][row] in one pass (to_tiled: dst rows = L, zero fill where map < 0)
int gather_rows_heads(const void* src, const int32_t* map, void* dst, int64_t batch, int heads, int64_t src_rows,
                      int64_t dst_rows, int64_t row_bytes, bool to_tiled, cudaStream_t st);
int combine_fwd(const void* out_s, const void* out_c, const void* gate, void* out, int64_t BH, int64_t Lq, int D,
                int be, int dtype, cudaStream_t st);
int combine_bwd(const void* dout, const void* gate, const void* out_c, void* d_out_c, void* dgate, int64_t BH,
                int64_t Lq, int D, int be, int dtype, cudaStream_t st);
// combine backward reading dout and the gate, and writing dgate, at raster rows; also stores dout in tile order
int combine_bwd_raster(const void* dout_raster, const void* gate_raster, const void* out_c, void* d_out_c,
                       void* dgate_raster, void* dout_tiled, const int32_t* map, int64_t raster_rows, int heads,
                       int64_t BH, int64_t Lq, int D, int be, int dtype, cudaStream_t st);
int sparse_fwd_scalar(const void* q, const void* k, const void* v, const int32_t* selected, const int32_t* kv_sizes,
                      void* out, float* lse2, int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk,
                      float scale, int dtype, cudaStream_t st);
int sparse_dq_scalar(const void* dout, const void* q, const void* k, const void* v, const void* out_s,
                     const float* lse2, const int32_t* selected, const int32_t* kv_sizes, float* delta, void* dq,
                     int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk, float scale, int dtype,
                     cudaStream_t st);
int sparse_dkdv_scalar(const void* dout, const void* q, const void* k, const void* v, const float* lse2,
                       const float* delta, const int32_t* counts, const int32_t* offsets, const int32_t* inverse,
                       const int32_t* kv_sizes, void* dk, void* dv, int64_t BH, int64_t Lq, int64_t Lkv, int D, int be,
                       int topk, float scale, int dtype, cudaStream_t st);

// ---- tensor-core kernels, bf16 or fp16, head dim 64 or 128, block volume 64, 128 or 256 (sparse_mma.cu) ------
bool sparse_tc_eligible(int D, int be, int dtype);
// redo_only: recompute only the 64-row query tiles whose first lse2 entry is NaN (the marker the
// tcgen05 forward leaves on a tile whose fixed softmax shift ran out of range).
// out_comb (optional): out_s + out_c[block] * gate is written there as well (gate may be null)
// dtype: the forward also exists for fp16 (it is the exact recomputation behind the fp16 tcgen05 forward)
int sparse_fwd_tc(const void* q, const void* k, const void* v, const int32_t* selected, const int32_t* kv_sizes,
                  void* out, float* lse2, int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk, float scale,
                  int dtype, bool redo_only, cudaStream_t st, const void* out_c = nullptr, const void* gate = nullptr,
                  void* out_comb = nullptr, int64_t kv_shard = 0, const int32_t* comb_map = nullptr,
                  int64_t comb_rows = 0, int comb_heads = 1);
int sparse_dq_tc(const void* dout, const void* q, const void* k, const void* v, const void* out_s, const float* lse2,
                 const int32_t* selected, const int32_t* kv_sizes, float* delta, void* dq, int64_t BH, int64_t Lq,
                 int64_t Lkv, int D, int be, int topk, float scale, int dtype, cudaStream_t st);
int sparse_dkdv_tc(const void* dout, const void* q, const void* k, const void* v, const float* lse2,
                   const float* delta, const int32_t* counts, const int32_t* offsets, const int32_t* inverse,
                   const int32_t* kv_sizes, void* dk, void* dv, int64_t BH, int64_t Lq, int64_t Lkv, int D, int be,
                   int topk, float scale, int dtype, cudaStream_t st);

// ---- tcgen05 / TMA kernels, bf16 or fp16 by `dtype` (sparse_umma.cu) -----------------------------------------------------
bool sparse_umma_eligible(int D, int be, int dtype, int topk);
int sparse_fwd_umma(const void* q, const void* k, const void* v, const int32_t* selected, const int32_t* kv_sizes,
                    void* out, float* lse2, int64_t BH, int64_t Lq, int64_t Lkv, int be, int topk, float scale,
                    int dtype, cudaStream_t st, const void* out_c = nullptr, const void* gate = nullptr,
                    void* out_comb = nullptr, int64_t kv_shard = 0,   // kv_shard: tokens per shard of a shard-major K/V buffer (0 = ordinary layout)
                    const int32_t* comb_map = nullptr, int64_t comb_rows = 0, int comb_heads = 1);
// comb_map (optional, with out_comb): tile-order token -> raster row (or -1); gate is then read, and out_comb written, in
// the raster layout [B, comb_rows, comb_heads, D] (BH = B * comb_heads) instead of tile order
int sparse_dq_umma(const void* dout, const void* q, const void* k, const void* v, const void* out_s,
                   const float* lse2, const int32_t* selected, const int32_t* kv_sizes, float* delta, void* dq,
                   int64_t BH, int64_t Lq, int64_t Lkv, int be, int topk, float scale, int dtype,
                   cudaStream_t st, const void* dq_mean = nullptr, const int32_t* q_sizes = nullptr,
                   int64_t kv_shard = 0, const int32_t* out_map = nullptr, int64_t out_rows = 0, int out_heads = 1);
int sparse_dkdv_umma(const void* dout, const void* q, const void* k, const void* v, const float* lse2,
                     const float* delta, const int32_t* counts, const int32_t* offsets, const int32_t* inverse,
                     const int32_t* kv_sizes, void* dk, void* dv, int64_t BH, int64_t Lq, int64_t Lkv, int be, int topk,
                     float scale, int dtype, cudaStream_t st, const void* dk_mean = nullptr,
                     const void* dv_mean = nullptr, void* ds_ws = nullptr, int64_t kv_shard = 0,
                     const int32_t* out_map = nullptr, int64_t out_rows = 0, int out_heads = 1);
// out_map (optional): dq (dk, dv) rows are written at the token's raster row of a [B, out_rows, out_heads, D] tensor
// the backward that forms dS once: the key-owned pass (above, with ds_ws and packed edges) stores it, this
// query-owned pass multiplies it by K
int64_t sparse_ds_workspace_bytes(int64_t BH, int64_t Lq, int be, int topk);
int sparse_dq_from_ds_umma(const void* k, const int32_t* selected, const int32_t* kv_sizes, const void* ds_ws, void* dq,
                           int64_t BH, int64_t Lq, int64_t Lkv, int be, int topk, float scale, int dtype,
                           cudaStream_t st, const void* dq_mean = nullptr, const int32_t* q_sizes = nullptr);
bool coarse_umma_eligible(int Qb, int Kb, int D, int dtype);
int coarse_fwd_umma(const void* qc, const void* kc, const void* vc, void* scores, void* probs, void* out_c, int64_t BH,
                    int Qb, int Kb, int D, float scale, int dtype, cudaStream_t st);
int coarse_bwd_umma(const void* d_out_c, const void* out_c, const void* qc, const void* kc, const void* vc,
                    const void* probs, void* ds, float* rowdot, void* dqc, void* dkc, void* dvc, int64_t BH, int Qb,
                    int Kb, int D, float scale, int dtype, cudaStream_t st);
int umma_selftest(const void* a, const void* b, float* out, int mode, cudaStream_t st);
int wait_timeout_selftest(unsigned long long limit_ns, int* gave_up, cudaStream_t st);
int device_status_fetch_and_clear(int* status);

}  // namespace vsa
