// extern "C" boundary of the library: argument checks, dispatch between the
// tensor-core and the scalar kernels, error text.  No allocation, no host sync.
#include <atomic>
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "kernels.h"

namespace vsa {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

static std::atomic<long long> g_launches{0};

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (e == cudaSuccess) return VSA_OK;
  return fail(VSA_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
}

// VSA_B200_KERNELS selects the fine-attention kernels (for cross-checks): "scalar" = CUDA cores
// everywhere, "mma" = warp-level mma.sync kernels, anything else = tcgen05 where available.
static bool scalar_forced() {
  const char* e = std::getenv("VSA_B200_KERNELS");
  return e && std::strcmp(e, "scalar") == 0;
}
static bool mma_forced() {
  const char* e = std::getenv("VSA_B200_KERNELS");
  return e && std::strcmp(e, "mma") == 0;
}

static int check_dtype(int dtype) {
  if (dtype != VSA_BF16 && dtype != VSA_F32 && dtype != VSA_F16)
    return fail(VSA_ERR_UNSUPPORTED, "dtype %d is not bf16 (0), fp32 (1) or fp16 (2)", dtype);
  return VSA_OK;
}

static int check_block_shape(int64_t BH, int64_t Lq, int64_t Lkv, int D, int be) {
  VSA_REQUIRE(BH >= 0 && Lq >= 0 && Lkv >= 0, "negative extent");
  VSA_REQUIRE(D >= 1 && be >= 1, "head dim and block volume must be positive");
  VSA_REQUIRE(Lq % be == 0 && Lkv % be == 0, "sequence lengths must be divisible by block_elements=%d", be);
  return VSA_OK;
}

}  // namespace vsa

using namespace vsa;

extern "C" {

const char* vsa_last_error_string(void) { return g_error; }

int vsa_version(void) { return 200; }

int64_t vsa_launch_count(void) { return (int64_t)g_launches.load(std::memory_order_relaxed); }

int vsa_block_mean3_fwd(const void* q, const void* k, const void* v, const int32_t* q_sizes, const int32_t* kv_sizes,
                        void* q_mean, void* k_mean, void* v_mean, int64_t BH, int64_t Lq, int64_t Lkv, int D, int be,
                        int dtype, void* stream) {
  int rc = check_dtype(dtype);
  if (rc) return rc;
  rc = check_block_shape(BH, Lq, Lkv, D, be);
  if (rc) return rc;
  VSA_REQUIRE(q && k && v && q_sizes && kv_sizes && q_mean && k_mean && v_mean, "block mean: null pointer");
  const void* x[3] = {q, k, v};
  void* out[3] = {q_mean, k_mean, v_mean};
  const int32_t* sizes[3] = {q_sizes, kv_sizes, kv_sizes};
  const int64_t L[3] = {Lq, Lkv, Lkv};
  return block_mean_fwd(x, out, sizes, L, 3, BH, D, be, dtype, (cudaStream_t)stream);
}

int vsa_block_mean_fwd(const void* x, const int32_t* sizes, void* mean, int64_t BH, int64_t L, int D, int be,
                       int dtype, void* stream) {
  int rc = check_dtype(dtype);
  if (rc) return rc;
  rc = check_block_shape(BH, L, L, D, be);
  if (rc) return rc;
  VSA_REQUIRE(x && sizes && mean, "block mean: null pointer");
  const void* xs[3] = {x, nullptr, nullptr};
  void* outs[3] = {mean, nullptr, nullptr};
  const int32_t* ss[3] = {sizes, nullptr, nullptr};
  const int64_t Ls[3] = {L, 0, 0};
  return block_mean_fwd(xs, outs, ss, Ls, 1, BH, D, be, dtype, (cudaStream_t)stream);
}

int vsa_block_mean_bwd_accumulate(void* dx, const void* dmean, const int32_t* sizes, int64_t BH, int64_t L, int D,
                                  int be, int dtype, void* stream) {
  int rc = check_dtype(dtype);
  if (rc) return rc;
  rc = check_block_shape(BH, L, L, D, be);
  if (rc) return rc;
  VSA_REQUIRE(dx && dmean && sizes, "block mean backward: null pointer");
  return block_mean_bwd(dx, dmean, sizes, BH, L, D, be, dtype, true, (cudaStream_t)stream);
}

int vsa_block_mean_bwd(void* dx, const void* dmean, const int32_t* sizes, int64_t BH, int64_t L, int D, int be,
                       int dtype, void* stream) {
  int rc = check_dtype(dtype);
  if (rc) return rc;
  rc = check_block_shape(BH, L, L, D, be);
  if (rc) return rc;
  VSA_REQUIRE(dx && dmean && sizes, "block mean backward: null pointer");
  return block_mean_bwd(dx, dmean, sizes, BH, L, D, be, dtype, false, (cudaStream_t)stream);
}

int vsa_coarse_fwd(const void* q_mean, const void* k_mean, const void* v_mean, void* scores, void* probs, void* out_c,
                   int64_t BH, int Qb, int Kb, int D, float scale, int dtype, void* stream) {
  int rc = check_dtype(dtype);
  if (rc) return rc;
  VSA_REQUIRE(BH >= 0 && Qb >= 0 && Kb >= 1 && D >= 1, "coarse forward: bad extents");
  VSA_REQUIRE(q_mean && k_mean && v_mean && scores && probs && out_c, "coarse forward: null pointer");
  if (!scalar_forced() && coarse_umma_eligible(Qb, Kb, D, dtype))
    return coarse_fwd_umma(q_mean, k_mean, v_mean, scores, probs, out_c, BH, Qb, Kb, D, scale, dtype, (cudaStream_t)stream);
  return coarse_fwd(q_mean, k_mean, v_mean, scores, probs, out_c, BH, Qb, Kb, D, scale, dtype, (cudaStream_t)stream);
}

int vsa_topk(const void* scores, int32_t* selected, int64_t rows, int Kb, int topk, int dtype, void* stream) {
  int rc = check_dtype(dtype);
  if (rc) return rc;
  VSA_REQUIRE(scores && selected, "topk: null pointer");
  VSA_REQUIRE(rows >= 0 && Kb >= 1, "topk: bad extents");
  VSA_REQUIRE(topk >= 1 && topk <= Kb, "topk must be in [1, %d]", Kb);
  return topk_select(scores, selected, rows, Kb, topk, dtype, (cudaStream_t)stream);
}

int vsa_coarse_bwd(const void* d_out_c, const void* out_c, const void* q_mean, const void* k_mean, const void* v_mean,
                   const void* probs, void* dscores_ws, float* rowdot_ws, void* dq_mean, void* dk_mean, void* dv_mean,
                   int64_t BH, int Qb, int Kb, int D, float scale, int dtype, void* stream) {
  int rc = check_dtype(dtype);
  if (rc) return rc;
  VSA_REQUIRE(BH >= 0 && Qb >= 0 && Kb >= 1 && D >= 1, "coarse backward: bad extents");
  VSA_REQUIRE(d_out_c && out_c && q_mean && k_mean && v_mean && probs && dscores_ws && rowdot_ws && dq_mean &&
                  dk_mean && dv_mean, "coarse backward: null pointer");
  if (!scalar_forced() && coarse_umma_eligible(Qb, Kb, D, dtype))
    return coarse_bwd_umma(d_out_c, out_c, q_mean, k_mean, v_mean, probs, dscores_ws, rowdot_ws, dq_mean, dk_mean,
                           dv_mean, BH, Qb, Kb, D, scale, dtype, (cudaStream_t)stream);
  return coarse_bwd(d_out_c, out_c, q_mean, k_mean, v_mean, probs, dscores_ws, rowdot_ws, dq_mean, dk_mean, dv_mean,
                    BH, Qb, Kb, D, scale, dtype, (cudaStream_t)stream);
}

static int check_sparse(int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk, int dtype) {
  int rc = check_dtype(dtype);
  if (rc) return rc;
  rc = check_block_shape(BH, Lq, Lkv, D, be);
  if (rc) return rc;
  VSA_REQUIRE(Lkv >= be, "at least one key block is required");
  VSA_REQUIRE(topk >= 1 && topk <= Lkv / be, "selected topk must be in [1, %lld]", (long long)(Lkv / be));
  return VSA_OK;
}

static int sparse_fwd_dispatch(const void* q, const void* k, const void* v, const int32_t* selected,
                               const int32_t* kv_sizes, void* out, float* lse2, const void* out_c, const void* gate,
                               void* out_comb, int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk,
                               float scale, int dtype, cudaStream_t st) {
  int rc;
  if (lse2 && !scalar_forced() && !mma_forced() && sparse_umma_eligible(D, be, dtype, topk)) {
    rc = sparse_fwd_umma(q, k, v, selected, kv_sizes, out, lse2, BH, Lq, Lkv, be, topk, scale, dtype, st, out_c, gate,
                         out_comb);
    if (rc) return rc;
    // exact recomputation of the (normally zero) tiles the fixed-shift softmax marked as out of range
    return sparse_fwd_tc(q, k, v, selected, kv_sizes, out, lse2, BH, Lq, Lkv, D, be, topk, scale, dtype, true, st, out_c,
                         gate, out_comb);
  }
  if (!scalar_forced() && sparse_tc_eligible(D, be, dtype))
    return sparse_fwd_tc(q, k, v, selected, kv_sizes, out, lse2, BH, Lq, Lkv, D, be, topk, scale, dtype, false, st, out_c,
                         gate, out_comb);
  rc = sparse_fwd_scalar(q, k, v, selected, kv_sizes, out, lse2, BH, Lq, Lkv, D, be, topk, scale, dtype, st);
  if (rc || !out_comb) return rc;
  return combine_fwd(out, out_c, gate, out_comb, BH, Lq, D, be, dtype, st);
}

int vsa_sparse_fwd(const void* q, const void* k, const void* v, const int32_t* selected, const int32_t* kv_sizes,
                   void* out, float* lse2, int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk, float scale,
                   int dtype, void* stream) {
  int rc = check_sparse(BH, Lq, Lkv, D, be, topk, dtype);
  if (rc) return rc;
  VSA_REQUIRE(q && k && v && selected && kv_sizes && out, "sparse forward: null pointer");
  return sparse_fwd_dispatch(q, k, v, selected, kv_sizes, out, lse2, nullptr, nullptr, nullptr, BH, Lq, Lkv, D, be, topk,
                             scale, dtype, (cudaStream_t)stream);
}

int vsa_sparse_fwd_combine(const void* q, const void* k, const void* v, const int32_t* selected,
                           const int32_t* kv_sizes, void* out_s, float* lse2, const void* out_c, const void* gate,
                           void* out, int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk, float scale,
                           int dtype, void* stream) {
  int rc = check_sparse(BH, Lq, Lkv, D, be, topk, dtype);
  if (rc) return rc;
  VSA_REQUIRE(q && k && v && selected && kv_sizes && out_s && out_c && out, "sparse forward + combine: null pointer");
  return sparse_fwd_dispatch(q, k, v, selected, kv_sizes, out_s, lse2, out_c, gate, out, BH, Lq, Lkv, D, be, topk, scale,
                             dtype, (cudaStream_t)stream);
}

int vsa_route_invert(const int32_t* selected, int32_t* counts, int32_t* offsets, int32_t* inverse,
                     int32_t* cursor_ws, int64_t BH, int Qb, int Kb, int topk, void* stream) {
  VSA_REQUIRE(selected && counts && offsets && inverse && cursor_ws, "route inversion: null pointer");
  VSA_REQUIRE(BH >= 0 && Qb >= 0 && Kb >= 1 && topk >= 1, "route inversion: bad extents");
  return route_invert(selected, counts, offsets, inverse, cursor_ws, BH, Qb, Kb, topk, (cudaStream_t)stream);
}

int vsa_route_invert_static(const int32_t* selected, int32_t* counts, int32_t* offsets, int32_t* inverse, int64_t BH,
                            int Qb, int Kb, int topk, void* stream) {
  VSA_REQUIRE(selected && counts && offsets && inverse, "static route inversion: null pointer");
  VSA_REQUIRE(BH >= 0 && Qb >= 0 && Kb >= 1 && topk >= 1, "static route inversion: bad extents");
  return route_invert_static(selected, counts, offsets, inverse, BH, Qb, Kb, topk, (cudaStream_t)stream);
}

int vsa_sparse_bwd_dq(const void* dout, const void* q, const void* k, const void* v, const void* out_s,
                      const float* lse2, const int32_t* selected, const int32_t* kv_sizes, float* delta, void* dq,
                      int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk, float scale, int dtype,
                      void* stream) {
  int rc = check_sparse(BH, Lq, Lkv, D, be, topk, dtype);
  if (rc) return rc;
  VSA_REQUIRE(dout && q && k && v && out_s && lse2 && selected && kv_sizes && delta && dq, "sparse dQ: null pointer");
  if (!scalar_forced() && !mma_forced() && sparse_umma_eligible(D, be, dtype, topk))
    return sparse_dq_umma(dout, q, k, v, out_s, lse2, selected, kv_sizes, delta, dq, BH, Lq, Lkv, be, topk, scale,
                          dtype, (cudaStream_t)stream);
  if (!scalar_forced() && sparse_tc_eligible(D, be, dtype))
    return sparse_dq_tc(dout, q, k, v, out_s, lse2, selected, kv_sizes, delta, dq, BH, Lq, Lkv, D, be, topk, scale,
                        dtype, (cudaStream_t)stream);
  return sparse_dq_scalar(dout, q, k, v, out_s, lse2, selected, kv_sizes, delta, dq, BH, Lq, Lkv, D, be, topk, scale,
                          dtype, (cudaStream_t)stream);
}

int vsa_sparse_bwd_dkdv(const void* dout, const void* q, const void* k, const void* v, const float* lse2,
                        const float* delta, const int32_t* counts, const int32_t* offsets, const int32_t* inverse,
                        const int32_t* kv_sizes, void* dk, void* dv, int64_t BH, int64_t Lq, int64_t Lkv, int D,
                        int be, int topk, float scale, int dtype, void* stream) {
  int rc = check_sparse(BH, Lq, Lkv, D, be, topk, dtype);
  if (rc) return rc;
  VSA_REQUIRE(dout && q && k && v && lse2 && delta && counts && offsets && inverse && kv_sizes && dk && dv,
              "sparse dK/dV: null pointer");
  if (!scalar_forced() && !mma_forced() && sparse_umma_eligible(D, be, dtype, topk))
    return sparse_dkdv_umma(dout, q, k, v, lse2, delta, counts, offsets, inverse, kv_sizes, dk, dv, BH, Lq, Lkv, be,
                            topk, scale, dtype, (cudaStream_t)stream);
  if (!scalar_forced() && sparse_tc_eligible(D, be, dtype))
    return sparse_dkdv_tc(dout, q, k, v, lse2, delta, counts, offsets, inverse, kv_sizes, dk, dv, BH, Lq, Lkv, D, be,
                          topk, scale, dtype, (cudaStream_t)stream);
  return sparse_dkdv_scalar(dout, q, k, v, lse2, delta, counts, offsets, inverse, kv_sizes, dk, dv, BH, Lq, Lkv, D, be,
                            topk, scale, dtype, (cudaStream_t)stream);
}

// The two backward passes with the block-mean backward folded into their stores (one rounding instead of a
// store, a reload and a second rounding; three launches and ~6 tensor-sized memory passes fewer per step).  On
// the tensor path the term is added in the epilogue; the other paths run the plain kernel and the accumulate
// kernel behind it, so the result is defined for every shape.
int vsa_sparse_bwd_dq_fused(const void* dout, const void* q, const void* k, const void* v, const void* out_s,
                            const float* lse2, const int32_t* selected, const int32_t* kv_sizes, float* delta, void* dq,
                            const void* dq_mean, const int32_t* q_sizes, int64_t BH, int64_t Lq, int64_t Lkv, int D,
                            int be, int topk, float scale, int dtype, void* stream) {
  int rc = check_sparse(BH, Lq, Lkv, D, be, topk, dtype);
  if (rc) return rc;
  VSA_REQUIRE(dout && q && k && v && out_s && lse2 && selected && kv_sizes && delta && dq && dq_mean && q_sizes,
              "sparse dQ (fused): null pointer");
  if (!scalar_forced() && !mma_forced() && sparse_umma_eligible(D, be, dtype, topk))
    return sparse_dq_umma(dout, q, k, v, out_s, lse2, selected, kv_sizes, delta, dq, BH, Lq, Lkv, be, topk, scale,
                          dtype, (cudaStream_t)stream, dq_mean, q_sizes);
  rc = vsa_sparse_bwd_dq(dout, q, k, v, out_s, lse2, selected, kv_sizes, delta, dq, BH, Lq, Lkv, D, be, topk, scale,
                         dtype, stream);
  if (rc) return rc;
  return block_mean_bwd(dq, dq_mean, q_sizes, BH, Lq, D, be, dtype, true, (cudaStream_t)stream);
}

int vsa_sparse_bwd_dkdv_fused(const void* dout, const void* q, const void* k, const void* v, const float* lse2,
                              const float* delta, const int32_t* counts, const int32_t* offsets,
                              const int32_t* inverse, const int32_t* kv_sizes, void* dk, void* dv,
                              const void* dk_mean, const void* dv_mean, int64_t BH, int64_t Lq, int64_t Lkv, int D,
                              int be, int topk, float scale, int dtype, void* stream) {
  int rc = check_sparse(BH, Lq, Lkv, D, be, topk, dtype);
  if (rc) return rc;
  VSA_REQUIRE(dout && q && k && v && lse2 && delta && counts && offsets && inverse && kv_sizes && dk && dv &&
                  dk_mean && dv_mean, "sparse dK/dV (fused): null pointer");
  if (!scalar_forced() && !mma_forced() && sparse_umma_eligible(D, be, dtype, topk))
    return sparse_dkdv_umma(dout, q, k, v, lse2, delta, counts, offsets, inverse, kv_sizes, dk, dv, BH, Lq, Lkv, be,
                            topk, scale, dtype, (cudaStream_t)stream, dk_mean, dv_mean);
  rc = vsa_sparse_bwd_dkdv(dout, q, k, v, lse2, delta, counts, offsets, inverse, kv_sizes, dk, dv, BH, Lq, Lkv, D, be,
                           topk, scale, dtype, stream);
  if (rc) return rc;
  rc = block_mean_bwd(dk, dk_mean, kv_sizes, BH, Lkv, D, be, dtype, true, (cudaStream_t)stream);
  if (rc) return rc;
  return block_mean_bwd(dv, dv_mean, kv_sizes, BH, Lkv, D, be, dtype, true, (cudaStream_t)stream);
}

// ---- the backward that forms dS once ---------------------------------------------------------------------
// vsa_sparse_bwd_dq + vsa_sparse_bwd_dkdv compute the scores and dP twice, once per pass (as the reference's
// _vsa_dq_kernel / _vsa_dkdv_kernel do).  The three entry points below compute them once: delta first, then the
// key-owned pass, which also writes every dS tile into a workspace, then a query-owned pass that only multiplies
// the stored tiles by K.  Tensor path only (vsa_sparse_bwd_ds_supported tells); the workspace holds 8 KB per
// (query tile, selected key tile), so callers with many slices run the two passes over groups of slices.
int vsa_route_invert_edges(const int32_t* selected, int32_t* counts, int32_t* offsets, int32_t* inverse_edges,
                           int32_t* cursor_ws, int64_t BH, int Qb, int Kb, int topk, void* stream) {
  VSA_REQUIRE(selected && counts && offsets && inverse_edges && cursor_ws, "route inversion: null pointer");
  VSA_REQUIRE(BH >= 0 && Qb >= 0 && Kb >= 1 && topk >= 1, "route inversion: bad extents");
  return route_invert(selected, counts, offsets, inverse_edges, cursor_ws, BH, Qb, Kb, topk, (cudaStream_t)stream, true);
}

int vsa_sparse_bwd_delta(const void* out_s, const void* dout, float* delta, int64_t BH, int64_t Lq, int D, int dtype,
                         void* stream) {
  int rc = check_dtype(dtype);
  if (rc) return rc;
  VSA_REQUIRE(out_s && dout && delta, "sparse delta: null pointer");
  VSA_REQUIRE(BH >= 0 && Lq >= 0 && D >= 1, "sparse delta: bad extents");
  return rowdot_rows(out_s, dout, delta, BH * Lq, D, dtype, (cudaStream_t)stream);
}

int vsa_sparse_bwd_ds_supported(int D, int be, int topk, int dtype) {
  return !scalar_forced() && !mma_forced() && sparse_umma_eligible(D, be, dtype, topk) && topk <= 2048 ? 1 : 0;
}

int64_t vsa_sparse_bwd_ds_workspace_bytes(int64_t BH, int64_t Lq, int be, int topk) {
  if (BH < 0 || Lq < 0 || be < 64 || be % 64 || topk < 0) return -1;
  return sparse_ds_workspace_bytes(BH, Lq, be, topk);
}

int vsa_sparse_bwd_dkdv_ds(const void* dout, const void* q, const void* k, const void* v, const float* lse2,
                           const float* delta, const int32_t* counts, const int32_t* offsets,
                           const int32_t* inverse_edges, const int32_t* kv_sizes, void* dk, void* dv,
                           const void* dk_mean, const void* dv_mean, void* ds_ws, int64_t BH, int64_t Lq, int64_t Lkv,
                           int D, int be, int topk, float scale, int dtype, void* stream) {
  int rc = check_sparse(BH, Lq, Lkv, D, be, topk, dtype);
  if (rc) return rc;
  VSA_REQUIRE(dout && q && k && v && lse2 && delta && counts && offsets && inverse_edges && kv_sizes && dk && dv && ds_ws,
              "sparse dK/dV (dS stored): null pointer");
  VSA_REQUIRE((dk_mean == nullptr) == (dv_mean == nullptr), "sparse dK/dV (dS stored): give both pooled gradients or neither");
  if (!vsa_sparse_bwd_ds_supported(D, be, topk, dtype))
    return fail(VSA_ERR_UNSUPPORTED, "sparse dK/dV (dS stored): needs bf16 or fp16, head dim 128, block volume 64, 128 or 256");
  return sparse_dkdv_umma(dout, q, k, v, lse2, delta, counts, offsets, inverse_edges, kv_sizes, dk, dv, BH, Lq, Lkv, be,
                          topk, scale, dtype, (cudaStream_t)stream, dk_mean, dv_mean, ds_ws);
}

int vsa_sparse_bwd_dq_from_ds(const void* k, const int32_t* selected, const int32_t* kv_sizes, const void* ds_ws,
                              void* dq, const void* dq_mean, const int32_t* q_sizes, int64_t BH, int64_t Lq,
                              int64_t Lkv, int D, int be, int topk, float scale, int dtype, void* stream) {
  int rc = check_sparse(BH, Lq, Lkv, D, be, topk, dtype);
  if (rc) return rc;
  VSA_REQUIRE(k && selected && kv_sizes && ds_ws && dq, "sparse dQ (from dS): null pointer");
  VSA_REQUIRE((dq_mean == nullptr) == (q_sizes == nullptr), "sparse dQ (from dS): give the pooled gradient and the query sizes, or neither");
  if (!vsa_sparse_bwd_ds_supported(D, be, topk, dtype))
    return fail(VSA_ERR_UNSUPPORTED, "sparse dQ (from dS): needs bf16 or fp16, head dim 128, block volume 64, 128 or 256");
  return sparse_dq_from_ds_umma(k, selected, kv_sizes, ds_ws, dq, BH, Lq, Lkv, be, topk, scale, dtype,
                                (cudaStream_t)stream, dq_mean, q_sizes);
}

// ---- shard-major K/V (sequence-parallel mode) --------------------------------------------------------------
// After an all-gather over W ranks the K/V shards lie one after another, [W][BH][Lkv/W][D].  These three entry
// points read (and, for dK/dV, write) that layout in place: row of (slice, token) = ((token / shard) * BH + slice)
// * shard + token % shard with shard = kv_shard tokens, so no re-layout copy follows the gather and the partial
// dK/dV are ready for the reduce-scatter.  Tensor path only (bf16 or fp16, D = 128, block volume 64, 128 or 256).
static int check_sharded(int64_t Lkv, int64_t kv_shard, int D, int be, int topk, int dtype, const char* what) {
  VSA_REQUIRE(kv_shard > 0 && Lkv % kv_shard == 0 && kv_shard % be == 0,
              "%s: kv_shard must divide Lkv and be a multiple of block_elements=%d", what, be);
  if (scalar_forced() || mma_forced() || !sparse_umma_eligible(D, be, dtype, topk))
    return fail(VSA_ERR_UNSUPPORTED, "%s: the shard-major layout needs bf16 or fp16, head dim 128, block volume 64, 128 or 256", what);
  return VSA_OK;
}

int vsa_sparse_sharded_supported(int D, int be, int topk, int dtype) {
  return !scalar_forced() && !mma_forced() && sparse_umma_eligible(D, be, dtype, topk) ? 1 : 0;
}

int vsa_sparse_fwd_combine_sharded(const void* q, const void* k_sh, const void* v_sh, const int32_t* selected,
                                   const int32_t* kv_sizes, void* out_s, float* lse2, const void* out_c,
                                   const void* gate, void* out, int64_t BH, int64_t Lq, int64_t Lkv, int64_t kv_shard,
                                   int D, int be, int topk, float scale, int dtype, void* stream) {
  int rc = check_sparse(BH, Lq, Lkv, D, be, topk, dtype);
  if (rc) return rc;
  VSA_REQUIRE(q && k_sh && v_sh && selected && kv_sizes && out_s && lse2, "sparse forward (sharded): null pointer");
  VSA_REQUIRE((out == nullptr) == (out_c == nullptr), "sparse forward (sharded): give out_c and out together, or neither");
  if ((rc = check_sharded(Lkv, kv_shard, D, be, topk, dtype, "sparse forward (sharded)"))) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  rc = sparse_fwd_umma(q, k_sh, v_sh, selected, kv_sizes, out_s, lse2, BH, Lq, Lkv, be, topk, scale, dtype, st, out_c, gate,
                       out, kv_shard);
  if (rc) return rc;
  return sparse_fwd_tc(q, k_sh, v_sh, selected, kv_sizes, out_s, lse2, BH, Lq, Lkv, D, be, topk, scale, dtype, true, st, out_c,
                       gate, out, kv_shard);
}

int vsa_sparse_bwd_dq_sharded(const void* dout, const void* q, const void* k_sh, const void* v_sh, const void* out_s,
                              const float* lse2, const int32_t* selected, const int32_t* kv_sizes, float* delta,
                              void* dq, const void* dq_mean, const int32_t* q_sizes, int64_t BH, int64_t Lq,
                              int64_t Lkv, int64_t kv_shard, int D, int be, int topk, float scale, int dtype,
                              void* stream) {
  int rc = check_sparse(BH, Lq, Lkv, D, be, topk, dtype);
  if (rc) return rc;
  VSA_REQUIRE(dout && q && k_sh && v_sh && out_s && lse2 && selected && kv_sizes && delta && dq,
              "sparse dQ (sharded): null pointer");
  VSA_REQUIRE((dq_mean == nullptr) == (q_sizes == nullptr), "sparse dQ (sharded): give the pooled gradient and the query sizes, or neither");
  if ((rc = check_sharded(Lkv, kv_shard, D, be, topk, dtype, "sparse dQ (sharded)"))) return rc;
  return sparse_dq_umma(dout, q, k_sh, v_sh, out_s, lse2, selected, kv_sizes, delta, dq, BH, Lq, Lkv, be, topk, scale,
                        dtype, (cudaStream_t)stream, dq_mean, q_sizes, kv_shard);
}

int vsa_sparse_bwd_dkdv_sharded(const void* dout, const void* q, const void* k_sh, const void* v_sh, const float* lse2,
                                const float* delta, const int32_t* counts, const int32_t* offsets,
                                const int32_t* inverse, const int32_t* kv_sizes, void* dk_sh, void* dv_sh,
                                const void* dk_mean, const void* dv_mean, int64_t BH, int64_t Lq, int64_t Lkv,
                                int64_t kv_shard, int D, int be, int topk, float scale, int dtype, void* stream) {
  int rc = check_sparse(BH, Lq, Lkv, D, be, topk, dtype);
  if (rc) return rc;
  VSA_REQUIRE(dout && q && k_sh && v_sh && lse2 && delta && counts && offsets && inverse && kv_sizes && dk_sh && dv_sh,
              "sparse dK/dV (sharded): null pointer");
  VSA_REQUIRE((dk_mean == nullptr) == (dv_mean == nullptr), "sparse dK/dV (sharded): give both pooled gradients or neither");
  if ((rc = check_sharded(Lkv, kv_shard, D, be, topk, dtype, "sparse dK/dV (sharded)"))) return rc;
  return sparse_dkdv_umma(dout, q, k_sh, v_sh, lse2, delta, counts, offsets, inverse, kv_sizes, dk_sh, dv_sh, BH, Lq, Lkv, be,
                          topk, scale, dtype, (cudaStream_t)stream, dk_mean, dv_mean, nullptr, kv_shard);
}

// ---- raster-order activations (tiling front end folded into the kernels' stores) ----------------------------
// A model holds q/k/v, the gate and the output as [B, S, H, D] in raster (t, h, w) token order; the kernels read
// tile-order [B*H, L, D] operands through TMA.  vsa_gather_rows_heads makes the operands in one pass each
// (gather + head transpose + zero padding); the three entry points below then read the gate and write the
// combined output and the three gradients straight at the tokens' raster rows, so nothing is moved back.
// map: tile-order token -> raster row or -1 (padding).  Tensor path only.
static int check_raster(const int32_t* map, int64_t rows, int heads, int64_t BH, int D, int be, int topk, int dtype,
                        const char* what) {
  VSA_REQUIRE(map != nullptr && rows >= 0 && heads >= 1 && BH % heads == 0, "%s: bad raster map, row count or head count", what);
  if (scalar_forced() || mma_forced() || !sparse_umma_eligible(D, be, dtype, topk))
    return fail(VSA_ERR_UNSUPPORTED, "%s: raster-order stores need bf16 or fp16, head dim 128, block volume 64, 128 or 256", what);
  return VSA_OK;
}

int vsa_sparse_kernel_family(int D, int be, int topk, int dtype) {
  if (scalar_forced()) return 0;
  if (!mma_forced() && sparse_umma_eligible(D, be, dtype, topk)) return 2;
  return sparse_tc_eligible(D, be, dtype) ? 1 : 0;
}

int vsa_sparse_raster_supported(int D, int be, int topk, int dtype) {
  return !scalar_forced() && !mma_forced() && sparse_umma_eligible(D, be, dtype, topk) ? 1 : 0;
}

int vsa_gather_rows_heads(const void* src, const int32_t* map, void* dst, int64_t batch, int heads, int64_t src_rows,
                          int64_t dst_rows, int64_t row_bytes, int to_tiled, void* stream) {
  VSA_REQUIRE(src && map && dst, "gather rows (heads): null pointer");
  VSA_REQUIRE(batch >= 0 && heads >= 0 && src_rows >= 0 && dst_rows >= 0 && row_bytes >= 0, "gather rows (heads): negative extent");
  return gather_rows_heads(src, map, dst, batch, heads, src_rows, dst_rows, row_bytes, to_tiled != 0, (cudaStream_t)stream);
}

int vsa_combine_bwd_raster(const void* dout_raster, const void* gate_raster, const void* out_c, void* d_out_c,
                           void* dgate_raster, void* dout_tiled, const int32_t* q_map, int64_t raster_rows, int heads,
                           int64_t BH, int64_t Lq, int D, int be, int dtype, void* stream) {
  int rc = check_dtype(dtype);
  if (rc) return rc;
  VSA_REQUIRE(dout_raster && out_c && d_out_c && dout_tiled && q_map, "combine backward (raster): null pointer");
  VSA_REQUIRE((gate_raster == nullptr) == (dgate_raster == nullptr), "combine backward (raster): give gate and dgate together, or neither");
  VSA_REQUIRE(BH >= 0 && Lq >= 0 && D >= 1 && be >= 1 && Lq % be == 0 && heads >= 1 && BH % heads == 0 && raster_rows >= 0,
              "combine backward (raster): bad extents");
  return combine_bwd_raster(dout_raster, gate_raster, out_c, d_out_c, dgate_raster, dout_tiled, q_map, raster_rows, heads, BH,
                            Lq, D, be, dtype, (cudaStream_t)stream);
}

int vsa_sparse_fwd_combine_raster(const void* q, const void* k, const void* v, const int32_t* selected,
                                  const int32_t* kv_sizes, void* out_s, float* lse2, const void* out_c,
                                  const void* gate_raster, void* out_raster, const int32_t* q_map, int64_t raster_rows,
                                  int heads, int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk, float scale,
                                  int dtype, void* stream) {
  int rc = check_sparse(BH, Lq, Lkv, D, be, topk, dtype);
  if (rc) return rc;
  VSA_REQUIRE(q && k && v && selected && kv_sizes && out_s && lse2 && out_c && out_raster,
              "sparse forward (raster): null pointer");
  if ((rc = check_raster(q_map, raster_rows, heads, BH, D, be, topk, dtype, "sparse forward (raster)"))) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  rc = sparse_fwd_umma(q, k, v, selected, kv_sizes, out_s, lse2, BH, Lq, Lkv, be, topk, scale, dtype, st, out_c,
                       gate_raster, out_raster, 0, q_map, raster_rows, heads);
  if (rc) return rc;
  return sparse_fwd_tc(q, k, v, selected, kv_sizes, out_s, lse2, BH, Lq, Lkv, D, be, topk, scale, dtype, true, st, out_c,
                       gate_raster, out_raster, 0, q_map, raster_rows, heads);
}

int vsa_sparse_bwd_dq_raster(const void* dout, const void* q, const void* k, const void* v, const void* out_s,
                             const float* lse2, const int32_t* selected, const int32_t* kv_sizes, float* delta,
                             void* dq_raster, const void* dq_mean, const int32_t* q_sizes, const int32_t* q_map,
                             int64_t raster_rows, int heads, int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk,
                             float scale, int dtype, void* stream) {
  int rc = check_sparse(BH, Lq, Lkv, D, be, topk, dtype);
  if (rc) return rc;
  VSA_REQUIRE(dout && q && k && v && out_s && lse2 && selected && kv_sizes && delta && dq_raster,
              "sparse dQ (raster): null pointer");
  VSA_REQUIRE((dq_mean == nullptr) == (q_sizes == nullptr), "sparse dQ (raster): give the pooled gradient and the query sizes, or neither");
  if ((rc = check_raster(q_map, raster_rows, heads, BH, D, be, topk, dtype, "sparse dQ (raster)"))) return rc;
  return sparse_dq_umma(dout, q, k, v, out_s, lse2, selected, kv_sizes, delta, dq_raster, BH, Lq, Lkv, be, topk, scale,
                        dtype, (cudaStream_t)stream, dq_mean, q_sizes, 0, q_map, raster_rows, heads);
}

int vsa_sparse_bwd_dkdv_raster(const void* dout, const void* q, const void* k, const void* v, const float* lse2,
                               const float* delta, const int32_t* counts, const int32_t* offsets,
                               const int32_t* inverse, const int32_t* kv_sizes, void* dk_raster, void* dv_raster,
                               const void* dk_mean, const void* dv_mean, const int32_t* kv_map, int64_t raster_rows,
                               int heads, int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk, float scale,
                               int dtype, void* stream) {
  int rc = check_sparse(BH, Lq, Lkv, D, be, topk, dtype);
  if (rc) return rc;
  VSA_REQUIRE(dout && q && k && v && lse2 && delta && counts && offsets && inverse && kv_sizes && dk_raster && dv_raster,
              "sparse dK/dV (raster): null pointer");
  VSA_REQUIRE((dk_mean == nullptr) == (dv_mean == nullptr), "sparse dK/dV (raster): give both pooled gradients or neither");
  if ((rc = check_raster(kv_map, raster_rows, heads, BH, D, be, topk, dtype, "sparse dK/dV (raster)"))) return rc;
  return sparse_dkdv_umma(dout, q, k, v, lse2, delta, counts, offsets, inverse, kv_sizes, dk_raster, dv_raster, BH, Lq,
                          Lkv, be, topk, scale, dtype, (cudaStream_t)stream, dk_mean, dv_mean, nullptr, 0, kv_map,
                          raster_rows, heads);
}

int vsa_gather_rows(const void* src, const int32_t* map, void* dst, int64_t batch, int64_t src_rows, int64_t dst_rows,
                    int64_t row_bytes, void* stream) {
  VSA_REQUIRE(src && map && dst, "gather rows: null pointer");
  VSA_REQUIRE(batch >= 0 && src_rows >= 0 && dst_rows >= 0 && row_bytes >= 0, "gather rows: negative extent");
  return gather_rows(src, map, dst, batch, src_rows, dst_rows, row_bytes, (cudaStream_t)stream);
}

int vsa_selftest_umma(const void* a, const void* b, float* out, int mode, void* stream) {
  VSA_REQUIRE(a && b && out && (mode == 0 || mode == 1), "selftest: bad argument");
  return umma_selftest(a, b, out, mode, (cudaStream_t)stream);
}

int64_t vsa_workspace_bytes(int which, int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk, int dtype) {
  if (BH < 0 || Lq < 0 || Lkv < 0 || D < 1 || be < 1 || topk < 0) return -1;
  if (dtype != VSA_BF16 && dtype != VSA_F32 && dtype != VSA_F16) return -1;
  const int64_t es = dtype == VSA_F32 ? 4 : 2, Qb = Lq / be, Kb = Lkv / be;
  switch (which) {
    case VSA_SCRATCH_SCORES: return BH * Qb * Kb * es;
    case VSA_SCRATCH_ROWDOT: return BH * Qb * 4;
    case VSA_SCRATCH_ROW_STATS: return BH * Lq * 4;
    case VSA_SCRATCH_CSR_ROWS: return BH * Kb * 4;
    case VSA_SCRATCH_CSR_EDGES: return BH * Qb * (int64_t)topk * 4;
    case VSA_SCRATCH_POOLED: return BH * Qb * (int64_t)D * es;
    case VSA_SCRATCH_DS_TILES: return be % 64 == 0 ? sparse_ds_workspace_bytes(BH, Lq, be, topk) : -1;
    default: return -1;
  }
}

int vsa_selftest_wait_timeout(int64_t limit_ns, int* gave_up, void* stream) {
  VSA_REQUIRE(gave_up, "wait self-test: null pointer");
  VSA_REQUIRE(limit_ns >= 1000 && limit_ns <= 100000000LL, "wait self-test: the limit must lie in [1 us, 100 ms]");
  return wait_timeout_selftest((unsigned long long)limit_ns, gave_up, (cudaStream_t)stream);
}

int vsa_device_status(int* status) {
  VSA_REQUIRE(status, "device status: null pointer");
  return device_status_fetch_and_clear(status);
}

int vsa_combine_fwd(const void* out_s, const void* out_c, const void* gate, void* out, int64_t BH, int64_t Lq, int D,
                    int be, int dtype, void* stream) {
  int rc = check_dtype(dtype);
  if (rc) return rc;
  rc = check_block_shape(BH, Lq, Lq, D, be);
  if (rc) return rc;
  VSA_REQUIRE(out_s && out_c && out, "combine: null pointer");
  return combine_fwd(out_s, out_c, gate, out, BH, Lq, D, be, dtype, (cudaStream_t)stream);
}

int vsa_combine_bwd(const void* dout, const void* gate, const void* out_c, void* d_out_c, void* dgate, int64_t BH,
                    int64_t Lq, int D, int be, int dtype, void* stream) {
  int rc = check_dtype(dtype);
  if (rc) return rc;
  rc = check_block_shape(BH, Lq, Lq, D, be);
  if (rc) return rc;
  VSA_REQUIRE(dout && out_c && d_out_c, "combine backward: null pointer");
  VSA_REQUIRE(gate || !dgate, "combine backward: dgate requested without a gate");
  return combine_bwd(dout, gate, out_c, d_out_c, dgate, BH, Lq, D, be, dtype, (cudaStream_t)stream);
}

}  // extern "C"
