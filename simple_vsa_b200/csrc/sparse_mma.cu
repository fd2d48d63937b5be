// Fine (block-sparse) attention on the warp-level tensor path: forward, the
// query-owned dQ pass and the key-owned dK/dV pass, for bf16 or fp16, head dim 64 or 128 and a
// logical block volume of 64, 128 or 256 tokens.
//
// Every kernel works on 64-token x head-dim tiles (16 KB at head dim 128, contiguous in global
// memory because a block's tokens are consecutive rows).  A logical block of 256
// tokens is four such tiles; the per-block size masks `sub*64 + col < size`, and a
// tile that lies wholly beyond the size is skipped.  Tiles are staged with
// cp.async into XOR-swizzled shared memory (16-byte chunk c of row r lives at
// chunk c ^ (r & 7)), double buffered, and consumed with ldmatrix + mma.sync
// m16n8k16 with fp32 accumulation.  Scores use scale*log2(e) and exp2, the saved
// statistic is row_max + log2(row_sum) (vsa/triton_impl.py:113-192 of the
// reference); P and dS are rounded to bf16 before their second GEMM
// (vsa/triton_impl.py:175,960,1106-1107).
#include "common.cuh"
#include "kernels.h"

namespace vsa {
namespace {

constexpr int kTile = 64;
constexpr int kThreads = 128;
template <typename K>
int set_smem(K kernel, int bytes, const char* what) {
  const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return fail(VSA_ERR_LAUNCH, "%s: cannot reserve %d bytes of shared memory: %s", what, bytes,
                                    cudaGetErrorString(e));
  return VSA_OK;
}


// the kernels exist once per head dim
namespace hd128 {
constexpr int kD = 128;
#include "sparse_mma_body.inl"
}  // namespace hd128
namespace hd64 {
constexpr int kD = 64;
#include "sparse_mma_body.inl"
}  // namespace hd64

}  // namespace

#define VSA_BY_HEAD_DIM(D_, call_) ((D_) == 64 ? hd64::call_ : hd128::call_)

bool sparse_tc_eligible(int D, int be, int dtype) {
  return (dtype == VSA_BF16 || dtype == VSA_F16) && (D == 128 || D == 64) && (be == 64 || be == 128 || be == 256);
}

int sparse_fwd_tc(const void* q, const void* k, const void* v, const int32_t* selected, const int32_t* kv_sizes,
                  void* out, float* lse2, int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk, float scale,
                  int dtype, bool redo_only, cudaStream_t st, const void* out_c, const void* gate, void* out_comb,
                  int64_t kv_shard, const int32_t* comb_map, int64_t comb_rows, int comb_heads) {
  const RasterMap rm{comb_map, (long long)comb_rows, comb_heads > 0 ? comb_heads : 1};
  if (BH == 0 || Lq == 0) return VSA_OK;
  if (kv_shard <= 0) kv_shard = Lkv;
  if (BH > 65535) return fail(VSA_ERR_UNSUPPORTED, "sparse forward: batch*heads %lld exceeds 65535", (long long)BH);
  if (dtype == VSA_F16)
    return VSA_BY_HEAD_DIM(D, launch_fwd<__half>(q, k, v, selected, kv_sizes, out, lse2, BH, Lq, Lkv, be, topk, scale,
                                                 redo_only, st, out_c, gate, out_comb, kv_shard, rm));
  return VSA_BY_HEAD_DIM(D, launch_fwd<__nv_bfloat16>(q, k, v, selected, kv_sizes, out, lse2, BH, Lq, Lkv, be, topk, scale,
                                                      redo_only, st, out_c, gate, out_comb, kv_shard, rm));
}

int sparse_dq_tc(const void* dout, const void* q, const void* k, const void* v, const void* out_s, const float* lse2,
                 const int32_t* selected, const int32_t* kv_sizes, float* delta, void* dq, int64_t BH, int64_t Lq,
                 int64_t Lkv, int D, int be, int topk, float scale, int dtype, cudaStream_t st) {
  if (BH == 0 || Lq == 0) return VSA_OK;
  if (BH > 65535) return fail(VSA_ERR_UNSUPPORTED, "sparse dQ: batch*heads %lld exceeds 65535", (long long)BH);
  if (dtype == VSA_F16)
    return VSA_BY_HEAD_DIM(D, launch_dq<__half>(dout, q, k, v, out_s, lse2, selected, kv_sizes, delta, dq, BH, Lq, Lkv, be,
                                                topk, scale, st));
  return VSA_BY_HEAD_DIM(D, launch_dq<__nv_bfloat16>(dout, q, k, v, out_s, lse2, selected, kv_sizes, delta, dq, BH, Lq, Lkv,
                                                     be, topk, scale, st));
}

int sparse_dkdv_tc(const void* dout, const void* q, const void* k, const void* v, const float* lse2,
                   const float* delta, const int32_t* counts, const int32_t* offsets, const int32_t* inverse,
                   const int32_t* kv_sizes, void* dk, void* dv, int64_t BH, int64_t Lq, int64_t Lkv, int D, int be,
                   int topk, float scale, int dtype, cudaStream_t st) {
  if (BH == 0 || Lkv == 0) return VSA_OK;
  if (BH > 65535) return fail(VSA_ERR_UNSUPPORTED, "sparse dK/dV: batch*heads %lld exceeds 65535", (long long)BH);
  if (dtype == VSA_F16)
    return VSA_BY_HEAD_DIM(D, launch_dkdv<__half>(dout, q, k, v, lse2, delta, counts, offsets, inverse, kv_sizes, dk, dv, BH,
                                                  Lq, Lkv, be, topk, scale, st));
  return VSA_BY_HEAD_DIM(D, launch_dkdv<__nv_bfloat16>(dout, q, k, v, lse2, delta, counts, offsets, inverse, kv_sizes, dk, dv,
                                                       BH, Lq, Lkv, be, topk, scale, st));
}

}  // namespace vsa
