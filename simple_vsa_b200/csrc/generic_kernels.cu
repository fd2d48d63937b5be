// Scalar (CUDA-core) kernels of the VSA path.
//
// Two roles: (1) the bandwidth-bound pieces of every configuration -- block
// means, pooled softmax, Top-K, gated combine, route inversion -- and (2) the
// fine attention forward/backward for shapes the tensor-core kernels do not
// cover (fp32 validation mode, block volumes other than 64/128/256, head dims
// other than 128).  Arithmetic follows the reference project's conventions:
// fp32 accumulation, base-2 log-sum-exp, masks from the per-block sizes.
#include <cuda_fp16.h>

#include <algorithm>
#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "kernels.h"

namespace vsa {

// Run `f` with a null pointer of the element type that `dtype` names (bf16, fp32 or fp16).
template <typename F>
static int dispatch_dtype(int dtype, F&& f) {
  switch (dtype) {
    case VSA_F32: return f(static_cast<float*>(nullptr));
    case VSA_F16: return f(static_cast<__half*>(nullptr));
    default: return f(static_cast<__nv_bfloat16*>(nullptr));
  }
}
#define VSA_TAG_TYPE(tag) typename std::remove_pointer<decltype(tag)>::type
static inline int elems_per_16_bytes(int dtype) { return dtype == VSA_F32 ? 4 : 8; }

// =========================================================================================
// Block means (vsa/common.py:55-82 of the reference): one CTA per (tensor, bh, block).
// Only the first sizes[b] rows of a block are read, so padding never reaches the sum.
// =========================================================================================
struct MeanJob {
  const void* x[3];
  void* out[3];
  const int32_t* sizes[3];
  int nb[3];
  long long first_cta[4];   // CTA index ranges per tensor
};

template <typename T>
__global__ void __launch_bounds__(128) block_mean_kernel(MeanJob job, int D, int be) {
  constexpr int VEC = 16 / sizeof(T);
  __shared__ __align__(16) float part_sm[128 * VEC];     // [row group][D] partial sums
  const long long cta = blockIdx.x;
  int t = 0;
  if (cta >= job.first_cta[1]) t = 1;
  if (cta >= job.first_cta[2]) t = 2;
  const long long local = cta - job.first_cta[t];
  const int nb = job.nb[t];
  const int blk = (int)(local % nb);
  const T* x = reinterpret_cast<const T*>(job.x[t]) + local * (long long)be * D;
  T* out = reinterpret_cast<T*>(job.out[t]) + local * (long long)D;
  int size = job.sizes[t][blk];
  size = size < 0 ? 0 : (size > be ? be : size);

  const int cpr = D / VEC;                     // 16-byte chunks per row
  const int rows_per_pass = blockDim.x / cpr;
  const int chunk = threadIdx.x % cpr;
  const int rgrp = threadIdx.x / cpr;
  float part[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) part[i] = 0.f;
  if (rgrp < rows_per_pass) {
    int r = rgrp;
    for (; r + 3 * rows_per_pass < size; r += 4 * rows_per_pass) {   // four independent 16-byte loads in flight
      uint4 raw[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        raw[u] = *reinterpret_cast<const uint4*>(x + (long long)(r + u * rows_per_pass) * D + chunk * VEC);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const T* e = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
        for (int i = 0; i < VEC; ++i) part[i] += Elem<T>::ld(e + i);
      }
    }
    for (; r < size; r += rows_per_pass) {
      const uint4 raw = *reinterpret_cast<const uint4*>(x + (long long)r * D + chunk * VEC);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int i = 0; i < VEC; ++i) part[i] += Elem<T>::ld(e + i);
    }
    float* dst = part_sm + rgrp * D + chunk * VEC;
#pragma unroll
    for (int i = 0; i < VEC; ++i) dst[i] = part[i];
  }
  __syncthreads();
  const float denom = (float)(size > 1 ? size : 1);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float sum = 0.f;
    for (int g = 0; g < rows_per_pass; ++g) sum += part_sm[g * D + d];     // fixed order: deterministic
    Elem<T>::st(out + d, sum / denom);
  }
}

// Warp-per-block form for rows of at most 32 sixteen-byte chunks (every head dim the tensor path serves):
// lane = (row parity group, chunk), eight independent loads in flight per lane, partial sums combined by
// shuffles in a fixed order.  No shared memory and no block barrier, so a CTA of four warps is four
// independent streams; the CTA-per-block kernel above spent a quarter of its time outside its loads.
template <typename T>
__global__ void __launch_bounds__(128) block_mean_warp_kernel(MeanJob job, int D, int be, long long total) {
  constexpr int VEC = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (unit >= total) return;
  int t = 0;
  if (unit >= job.first_cta[1]) t = 1;
  if (unit >= job.first_cta[2]) t = 2;
  // (picked with selects: indexing the parameter struct with a run-time index would copy it to the stack)
  const long long first = t == 0 ? job.first_cta[0] : (t == 1 ? job.first_cta[1] : job.first_cta[2]);
  const int nb = t == 0 ? job.nb[0] : (t == 1 ? job.nb[1] : job.nb[2]);
  const void* xin = t == 0 ? job.x[0] : (t == 1 ? job.x[1] : job.x[2]);
  void* xout = t == 0 ? job.out[0] : (t == 1 ? job.out[1] : job.out[2]);
  const int32_t* sz = t == 0 ? job.sizes[0] : (t == 1 ? job.sizes[1] : job.sizes[2]);
  const long long local = unit - first;
  const int blk = (int)(local % nb);
  const T* x = reinterpret_cast<const T*>(xin) + local * (long long)be * D;
  T* out = reinterpret_cast<T*>(xout) + local * (long long)D;
  int size = sz[blk];
  size = size < 0 ? 0 : (size > be ? be : size);
  const int cpr = D / VEC, rpl = 32 / cpr;       // chunks per row, rows per warp-wide load
  const int chunk = lane % cpr, rsub = lane / cpr;
  const T* px = x + chunk * VEC;
  float part[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) part[i] = 0.f;
  int r = rsub;
  for (; r + 7 * rpl < size; r += 8 * rpl) {
    uint4 raw[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) raw[u] = *reinterpret_cast<const uint4*>(px + (long long)(r + u * rpl) * D);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const T* e = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
      for (int i = 0; i < VEC; ++i) part[i] += Elem<T>::ld(e + i);
    }
  }
  for (; r < size; r += rpl) {
    const uint4 raw = *reinterpret_cast<const uint4*>(px + (long long)r * D);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < VEC; ++i) part[i] += Elem<T>::ld(e + i);
  }
  for (int o = cpr; o < 32; o <<= 1) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) part[i] += __shfl_xor_sync(0xffffffffu, part[i], o);
  }
  if (rsub == 0) {
    const float denom = (float)(size > 1 ? size : 1);
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < VEC; ++i) Elem<T>::st(e + i, part[i] / denom);
    *reinterpret_cast<uint4*>(out + chunk * VEC) = raw;
  }
}

template <typename T>
static int launch_block_mean(MeanJob job, int ntensors, int64_t BH, int D, int be, cudaStream_t st) {
  constexpr int VEC = 16 / sizeof(T);
  if (D % VEC != 0 || D / VEC > 128 || D > 256)
    return fail(VSA_ERR_UNSUPPORTED, "block mean: head dim %d must be a multiple of %d and <= 256", D, VEC);
  long long total = 0;
  for (int t = 0; t < 3; ++t) {
    job.first_cta[t] = total;
    if (t < ntensors) total += BH * job.nb[t];
  }
  job.first_cta[3] = total;
  for (int t = ntensors; t < 3; ++t) job.first_cta[t] = total + 1;  // never matched
  if (total == 0) return VSA_OK;
  if (total > 0x7fffffffLL) return fail(VSA_ERR_UNSUPPORTED, "block mean: too many blocks");
  const int cpr = D / VEC;
  if (cpr <= 32 && 32 % cpr == 0) {
    block_mean_warp_kernel<T><<<(unsigned)((total + 3) / 4), 128, 0, st>>>(job, D, be, total);
    return check_launch("block_mean_warp_kernel");
  }
  block_mean_kernel<T><<<(unsigned)total, 128, 0, st>>>(job, D, be);
  return check_launch("block_mean_kernel");
}

int block_mean_fwd(const void* const* x, void* const* out, const int32_t* const* sizes, const int64_t* L,
                   int ntensors, int64_t BH, int D, int be, int dtype, cudaStream_t st) {
  MeanJob job{};
  for (int t = 0; t < ntensors; ++t) {
    job.x[t] = x[t];
    job.out[t] = out[t];
    job.sizes[t] = sizes[t];
    job.nb[t] = (int)(L[t] / be);
  }
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = VSA_TAG_TYPE(tag);
    return launch_block_mean<T>(job, ntensors, BH, D, be, st);
  });
}

// Block-mean backward (vsa/fused_common.py:62-103 of the reference).  ACCUM adds into
// dx on valid rows and leaves padding rows alone; otherwise padding rows are zeroed.
template <typename T, bool ACCUM>
__global__ void __launch_bounds__(128) block_mean_bwd_kernel(T* __restrict__ dx, const T* __restrict__ dmean,
                                                            const int32_t* __restrict__ sizes, int nb, int D, int be) {
  constexpr int VEC = 16 / sizeof(T);
  const long long local = blockIdx.x;
  const int blk = (int)(local % nb);
  int size = sizes[blk];
  size = size < 0 ? 0 : (size > be ? be : size);
  const float inv = 1.f / (float)(size > 1 ? size : 1);
  T* x = dx + local * (long long)be * D;
  const T* g = dmean + local * (long long)D;
  const int cpr = D / VEC;
  const int rows_per_pass = blockDim.x / cpr;
  const int chunk = threadIdx.x % cpr;
  const int rgrp = threadIdx.x / cpr;
  if (rgrp >= rows_per_pass) return;
  float gv[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) gv[i] = Elem<T>::ld(g + chunk * VEC + i) * inv;
  const int last = ACCUM ? size : be;
  for (int r = rgrp; r < last; r += rows_per_pass) {
    uint4* p = reinterpret_cast<uint4*>(x + (long long)r * D + chunk * VEC);
    uint4 raw = ACCUM ? *p : make_uint4(0, 0, 0, 0);
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const float base = ACCUM ? Elem<T>::ld(e + i) : 0.f;
      Elem<T>::st(e + i, r < size ? base + gv[i] : 0.f);
    }
    *p = raw;
  }
}

int block_mean_bwd(void* dx, const void* dmean, const int32_t* sizes, int64_t BH, int64_t L, int D, int be,
                   int dtype, bool accumulate, cudaStream_t st) {
  const int nb = (int)(L / be);
  const long long total = BH * nb;
  if (total == 0) return VSA_OK;
  const int vec = elems_per_16_bytes(dtype);
  if (D % vec != 0 || D / vec > 128)
    return fail(VSA_ERR_UNSUPPORTED, "block mean backward: head dim %d must be a multiple of %d and <= 256", D, vec);
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = VSA_TAG_TYPE(tag);
    if (accumulate)
      block_mean_bwd_kernel<T, true><<<(unsigned)total, 128, 0, st>>>((T*)dx, (const T*)dmean, sizes, nb, D, be);
    else
      block_mean_bwd_kernel<T, false><<<(unsigned)total, 128, 0, st>>>((T*)dx, (const T*)dmean, sizes, nb, D, be);
    return check_launch("block_mean_bwd_kernel");
  });
}

// =========================================================================================
// Small batched GEMM with arbitrary strides (the pooled attention and its backward).
// C[b][m][n] = epilogue(sum_k A[b][m][k] * B[b][k][n]); 64x64 tile, 16-deep, 4x4 per thread.
// =========================================================================================
struct EpiScores {   // scores = round(round(acc) * scale)            vsa/common.py:164
  float scale;
  template <typename T> __device__ void operator()(T* C, long long idx, long long, int, int, float acc) const {
    Elem<T>::st(C + idx, Elem<T>::round(acc) * scale);
  }
};
struct EpiStore {    // plain rounding store
  template <typename T> __device__ void operator()(T* C, long long idx, long long, int, int, float acc) const {
    Elem<T>::st(C + idx, acc);
  }
};
template <typename T> struct EpiSoftmaxBwd {   // dS = P * (dP - rowdot) * scale
  const T* probs;
  const float* rowdot;   // [batch*M]
  float scale;
  int M;
  __device__ void operator()(T* C, long long idx, long long b, int m, int, float acc) const {
    const float p = Elem<T>::ld(probs + idx);
    Elem<T>::st(C + idx, p * (acc - rowdot[b * M + m]) * scale);
  }
};

template <typename T, typename Epi>
__global__ void __launch_bounds__(256) gemm_kernel(const T* __restrict__ A, long long a_bs, int a_rs, int a_cs,
                                                   const T* __restrict__ B, long long b_bs, int b_rs, int b_cs,
                                                   T* __restrict__ C, long long c_bs, int M, int N, int K, Epi epi) {
  __shared__ float As[16][68];
  __shared__ float Bs[16][68];
  const long long b = blockIdx.z;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  A += b * a_bs;
  B += b * b_bs;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += 16) {
    // each thread stages 4 elements of A and of B; the fast index follows the unit stride
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = threadIdx.x + i * 256;          // 0..1023
      int mm, kk;
      if (a_cs == 1) { kk = e % 16; mm = e / 16; } else { mm = e % 64; kk = e / 64; }
      float va = 0.f;
      if (m0 + mm < M && k0 + kk < K) va = Elem<T>::ld(A + (long long)(m0 + mm) * a_rs + (long long)(k0 + kk) * a_cs);
      As[kk][mm] = va;
      int nn, kb;
      if (b_rs == 1) { kb = e % 16; nn = e / 16; } else { nn = e % 64; kb = e / 64; }
      float vb = 0.f;
      if (n0 + nn < N && k0 + kb < K) vb = Elem<T>::ld(B + (long long)(k0 + kb) * b_rs + (long long)(n0 + nn) * b_cs);
      Bs[kb][nn] = vb;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], bb[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bb[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) epi(C, b * c_bs + (long long)m * N + n, b, m, n, acc[i][j]);
    }
  }
}

template <typename T, typename Epi>
static int gemm(const T* A, long long a_bs, int a_rs, int a_cs, const T* B, long long b_bs, int b_rs, int b_cs,
                T* C, int64_t batch, int M, int N, int K, Epi epi, cudaStream_t st, const char* what) {
  if (batch == 0 || M == 0 || N == 0) return VSA_OK;
  if (batch > 65535) return fail(VSA_ERR_UNSUPPORTED, "%s: batch*heads %lld exceeds 65535", what, (long long)batch);
  dim3 grid((N + 63) / 64, (M + 63) / 64, (unsigned)batch);
  gemm_kernel<T, Epi><<<grid, 256, 0, st>>>(A, a_bs, a_rs, a_cs, B, b_bs, b_rs, b_cs, C, (long long)M * N, M, N, K, epi);
  return check_launch(what);
}

// Row softmax of the pooled scores: probs = round(softmax_fp32(scores)).
template <typename T>
__global__ void __launch_bounds__(128) softmax_rows_kernel(const T* __restrict__ scores, T* __restrict__ probs, int n) {
  __shared__ float red[4];
  const T* s = scores + (long long)blockIdx.x * n;
  T* p = probs + (long long)blockIdx.x * n;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < n; i += blockDim.x) mx = fmaxf(mx, Elem<T>::ld(s + i));
  mx = warp_max(mx);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  __syncthreads();
  float sum = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) sum += expf(Elem<T>::ld(s + i) - mx);
  sum = warp_sum(sum);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
  __syncthreads();
  sum = red[0] + red[1] + red[2] + red[3];
  const float inv = 1.f / sum;
  for (int i = threadIdx.x; i < n; i += blockDim.x) Elem<T>::st(p + i, expf(Elem<T>::ld(s + i) - mx) * inv);
}

// The same for rows of up to 3072 scores: one warp per row, the row in registers (read once, one expf per
// element), reductions by shuffles only.  Same arithmetic as above: fp32 max, expf, fp32 sum, one rounding.
template <typename T, int SLOTS>
__global__ void __launch_bounds__(256) softmax_rows_warp_kernel(const T* __restrict__ scores, T* __restrict__ probs,
                                                                long long rows, int n) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* s = scores + row * n;
  T* p = probs + row * n;
  float x[SLOTS];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < SLOTS; ++j) {
    const int i = j * 32 + lane;
    x[j] = i < n ? Elem<T>::ld(s + i) : -INFINITY;
    mx = fmaxf(mx, x[j]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < SLOTS; ++j) {
    x[j] = expf(x[j] - mx);          // exp(-inf) = 0 for the slots beyond the row
    sum += x[j];
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
#pragma unroll
  for (int j = 0; j < SLOTS; ++j) {
    const int i = j * 32 + lane;
    if (i < n) Elem<T>::st(p + i, x[j] * inv);
  }
}

template <typename T>
static int launch_softmax_rows(const T* scores, T* probs, long long rows, int n, cudaStream_t st) {
  const unsigned grid = (unsigned)((rows + 7) / 8);
  if (n <= 512) {
    softmax_rows_warp_kernel<T, 16><<<grid, 256, 0, st>>>(scores, probs, rows, n);
  } else if (n <= 1536) {
    softmax_rows_warp_kernel<T, 48><<<grid, 256, 0, st>>>(scores, probs, rows, n);
  } else if (n <= 3072) {
    softmax_rows_warp_kernel<T, 96><<<grid, 256, 0, st>>>(scores, probs, rows, n);
  } else {
    softmax_rows_kernel<T><<<(unsigned)rows, 128, 0, st>>>(scores, probs, n);
  }
  return check_launch("softmax_rows_kernel");
}

// rowdot[r] = sum_d a[r,d] * b[r,d]  (one warp per row)
template <typename T>
__global__ void rowdot_kernel(const T* __restrict__ a, const T* __restrict__ b, float* __restrict__ out, long long rows, int D) {
  const long long r = (long long)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  if (r >= rows) return;
  float s = 0.f;
  for (int d = threadIdx.x & 31; d < D; d += 32) s += Elem<T>::ld(a + r * D + d) * Elem<T>::ld(b + r * D + d);
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) out[r] = s;
}

int softmax_rows(const void* scores, void* probs, int64_t rows, int n, int dtype, cudaStream_t st) {
  if (rows == 0) return VSA_OK;
  if (rows > 0x7fffffffLL) return fail(VSA_ERR_UNSUPPORTED, "pooled softmax: too many rows");
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = VSA_TAG_TYPE(tag);
    return launch_softmax_rows<T>((const T*)scores, (T*)probs, rows, n, st);
  });
}

int rowdot_rows(const void* a, const void* b, float* out, int64_t rows, int D, int dtype, cudaStream_t st) {
  if (rows == 0) return VSA_OK;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = VSA_TAG_TYPE(tag);
    rowdot_kernel<T><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>((const T*)a, (const T*)b, out, rows, D);
    return check_launch("rowdot_kernel");
  });
}

template <typename T>
static int coarse_fwd_t(const T* qc, const T* kc, const T* vc, T* scores, T* probs, T* out_c,
                        int64_t BH, int Qb, int Kb, int D, float scale, cudaStream_t st) {
  // scores[Qb,Kb] = qc[Qb,D] * kc[Kb,D]^T
  int rc = gemm<T>(qc, (long long)Qb * D, D, 1, kc, (long long)Kb * D, 1, D, scores, BH, Qb, Kb, D,
                   EpiScores{scale}, st, "coarse scores");
  if (rc) return rc;
  const long long rows = BH * Qb;
  if (rows > 0x7fffffffLL) return fail(VSA_ERR_UNSUPPORTED, "coarse softmax: too many rows");
  rc = launch_softmax_rows<T>(scores, probs, rows, Kb, st);
  if (rc) return rc;
  // out_c[Qb,D] = probs[Qb,Kb] * vc[Kb,D]
  return gemm<T>(probs, (long long)Qb * Kb, Kb, 1, vc, (long long)Kb * D, D, 1, out_c, BH, Qb, D, Kb, EpiStore{}, st,
                 "coarse output");
}

int coarse_fwd(const void* qc, const void* kc, const void* vc, void* scores, void* probs, void* out_c, int64_t BH,
               int Qb, int Kb, int D, float scale, int dtype, cudaStream_t st) {
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = VSA_TAG_TYPE(tag);
    return coarse_fwd_t<T>((const T*)qc, (const T*)kc, (const T*)vc, (T*)scores, (T*)probs, (T*)out_c, BH, Qb, Kb, D,
                           scale, st);
  });
}

template <typename T>
static int coarse_bwd_t(const T* d_out_c, const T* out_c, const T* qc, const T* kc, const T* vc, const T* probs,
                        T* ds, float* rowdot, T* dqc, T* dkc, T* dvc, int64_t BH, int Qb, int Kb, int D, float scale,
                        cudaStream_t st) {
  const long long rows = BH * Qb;
  if (rows == 0) return VSA_OK;
  rowdot_kernel<T><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(d_out_c, out_c, rowdot, rows, D);
  int rc = check_launch("rowdot_kernel");
  if (rc) return rc;
  // dV_c[Kb,D] = probs^T[Kb,Qb] * d_out_c[Qb,D]
  rc = gemm<T>(probs, (long long)Qb * Kb, 1, Kb, d_out_c, (long long)Qb * D, D, 1, dvc, BH, Kb, D, Qb, EpiStore{}, st,
               "coarse dV");
  if (rc) return rc;
  // dS[Qb,Kb] = probs * (d_out_c[Qb,D] * vc[Kb,D]^T - rowdot) * scale
  rc = gemm<T>(d_out_c, (long long)Qb * D, D, 1, vc, (long long)Kb * D, 1, D, ds, BH, Qb, Kb, D,
               EpiSoftmaxBwd<T>{probs, rowdot, scale, Qb}, st, "coarse dS");
  if (rc) return rc;
  // dQ_c[Qb,D] = dS[Qb,Kb] * kc[Kb,D]
  rc = gemm<T>(ds, (long long)Qb * Kb, Kb, 1, kc, (long long)Kb * D, D, 1, dqc, BH, Qb, D, Kb, EpiStore{}, st,
               "coarse dQ");
  if (rc) return rc;
  // dK_c[Kb,D] = dS^T[Kb,Qb] * qc[Qb,D]
  return gemm<T>(ds, (long long)Qb * Kb, 1, Kb, qc, (long long)Qb * D, D, 1, dkc, BH, Kb, D, Qb, EpiStore{}, st,
                 "coarse dK");
}

int coarse_bwd(const void* d_out_c, const void* out_c, const void* qc, const void* kc, const void* vc,
               const void* probs, void* ds, float* rowdot, void* dqc, void* dkc, void* dvc, int64_t BH, int Qb, int Kb,
               int D, float scale, int dtype, cudaStream_t st) {
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = VSA_TAG_TYPE(tag);
    return coarse_bwd_t<T>((const T*)d_out_c, (const T*)out_c, (const T*)qc, (const T*)kc, (const T*)vc,
                           (const T*)probs, (T*)ds, rowdot, (T*)dqc, (T*)dkc, (T*)dvc, BH, Qb, Kb, D, scale, st);
  });
}

// =========================================================================================
// Top-K by radix select (vsa/torch_impl.py:85 of the reference).  Every id with a key above the
// k-th largest, plus the lowest-numbered ids equal to it, are written in ascending id order.
// Long rows (> 3072 scores): one CTA per row, keys in shared memory, four 8-bit histogram passes.
// =========================================================================================
constexpr int kTopkThreads = 256;
constexpr int kTopkMaxCols = 8192;

__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

template <typename T>
__global__ void __launch_bounds__(kTopkThreads) topk_kernel(const T* __restrict__ scores, int32_t* __restrict__ selected,
                                                            int n, int topk) {
  extern __shared__ uint32_t keys[];       // [n]
  __shared__ int hist[256];
  __shared__ uint32_t sh_prefix;
  __shared__ int sh_k;
  __shared__ int warp_cnt[2][kTopkThreads / 32];
  const T* s = scores + (long long)blockIdx.x * n;
  int32_t* out = selected + (long long)blockIdx.x * topk;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  for (int i = tid; i < n; i += kTopkThreads) keys[i] = order_key(Elem<T>::ld(s + i));
  if (tid == 0) { sh_prefix = 0; sh_k = topk; }
  __syncthreads();

  for (int pass = 3; pass >= 0; --pass) {
    hist[tid] = 0;
    __syncthreads();
    const uint32_t prefix = sh_prefix;
    const int k = sh_k;
    const int shift = pass * 8;
    const uint32_t hi_mask = pass == 3 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = tid; i < n; i += kTopkThreads) {
      const uint32_t key = keys[i];
      if ((key & hi_mask) == prefix) atomicAdd(&hist[(key >> shift) & 255], 1);
    }
    __syncthreads();
    if (warp == 0) {
      // lane l owns bins [255-8l-7, 255-8l]; scan from the top bin down
      int mine = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) mine += hist[255 - 8 * lane - j];
      int incl = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      const int above = incl - mine;                  // elements in bins above this lane's range
      if (above < k && k <= incl) {
        int run = above;
        for (int j = 0; j < 8; ++j) {
          const int bin = 255 - 8 * lane - j;
          const int c = hist[bin];
          if (k <= run + c) {
            sh_prefix = prefix | ((uint32_t)bin << shift);
            sh_k = k - run;
            break;
          }
          run += c;
        }
      }
    }
    __syncthreads();
  }
  const uint32_t thr = sh_prefix;
  const int take_eq = sh_k;        // how many ids equal to the threshold are kept (>= 1)

  int eq_seen = 0, written = 0;
  for (int base = 0; base < n; base += kTopkThreads) {
    const int i = base + tid;
    const uint32_t key = i < n ? keys[i] : 0u;
    const bool gt = i < n && key > thr;
    const bool eq = i < n && key == thr;
    const unsigned eq_b = __ballot_sync(0xffffffffu, eq);
    if (lane == 0) warp_cnt[0][warp] = __popc(eq_b);
    __syncthreads();
    int eq_before = eq_seen, eq_total = 0;
#pragma unroll
    for (int w = 0; w < kTopkThreads / 32; ++w) {
      const int c = warp_cnt[0][w];
      if (w < warp) eq_before += c;
      eq_total += c;
    }
    eq_before += __popc(eq_b & ((1u << lane) - 1u));
    const bool take = gt || (eq && eq_before < take_eq);
    const unsigned tk_b = __ballot_sync(0xffffffffu, take);
    if (lane == 0) warp_cnt[1][warp] = __popc(tk_b);
    __syncthreads();
    int pos = written, tk_total = 0;
#pragma unroll
    for (int w = 0; w < kTopkThreads / 32; ++w) {
      const int c = warp_cnt[1][w];
      if (w < warp) pos += c;
      tk_total += c;
    }
    pos += __popc(tk_b & ((1u << lane) - 1u));
    if (take && pos < topk) out[pos] = i;
    eq_seen += eq_total;
    written += tk_total;
    __syncthreads();
  }
}

// Rows of up to 3072 scores: one WARP per row, the keys in registers (lane l holds ids l, l+32, ...), no shared
// memory and no block-wide barrier.  The k-th largest key is built bit by bit from the top ("is the number of
// keys >= candidate still >= k?": a compare-and-count over the registers and one redux.sync per bit); 16-bit
// inputs need 16 bits only, because the low bits of their keys carry no information once masked.  Then one pass
// over the registers in id order writes every id above the threshold and the lowest ids equal to it.
template <typename T> struct KeyBits { static constexpr int low = 0; };
template <> struct KeyBits<__nv_bfloat16> { static constexpr int low = 16; };
template <> struct KeyBits<__half> { static constexpr int low = 13; };

// VEC = 1: lane l holds keys l, l + 32, ... (any row length and alignment).  VEC = 16 / sizeof(T): lane l holds VEC
// consecutive keys per 16-byte load, slot j <-> key ((j / VEC) * 32 + l) * VEC + j % VEC; eight (four) times fewer
// load instructions, each a full 512-byte warp access.  Needs rows that start on 16 bytes (n a multiple of VEC).
template <typename T, int SLOTS, int VEC>
__global__ void __launch_bounds__(256) topk_warp_kernel(const T* __restrict__ scores, int32_t* __restrict__ selected,
                                                        long long rows, int n, int topk) {
  static_assert(SLOTS % VEC == 0, "slots come in groups of VEC");
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* s = scores + row * n;
  int32_t* out = selected + row * topk;
  constexpr int kLow = KeyBits<T>::low;
  constexpr uint32_t kMask = kLow ? ~((1u << kLow) - 1u) : 0xffffffffu;
  auto id_of = [&](int j) -> int { return ((j / VEC) * 32 + lane) * VEC + (j % VEC); };
  uint32_t key[SLOTS];
  if (VEC == 1) {
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) {
      const int i = id_of(j);
      key[j] = i < n ? (order_key(Elem<T>::ld(s + i)) & kMask) : 0u;     // 0 sorts below every candidate
    }
  } else {
#pragma unroll
    for (int g = 0; g < SLOTS / VEC; ++g) {
      const int i0 = (g * 32 + lane) * VEC;
      uint4 raw = make_uint4(0, 0, 0, 0);
      if (i0 < n) raw = *reinterpret_cast<const uint4*>(s + i0);         // n is a multiple of VEC: all or nothing
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int x = 0; x < VEC; ++x) key[g * VEC + x] = i0 < n ? (order_key(Elem<T>::ld(e + x)) & kMask) : 0u;
    }
  }
  uint32_t thr = 0;
#pragma unroll 1
  for (int b = 31; b >= kLow; --b) {
    const uint32_t t = thr | (1u << b);
    int cnt = 0;
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) cnt += key[j] >= t ? 1 : 0;
    cnt = __reduce_add_sync(0xffffffffu, cnt);
    if (cnt >= topk) thr = t;
  }
  int above = 0;
#pragma unroll
  for (int j = 0; j < SLOTS; ++j) above += key[j] > thr ? 1 : 0;
  above = __reduce_add_sync(0xffffffffu, above);
  const int take_eq = topk - above;            // ids equal to the threshold that are kept (lowest first)
  // The best-scoring block goes first (lowest id among equals, so it is in the kept set), the rest follow in
  // ascending id order.  The order of a route does not change what is attended to, but the fine forward takes its
  // softmax shift from the first pair of tiles it meets: with the best block there the shift is next to the row
  // maximum, P stays near or below 1, and the out-of-range recomputation stays the exception on real score
  // distributions (above all for fp16, whose P overflows 2^16).
  uint32_t best = 0;
#pragma unroll
  for (int j = 0; j < SLOTS; ++j) best = key[j] > best ? key[j] : best;      // slots beyond n hold 0
  best = __reduce_max_sync(0xffffffffu, best);
  int first = 0x7fffffff;
#pragma unroll
  for (int j = SLOTS - 1; j >= 0; --j) {
    const int i = id_of(j);
    first = (key[j] == best && i < n) ? i : first;                         // ids of a lane ascend with j: the lowest wins
  }
  const int lead = __reduce_min_sync(0xffffffffu, first);
  if (lane == 0) out[0] = lead;
  const unsigned lt = (1u << lane) - 1u;
  int written = 1, eq_seen = 0;
  // groups of VEC slots; inside a group ids ascend by (lane, slot), so an element's rank is the count over lower lanes
  // (all slots of the group) plus the count over its own earlier slots
#pragma unroll
  for (int g = 0; g < SLOTS / VEC; ++g) {
    unsigned eq_b[VEC];
    bool eq[VEC], gt[VEC];
    int eq_lower = 0, eq_all = 0;
#pragma unroll
    for (int x = 0; x < VEC; ++x) {
      const int j = g * VEC + x;
      gt[x] = key[j] > thr;
      eq[x] = key[j] == thr && id_of(j) < n;
      eq_b[x] = __ballot_sync(0xffffffffu, eq[x]);
      eq_lower += __popc(eq_b[x] & lt);
      eq_all += __popc(eq_b[x]);
    }
    bool take[VEC];
    int tk_lower = 0, tk_all = 0, own_eq = 0;
    unsigned tk_b[VEC];
#pragma unroll
    for (int x = 0; x < VEC; ++x) {
      const int j = g * VEC + x;
      const bool kept = gt[x] || (eq[x] && eq_seen + eq_lower + own_eq < take_eq);
      own_eq += eq[x] ? 1 : 0;
      take[x] = kept && id_of(j) != lead;
      tk_b[x] = __ballot_sync(0xffffffffu, take[x]);
      tk_lower += __popc(tk_b[x] & lt);
      tk_all += __popc(tk_b[x]);
    }
    int own_tk = 0;
#pragma unroll
    for (int x = 0; x < VEC; ++x) {
      const int pos = written + tk_lower + own_tk;
      if (take[x] && pos < topk) out[pos] = id_of(g * VEC + x);
      own_tk += take[x] ? 1 : 0;
    }
    eq_seen += eq_all;
    written += tk_all;
  }
}

int topk_select(const void* scores, int32_t* selected, int64_t rows, int Kb, int topk, int dtype, cudaStream_t st) {
  if (rows == 0) return VSA_OK;
  if (Kb > kTopkMaxCols) return fail(VSA_ERR_UNSUPPORTED, "topk: %d key blocks exceed the supported %d", Kb, kTopkMaxCols);
  if (rows > 0x7fffffffLL) return fail(VSA_ERR_UNSUPPORTED, "topk: too many rows");
  const size_t smem = (size_t)Kb * sizeof(uint32_t);
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = VSA_TAG_TYPE(tag);
    const unsigned grid = (unsigned)((rows + 7) / 8);
    constexpr int kVec = 16 / (int)sizeof(T);
    const bool wide = Kb % kVec == 0 && reinterpret_cast<uintptr_t>(scores) % 16 == 0;
    auto launch = [&](auto narrow, auto vector) -> int {
      if (wide) vector<<<grid, 256, 0, st>>>((const T*)scores, selected, rows, Kb, topk);
      else narrow<<<grid, 256, 0, st>>>((const T*)scores, selected, rows, Kb, topk);
      return check_launch("topk_warp_kernel");
    };
    if (Kb <= 512) return launch(topk_warp_kernel<T, 16, 1>, topk_warp_kernel<T, 16, kVec>);
    if (Kb <= 1536) return launch(topk_warp_kernel<T, 48, 1>, topk_warp_kernel<T, 48, kVec>);
    if (Kb <= 3072) return launch(topk_warp_kernel<T, 96, 1>, topk_warp_kernel<T, 96, kVec>);
    topk_kernel<T><<<(unsigned)rows, kTopkThreads, smem, st>>>((const T*)scores, selected, Kb, topk);
    return check_launch("topk_kernel");
  });
}

// =========================================================================================
// Route inversion (vsa/triton_impl.py:476-595 of the reference): count, scan, scatter.
// =========================================================================================
__global__ void route_count_kernel(const int32_t* __restrict__ selected, int32_t* __restrict__ counts,
                                   long long edges_total, int edges_per_bh, int Kb) {
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= edges_total) return;
  const long long bh = e / edges_per_bh;
  const int kv = selected[e];
  if ((unsigned)kv < (unsigned)Kb) atomicAdd(&counts[bh * Kb + kv], 1);
}

__global__ void __launch_bounds__(256) route_scan_kernel(const int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
                                                         int32_t* __restrict__ cursor, int Kb) {
  __shared__ int warp_tot[8];
  __shared__ int carry_sm;
  const long long bh = blockIdx.x;
  const int32_t* c = counts + bh * Kb;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_sm = 0;
  __syncthreads();
  for (int base = 0; base < Kb; base += 256) {
    const int i = base + threadIdx.x;
    const int v = i < Kb ? c[i] : 0;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int before = carry_sm;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    if (i < Kb) {
      offsets[bh * Kb + i] = before + incl - v;
      cursor[bh * Kb + i] = before + incl - v;
    }
    __syncthreads();
    if (threadIdx.x == 255) carry_sm = before + incl;
    __syncthreads();
  }
}

// What a row of the inverse table holds per in-edge: the query block id (the reference's table), or, packed,
// (query block << 11) | position of the key block in that query block's route -- which names the edge itself.
__device__ __forceinline__ int32_t route_entry(int edge_in_slice, int topk, bool packed) {
  const int qb = edge_in_slice / topk;
  return packed ? (int32_t)((qb << 11) | (edge_in_slice - qb * topk)) : (int32_t)qb;
}

__global__ void route_scatter_kernel(const int32_t* __restrict__ selected, int32_t* __restrict__ cursor,
                                     int32_t* __restrict__ inverse, long long edges_total, int edges_per_bh, int Kb,
                                     int topk, bool packed) {
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= edges_total) return;
  const long long bh = e / edges_per_bh;
  const int within = (int)(e - bh * edges_per_bh);
  const int kv = selected[e];
  if ((unsigned)kv >= (unsigned)Kb) return;
  const int slot = atomicAdd(&cursor[bh * Kb + kv], 1);
  inverse[bh * edges_per_bh + slot] = route_entry(within, topk, packed);
}

// Chunked forms of the two passes for key-block counts that fit in shared memory: a CTA owns a contiguous chunk
// of one slice's edges, histograms it in shared memory, and touches global memory with ONE atomic per key block
// it met (the plain forms above pay one global atomic per edge: 20.7 M at the 92k-token shape, now 1.8 M).
// In the scatter pass the global atomic claims a run of slots for the CTA's edges of that key block; positions
// inside the run come from a second shared-memory counter.  Order inside a key row stays unspecified.
constexpr int kRouteChunkThreads = 512;
constexpr int kRouteMaxSmemKb = 6144;        // 2 x int32 [Kb] <= 48 KB

__global__ void __launch_bounds__(kRouteChunkThreads)
route_count_chunk_kernel(const int32_t* __restrict__ selected, int32_t* __restrict__ counts, int edges_per_bh,
                         int chunk, int Kb) {
  extern __shared__ int32_t route_sm[];
  int32_t* hist = route_sm;
  const long long bh = blockIdx.y;
  const int e0 = blockIdx.x * chunk, e1 = min(edges_per_bh, e0 + chunk);
  const int32_t* sel = selected + bh * edges_per_bh;
  for (int i = threadIdx.x; i < Kb; i += kRouteChunkThreads) hist[i] = 0;
  __syncthreads();
  for (int e = e0 + threadIdx.x; e < e1; e += kRouteChunkThreads) {
    const int kv = sel[e];
    if ((unsigned)kv < (unsigned)Kb) atomicAdd(&hist[kv], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < Kb; i += kRouteChunkThreads) {
    const int c = hist[i];
    if (c) atomicAdd(&counts[bh * Kb + i], c);
  }
}

__global__ void __launch_bounds__(kRouteChunkThreads)
route_scatter_chunk_kernel(const int32_t* __restrict__ selected, int32_t* __restrict__ cursor,
                           int32_t* __restrict__ inverse, int edges_per_bh, int chunk, int Kb, int topk, bool packed) {
  extern __shared__ int32_t route_sm[];
  int32_t* hist = route_sm;            // count of this chunk per key block, then the first claimed slot
  int32_t* next = route_sm + Kb;       // slots handed out so far inside the claimed run
  const long long bh = blockIdx.y;
  const int e0 = blockIdx.x * chunk, e1 = min(edges_per_bh, e0 + chunk);
  const int32_t* sel = selected + bh * edges_per_bh;
  for (int i = threadIdx.x; i < Kb; i += kRouteChunkThreads) {
    hist[i] = 0;
    next[i] = 0;
  }
  __syncthreads();
  for (int e = e0 + threadIdx.x; e < e1; e += kRouteChunkThreads) {
    const int kv = sel[e];
    if ((unsigned)kv < (unsigned)Kb) atomicAdd(&hist[kv], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < Kb; i += kRouteChunkThreads) {
    const int c = hist[i];
    if (c) hist[i] = atomicAdd(&cursor[bh * Kb + i], c);
  }
  __syncthreads();
  int32_t* inv = inverse + bh * edges_per_bh;
  for (int e = e0 + threadIdx.x; e < e1; e += kRouteChunkThreads) {
    const int kv = sel[e];
    if ((unsigned)kv >= (unsigned)Kb) continue;
    inv[hist[kv] + atomicAdd(&next[kv], 1)] = route_entry(e, topk, packed);
  }
}

int route_invert(const int32_t* selected, int32_t* counts, int32_t* offsets, int32_t* inverse, int32_t* cursor,
                 int64_t BH, int Qb, int Kb, int topk, cudaStream_t st, bool packed) {
  const long long per = (long long)Qb * topk;
  if (packed && (topk > 2048 || Qb >= (1 << 20)))
    return fail(VSA_ERR_UNSUPPORTED, "route inversion: packed edges need topk <= 2048 and fewer than 2^20 query blocks");
  const long long total = BH * per;
  if (BH == 0 || Kb == 0) return VSA_OK;
  if (per > 0x7fffffffLL) return fail(VSA_ERR_UNSUPPORTED, "route inversion: too many edges per slice");
  if (cudaMemsetAsync(counts, 0, sizeof(int32_t) * BH * Kb, st) != cudaSuccess)
    return fail(VSA_ERR_LAUNCH, "route inversion: memset failed: %s", cudaGetErrorString(cudaGetLastError()));
  const bool chunked = Kb <= kRouteMaxSmemKb && BH <= 65535;
  // chunks of >= 8192 edges, at most 64 per slice: enough CTAs to fill the GPU, few enough global atomics
  const int chunks = (int)std::max<long long>(1, std::min<long long>(64, per / 8192));
  const int chunk = (int)((per + chunks - 1) / chunks);
  const dim3 grid((unsigned)chunks, (unsigned)BH);
  int rc = VSA_OK;
  if (total > 0) {
    if (chunked) {
      route_count_chunk_kernel<<<grid, kRouteChunkThreads, sizeof(int32_t) * Kb, st>>>(selected, counts, (int)per, chunk, Kb);
      rc = check_launch("route_count_chunk_kernel");
    } else {
      const unsigned blocks = (unsigned)((total + 255) / 256);
      route_count_kernel<<<blocks, 256, 0, st>>>(selected, counts, total, (int)per, Kb);
      rc = check_launch("route_count_kernel");
    }
    if (rc) return rc;
  }
  route_scan_kernel<<<(unsigned)BH, 256, 0, st>>>(counts, offsets, cursor, Kb);
  rc = check_launch("route_scan_kernel");
  if (rc) return rc;
  if (total > 0) {
    if (chunked) {
      route_scatter_chunk_kernel<<<grid, kRouteChunkThreads, 2 * sizeof(int32_t) * Kb, st>>>(selected, cursor, inverse,
                                                                                            (int)per, chunk, Kb, topk, packed);
      rc = check_launch("route_scatter_chunk_kernel");
    } else {
      const unsigned blocks = (unsigned)((total + 255) / 256);
      route_scatter_kernel<<<blocks, 256, 0, st>>>(selected, cursor, inverse, total, (int)per, Kb, topk, packed);
      rc = check_launch("route_scatter_kernel");
    }
  }
  return rc;
}

// -----------------------------------------------------------------------------------------
// Route inversion for callers that cannot hand over scratch memory.
//
// Some hosts of this library may not allocate device memory at the point where they need the
// inverse routing: a serving process that gave the whole GPU to its own memory pool at start-up
// (a later cudaMalloc simply fails), or a latency-critical loop in which cudaMalloc is banned
// because it synchronises the device.  For them the per-key-block cursor that the scatter step
// needs lives in the fixed array below instead of a caller-provided buffer.  The array belongs to
// the library image: every GPU that loads the library holds these 1 MiB until the process exits.
//
// In host code the name `g_static_cursor` is only a handle for the symbol, not a device address;
// the device address is looked up once per device with cudaGetSymbolAddress (with that device
// current) and that pointer is what the kernels receive.
// -----------------------------------------------------------------------------------------
constexpr long long kStaticCursorEntries = 1LL << 18;          // batch*heads*key_blocks <= 262,144
static __device__ __align__(256) int32_t g_static_cursor[kStaticCursorEntries];

static int32_t* static_cursor_for_current_device(int* rc_out) {
  constexpr int kMaxDevices = 64;
  static int32_t* ptrs[kMaxDevices] = {};
  static std::mutex mu;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    *rc_out = fail(VSA_ERR_LAUNCH, "static route inversion: cannot identify the current device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_cursor);
    if (e != cudaSuccess || !p) {
      *rc_out = fail(VSA_ERR_LAUNCH, "static route inversion: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    ptrs[dev] = static_cast<int32_t*>(p);
  }
  *rc_out = VSA_OK;
  return ptrs[dev];
}

int route_invert_static(const int32_t* selected, int32_t* counts, int32_t* offsets, int32_t* inverse, int64_t BH,
                        int Qb, int Kb, int topk, cudaStream_t st) {
  if (BH * (long long)Kb > kStaticCursorEntries)
    return fail(VSA_ERR_UNSUPPORTED,
                "static route inversion: batch*heads*key_blocks = %lld exceeds the built-in scratch of %lld entries; "
                "use vsa_route_invert with a caller-provided cursor buffer",
                (long long)(BH * (long long)Kb), kStaticCursorEntries);
  int rc = VSA_OK;
  int32_t* cursor = static_cursor_for_current_device(&rc);
  if (!cursor) return rc;
  // the scan step rewrites every cursor entry it will use, so nothing left by an earlier call survives
  return route_invert(selected, counts, offsets, inverse, cursor, BH, Qb, Kb, topk, st, false);
}

// =========================================================================================
// Gated combine (vsa/fused_common.py:175-256 of the reference).
// =========================================================================================
template <typename T, bool GATE>
__global__ void __launch_bounds__(256) combine_fwd_kernel(const T* __restrict__ out_s, const T* __restrict__ out_c,
                                                          const T* __restrict__ gate, T* __restrict__ out,
                                                          long long chunks, int D, int be) {
  constexpr int VEC = 16 / sizeof(T);
  const int cpr = D / VEC;
  for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < chunks;
       c += (long long)gridDim.x * blockDim.x) {
    const long long row = c / cpr;
    const int ch = (int)(c - row * cpr);
    const long long blk = row / be;
    const uint4 s_raw = *reinterpret_cast<const uint4*>(out_s + c * VEC);
    const uint4 c_raw = *reinterpret_cast<const uint4*>(out_c + blk * D + ch * VEC);
    uint4 g_raw = make_uint4(0, 0, 0, 0);
    if (GATE) g_raw = *reinterpret_cast<const uint4*>(gate + c * VEC);
    uint4 o_raw;
    const T* se = reinterpret_cast<const T*>(&s_raw);
    const T* ce = reinterpret_cast<const T*>(&c_raw);
    const T* ge = reinterpret_cast<const T*>(&g_raw);
    T* oe = reinterpret_cast<T*>(&o_raw);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      float cv = Elem<T>::ld(ce + i);
      if (GATE) cv *= Elem<T>::ld(ge + i);
      Elem<T>::st(oe + i, Elem<T>::ld(se + i) + cv);
    }
    *reinterpret_cast<uint4*>(out + c * VEC) = o_raw;
  }
}

int combine_fwd(const void* out_s, const void* out_c, const void* gate, void* out, int64_t BH, int64_t Lq, int D,
                int be, int dtype, cudaStream_t st) {
  const int vec = elems_per_16_bytes(dtype);
  if (D % vec != 0) return fail(VSA_ERR_UNSUPPORTED, "combine: head dim %d must be a multiple of %d", D, vec);
  const long long chunks = BH * Lq * (D / vec);
  if (chunks == 0) return VSA_OK;
  long long blocks = (chunks + 255) / 256;
  if (blocks > 148LL * 64) blocks = 148LL * 64;
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = VSA_TAG_TYPE(tag);
    if (gate)
      combine_fwd_kernel<T, true><<<(unsigned)blocks, 256, 0, st>>>((const T*)out_s, (const T*)out_c, (const T*)gate,
                                                                   (T*)out, chunks, D, be);
    else
      combine_fwd_kernel<T, false><<<(unsigned)blocks, 256, 0, st>>>((const T*)out_s, (const T*)out_c, (const T*)gate,
                                                                    (T*)out, chunks, D, be);
    return check_launch("combine_fwd_kernel");
  });
}

// One CTA per (bh, query block): d_out_c = sum over ALL be rows of dout*gate (padded
// query rows included), dgate = dout * out_c[block], both from a single read of dout.
template <typename T, bool GATE>
__global__ void __launch_bounds__(128) combine_bwd_kernel(const T* __restrict__ dout, const T* __restrict__ gate,
                                                          const T* __restrict__ out_c, T* __restrict__ d_out_c,
                                                          T* __restrict__ dgate, int D, int be) {
  constexpr int VEC = 16 / sizeof(T);
  __shared__ __align__(16) float part_sm[128 * VEC];     // [row group][D] partial sums
  const long long blk = blockIdx.x;
  const T* g_do = dout + blk * (long long)be * D;
  const T* g_gate = GATE ? gate + blk * (long long)be * D : nullptr;
  T* g_dgate = (GATE && dgate) ? dgate + blk * (long long)be * D : nullptr;
  const int cpr = D / VEC;
  const int rows_per_pass = blockDim.x / cpr;
  const int chunk = threadIdx.x % cpr;
  const int rgrp = threadIdx.x / cpr;
  if (rgrp < rows_per_pass) {
    float cvec[VEC], part[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      cvec[i] = Elem<T>::ld(out_c + blk * D + chunk * VEC + i);
      part[i] = 0.f;
    }
#pragma unroll 4
    for (int r = rgrp; r < be; r += rows_per_pass) {
      const long long off = (long long)r * D + chunk * VEC;
      const uint4 d_raw = *reinterpret_cast<const uint4*>(g_do + off);
      const T* de = reinterpret_cast<const T*>(&d_raw);
      if (GATE) {
        const uint4 g_raw = *reinterpret_cast<const uint4*>(g_gate + off);
        const T* ge = reinterpret_cast<const T*>(&g_raw);
        uint4 o_raw;
        T* oe = reinterpret_cast<T*>(&o_raw);
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          const float dv = Elem<T>::ld(de + i);
          part[i] += dv * Elem<T>::ld(ge + i);
          Elem<T>::st(oe + i, dv * cvec[i]);
        }
        if (g_dgate) *reinterpret_cast<uint4*>(g_dgate + off) = o_raw;
      } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) part[i] += Elem<T>::ld(de + i);
      }
    }
    float* dst = part_sm + rgrp * D + chunk * VEC;
#pragma unroll
    for (int i = 0; i < VEC; ++i) dst[i] = part[i];
  }
  __syncthreads();
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float sum = 0.f;
    for (int g = 0; g < rows_per_pass; ++g) sum += part_sm[g * D + d];     // fixed order: deterministic
    Elem<T>::st(d_out_c + blk * D + d, sum);
  }
}

int combine_bwd(const void* dout, const void* gate, const void* out_c, void* d_out_c, void* dgate, int64_t BH,
                int64_t Lq, int D, int be, int dtype, cudaStream_t st) {
  const int vec = elems_per_16_bytes(dtype);
  if (D % vec != 0 || D / vec > 128 || D > 256)
    return fail(VSA_ERR_UNSUPPORTED, "combine backward: head dim %d must be a multiple of %d and <= 256", D, vec);
  const long long blocks = BH * (Lq / be);
  if (blocks == 0) return VSA_OK;
  if (blocks > 0x7fffffffLL) return fail(VSA_ERR_UNSUPPORTED, "combine backward: too many blocks");
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = VSA_TAG_TYPE(tag);
    if (gate)
      combine_bwd_kernel<T, true><<<(unsigned)blocks, 128, 0, st>>>((const T*)dout, (const T*)gate, (const T*)out_c,
                                                                   (T*)d_out_c, (T*)dgate, D, be);
    else
      combine_bwd_kernel<T, false><<<(unsigned)blocks, 128, 0, st>>>((const T*)dout, (const T*)gate, (const T*)out_c,
                                                                    (T*)d_out_c, (T*)dgate, D, be);
    return check_launch("combine_bwd_kernel");
  });
}

// Combine backward for raster-order activations, with the tile-order copy of dout as a by-product.  dout and the
// gate are read at each token's raster row ([B][S][H][D], see RasterMap), dgate is written there, and every row of
// dout is also stored in tile order ([BH][Lq][D], zeros in the padding rows) for the TMA loads of the fine backward:
// one pass instead of two gathers, the combine backward and an un-tiling of dgate.
template <typename T, bool GATE>
__global__ void __launch_bounds__(128) combine_bwd_raster_kernel(const T* __restrict__ dout_raster, const T* __restrict__ gate_raster,
                                                                 const T* __restrict__ out_c, T* __restrict__ d_out_c,
                                                                 T* __restrict__ dgate_raster, T* __restrict__ dout_tiled,
                                                                 RasterMap rm, int blocks_per_slice, int D, int be) {
  constexpr int VEC = 16 / sizeof(T);
  __shared__ __align__(16) float part_sm[128 * VEC];     // [row group][D] partial sums
  const long long blk = blockIdx.x;
  const long long bh = blk / blocks_per_slice;
  const long long token0 = (blk - bh * blocks_per_slice) * (long long)be;
  T* t_do = dout_tiled + blk * (long long)be * D;
  const int cpr = D / VEC;
  const int rows_per_pass = blockDim.x / cpr;
  const int chunk = threadIdx.x % cpr;
  const int rgrp = threadIdx.x / cpr;
  if (rgrp < rows_per_pass) {
    float cvec[VEC], part[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      cvec[i] = Elem<T>::ld(out_c + blk * D + chunk * VEC + i);
      part[i] = 0.f;
    }
#pragma unroll 4
    for (int r = rgrp; r < be; r += rows_per_pass) {
      const long long rrow = raster_row(rm, bh, token0 + r);
      uint4 d_raw = make_uint4(0, 0, 0, 0);
      if (rrow >= 0) {
        const long long roff = rrow * D + chunk * VEC;
        d_raw = *reinterpret_cast<const uint4*>(dout_raster + roff);
        const T* de = reinterpret_cast<const T*>(&d_raw);
        if (GATE) {
          const uint4 g_raw = *reinterpret_cast<const uint4*>(gate_raster + roff);
          const T* ge = reinterpret_cast<const T*>(&g_raw);
          uint4 o_raw;
          T* oe = reinterpret_cast<T*>(&o_raw);
#pragma unroll
          for (int i = 0; i < VEC; ++i) {
            const float dv = Elem<T>::ld(de + i);
            part[i] += dv * Elem<T>::ld(ge + i);
            Elem<T>::st(oe + i, dv * cvec[i]);
          }
          if (dgate_raster) *reinterpret_cast<uint4*>(dgate_raster + roff) = o_raw;
        } else {
#pragma unroll
          for (int i = 0; i < VEC; ++i) part[i] += Elem<T>::ld(de + i);
        }
      }
      *reinterpret_cast<uint4*>(t_do + (long long)r * D + chunk * VEC) = d_raw;
    }
    float* dst = part_sm + rgrp * D + chunk * VEC;
#pragma unroll
    for (int i = 0; i < VEC; ++i) dst[i] = part[i];
  }
  __syncthreads();
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float sum = 0.f;
    for (int g = 0; g < rows_per_pass; ++g) sum += part_sm[g * D + d];     // fixed order: deterministic
    Elem<T>::st(d_out_c + blk * D + d, sum);
  }
}

int combine_bwd_raster(const void* dout_raster, const void* gate_raster, const void* out_c, void* d_out_c,
                       void* dgate_raster, void* dout_tiled, const int32_t* map, int64_t raster_rows, int heads,
                       int64_t BH, int64_t Lq, int D, int be, int dtype, cudaStream_t st) {
  const int vec = elems_per_16_bytes(dtype);
  if (D % vec != 0 || D / vec > 128 || D > 256)
    return fail(VSA_ERR_UNSUPPORTED, "combine backward (raster): head dim %d must be a multiple of %d and <= 256", D, vec);
  const long long blocks = BH * (Lq / be);
  if (blocks == 0) return VSA_OK;
  if (blocks > 0x7fffffffLL || BH > 65535) return fail(VSA_ERR_UNSUPPORTED, "combine backward (raster): too many blocks or slices");
  const RasterMap rm{map, (long long)raster_rows, heads};
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = VSA_TAG_TYPE(tag);
    if (gate_raster)
      combine_bwd_raster_kernel<T, true><<<(unsigned)blocks, 128, 0, st>>>((const T*)dout_raster, (const T*)gate_raster, (const T*)out_c,
                                                                          (T*)d_out_c, (T*)dgate_raster, (T*)dout_tiled, rm,
                                                                          (int)(Lq / be), D, be);
    else
      combine_bwd_raster_kernel<T, false><<<(unsigned)blocks, 128, 0, st>>>((const T*)dout_raster, nullptr, (const T*)out_c,
                                                                           (T*)d_out_c, nullptr, (T*)dout_tiled, rm,
                                                                           (int)(Lq / be), D, be);
    return check_launch("combine_bwd_raster_kernel");
  });
}

// =========================================================================================
// Row gather with zero fill: dst[b, r, :] = map[r] >= 0 ? src[b, map[r], :] : 0.
// One kernel serves both directions of the 3-D tiling front end (vsa/fastvideo_tiling.py:128-145 of
// the reference): raster -> zero-padded tile-contiguous layout, and back.  Pure HBM traffic:
// every byte is read once and written once.
// =========================================================================================
template <typename W>
__global__ void __launch_bounds__(256) gather_rows_kernel(const W* __restrict__ src, const int32_t* __restrict__ map,
                                                          W* __restrict__ dst, long long src_rows, long long dst_rows,
                                                          int words_per_row, long long total_rows) {
  // blockDim = (tx, ty): ty destination rows per block, tx threads walking the words of a row, so that the row
  // index is split once per row and thread and the inner loop has no division
  for (long long row_all = (long long)blockIdx.x * blockDim.y + threadIdx.y; row_all < total_rows;
       row_all += (long long)gridDim.x * blockDim.y) {
    const long long b = row_all / dst_rows;
    const long long r = row_all - b * dst_rows;
    const int m = map[r];
    W* d = dst + row_all * words_per_row;
    if (m >= 0) {
      const W* s = src + (b * src_rows + m) * words_per_row;
      for (int w = threadIdx.x; w < words_per_row; w += blockDim.x) d[w] = s[w];
    } else {
      for (int w = threadIdx.x; w < words_per_row; w += blockDim.x) d[w] = W{};
    }
  }
}

int gather_rows(const void* src, const int32_t* map, void* dst, int64_t batch, int64_t src_rows, int64_t dst_rows,
                int64_t row_bytes, cudaStream_t st) {
  if (batch == 0 || dst_rows == 0 || row_bytes == 0) return VSA_OK;
  const bool wide = row_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(dst) % 16 == 0;
  if (!wide && row_bytes % 2 != 0) return fail(VSA_ERR_UNSUPPORTED, "gather rows: row size %lld bytes is odd", (long long)row_bytes);
  const int unit = wide ? 16 : (row_bytes % 4 == 0 ? 4 : 2);
  const long long wpr = row_bytes / unit;
  if (wpr > 0x7fffffffLL) return fail(VSA_ERR_UNSUPPORTED, "gather rows: row too long");
  const long long rows = batch * dst_rows;
  unsigned tx = 1;
  while (tx < 256 && tx < wpr) tx <<= 1;
  const dim3 block(tx, 256 / tx);
  long long blocks = (rows + block.y - 1) / block.y;
  if (blocks > 148LL * 64) blocks = 148LL * 64;
  if (unit == 16)
    gather_rows_kernel<uint4><<<(unsigned)blocks, block, 0, st>>>((const uint4*)src, map, (uint4*)dst, src_rows, dst_rows, (int)wpr, rows);
  else if (unit == 4)
    gather_rows_kernel<uint32_t><<<(unsigned)blocks, block, 0, st>>>((const uint32_t*)src, map, (uint32_t*)dst, src_rows, dst_rows, (int)wpr, rows);
  else
    gather_rows_kernel<uint16_t><<<(unsigned)blocks, block, 0, st>>>((const uint16_t*)src, map, (uint16_t*)dst, src_rows, dst_rows, (int)wpr, rows);
  return check_launch("gather_rows_kernel");
}

// Row gather that also moves the head axis: raster-order activations [B][S][H][row] <-> tile-order operands
// [B][H][L][row].  TO_TILED: dst (b, h, l) = src (b, map[l], h), zero where map[l] < 0 (the padding rows of a
// clipped tile); otherwise dst (b, s, h) = src (b, h, map[s]).  One pass instead of a gather plus a transpose.
template <bool TO_TILED>
__global__ void __launch_bounds__(256) gather_rows_heads_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ map,
                                                                uint4* __restrict__ dst, int heads, long long src_rows,
                                                                long long dst_rows, int words_per_row, long long total_words) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total_words;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row_all = i / words_per_row;
    const int w = (int)(i - row_all * words_per_row);
    long long b, r;
    int h;
    if (TO_TILED) {                       // destination [B][H][dst_rows]
      const long long bh = row_all / dst_rows;
      r = row_all - bh * dst_rows;
      b = bh / heads;
      h = (int)(bh - b * heads);
    } else {                              // destination [B][dst_rows][H]
      const long long bs = row_all / heads;
      h = (int)(row_all - bs * heads);
      b = bs / dst_rows;
      r = bs - b * dst_rows;
    }
    const int m = map[r];
    uint4 val = make_uint4(0, 0, 0, 0);
    if (m >= 0)
      val = TO_TILED ? src[((b * src_rows + m) * heads + h) * words_per_row + w]
                     : src[((b * heads + h) * src_rows + m) * words_per_row + w];
    dst[i] = val;
  }
}

// The same move for rows of 2^k 16-byte words (k <= 8) and fewer than 2^31 rows per side, which is every case the
// attention path produces.  A block owns 256 >> k consecutive DESTINATION tokens of one batch entry and walks the
// heads in its inner loop, so that everything it touches within a few microseconds lies together in memory on both
// sides: whole [H x row] token records on the raster side, runs of consecutive tile-order rows per head on the other
// (a loop over independent rows leaves one side as scattered 256-byte pieces, which DRAM serves at half rate).
template <bool TO_TILED>
__global__ void __launch_bounds__(256) gather_rows_heads_pow2_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ map,
                                                                     uint4* __restrict__ dst, unsigned heads, unsigned src_rows,
                                                                     unsigned dst_rows, int log2_words, unsigned groups_per_batch,
                                                                     unsigned total_groups) {
  const unsigned rows_per_block = 256u >> log2_words;
  const unsigned w = threadIdx.x & ((1u << log2_words) - 1u);
  for (unsigned g = blockIdx.x; g < total_groups; g += gridDim.x) {
    const unsigned b = g / groups_per_batch;
    const unsigned r = (g - b * groups_per_batch) * rows_per_block + (threadIdx.x >> log2_words);
    if (r >= dst_rows) continue;
    const int m = map[r];
#pragma unroll 4
    for (unsigned h = 0; h < heads; ++h) {
      uint4 val = make_uint4(0, 0, 0, 0);
      if (m >= 0) {
        const unsigned long long srow = TO_TILED ? ((unsigned long long)b * src_rows + (unsigned)m) * heads + h
                                                 : ((unsigned long long)b * heads + h) * src_rows + (unsigned)m;
        val = src[(srow << log2_words) + w];
      }
      const unsigned long long drow = TO_TILED ? ((unsigned long long)b * heads + h) * dst_rows + r
                                               : ((unsigned long long)b * dst_rows + r) * heads + h;
      dst[(drow << log2_words) + w] = val;
    }
  }
}

int gather_rows_heads(const void* src, const int32_t* map, void* dst, int64_t batch, int heads, int64_t src_rows,
                      int64_t dst_rows, int64_t row_bytes, bool to_tiled, cudaStream_t st) {
  if (batch == 0 || heads == 0 || dst_rows == 0 || row_bytes == 0) return VSA_OK;
  if (row_bytes % 16 || reinterpret_cast<uintptr_t>(src) % 16 || reinterpret_cast<uintptr_t>(dst) % 16)
    return fail(VSA_ERR_UNSUPPORTED, "gather rows (heads): rows must be multiples of 16 bytes and 16-byte aligned");
  const long long wpr = row_bytes / 16;
  const long long rows = batch * heads * dst_rows;
  int log2_words = 0;
  while ((1LL << log2_words) < wpr) ++log2_words;
  if ((1LL << log2_words) == wpr && log2_words <= 8 && dst_rows < 0x7fffffffLL && src_rows < 0x7fffffffLL) {
    const long long rows_per_block = 256 >> log2_words;
    const long long groups_per_batch = (dst_rows + rows_per_block - 1) / rows_per_block;
    const long long groups = batch * groups_per_batch;
    if (groups < 0xffffffffLL) {
      const unsigned blocks = (unsigned)(groups < 148LL * 64 ? groups : 148LL * 64);
      if (to_tiled)
        gather_rows_heads_pow2_kernel<true><<<blocks, 256, 0, st>>>((const uint4*)src, map, (uint4*)dst, (unsigned)heads,
                                                                    (unsigned)src_rows, (unsigned)dst_rows, log2_words,
                                                                    (unsigned)groups_per_batch, (unsigned)groups);
      else
        gather_rows_heads_pow2_kernel<false><<<blocks, 256, 0, st>>>((const uint4*)src, map, (uint4*)dst, (unsigned)heads,
                                                                     (unsigned)src_rows, (unsigned)dst_rows, log2_words,
                                                                     (unsigned)groups_per_batch, (unsigned)groups);
      return check_launch("gather_rows_heads_pow2_kernel");
    }
  }
  const long long total = rows * wpr;
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 32) blocks = 148LL * 32;
  if (to_tiled)
    gather_rows_heads_kernel<true><<<(unsigned)blocks, 256, 0, st>>>((const uint4*)src, map, (uint4*)dst, heads, src_rows,
                                                                     dst_rows, (int)wpr, total);
  else
    gather_rows_heads_kernel<false><<<(unsigned)blocks, 256, 0, st>>>((const uint4*)src, map, (uint4*)dst, heads, src_rows,
                                                                      dst_rows, (int)wpr, total);
  return check_launch("gather_rows_heads_kernel");
}

// =========================================================================================
// Scalar fine attention (any block volume, any head dim <= 256, bf16 or fp32): one warp
// per query row (forward, dQ) or per key row (dK/dV).  Lane l holds dims l, l+32, ...
// =========================================================================================
constexpr int kMaxDimRegs = 8;    // head dim <= 256

template <typename T>
__device__ __forceinline__ void load_row(const T* p, int D, int lane, float (&r)[kMaxDimRegs]) {
#pragma unroll
  for (int i = 0; i < kMaxDimRegs; ++i) {
    const int d = lane + 32 * i;
    r[i] = d < D ? Elem<T>::ld(p + d) : 0.f;
  }
}
__device__ __forceinline__ float dot_regs(const float (&a)[kMaxDimRegs], const float (&b)[kMaxDimRegs]) {
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxDimRegs; ++i) s = fmaf(a[i], b[i], s);
  return s;
}

template <typename T>
__global__ void __launch_bounds__(256) sparse_fwd_scalar_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                                const T* __restrict__ v,
                                                                const int32_t* __restrict__ selected,
                                                                const int32_t* __restrict__ kv_sizes,
                                                                T* __restrict__ out, float* __restrict__ lse2,
                                                                long long Lq, long long Lkv, int D, int be, int topk,
                                                                float scale) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= Lq) return;
  const long long bh = blockIdx.y;
  const int Qb = (int)(Lq / be);
  const int qb = (int)(row / be);
  const float c = scale * kLog2e;
  float qr[kMaxDimRegs], acc[kMaxDimRegs] = {}, kr[kMaxDimRegs], vr[kMaxDimRegs];
  load_row(q + (bh * Lq + row) * D, D, lane, qr);
  float m = -INFINITY, l = 0.f;
  const int32_t* sel = selected + (bh * Qb + qb) * (long long)topk;
  for (int s = 0; s < topk; ++s) {
    const int kvb = sel[s];
    int size = (unsigned)kvb < (unsigned)(Lkv / be) ? kv_sizes[kvb] : 0;     // an id outside the table is an empty block
    size = size > be ? be : size;
    const T* kp = k + (bh * Lkv + (long long)kvb * be) * D;
    const T* vp = v + (bh * Lkv + (long long)kvb * be) * D;
    for (int j = 0; j < size; ++j) {
      load_row(kp + (long long)j * D, D, lane, kr);
      load_row(vp + (long long)j * D, D, lane, vr);
      const float sc = warp_sum(dot_regs(qr, kr)) * c;
      const float mn = fmaxf(m, sc);
      const float alpha = exp2f(m - mn);          // m == -inf on the first token gives 0
      const float p = exp2f(sc - mn);
      l = l * alpha + p;
#pragma unroll
      for (int i = 0; i < kMaxDimRegs; ++i) acc[i] = fmaf(p, vr[i], acc[i] * alpha);
      m = mn;
    }
  }
  const float inv = 1.f / l;
  T* op = out + (bh * Lq + row) * D;
#pragma unroll
  for (int i = 0; i < kMaxDimRegs; ++i) {
    const int d = lane + 32 * i;
    if (d < D) Elem<T>::st(op + d, acc[i] * inv);
  }
  if (lse2 && lane == 0) lse2[bh * Lq + row] = m + log2f(l);
}

template <typename T>
__global__ void __launch_bounds__(256) sparse_dq_scalar_kernel(const T* __restrict__ dout, const T* __restrict__ q,
                                                               const T* __restrict__ k, const T* __restrict__ v,
                                                               const T* __restrict__ out_s, const float* __restrict__ lse2,
                                                               const int32_t* __restrict__ selected,
                                                               const int32_t* __restrict__ kv_sizes,
                                                               float* __restrict__ delta, T* __restrict__ dq,
                                                               long long Lq, long long Lkv, int D, int be, int topk,
                                                               float scale) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= Lq) return;
  const long long bh = blockIdx.y;
  const int Qb = (int)(Lq / be);
  const int qb = (int)(row / be);
  const float c = scale * kLog2e;
  float qr[kMaxDimRegs], dor[kMaxDimRegs], acc[kMaxDimRegs] = {}, kr[kMaxDimRegs], vr[kMaxDimRegs];
  load_row(q + (bh * Lq + row) * D, D, lane, qr);
  load_row(dout + (bh * Lq + row) * D, D, lane, dor);
  load_row(out_s + (bh * Lq + row) * D, D, lane, kr);
  const float dl = warp_sum(dot_regs(kr, dor));
  if (lane == 0) delta[bh * Lq + row] = dl;
  const float lse = lse2[bh * Lq + row];
  const int32_t* sel = selected + (bh * Qb + qb) * (long long)topk;
  for (int s = 0; s < topk; ++s) {
    const int kvb = sel[s];
    int size = (unsigned)kvb < (unsigned)(Lkv / be) ? kv_sizes[kvb] : 0;     // an id outside the table is an empty block
    size = size > be ? be : size;
    const T* kp = k + (bh * Lkv + (long long)kvb * be) * D;
    const T* vp = v + (bh * Lkv + (long long)kvb * be) * D;
    for (int j = 0; j < size; ++j) {
      load_row(kp + (long long)j * D, D, lane, kr);
      load_row(vp + (long long)j * D, D, lane, vr);
      const float sc = warp_sum(dot_regs(qr, kr)) * c;
      const float dp = warp_sum(dot_regs(dor, vr));
      const float ds = exp2f(sc - lse) * (dp - dl) * scale;
#pragma unroll
      for (int i = 0; i < kMaxDimRegs; ++i) acc[i] = fmaf(ds, kr[i], acc[i]);
    }
  }
  T* op = dq + (bh * Lq + row) * D;
#pragma unroll
  for (int i = 0; i < kMaxDimRegs; ++i) {
    const int d = lane + 32 * i;
    if (d < D) Elem<T>::st(op + d, acc[i]);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) sparse_dkdv_scalar_kernel(
    const T* __restrict__ dout, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
    const float* __restrict__ lse2, const float* __restrict__ delta, const int32_t* __restrict__ counts,
    const int32_t* __restrict__ offsets, const int32_t* __restrict__ inverse, const int32_t* __restrict__ kv_sizes,
    T* __restrict__ dk, T* __restrict__ dv, long long Lq, long long Lkv, int D, int be, int topk, float scale) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= Lkv) return;
  const long long bh = blockIdx.y;
  const int Kb = (int)(Lkv / be), Qb = (int)(Lq / be);
  const int kvb = (int)(row / be);
  const int pos = (int)(row - (long long)kvb * be);
  const float c = scale * kLog2e;
  float kr[kMaxDimRegs], vr[kMaxDimRegs], dka[kMaxDimRegs] = {}, dva[kMaxDimRegs] = {}, qr[kMaxDimRegs], dor[kMaxDimRegs];
  if (pos < kv_sizes[kvb]) {
    load_row(k + (bh * Lkv + row) * D, D, lane, kr);
    load_row(v + (bh * Lkv + row) * D, D, lane, vr);
    const int cnt = counts[bh * Kb + kvb];
    const int32_t* inv = inverse + bh * (long long)Qb * topk + offsets[bh * Kb + kvb];
    for (int e = 0; e < cnt; ++e) {
      const long long r0 = (long long)inv[e] * be;
      for (int r = 0; r < be; ++r) {
        const long long qi = bh * Lq + r0 + r;
        load_row(q + qi * D, D, lane, qr);
        load_row(dout + qi * D, D, lane, dor);
        const float sc = warp_sum(dot_regs(qr, kr)) * c;
        const float dp = warp_sum(dot_regs(dor, vr));
        const float p = exp2f(sc - lse2[qi]);
        const float ds = p * (dp - delta[qi]);
#pragma unroll
        for (int i = 0; i < kMaxDimRegs; ++i) {
          dka[i] = fmaf(ds, qr[i], dka[i]);
          dva[i] = fmaf(p, dor[i], dva[i]);
        }
      }
    }
  }
  T* dkp = dk + (bh * Lkv + row) * D;
  T* dvp = dv + (bh * Lkv + row) * D;
#pragma unroll
  for (int i = 0; i < kMaxDimRegs; ++i) {
    const int d = lane + 32 * i;
    if (d < D) {
      Elem<T>::st(dkp + d, dka[i] * scale);
      Elem<T>::st(dvp + d, dva[i]);
    }
  }
}

static int check_scalar_shape(int64_t BH, int D, const char* what) {
  if (D > 32 * kMaxDimRegs) return fail(VSA_ERR_UNSUPPORTED, "%s: head dim %d exceeds 256", what, D);
  if (BH > 65535) return fail(VSA_ERR_UNSUPPORTED, "%s: batch*heads %lld exceeds 65535", what, (long long)BH);
  return VSA_OK;
}

int sparse_fwd_scalar(const void* q, const void* k, const void* v, const int32_t* selected, const int32_t* kv_sizes,
                      void* out, float* lse2, int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk,
                      float scale, int dtype, cudaStream_t st) {
  int rc = check_scalar_shape(BH, D, "sparse forward");
  if (rc) return rc;
  if (BH == 0 || Lq == 0) return VSA_OK;
  dim3 grid((unsigned)((Lq + 7) / 8), (unsigned)BH);
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = VSA_TAG_TYPE(tag);
    sparse_fwd_scalar_kernel<T><<<grid, 256, 0, st>>>((const T*)q, (const T*)k, (const T*)v, selected, kv_sizes, (T*)out,
                                                      lse2, Lq, Lkv, D, be, topk, scale);
    return check_launch("sparse_fwd_scalar_kernel");
  });
}

int sparse_dq_scalar(const void* dout, const void* q, const void* k, const void* v, const void* out_s,
                     const float* lse2, const int32_t* selected, const int32_t* kv_sizes, float* delta, void* dq,
                     int64_t BH, int64_t Lq, int64_t Lkv, int D, int be, int topk, float scale, int dtype,
                     cudaStream_t st) {
  int rc = check_scalar_shape(BH, D, "sparse dQ");
  if (rc) return rc;
  if (BH == 0 || Lq == 0) return VSA_OK;
  dim3 grid((unsigned)((Lq + 7) / 8), (unsigned)BH);
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = VSA_TAG_TYPE(tag);
    sparse_dq_scalar_kernel<T><<<grid, 256, 0, st>>>((const T*)dout, (const T*)q, (const T*)k, (const T*)v,
                                                     (const T*)out_s, lse2, selected, kv_sizes, delta, (T*)dq, Lq, Lkv,
                                                     D, be, topk, scale);
    return check_launch("sparse_dq_scalar_kernel");
  });
}

int sparse_dkdv_scalar(const void* dout, const void* q, const void* k, const void* v, const float* lse2,
                       const float* delta, const int32_t* counts, const int32_t* offsets, const int32_t* inverse,
                       const int32_t* kv_sizes, void* dk, void* dv, int64_t BH, int64_t Lq, int64_t Lkv, int D, int be,
                       int topk, float scale, int dtype, cudaStream_t st) {
  int rc = check_scalar_shape(BH, D, "sparse dK/dV");
  if (rc) return rc;
  if (BH == 0 || Lkv == 0) return VSA_OK;
  dim3 grid((unsigned)((Lkv + 7) / 8), (unsigned)BH);
  return dispatch_dtype(dtype, [&](auto* tag) {
    using T = VSA_TAG_TYPE(tag);
    sparse_dkdv_scalar_kernel<T><<<grid, 256, 0, st>>>((const T*)dout, (const T*)q, (const T*)k, (const T*)v, lse2, delta,
                                                       counts, offsets, inverse, kv_sizes, (T*)dk, (T*)dv, Lq, Lkv, D, be,
                                                       topk, scale);
    return check_launch("sparse_dkdv_scalar_kernel");
  });
}

}  // namespace vsa
