// Shared helpers of the VSA kernels: status handling, element traits,
// warp-level primitives and the sm_100a PTX wrappers the tensor-core kernels use.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/vsa_b200.h"

namespace vsa {

constexpr float kLog2e = 1.4426950408889634f;

// ---- error reporting ------------------------------------------------------------------
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);
int check_launch(const char* what);

#define VSA_REQUIRE(cond, ...)                                      \
  do {                                                              \
    if (!(cond)) return ::vsa::fail(VSA_ERR_BAD_ARGUMENT, __VA_ARGS__); \
  } while (0)

// ---- element traits ---------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
  __device__ __forceinline__ static float ld(const float* p) { return *p; }
  __device__ __forceinline__ static void st(float* p, float x) { *p = x; }
  __device__ __forceinline__ static float round(float x) { return x; }
};
template <> struct Elem<__nv_bfloat16> {
  __device__ __forceinline__ static float ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  __device__ __forceinline__ static void st(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }
  __device__ __forceinline__ static float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
  __device__ __forceinline__ static float to(__nv_bfloat16 x) { return __bfloat162float(x); }
  __device__ __forceinline__ static __nv_bfloat16 from(float x) { return __float2bfloat16_rn(x); }
  __device__ __forceinline__ static uint32_t pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};

template <> struct Elem<__half> {
  __device__ __forceinline__ static float ld(const __half* p) { return __half2float(*p); }
  __device__ __forceinline__ static void st(__half* p, float x) { *p = __float2half_rn(x); }
  __device__ __forceinline__ static float round(float x) { return __half2float(__float2half_rn(x)); }
  __device__ __forceinline__ static float to(__half x) { return __half2float(x); }
  __device__ __forceinline__ static __half from(float x) { return __float2half_rn(x); }
  __device__ __forceinline__ static uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};

// ---- warp helpers -----------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}
__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) { return Elem<__nv_bfloat16>::pack(lo, hi); }

// Row of token `token` of slice `bh` in a K/V-shaped tensor.  Ordinary tensors are [BH][Lkv][D] (shard == Lkv).  A
// sequence-parallel all-gather leaves the shards of the W ranks one after another, [W][BH][Lkv/W][D]; with
// shard = Lkv/W the same formula addresses that buffer in place, so nothing has to be re-laid-out after the gather
// (and partial dK/dV written the same way are ready for the reduce-scatter).  A 64-token tile never straddles two
// shards because the shard length is a multiple of the block volume.
__device__ __forceinline__ long long kv_tensor_row(long long bh, long long BH, long long token, long long shard) {
  const long long r = token / shard;
  return (r * BH + bh) * shard + (token - r * shard);
}

// Optional re-layout of per-token rows on the way in or out of a kernel.  The attention kernels work on tile-order
// tensors [BH][L][D] (L = blocks x block volume, padding rows included); a model keeps its activations in raster
// order [B][S][H][D].  With a map, tile-order token t of slice (b, h) lives at raster row (b*S + map[t])*H + h;
// map[t] < 0 marks a padding row, which has no raster counterpart.  map == nullptr: no re-layout.
struct RasterMap {
  const int32_t* map;
  long long rows;   // S
  int heads;        // H
};
__device__ __forceinline__ long long raster_row(const RasterMap& rm, long long bh, long long token) {
  const int s = rm.map[token];
  if (s < 0) return -1;
  const int b = (int)bh / rm.heads;          // bh < 65536: a 32-bit division
  return ((long long)b * rm.rows + s) * rm.heads + ((int)bh - b * rm.heads);
}

// Gated combine of eight 16-bit values: out = out_s + out_c * gate (gate optional) in fp32, one rounding -- the
// arithmetic of the stand-alone combine pass, so fusing it into a kernel's store changes no bit.
template <typename T>
__device__ __forceinline__ uint4 combine_x8(const uint4& s_raw, const uint4& c_raw, const uint4& g_raw, bool has_gate) {
  uint4 o_raw;
  const T* se = reinterpret_cast<const T*>(&s_raw);
  const T* ce = reinterpret_cast<const T*>(&c_raw);
  const T* ge = reinterpret_cast<const T*>(&g_raw);
  T* oe = reinterpret_cast<T*>(&o_raw);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float cv = Elem<T>::to(ce[i]);
    if (has_gate) cv *= Elem<T>::to(ge[i]);
    oe[i] = Elem<T>::from(Elem<T>::to(se[i]) + cv);
  }
  return o_raw;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- cp.async / ldmatrix / mma.sync (legacy tensor path used by the first-generation kernels)
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// the same product with fp16 operands
__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T> __device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  mma_bf16(d, a, b0, b1);
}
template <> __device__ __forceinline__ void mma_16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  mma_f16(d, a, b0, b1);
}

}  // namespace vsa
