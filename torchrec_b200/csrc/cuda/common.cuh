// Shared device helpers for the sm_100a kernels of torchrec_b200.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace trb {

constexpr int kMaxPeers = 16;

// Pointers of one symmetric buffer on every rank, passed by value to a kernel.
struct PeerPtrs {
  void* p[kMaxPeers];
};

enum OutDtype : int { OUT_F32 = 0, OUT_F16 = 1, OUT_BF16 = 2 };

__device__ __forceinline__ float4 f4zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }

// ---- 4-element vector load/store with conversion to fp32 -------------------------------
template <typename T>
struct Vec4;

template <>
struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
  static __device__ __forceinline__ float4 load_plain(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};

template <>
struct Vec4<__half> {
  static __device__ __forceinline__ float4 cvt(uint2 raw) {
    __half2 a = *reinterpret_cast<__half2*>(&raw.x);
    __half2 b = *reinterpret_cast<__half2*>(&raw.y);
    float2 fa = __half22float2(a), fb = __half22float2(b);
    return make_float4(fa.x, fa.y, fb.x, fb.y);
  }
  static __device__ __forceinline__ float4 load(const __half* p) { return cvt(__ldg(reinterpret_cast<const uint2*>(p))); }
  static __device__ __forceinline__ float4 load_plain(const __half* p) { return cvt(*reinterpret_cast<const uint2*>(p)); }
  static __device__ __forceinline__ void store(__half* p, float4 v) {
    __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&a);
    raw.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
  }
};

template <>
struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 cvt(uint2 raw) {
    // bf16 -> fp32 is a 16-bit shift
    return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                       __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
  }
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) { return cvt(__ldg(reinterpret_cast<const uint2*>(p))); }
  static __device__ __forceinline__ float4 load_plain(const __nv_bfloat16* p) { return cvt(*reinterpret_cast<const uint2*>(p)); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&a);
    raw.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
  }
};

// store 4 fp32 values at element offset `e` of a row whose dtype is chosen at run time
__device__ __forceinline__ void store4_dyn(void* base, int64_t e, float4 v, int dtype) {
  if (dtype == OUT_F32) {
    Vec4<float>::store(reinterpret_cast<float*>(base) + e, v);
  } else if (dtype == OUT_F16) {
    Vec4<__half>::store(reinterpret_cast<__half*>(base) + e, v);
  } else {
    Vec4<__nv_bfloat16>::store(reinterpret_cast<__nv_bfloat16*>(base) + e, v);
  }
}

__device__ __forceinline__ float4 load4_dyn(const void* base, int64_t e, int dtype) {
  if (dtype == OUT_F32) return Vec4<float>::load_plain(reinterpret_cast<const float*>(base) + e);
  if (dtype == OUT_F16) return Vec4<__half>::load_plain(reinterpret_cast<const __half*>(base) + e);
  return Vec4<__nv_bfloat16>::load_plain(reinterpret_cast<const __nv_bfloat16*>(base) + e);
}

// vectorised fp32 reduction into (possibly peer) global memory: one 16-byte red per lane
__device__ __forceinline__ void red_add_f32x4(float* addr, float4 v) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace trb

#define TRB_CUDA_CHECK(expr)                                                                  \
  do {                                                                                        \
    cudaError_t _e = (expr);                                                                  \
    TORCH_CHECK(_e == cudaSuccess, "CUDA error ", cudaGetErrorString(_e), " at ", __FILE__, ":", __LINE__); \
  } while (0)
