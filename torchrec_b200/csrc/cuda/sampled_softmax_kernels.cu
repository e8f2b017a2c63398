// Cross entropy of a sampled softmax whose class 0 is the positive: per row p, over the scores [pos[p], neg[p, 0..N)],
//   loss[p] = logsumexp - pos[p],   and in the same pass the gradient:  neg[p, :] <- softmax * gscale (in place, bf16),
//   dpos[p] = (softmax_0 - 1) * gscale.
// One block per row; a row of up to 8192 bf16 scores stays in registers between the three sweeps (max, sum, write), longer rows
// are re-read.  The library route casts the [P, 1 + N] scores to fp32, runs log-softmax forward and backward and casts back:
// about five passes over a tensor that is read once and written once here.  (The reference model ends in a dense projection
// over the whole vocabulary and nn.CrossEntropyLoss, examples/bert4rec/bert4rec_main.py of the reference.)
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_bf16.h>
#include <torch/library.h>

#include "common.cuh"

namespace trb {

constexpr int kCeThreads = 256;
constexpr int kCeCache = 4;  // 16-byte vectors per thread kept in registers: 256 * 4 * 8 = 8192 scores

__device__ __forceinline__ float ce_block_reduce(float v, bool is_max, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, other) : v + other;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();  // red may still be read from the previous reduction
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int w = 1; w < kCeThreads / 32; ++w) r = is_max ? fmaxf(r, red[w]) : r + red[w];
  return r;
}

__global__ void __launch_bounds__(kCeThreads) sampled_ce_kernel(const float* __restrict__ pos, __nv_bfloat16* __restrict__ neg, float* __restrict__ loss,
                                                                float* __restrict__ dpos, int64_t ld, int N, float gscale) {
  __shared__ float red[kCeThreads / 32];
  const int64_t p = blockIdx.x;
  __nv_bfloat16* row = neg + p * ld;
  const int nvec = N / 8;  // N % 8 == 0
  uint4 cache[kCeCache];
  const float pv = pos[p];
  float m = pv;
#pragma unroll
  for (int c = 0; c < kCeCache; ++c) {
    const int v = threadIdx.x + c * kCeThreads;
    cache[c] = v < nvec ? *reinterpret_cast<const uint4*>(row + v * 8) : make_uint4(0xff80ff80u, 0xff80ff80u, 0xff80ff80u, 0xff80ff80u);  // -inf
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&cache[c]);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      m = fmaxf(m, fmaxf(f.x, f.y));
    }
  }
  for (int v = threadIdx.x + kCeCache * kCeThreads; v < nvec; v += kCeThreads) {
    const uint4 raw = *reinterpret_cast<const uint4*>(row + v * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      m = fmaxf(m, fmaxf(f.x, f.y));
    }
  }
  m = ce_block_reduce(m, true, red);
  constexpr float kLog2e = 1.4426950408889634f;
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < kCeCache; ++c) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&cache[c]);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      s += exp2f((f.x - m) * kLog2e) + exp2f((f.y - m) * kLog2e);
    }
  }
  for (int v = threadIdx.x + kCeCache * kCeThreads; v < nvec; v += kCeThreads) {
    const uint4 raw = *reinterpret_cast<const uint4*>(row + v * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      s += exp2f((f.x - m) * kLog2e) + exp2f((f.y - m) * kLog2e);
    }
  }
  s = ce_block_reduce(s, false, red) + exp2f((pv - m) * kLog2e);
  const float inv = gscale / s;
  if (threadIdx.x == 0) {
    loss[p] = m + logf(s) - pv;
    dpos[p] = exp2f((pv - m) * kLog2e) * inv - gscale;
  }
#pragma unroll
  for (int c = 0; c < kCeCache; ++c) {
    const int v = threadIdx.x + c * kCeThreads;
    if (v >= nvec) continue;
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&cache[c]);
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      oh[k] = __floats2bfloat162_rn(exp2f((f.x - m) * kLog2e) * inv, exp2f((f.y - m) * kLog2e) * inv);
    }
    *reinterpret_cast<uint4*>(row + v * 8) = o;
  }
  for (int v = threadIdx.x + kCeCache * kCeThreads; v < nvec; v += kCeThreads) {
    const uint4 raw = *reinterpret_cast<const uint4*>(row + v * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      oh[k] = __floats2bfloat162_rn(exp2f((f.x - m) * kLog2e) * inv, exp2f((f.y - m) * kLog2e) * inv);
    }
    *reinterpret_cast<uint4*>(row + v * 8) = o;
  }
}

// neg [P_rows >= P, N] bf16 is overwritten with the gradient of its first P rows; returns (loss [P], dpos [P])
std::tuple<at::Tensor, at::Tensor> sampled_ce_fwd_bwd(const at::Tensor& pos, at::Tensor neg, double gscale) {
  TORCH_CHECK(pos.is_cuda() && pos.scalar_type() == at::kFloat && pos.dim() == 1 && pos.is_contiguous());
  TORCH_CHECK(neg.is_cuda() && neg.scalar_type() == at::kBFloat16 && neg.dim() == 2 && neg.stride(1) == 1 && neg.size(0) >= pos.size(0));
  const int64_t P = pos.size(0);
  const int N = int(neg.size(1));
  TORCH_CHECK(N >= 8 && N % 8 == 0 && neg.stride(0) % 8 == 0 && reinterpret_cast<uintptr_t>(neg.data_ptr()) % 16 == 0,
              "sampled_ce: the number of negatives and the row pitch must be multiples of 8");
  c10::cuda::CUDAGuard guard(pos.device());
  at::Tensor loss = at::empty({P}, pos.options()), dpos = at::empty({P}, pos.options());
  if (P == 0) return {loss, dpos};
  sampled_ce_kernel<<<unsigned(P), kCeThreads, 0, at::cuda::getCurrentCUDAStream()>>>(pos.data_ptr<float>(), reinterpret_cast<__nv_bfloat16*>(neg.data_ptr()),
                                                                                     loss.data_ptr<float>(), dpos.data_ptr<float>(), neg.stride(0), N, float(gscale));
  TRB_CUDA_CHECK(cudaGetLastError());
  return {loss, dpos};
}

}  // namespace trb

TORCH_LIBRARY_FRAGMENT(trb200, m) { m.def("sampled_ce_fwd_bwd(Tensor pos, Tensor(a!) neg, float gscale) -> (Tensor, Tensor)"); }

TORCH_LIBRARY_IMPL(trb200, CUDA, m) { m.impl("sampled_ce_fwd_bwd", &trb::sampled_ce_fwd_bwd); }
