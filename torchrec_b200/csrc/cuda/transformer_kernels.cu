// Memory-bound pieces of a transformer block over packed (unpadded) tokens, each fused into one pass over the activations:
//
//   ln_residual_fwd   s = r + dropout(a)         (the residual stream; `a` may be absent: s = r)
//                     y = LayerNorm(s) * gamma + beta
//   ln_residual_bwd   from dy (and the gradient that reaches s from later blocks) -> ds, da, dgamma, dbeta
//   gelu_dropout_fwd  h = dropout(gelu(z));   gelu_dropout_bwd   dz = dh * mask * gelu'(z)
//
// Dropout masks are never stored: an element is kept iff its 16 bits of hash(seed, position) fall below the keep threshold
// (the keep probability is rounded to a multiple of 2^-16 and the rescale factor matches the rounded value), and the backward
// recomputes the same hash.  One warp owns one token row (D <= 1024, D % 256 == 0: every lane moves 16 bytes at a
// time); statistics are fp32.  The reference model runs these as separate library kernels on padded [B, L, D] tensors
// (examples/bert4rec/models/bert4rec.py of the reference: nn.LayerNorm, nn.Dropout, GELU between nn.Linear layers).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_bf16.h>
#include <torch/library.h>

#include "common.cuh"

namespace trb {

// splitmix64 finaliser over (seed, index)
// 64 hash bits -> four 16-bit lanes
__device__ __forceinline__ uint64_t drop_hash64(uint64_t seed, uint64_t i) {
  uint64_t z = seed + (i + 1) * 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

struct Drop {
  uint64_t seed;
  uint32_t keep_below;  // an element is kept iff its 16 random bits are below this (p == 0: everything is kept, nothing is hashed)
  float scale;          // 1 / (realised keep probability): keep_below is a multiple of 2^-16, the scale matches it exactly
  int on;
  // the eight factors of elements [i8 * 8, i8 * 8 + 8): two hashes, sixteen bits per element
  __device__ __forceinline__ void factors8(uint64_t i8, float (&f)[8]) const {
    if (!on) {
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] = 1.f;
      return;
    }
    const uint64_t h0 = drop_hash64(seed, i8 * 2), h1 = drop_hash64(seed, i8 * 2 + 1);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      f[k] = uint32_t((h0 >> (16 * k)) & 0xffff) < keep_below ? scale : 0.f;
      f[4 + k] = uint32_t((h1 >> (16 * k)) & 0xffff) < keep_below ? scale : 0.f;
    }
  }
};

static Drop make_drop(double p, int64_t seed) {
  Drop d;
  d.on = p > 0.0 ? 1 : 0;
  d.seed = uint64_t(seed);
  const double keep = std::min(65536.0, std::max(1.0, std::floor((1.0 - p) * 65536.0 + 0.5)));
  d.keep_below = uint32_t(keep);
  d.scale = d.on ? float(65536.0 / keep) : 1.f;
  return d;
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 f = __bfloat1622float2(h[k]);
    v[2 * k] = f.x;
    v[2 * k + 1] = f.y;
  }
}

__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// kChunks = D / 256: every lane holds kChunks groups of 8 consecutive elements (group c starts at c * 256 + lane * 8)
template <int kChunks>
__global__ void __launch_bounds__(256) ln_residual_fwd_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ r,
                                                              const float* __restrict__ gamma, const float* __restrict__ beta,
                                                              __nv_bfloat16* __restrict__ s_out, __nv_bfloat16* __restrict__ y,
                                                              float* __restrict__ mean_out, float* __restrict__ rstd_out, int64_t T,
                                                              float eps, Drop drop) {
  constexpr int D = kChunks * 256;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (row >= T) return;
  float s[kChunks][8];
  float sum = 0.f;
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int e = c * 256 + lane * 8;
    load8(r + row * D + e, s[c]);
    if (a != nullptr) {
      float av[8], fk[8];
      load8(a + row * D + e, av);
      drop.factors8((uint64_t(row) * D + e) >> 3, fk);
#pragma unroll
      for (int k = 0; k < 8; ++k) s[c][k] += av[k] * fk[k];
      // the residual stream is stored in bf16: normalise what the next block will read, not the unrounded sum
#pragma unroll
      for (int k = 0; k < 8; ++k) s[c][k] = __bfloat162float(__float2bfloat16(s[c][k]));
      store8(s_out + row * D + e, s[c]);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) sum += s[c][k];
  }
  const float mean = warp_sum(sum) * (1.f / D);
  float var = 0.f;
#pragma unroll
  for (int c = 0; c < kChunks; ++c)
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float d = s[c][k] - mean;
      var += d * d;
    }
  const float rstd = rsqrtf(warp_sum(var) * (1.f / D) + eps);
  if (lane == 0) {
    mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int e = c * 256 + lane * 8;
    float out[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) out[k] = (s[c][k] - mean) * rstd * gamma[e + k] + beta[e + k];
    store8(y + row * D + e, out);
  }
}

// ds = LN backward of dy (+ ds_extra); da = ds * mask * scale; dgamma / dbeta: per-block partial sums, then atomics.
template <int kChunks>
__global__ void __launch_bounds__(256) ln_residual_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ ds_extra,
                                                              const __nv_bfloat16* __restrict__ s, const float* __restrict__ gamma,
                                                              const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                                                              __nv_bfloat16* __restrict__ ds_out, __nv_bfloat16* __restrict__ da_out,
                                                              float* __restrict__ dgamma, float* __restrict__ dbeta, int64_t T, Drop drop,
                                                              int rows_per_warp) {
  constexpr int D = kChunks * 256;
  __shared__ float sh[8][D];  // 32 KB at D = 1024: used for dgamma first, then for dbeta
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  float g_acc[kChunks][8], b_acc[kChunks][8], gm[kChunks][8];
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int e = c * 256 + lane * 8;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      g_acc[c][k] = 0.f;
      b_acc[c][k] = 0.f;
      gm[c][k] = gamma[e + k];
    }
  }
  for (int i = 0; i < rows_per_warp; ++i) {
    const int64_t row = warp * rows_per_warp + i;
    if (row >= T) break;
    const float mean = mean_in[row], rstd = rstd_in[row];
    float xh[kChunks][8], dxh[kChunks][8];
    float m1 = 0.f, m2 = 0.f;
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
      const int e = c * 256 + lane * 8;
      float dyv[8], sv[8];
      load8(dy + row * D + e, dyv);
      load8(s + row * D + e, sv);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        xh[c][k] = (sv[k] - mean) * rstd;
        dxh[c][k] = dyv[k] * gm[c][k];
        m1 += dxh[c][k];
        m2 += dxh[c][k] * xh[c][k];
        g_acc[c][k] += dyv[k] * xh[c][k];
        b_acc[c][k] += dyv[k];
      }
    }
    m1 = warp_sum(m1) * (1.f / D);
    m2 = warp_sum(m2) * (1.f / D);
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
      const int e = c * 256 + lane * 8;
      float dsv[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) dsv[k] = rstd * (dxh[c][k] - m1 - xh[c][k] * m2);
      if (ds_extra != nullptr) {
        float ex[8];
        load8(ds_extra + row * D + e, ex);
#pragma unroll
        for (int k = 0; k < 8; ++k) dsv[k] += ex[k];
      }
      store8(ds_out + row * D + e, dsv);
      if (da_out != nullptr) {
        float dav[8], fk[8];
        drop.factors8((uint64_t(row) * D + e) >> 3, fk);
#pragma unroll
        for (int k = 0; k < 8; ++k) dav[k] = dsv[k] * fk[k];
        store8(da_out + row * D + e, dav);
      }
    }
  }
  // block reduction of the parameter gradients, one atomic per element and block
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
      const int e = c * 256 + lane * 8;
#pragma unroll
      for (int k = 0; k < 8; ++k) sh[wib][e + k] = pass == 0 ? g_acc[c][k] : b_acc[c][k];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < D; e += blockDim.x) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) t += sh[w][e];
      atomicAdd((pass == 0 ? dgamma : dbeta) + e, t);
    }
    __syncthreads();
  }
}

// Phi(x) = 0.5 (1 + erf(x / sqrt 2)) and e = exp(-x^2 / 2) from one exponential: erfc by the rational approximation 7.1.26 of
// Abramowitz & Stegun (absolute error below 1.5e-7, far under the bf16 output's resolution); about a third of the
// instructions of the library's erff, which made these kernels instruction-bound.
__device__ __forceinline__ void gelu_parts(float x, float& cdf, float& e) {
  const float ax = fabsf(x) * 0.70710678118654752f;
  const float t = __frcp_rn(fmaf(0.3275911f, ax, 1.f));
  e = exp2f(-0.72134752044448170f * x * x);
  const float poly = fmaf(fmaf(fmaf(fmaf(1.061405429f, t, -1.453152027f), t, 1.421413741f), t, -0.284496736f), t, 0.254829592f) * t;
  const float half_erfc = 0.5f * poly * e;
  cdf = x >= 0.f ? 1.f - half_erfc : half_erfc;
}
__device__ __forceinline__ float gelu_f(float x) {
  float cdf, e;
  gelu_parts(x, cdf, e);
  return x * cdf;
}
__device__ __forceinline__ float gelu_grad_f(float x) {
  float cdf, e;
  gelu_parts(x, cdf, e);
  return fmaf(x * 0.3989422804014327f, e, cdf);
}

template <bool kBackward>
__global__ void __launch_bounds__(256) gelu_dropout_kernel(const __nv_bfloat16* __restrict__ z, const __nv_bfloat16* __restrict__ dh,
                                                           __nv_bfloat16* __restrict__ out, int64_t n8, Drop drop) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  float zv[8], o[8], fk[8];
  load8(z + i * 8, zv);
  drop.factors8(uint64_t(i), fk);
  if (kBackward) {
    float g[8];
    load8(dh + i * 8, g);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = g[k] * fk[k] * gelu_grad_f(zv[k]);
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = gelu_f(zv[k]) * fk[k];
  }
  store8(out + i * 8, o);
}

// ---- host side -----------------------------------------------------------------------------------------------------
static void check_rows(const at::Tensor& t, int64_t T, int64_t D, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous() && t.dim() == 2 && t.size(0) == T && t.size(1) == D, name,
              ": contiguous bf16 [tokens, D] expected");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 == 0, name, ": 16-byte aligned storage expected");
}

#define TRB_DISPATCH_CHUNKS(D, ...)                                   \
  [&] {                                                               \
    const int chunks_ = int((D) / 256);                               \
    if (chunks_ == 1) { constexpr int kChunks = 1; __VA_ARGS__(); }   \
    else if (chunks_ == 2) { constexpr int kChunks = 2; __VA_ARGS__(); } \
    else if (chunks_ == 3) { constexpr int kChunks = 3; __VA_ARGS__(); } \
    else { constexpr int kChunks = 4; __VA_ARGS__(); }                \
  }()

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> ln_residual_fwd(const c10::optional<at::Tensor>& a, const at::Tensor& r,
                                                                         const at::Tensor& gamma, const at::Tensor& beta, double p,
                                                                         int64_t seed, double eps) {
  const int64_t T = r.size(0), D = r.size(1);
  TORCH_CHECK(D % 256 == 0 && D <= 1024, "D must be 256, 512, 768 or 1024");
  check_rows(r, T, D, "r");
  const bool has_a = a.has_value() && a->defined();
  if (has_a) check_rows(*a, T, D, "a");
  TORCH_CHECK(gamma.is_cuda() && gamma.scalar_type() == at::kFloat && gamma.numel() == D && beta.scalar_type() == at::kFloat && beta.numel() == D);
  c10::cuda::CUDAGuard guard(r.device());
  at::Tensor s = has_a ? at::empty_like(r) : at::empty({0}, r.options());  // without `a` the stream is `r` itself: nothing to write
  at::Tensor y = at::empty_like(r);
  at::Tensor mean = at::empty({T}, r.options().dtype(at::kFloat)), rstd = at::empty({T}, r.options().dtype(at::kFloat));
  if (T == 0) return {s, y, mean, rstd};
  const Drop drop = make_drop(has_a ? p : 0.0, seed);
  const int64_t blocks = (T * 32 + 255) / 256;
  auto stream = at::cuda::getCurrentCUDAStream();
  TRB_DISPATCH_CHUNKS(D, [&] {
    ln_residual_fwd_kernel<kChunks><<<blocks, 256, 0, stream>>>(
        has_a ? reinterpret_cast<const __nv_bfloat16*>(a->data_ptr()) : nullptr, reinterpret_cast<const __nv_bfloat16*>(r.data_ptr()),
        gamma.data_ptr<float>(), beta.data_ptr<float>(), has_a ? reinterpret_cast<__nv_bfloat16*>(s.data_ptr()) : nullptr,
        reinterpret_cast<__nv_bfloat16*>(y.data_ptr()), mean.data_ptr<float>(), rstd.data_ptr<float>(), T, float(eps), drop);
  });
  TRB_CUDA_CHECK(cudaGetLastError());
  return {s, y, mean, rstd};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> ln_residual_bwd(const c10::optional<at::Tensor>& ds_extra, const at::Tensor& dy,
                                                                         const at::Tensor& s, const at::Tensor& gamma,
                                                                         const at::Tensor& mean, const at::Tensor& rstd, double p,
                                                                         int64_t seed, bool has_a) {
  const int64_t T = s.size(0), D = s.size(1);
  TORCH_CHECK(D % 256 == 0 && D <= 1024, "D must be 256, 512, 768 or 1024");
  check_rows(s, T, D, "s");
  check_rows(dy, T, D, "dy");
  const bool extra = ds_extra.has_value() && ds_extra->defined();
  if (extra) check_rows(*ds_extra, T, D, "ds_extra");
  TORCH_CHECK(mean.scalar_type() == at::kFloat && mean.numel() == T && rstd.scalar_type() == at::kFloat && rstd.numel() == T);
  c10::cuda::CUDAGuard guard(s.device());
  at::Tensor ds = at::empty_like(s);
  at::Tensor da = has_a ? at::empty_like(s) : at::empty({0}, s.options());
  at::Tensor dgamma = at::zeros({D}, s.options().dtype(at::kFloat)), dbeta = at::zeros({D}, s.options().dtype(at::kFloat));
  if (T == 0) return {ds, da, dgamma, dbeta};
  const Drop drop = make_drop(has_a ? p : 0.0, seed);
  // about four waves of blocks: few enough atomics on dgamma / dbeta, enough warps to hide latency
  const int64_t target_warps = 148 * 8 * 8 * 4;
  const int rows_per_warp = int(std::max<int64_t>(1, (T + target_warps - 1) / target_warps));
  const int64_t warps = (T + rows_per_warp - 1) / rows_per_warp;
  const int64_t blocks = (warps * 32 + 255) / 256;
  auto stream = at::cuda::getCurrentCUDAStream();
  TRB_DISPATCH_CHUNKS(D, [&] {
    ln_residual_bwd_kernel<kChunks><<<blocks, 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(dy.data_ptr()), extra ? reinterpret_cast<const __nv_bfloat16*>(ds_extra->data_ptr()) : nullptr,
        reinterpret_cast<const __nv_bfloat16*>(s.data_ptr()), gamma.data_ptr<float>(), mean.data_ptr<float>(), rstd.data_ptr<float>(),
        reinterpret_cast<__nv_bfloat16*>(ds.data_ptr()), has_a ? reinterpret_cast<__nv_bfloat16*>(da.data_ptr()) : nullptr,
        dgamma.data_ptr<float>(), dbeta.data_ptr<float>(), T, drop, rows_per_warp);
  });
  TRB_CUDA_CHECK(cudaGetLastError());
  return {ds, da, dgamma, dbeta};
}

static at::Tensor gelu_dropout_impl(const at::Tensor& z, const c10::optional<at::Tensor>& dh, double p, int64_t seed) {
  TORCH_CHECK(z.is_cuda() && z.scalar_type() == at::kBFloat16 && z.is_contiguous() && z.numel() % 8 == 0, "contiguous bf16 tensor with a multiple of 8 elements expected");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(z.data_ptr()) % 16 == 0);
  c10::cuda::CUDAGuard guard(z.device());
  at::Tensor out = at::empty_like(z);
  const int64_t n8 = z.numel() / 8;
  if (n8 == 0) return out;
  const Drop drop = make_drop(p, seed);
  const int64_t blocks = (n8 + 255) / 256;
  auto stream = at::cuda::getCurrentCUDAStream();
  if (dh.has_value() && dh->defined()) {
    TORCH_CHECK(dh->is_cuda() && dh->scalar_type() == at::kBFloat16 && dh->is_contiguous() && dh->numel() == z.numel());
    gelu_dropout_kernel<true><<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(z.data_ptr()),
                                                          reinterpret_cast<const __nv_bfloat16*>(dh->data_ptr()),
                                                          reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), n8, drop);
  } else {
    gelu_dropout_kernel<false><<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(z.data_ptr()), nullptr,
                                                           reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), n8, drop);
  }
  TRB_CUDA_CHECK(cudaGetLastError());
  return out;
}

at::Tensor gelu_dropout_fwd(const at::Tensor& z, double p, int64_t seed) { return gelu_dropout_impl(z, c10::nullopt, p, seed); }
at::Tensor gelu_dropout_bwd(const at::Tensor& dh, const at::Tensor& z, double p, int64_t seed) { return gelu_dropout_impl(z, dh, p, seed); }

}  // namespace trb

TORCH_LIBRARY_FRAGMENT(trb200, m) {
  m.def("ln_residual_fwd(Tensor? a, Tensor r, Tensor gamma, Tensor beta, float p, int seed, float eps) -> (Tensor, Tensor, Tensor, Tensor)");
  m.def("ln_residual_bwd(Tensor? ds_extra, Tensor dy, Tensor s, Tensor gamma, Tensor mean, Tensor rstd, float p, int seed, bool has_a) -> (Tensor, Tensor, Tensor, Tensor)");
  m.def("gelu_dropout_fwd(Tensor z, float p, int seed) -> Tensor");
  m.def("gelu_dropout_bwd(Tensor dh, Tensor z, float p, int seed) -> Tensor");
}

TORCH_LIBRARY_IMPL(trb200, CUDA, m) {
  m.impl("ln_residual_fwd", &trb::ln_residual_fwd);
  m.impl("ln_residual_bwd", &trb::ln_residual_bwd);
  m.impl("gelu_dropout_fwd", &trb::gelu_dropout_fwd);
  m.impl("gelu_dropout_bwd", &trb::gelu_dropout_bwd);
}
