// Elementwise / reduction kernels around the tensor-core GEMMs of the dense towers, and the DLRM dot
// interaction.  All are HBM-bound: each makes one pass over its operands with 16-byte accesses.
//
// Counterparts in the reference are plain torch ops (torchrec/modules/crossnet.py:178-181,
// torchrec/models/dlrm.py:216-219).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "common.cuh"
#include "dot_mma.cuh"

namespace trb {

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

// ---- dz = dy * act'(y) -------------------------------------------------------------------------
__global__ void __launch_bounds__(256) act_backward_kernel(const bf16x8* __restrict__ dy, const bf16x8* __restrict__ y,
                                                           bf16x8* __restrict__ dz, int64_t n8, int act) {
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += int64_t(gridDim.x) * blockDim.x) {
    bf16x8 a = dy[i], b = y[i], o;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 fa = __bfloat1622float2(a.v[k]), fb = __bfloat1622float2(b.v[k]);
      float2 r;
      if (act == 1) {
        r.x = fb.x > 0.f ? fa.x : 0.f;
        r.y = fb.y > 0.f ? fa.y : 0.f;
      } else {
        r.x = fa.x * fb.x * (1.f - fb.x);
        r.y = fa.y * fb.y * (1.f - fb.y);
      }
      o.v[k] = __floats2bfloat162_rn(r.x, r.y);
    }
    dz[i] = o;
  }
}

at::Tensor act_backward_bf16(const at::Tensor& dy, const at::Tensor& y, int64_t act) {
  TORCH_CHECK(dy.scalar_type() == at::kBFloat16 && y.scalar_type() == at::kBFloat16);
  TORCH_CHECK(dy.is_contiguous() && y.is_contiguous() && dy.numel() == y.numel() && dy.numel() % 8 == 0);
  c10::cuda::CUDAGuard guard(dy.device());
  at::Tensor dz = at::empty_like(dy);
  const int64_t n8 = dy.numel() / 8;
  if (n8 == 0) return dz;
  const int64_t blocks = std::min<int64_t>((n8 + 255) / 256, 148 * 16);
  act_backward_kernel<<<blocks, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const bf16x8*>(dy.data_ptr()), reinterpret_cast<const bf16x8*>(y.data_ptr()),
      reinterpret_cast<bf16x8*>(dz.data_ptr()), n8, int(act));
  TRB_CUDA_CHECK(cudaGetLastError());
  return dz;
}

// ---- cross layer backward: du = dy * x0 ; dx0 = dy * u ------------------------------------------
__global__ void __launch_bounds__(256) cross_bwd_kernel(const bf16x8* __restrict__ dy, const bf16x8* __restrict__ x0,
                                                        const bf16x8* __restrict__ u, bf16x8* __restrict__ du,
                                                        bf16x8* __restrict__ dx0, int64_t n8) {
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += int64_t(gridDim.x) * blockDim.x) {
    bf16x8 a = dy[i], b = x0[i], c = u[i], o1, o2;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 fa = __bfloat1622float2(a.v[k]), fb = __bfloat1622float2(b.v[k]), fc = __bfloat1622float2(c.v[k]);
      o1.v[k] = __floats2bfloat162_rn(fa.x * fb.x, fa.y * fb.y);
      o2.v[k] = __floats2bfloat162_rn(fa.x * fc.x, fa.y * fc.y);
    }
    du[i] = o1;
    dx0[i] = o2;
  }
}

std::tuple<at::Tensor, at::Tensor> cross_bwd_elementwise(const at::Tensor& dy, const at::Tensor& x0,
                                                         const at::Tensor& u) {
  TORCH_CHECK(dy.scalar_type() == at::kBFloat16 && x0.scalar_type() == at::kBFloat16 && u.scalar_type() == at::kBFloat16);
  TORCH_CHECK(dy.is_contiguous() && x0.is_contiguous() && u.is_contiguous() && dy.numel() % 8 == 0);
  c10::cuda::CUDAGuard guard(dy.device());
  at::Tensor du = at::empty_like(dy), dx0 = at::empty_like(dy);
  const int64_t n8 = dy.numel() / 8;
  if (n8 == 0) return {du, dx0};
  const int64_t blocks = std::min<int64_t>((n8 + 255) / 256, 148 * 16);
  cross_bwd_kernel<<<blocks, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const bf16x8*>(dy.data_ptr()), reinterpret_cast<const bf16x8*>(x0.data_ptr()),
      reinterpret_cast<const bf16x8*>(u.data_ptr()), reinterpret_cast<bf16x8*>(du.data_ptr()),
      reinterpret_cast<bf16x8*>(dx0.data_ptr()), n8);
  TRB_CUDA_CHECK(cudaGetLastError());
  return {du, dx0};
}

// ---- cross layer backward, fused over the layer stack ---------------------------------------------
//   du      = dy * x0
//   dx0_out = dy * u (+ dx0_in) (+ dy)        running gradient of x0 over the layers (the "+ dy" closes layer 0,
//                                            whose x input is x0 itself)
//   db     += column sums of du               bias gradient, fp32 atomics
// A warp covers 256 consecutive columns of a row (16 bytes per lane), the 8 warps of a CTA walk rows 8 apart.
__global__ void __launch_bounds__(256) cross_bwd_fused_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x0,
                                                              const __nv_bfloat16* __restrict__ u, const __nv_bfloat16* dx0_in,
                                                              __nv_bfloat16* __restrict__ du, __nv_bfloat16* dx0_out,
                                                              float* __restrict__ db, int64_t M, int N, int rows_per_cta, int add_dy) {
  __shared__ float red[8][256];
  const int lane = threadIdx.x & 31, rg = threadIdx.x >> 5;
  const int col = blockIdx.x * 256 + lane * 8;
  const int64_t r0 = int64_t(blockIdx.y) * rows_per_cta;
  const int64_t r1 = min(M, r0 + rows_per_cta);
  float cs[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) cs[k] = 0.f;
  if (col < N) {
    for (int64_t r = r0 + rg; r < r1; r += 8) {
      const int64_t i = r * N + col;
      const bf16x8 a = *reinterpret_cast<const bf16x8*>(dy + i);
      const bf16x8 b = *reinterpret_cast<const bf16x8*>(x0 + i);
      const bf16x8 c = *reinterpret_cast<const bf16x8*>(u + i);
      bf16x8 acc;
      if (dx0_in) acc = *reinterpret_cast<const bf16x8*>(dx0_in + i);
      bf16x8 o1, o2;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 fa = __bfloat1622float2(a.v[k]), fb = __bfloat1622float2(b.v[k]), fc = __bfloat1622float2(c.v[k]);
        o1.v[k] = __floats2bfloat162_rn(fa.x * fb.x, fa.y * fb.y);
        // the bias gradient sums the values that the weight-gradient GEMM will read, i.e. the rounded ones
        const float2 fo = __bfloat1622float2(o1.v[k]);
        cs[2 * k] += fo.x;
        cs[2 * k + 1] += fo.y;
        float gx = fa.x * fc.x, gy = fa.y * fc.y;
        if (dx0_in) {
          const float2 fd = __bfloat1622float2(acc.v[k]);
          gx += fd.x;
          gy += fd.y;
        }
        if (add_dy) {
          gx += fa.x;
          gy += fa.y;
        }
        o2.v[k] = __floats2bfloat162_rn(gx, gy);
      }
      *reinterpret_cast<bf16x8*>(du + i) = o1;
      *reinterpret_cast<bf16x8*>(dx0_out + i) = o2;
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) red[rg][lane * 8 + k] = cs[k];
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) s += red[k][threadIdx.x];
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < N) atomicAdd(db + c, s);
}

// returns (du, dx0_out, db); dx0_out aliases dx0_in when that is given
std::tuple<at::Tensor, at::Tensor, at::Tensor> cross_bwd_fused(const at::Tensor& dy, const at::Tensor& x0, const at::Tensor& u,
                                                               const c10::optional<at::Tensor>& dx0_in, bool add_dy) {
  TORCH_CHECK(dy.scalar_type() == at::kBFloat16 && x0.scalar_type() == at::kBFloat16 && u.scalar_type() == at::kBFloat16);
  TORCH_CHECK(dy.dim() == 2 && dy.is_contiguous() && x0.is_contiguous() && u.is_contiguous() && dy.size(1) % 8 == 0);
  TORCH_CHECK(x0.sizes() == dy.sizes() && u.sizes() == dy.sizes());
  c10::cuda::CUDAGuard guard(dy.device());
  const int64_t M = dy.size(0);
  const int N = int(dy.size(1));
  at::Tensor du = at::empty_like(dy);
  at::Tensor dx0_out;
  const __nv_bfloat16* in_ptr = nullptr;
  if (dx0_in.has_value() && dx0_in->defined()) {
    TORCH_CHECK(dx0_in->scalar_type() == at::kBFloat16 && dx0_in->is_contiguous() && dx0_in->sizes() == dy.sizes());
    dx0_out = *dx0_in;
    in_ptr = reinterpret_cast<const __nv_bfloat16*>(dx0_in->data_ptr());
  } else {
    dx0_out = at::empty_like(dy);
  }
  at::Tensor db = at::zeros({N}, dy.options().dtype(at::kFloat));
  if (M == 0) return {du, dx0_out, db};
  const int col_tiles = (N + 255) / 256;
  const int row_splits = int(std::max<int64_t>(1, std::min<int64_t>((M + 63) / 64, (148 * 8 + col_tiles - 1) / col_tiles)));
  const int rows_per_cta = int((M + row_splits - 1) / row_splits);
  dim3 grid(col_tiles, row_splits);
  cross_bwd_fused_kernel<<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const __nv_bfloat16*>(dy.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(x0.data_ptr()),
      reinterpret_cast<const __nv_bfloat16*>(u.data_ptr()), in_ptr, reinterpret_cast<__nv_bfloat16*>(du.data_ptr()),
      reinterpret_cast<__nv_bfloat16*>(dx0_out.data_ptr()), db.data_ptr<float>(), M, N, rows_per_cta, add_dy ? 1 : 0);
  TRB_CUDA_CHECK(cudaGetLastError());
  return {du, dx0_out, db};
}

// ---- column sum of a bf16 [M, N] matrix -> fp32 [N] (bias gradient) --------------------------------
// grid.x tiles columns (64 per CTA), grid.y splits rows; partial sums are combined with fp32 atomics.
__global__ void __launch_bounds__(256) colsum_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out,
                                                     int64_t M, int N, int rows_per_cta) {
  __shared__ float red[8][64];
  const int c2 = threadIdx.x & 31;   // column pair inside the tile
  const int rg = threadIdx.x >> 5;   // row group 0..7
  const int col = blockIdx.x * 64 + c2 * 2;
  const int64_t r0 = int64_t(blockIdx.y) * rows_per_cta;
  const int64_t r1 = min(M, r0 + rows_per_cta);
  float s0 = 0.f, s1 = 0.f;
  if (col < N) {
    for (int64_t r = r0 + rg; r < r1; r += 8) {
      __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(x + r * N + col);
      float2 f = __bfloat1622float2(v);
      s0 += f.x;
      s1 += f.y;
    }
  }
  red[rg][c2 * 2] = s0;
  red[rg][c2 * 2 + 1] = s1;
  __syncthreads();
  if (threadIdx.x < 64) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) s += red[k][threadIdx.x];
    const int c = blockIdx.x * 64 + threadIdx.x;
    if (c < N) atomicAdd(out + c, s);
  }
}

// column sums of x; with `acc` they are ADDED into that fp32 [N] tensor (a bias gradient landing in a flat gradient buffer)
static at::Tensor colsum_impl(const at::Tensor& x, c10::optional<at::Tensor> acc) {
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.is_contiguous() && x.size(1) % 2 == 0);
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t M = x.size(0);
  const int N = int(x.size(1));
  at::Tensor out;
  if (acc.has_value() && acc->defined()) {
    out = *acc;
    TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kFloat && out.numel() == N && out.is_contiguous());
  } else {
    out = at::zeros({N}, x.options().dtype(at::kFloat));
  }
  if (M == 0) return out;
  const int col_tiles = (N + 63) / 64;
  int row_splits = int(std::max<int64_t>(1, std::min<int64_t>((148 * 8) / col_tiles, (M + 255) / 256)));
  const int rows_per_cta = int((M + row_splits - 1) / row_splits);
  dim3 grid(col_tiles, row_splits);
  colsum_kernel<<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), out.data_ptr<float>(), M, N, rows_per_cta);
  TRB_CUDA_CHECK(cudaGetLastError());
  return out;
}

at::Tensor colsum_bf16(const at::Tensor& x) { return colsum_impl(x, c10::nullopt); }

void colsum_bf16_acc(const at::Tensor& x, at::Tensor acc) { colsum_impl(x, acc); }

// ---- dot interaction ------------------------------------------------------------------------------
// One CTA per sample.  X = [dense; sparse] is staged in shared memory as fp32 with a padded pitch.
template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

template <typename T>
__global__ void __launch_bounds__(128) dot_fwd_kernel(const T* __restrict__ dense, const T* __restrict__ sparse,
                                                      T* __restrict__ out, int F, int D, int out_dim) {
  extern __shared__ float sm[];
  const int n = F + 1, pitch = D + 1;
  const int64_t b = blockIdx.x;
  for (int i = threadIdx.x; i < n * D; i += blockDim.x) {
    const int r = i / D, d = i - r * D;
    sm[r * pitch + d] = r == 0 ? to_f<T>(dense[b * D + d]) : to_f<T>(sparse[(b * F + (r - 1)) * D + d]);
  }
  __syncthreads();
  T* o = out + b * out_dim;
  for (int d = threadIdx.x; d < D; d += blockDim.x) o[d] = from_f<T>(sm[d]);
  const int npairs = n * (n - 1) / 2;
  for (int pi = threadIdx.x; pi < npairs; pi += blockDim.x) {
    // pair index -> (i, j), i < j, row-major over the strict upper triangle
    int i = 0, rem = pi;
    while (rem >= n - 1 - i) { rem -= n - 1 - i; ++i; }
    const int j = i + 1 + rem;
    float s = 0.f;
    for (int d = 0; d < D; ++d) s = fmaf(sm[i * pitch + d], sm[j * pitch + d], s);
    o[D + pi] = from_f<T>(s);
  }
}

template <typename T>
__global__ void __launch_bounds__(128) dot_bwd_kernel(const T* __restrict__ dout, const T* __restrict__ dense,
                                                      const T* __restrict__ sparse, T* __restrict__ ddense,
                                                      T* __restrict__ dsparse, int F, int D, int out_dim) {
  extern __shared__ float sm[];
  const int n = F + 1, pitch = D + 1;
  float* X = sm;                 // [n, pitch]
  float* dZ = sm + n * pitch;    // [n, n] symmetric, zero diagonal
  const int64_t b = blockIdx.x;
  for (int i = threadIdx.x; i < n * D; i += blockDim.x) {
    const int r = i / D, d = i - r * D;
    X[r * pitch + d] = r == 0 ? to_f<T>(dense[b * D + d]) : to_f<T>(sparse[(b * F + (r - 1)) * D + d]);
  }
  for (int i = threadIdx.x; i < n * n; i += blockDim.x) dZ[i] = 0.f;
  __syncthreads();
  const T* go = dout + b * out_dim;
  const int npairs = n * (n - 1) / 2;
  for (int pi = threadIdx.x; pi < npairs; pi += blockDim.x) {
    int i = 0, rem = pi;
    while (rem >= n - 1 - i) { rem -= n - 1 - i; ++i; }
    const int j = i + 1 + rem;
    const float g = to_f<T>(go[D + pi]);
    dZ[i * n + j] = g;
    dZ[j * n + i] = g;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < n * D; idx += blockDim.x) {
    const int i = idx / D, d = idx - i * D;
    float s = 0.f;
    for (int j = 0; j < n; ++j) s = fmaf(dZ[i * n + j], X[j * pitch + d], s);
    if (i == 0) ddense[b * D + d] = from_f<T>(s + to_f<T>(go[d]));
    else dsparse[(b * F + (i - 1)) * D + d] = from_f<T>(s);
  }
}

at::Tensor dot_interaction_fwd(const at::Tensor& dense, const at::Tensor& sparse) {
  TORCH_CHECK(dense.dim() == 2 && sparse.dim() == 3 && dense.is_contiguous() && sparse.is_contiguous());
  TORCH_CHECK(dense.scalar_type() == sparse.scalar_type());
  c10::cuda::CUDAGuard guard(dense.device());
  const int64_t B = dense.size(0);
  const int D = int(dense.size(1)), F = int(sparse.size(1));
  const int n = F + 1;
  const int out_dim = D + n * (n - 1) / 2;
  at::Tensor out = at::empty({B, out_dim}, dense.options());
  if (B == 0) return out;
  const size_t smem = size_t(n) * (D + 1) * sizeof(float);
  auto stream = at::cuda::getCurrentCUDAStream();
  if (dense.scalar_type() == at::kFloat) {
    cudaFuncSetAttribute(dot_fwd_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    dot_fwd_kernel<float><<<B, 128, smem, stream>>>(dense.data_ptr<float>(), sparse.data_ptr<float>(),
                                                    out.data_ptr<float>(), F, D, out_dim);
  } else if (dot_mma_ok(F, D)) {
    TORCH_CHECK(dense.scalar_type() == at::kBFloat16);
    const size_t msmem = dot_fwd_mma_smem(D);
    if (msmem > 48 * 1024) cudaFuncSetAttribute(dot_fwd_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(msmem));
    dot_fwd_mma_kernel<<<(B + kDotWarps - 1) / kDotWarps, 32 * kDotWarps, msmem, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(dense.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(sparse.data_ptr()),
        reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), B, F, D, out_dim);
  } else {
    TORCH_CHECK(dense.scalar_type() == at::kBFloat16);
    cudaFuncSetAttribute(dot_fwd_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    dot_fwd_kernel<__nv_bfloat16><<<B, 128, smem, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(dense.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(sparse.data_ptr()),
        reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), F, D, out_dim);
  }
  TRB_CUDA_CHECK(cudaGetLastError());
  return out;
}

std::tuple<at::Tensor, at::Tensor> dot_interaction_bwd(const at::Tensor& dout, const at::Tensor& dense,
                                                       const at::Tensor& sparse) {
  c10::cuda::CUDAGuard guard(dense.device());
  const int64_t B = dense.size(0);
  const int D = int(dense.size(1)), F = int(sparse.size(1));
  const int n = F + 1;
  const int out_dim = D + n * (n - 1) / 2;
  TORCH_CHECK(dout.is_contiguous() && dout.size(1) == out_dim && dout.scalar_type() == dense.scalar_type());
  at::Tensor dd = at::empty_like(dense), ds = at::empty_like(sparse);
  if (B == 0) return {dd, ds};
  const size_t smem = (size_t(n) * (D + 1) + size_t(n) * n) * sizeof(float);
  auto stream = at::cuda::getCurrentCUDAStream();
  if (dense.scalar_type() == at::kFloat) {
    cudaFuncSetAttribute(dot_bwd_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    dot_bwd_kernel<float><<<B, 128, smem, stream>>>(dout.data_ptr<float>(), dense.data_ptr<float>(),
                                                    sparse.data_ptr<float>(), dd.data_ptr<float>(),
                                                    ds.data_ptr<float>(), F, D, out_dim);
  } else if (dot_mma_ok(F, D)) {
    const size_t msmem = dot_bwd_mma_smem(D);
    if (msmem > 48 * 1024) cudaFuncSetAttribute(dot_bwd_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(msmem));
    dot_bwd_mma_kernel<<<(B + kDotWarps - 1) / kDotWarps, 32 * kDotWarps, msmem, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(dout.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(dense.data_ptr()),
        reinterpret_cast<const __nv_bfloat16*>(sparse.data_ptr()), reinterpret_cast<__nv_bfloat16*>(dd.data_ptr()),
        reinterpret_cast<__nv_bfloat16*>(ds.data_ptr()), B, F, D, out_dim);
  } else {
    cudaFuncSetAttribute(dot_bwd_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    dot_bwd_kernel<__nv_bfloat16><<<B, 128, smem, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(dout.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(dense.data_ptr()),
        reinterpret_cast<const __nv_bfloat16*>(sparse.data_ptr()), reinterpret_cast<__nv_bfloat16*>(dd.data_ptr()),
        reinterpret_cast<__nv_bfloat16*>(ds.data_ptr()), F, D, out_dim);
  }
  TRB_CUDA_CHECK(cudaGetLastError());
  return {dd, ds};
}

}  // namespace trb

TORCH_LIBRARY_FRAGMENT(trb200, m) {
  m.def("act_backward_bf16(Tensor dy, Tensor y, int act) -> Tensor");
  m.def("cross_bwd_elementwise(Tensor dy, Tensor x0, Tensor u) -> (Tensor, Tensor)");
  m.def("cross_bwd_fused(Tensor dy, Tensor x0, Tensor u, Tensor(a!)? dx0_in, bool add_dy) -> (Tensor, Tensor(a!), Tensor)");
  m.def("colsum_bf16(Tensor x) -> Tensor");
  m.def("colsum_bf16_acc(Tensor x, Tensor(a!) acc) -> ()");
  m.def("dot_interaction_fwd(Tensor dense, Tensor sparse) -> Tensor");
  m.def("dot_interaction_bwd(Tensor dout, Tensor dense, Tensor sparse) -> (Tensor, Tensor)");
}

TORCH_LIBRARY_IMPL(trb200, CUDA, m) {
  m.impl("act_backward_bf16", &trb::act_backward_bf16);
  m.impl("cross_bwd_elementwise", &trb::cross_bwd_elementwise);
  m.impl("cross_bwd_fused", &trb::cross_bwd_fused);
  m.impl("colsum_bf16", &trb::colsum_bf16);
  m.impl("colsum_bf16_acc", &trb::colsum_bf16_acc);
  m.impl("dot_interaction_fwd", &trb::dot_interaction_fwd);
  m.impl("dot_interaction_bwd", &trb::dot_interaction_bwd);
}
