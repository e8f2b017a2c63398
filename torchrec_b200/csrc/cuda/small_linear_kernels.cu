// Linear layers whose shape does not fit a tensor-core tile, on the CUDA cores and bound by memory:
//
//   small K   the first layer of a bottom MLP reads a handful of dense features (K = 13 for the Criteo models): a thread keeps the
//             weights of four output columns in registers and walks the rows.  The weight gradient walks the rows
//             once with K accumulators per output column and adds its partial sums into the fp32 gradient.
//   N = 1     the logit layer: one warp per row for the forward; the backward writes dx = dy * w and reduces dw and db in one pass.
//
// The bf16 TMA operands of the tcgen05 GEMM need row pitches of 16 bytes (K % 8 == 0, N % 8 == 0), which K = 13 and N = 1 do not
// meet; the reference hands both layers to the library's GEMM (torchrec/modules/mlp.py:20-90).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_bf16.h>
#include <torch/library.h>

#include "common.cuh"

namespace trb {

constexpr int kSmallKMax = 32;

__device__ __forceinline__ float small_act(float v, int act) {
  if (act == 1) return v > 0.f ? v : 0.f;
  if (act == 2) return 1.f / (1.f + __expf(-v));
  return v;
}

// y[m, n] = act(sum_k x[m, k] w[n, k] + b[n]);  x bf16 [M, K], w fp32 [N, K], y bf16 [M, N], N % 4 == 0, K <= KP
// A thread keeps the weights of four neighbouring columns in registers and walks the rows of a 64-row tile whose x values sit in
// shared memory (one broadcast read per row and four values); `tpr` threads (a power of two) cover a row, grid.y the column chunks.
template <int KP>
__global__ void __launch_bounds__(256) small_k_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                                                          __nv_bfloat16* __restrict__ y, int64_t M, int N, int K, int act, int tpr) {
  constexpr int kRows = 64;
  __shared__ __align__(16) float xs[kRows][KP];
  const int cq = blockIdx.y * tpr + (threadIdx.x & (tpr - 1));  // column quad
  const int rl = threadIdx.x / tpr, rpp = 256 / tpr;
  const bool live = 4 * cq < N;
  float wr[4][KP], br[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    br[j] = (live && bias) ? bias[4 * cq + j] : 0.f;
#pragma unroll
    for (int k = 0; k < KP; ++k) wr[j][k] = (live && k < K) ? w[int64_t(4 * cq + j) * K + k] : 0.f;
  }
  const int64_t tiles = (M + kRows - 1) / kRows;
  for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const int64_t r0 = tile * kRows;
    const int nr = M - r0 < kRows ? int(M - r0) : kRows;
    __syncthreads();
    for (int i = threadIdx.x; i < kRows * KP; i += 256) {
      const int r = i / KP, k = i - r * KP;
      xs[r][k] = (r < nr && k < K) ? __bfloat162float(x[(r0 + r) * K + k]) : 0.f;
    }
    __syncthreads();
    if (!live) continue;
    for (int r = rl; r < nr; r += rpp) {
      float acc[4] = {br[0], br[1], br[2], br[3]};
#pragma unroll
      for (int k4 = 0; k4 < KP; k4 += 4) {
        const float4 xv = *reinterpret_cast<const float4*>(&xs[r][k4]);
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[j] += xv.x * wr[j][k4] + xv.y * wr[j][k4 + 1] + xv.z * wr[j][k4 + 2] + xv.w * wr[j][k4 + 3];
      }
      __align__(8) __nv_bfloat162 o[2] = {__floats2bfloat162_rn(small_act(acc[0], act), small_act(acc[1], act)),
                                          __floats2bfloat162_rn(small_act(acc[2], act), small_act(acc[3], act))};
      *reinterpret_cast<uint2*>(y + (r0 + r) * N + 4 * cq) = *reinterpret_cast<const uint2*>(o);
    }
  }
}

// dw[n, k] += sum_m dz[m, n] x[m, k];  dz bf16 [M, N] (N even), x bf16 [M, K], K <= KP
// grid (row chunks, column-pair chunks of 256); every thread owns two neighbouring columns
template <int KP>
__global__ void __launch_bounds__(256) small_k_wgrad_kernel(const __nv_bfloat16* __restrict__ dz, const __nv_bfloat16* __restrict__ x, float* __restrict__ dw,
                                                            int64_t M, int N, int K, int64_t rows_per_block) {
  constexpr int kRows = 128;
  __shared__ __align__(16) float xs[kRows][KP];
  const int cp = blockIdx.y * 256 + threadIdx.x;  // column pair
  const bool live = 2 * cp < N;
  const int64_t r_lo = int64_t(blockIdx.x) * rows_per_block;
  const int64_t r_hi = r_lo + rows_per_block < M ? r_lo + rows_per_block : M;
  float a0[KP], a1[KP];
#pragma unroll
  for (int k = 0; k < KP; ++k) a0[k] = a1[k] = 0.f;
  for (int64_t r0 = r_lo; r0 < r_hi; r0 += kRows) {
    const int nr = r_hi - r0 < kRows ? int(r_hi - r0) : kRows;
    __syncthreads();
    for (int i = threadIdx.x; i < kRows * KP; i += 256) {
      const int r = i / KP, k = i - r * KP;
      xs[r][k] = (r < nr && k < K) ? __bfloat162float(x[(r0 + r) * K + k]) : 0.f;
    }
    __syncthreads();
    if (!live) continue;
    for (int rb = 0; rb < nr; rb += 8) {  // eight loads in flight per thread before the arithmetic (rows past nr: x is zero)
      float2 g[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int r = rb + u < nr ? rb + u : nr - 1;
        g[u] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dz + (r0 + r) * N + 2 * cp));
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
#pragma unroll
        for (int k4 = 0; k4 < KP; k4 += 4) {
          const float4 xv = *reinterpret_cast<const float4*>(&xs[(rb + u) & (kRows - 1)][k4]);
          const float gx = rb + u < nr ? g[u].x : 0.f, gy = rb + u < nr ? g[u].y : 0.f;
          a0[k4] += gx * xv.x; a0[k4 + 1] += gx * xv.y; a0[k4 + 2] += gx * xv.z; a0[k4 + 3] += gx * xv.w;
          a1[k4] += gy * xv.x; a1[k4 + 1] += gy * xv.y; a1[k4 + 2] += gy * xv.z; a1[k4 + 3] += gy * xv.w;
        }
      }
    }
  }
  if (!live) return;
#pragma unroll
  for (int k = 0; k < KP; ++k) {
    if (k < K) {
      atomicAdd(dw + int64_t(2 * cp) * K + k, a0[k]);
      atomicAdd(dw + int64_t(2 * cp + 1) * K + k, a1[k]);
    }
  }
}

// y[m] = sum_k x[m, k] w[k] + b;  x bf16 [M, K], K % 8 == 0; one warp per row
__global__ void __launch_bounds__(256) out1_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                                                       float* __restrict__ y, int64_t M, int K) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = (int64_t(gridDim.x) * blockDim.x) >> 5;
  const float b = bias ? bias[0] : 0.f;
  for (int64_t m = warp; m < M; m += nwarps) {
    float acc = 0.f;
    for (int k0 = lane * 8; k0 < K; k0 += 256) {
      const uint4 raw = *reinterpret_cast<const uint4*>(x + m * K + k0);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
      const float4 w0 = *reinterpret_cast<const float4*>(w + k0);
      const float4 w1 = *reinterpret_cast<const float4*>(w + k0 + 4);
      const float2 p0 = __bfloat1622float2(h[0]), p1 = __bfloat1622float2(h[1]), p2 = __bfloat1622float2(h[2]), p3 = __bfloat1622float2(h[3]);
      acc += p0.x * w0.x + p0.y * w0.y + p1.x * w0.z + p1.y * w0.w + p2.x * w1.x + p2.y * w1.y + p3.x * w1.z + p3.y * w1.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) y[m] = acc + b;
  }
}

// dx[m, k] = dy[m] w[k] (bf16);  dw[k] += sum_m dy[m] x[m, k];  db += sum_m dy[m];  K % 8 == 0, K <= 1024
__global__ void __launch_bounds__(256) out1_bwd_kernel(const float* __restrict__ dy, const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                                       __nv_bfloat16* __restrict__ dx, float* __restrict__ dw, float* __restrict__ db, int64_t M, int K) {
  __shared__ float red[8][256 + 1];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int64_t warp = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = (int64_t(gridDim.x) * blockDim.x) >> 5;
  for (int pass = 0; pass * 256 < K; ++pass) {
    const int k0 = pass * 256 + lane * 8;
    const bool live = k0 < K;
    float wv[8], acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      wv[j] = live ? w[k0 + j] : 0.f;
      acc[j] = 0.f;
    }
    float dsum = 0.f;
    for (int64_t m = warp; m < M; m += nwarps) {
      const float g = dy[m];
      dsum += g;
      if (!live) continue;
      const uint4 raw = *reinterpret_cast<const uint4*>(x + m * K + k0);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
      __align__(16) __nv_bfloat162 o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 p = __bfloat1622float2(h[j]);
        acc[2 * j] += g * p.x;
        acc[2 * j + 1] += g * p.y;
        o[j] = __floats2bfloat162_rn(g * wv[2 * j], g * wv[2 * j + 1]);
      }
      if (dx) *reinterpret_cast<uint4*>(dx + m * K + k0) = *reinterpret_cast<const uint4*>(o);
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 8; ++j) red[wib][lane * 8 + j] = acc[j];
    __syncthreads();
    {
      const int k = pass * 256 + threadIdx.x;
      if (k < K) {
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < 8; ++q) s += red[q][threadIdx.x];
        atomicAdd(dw + k, s);
      }
    }
    if (pass == 0 && db != nullptr && lane == 0) atomicAdd(db, dsum);
  }
}

static int small_grid(int64_t work_items, int per_block) {
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return int(std::max<int64_t>(1, std::min<int64_t>((work_items + per_block - 1) / per_block, int64_t(sms) * 8)));
}

at::Tensor linear_small_k_fwd(const at::Tensor& x, const at::Tensor& w, const c10::optional<at::Tensor>& bias, int64_t act) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.is_contiguous(), "x must be a contiguous bf16 CUDA matrix");
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == at::kFloat && w.dim() == 2 && w.is_contiguous() && w.size(1) == x.size(1));
  const int64_t M = x.size(0);
  const int N = int(w.size(0)), K = int(w.size(1));
  TORCH_CHECK(K >= 1 && K <= kSmallKMax && N % 4 == 0 && N >= 4, "linear_small_k: K <= 32 and N % 4 == 0");
  if (bias.has_value()) TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == at::kFloat && bias->numel() == N && bias->is_contiguous());
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor y = at::empty({M, N}, x.options());
  if (M == 0) return y;
  auto stream = at::cuda::getCurrentCUDAStream();
  const int quads = N / 4;
  int tpr = 1;
  while (tpr < quads && tpr < 256) tpr *= 2;
  const int col_chunks = (quads + tpr - 1) / tpr;
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const int64_t tiles = (M + 63) / 64;
  const dim3 grid(unsigned(std::max<int64_t>(1, std::min<int64_t>(tiles, (int64_t(sms) * 4 + col_chunks - 1) / col_chunks))), unsigned(col_chunks));
  const auto* xp = reinterpret_cast<const __nv_bfloat16*>(x.data_ptr());
  const float* bp = bias.has_value() ? bias->data_ptr<float>() : nullptr;
  auto* yp = reinterpret_cast<__nv_bfloat16*>(y.data_ptr());
  if (K <= 8) small_k_fwd_kernel<8><<<grid, 256, 0, stream>>>(xp, w.data_ptr<float>(), bp, yp, M, N, K, int(act), tpr);
  else if (K <= 16) small_k_fwd_kernel<16><<<grid, 256, 0, stream>>>(xp, w.data_ptr<float>(), bp, yp, M, N, K, int(act), tpr);
  else small_k_fwd_kernel<32><<<grid, 256, 0, stream>>>(xp, w.data_ptr<float>(), bp, yp, M, N, K, int(act), tpr);
  TRB_CUDA_CHECK(cudaGetLastError());
  return y;
}

void linear_small_k_wgrad_acc(const at::Tensor& dz, const at::Tensor& x, at::Tensor dw) {
  TORCH_CHECK(dz.is_cuda() && dz.scalar_type() == at::kBFloat16 && dz.dim() == 2 && dz.is_contiguous());
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.is_contiguous() && x.size(0) == dz.size(0));
  const int64_t M = dz.size(0);
  const int N = int(dz.size(1)), K = int(x.size(1));
  TORCH_CHECK(dw.is_cuda() && dw.scalar_type() == at::kFloat && dw.is_contiguous() && dw.numel() == int64_t(N) * K);
  TORCH_CHECK(K >= 1 && K <= kSmallKMax && N % 2 == 0, "linear_small_k: K <= 32 and N even");
  if (M == 0) return;
  c10::cuda::CUDAGuard guard(dz.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const int col_chunks = (N / 2 + 255) / 256;
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const int64_t row_blocks = std::max<int64_t>(1, std::min<int64_t>((M + 127) / 128, (2 * sms + col_chunks - 1) / col_chunks));
  int64_t rows_per_block = (M + row_blocks - 1) / row_blocks;
  rows_per_block = (rows_per_block + 127) / 128 * 128;
  const dim3 grid(unsigned((M + rows_per_block - 1) / rows_per_block), unsigned(col_chunks));
  const auto* dzp = reinterpret_cast<const __nv_bfloat16*>(dz.data_ptr());
  const auto* xp = reinterpret_cast<const __nv_bfloat16*>(x.data_ptr());
  if (K <= 8) small_k_wgrad_kernel<8><<<grid, 256, 0, stream>>>(dzp, xp, dw.data_ptr<float>(), M, N, K, rows_per_block);
  else if (K <= 16) small_k_wgrad_kernel<16><<<grid, 256, 0, stream>>>(dzp, xp, dw.data_ptr<float>(), M, N, K, rows_per_block);
  else small_k_wgrad_kernel<32><<<grid, 256, 0, stream>>>(dzp, xp, dw.data_ptr<float>(), M, N, K, rows_per_block);
  TRB_CUDA_CHECK(cudaGetLastError());
}

at::Tensor linear_out1_fwd(const at::Tensor& x, const at::Tensor& w, const c10::optional<at::Tensor>& bias) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.is_contiguous());
  const int64_t M = x.size(0);
  const int K = int(x.size(1));
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == at::kFloat && w.is_contiguous() && w.numel() == K && K % 8 == 0 && K <= 1024);
  if (bias.has_value()) TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == at::kFloat && bias->numel() == 1);
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor y = at::empty({M, 1}, x.options().dtype(at::kFloat));
  if (M == 0) return y;
  auto stream = at::cuda::getCurrentCUDAStream();
  out1_fwd_kernel<<<small_grid(M, 8 * 4), 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), w.data_ptr<float>(),
                                                            bias.has_value() ? bias->data_ptr<float>() : nullptr, y.data_ptr<float>(), M, K);
  TRB_CUDA_CHECK(cudaGetLastError());
  return y;
}

// returns dx (bf16 [M, K]) when need_dx, an empty tensor otherwise; dw and db are accumulated into
at::Tensor linear_out1_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& w, at::Tensor dw, const c10::optional<at::Tensor>& db, bool need_dx) {
  TORCH_CHECK(dy.is_cuda() && dy.scalar_type() == at::kFloat && dy.is_contiguous() && dy.numel() == x.size(0));
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.is_contiguous());
  const int64_t M = x.size(0);
  const int K = int(x.size(1));
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == at::kFloat && w.is_contiguous() && w.numel() == K && K % 8 == 0 && K <= 1024);
  TORCH_CHECK(dw.is_cuda() && dw.scalar_type() == at::kFloat && dw.is_contiguous() && dw.numel() == K);
  if (db.has_value()) TORCH_CHECK(db->is_cuda() && db->scalar_type() == at::kFloat && db->numel() == 1);
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor dx = need_dx ? at::empty({M, K}, x.options()) : at::empty({0}, x.options());
  if (M == 0) return dx;
  auto stream = at::cuda::getCurrentCUDAStream();
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const int blocks = int(std::max<int64_t>(1, std::min<int64_t>((M + 63) / 64, int64_t(sms) * 4)));
  out1_bwd_kernel<<<blocks, 256, 0, stream>>>(dy.data_ptr<float>(), reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), w.data_ptr<float>(),
                                              need_dx ? reinterpret_cast<__nv_bfloat16*>(dx.data_ptr()) : nullptr, dw.data_ptr<float>(),
                                              db.has_value() ? db->data_ptr<float>() : nullptr, M, K);
  TRB_CUDA_CHECK(cudaGetLastError());
  return dx;
}

}  // namespace trb

TORCH_LIBRARY_FRAGMENT(trb200, m) {
  m.def("linear_small_k_fwd(Tensor x, Tensor w, Tensor? bias, int act) -> Tensor");
  m.def("linear_small_k_wgrad_acc(Tensor dz, Tensor x, Tensor(a!) dw) -> ()");
  m.def("linear_out1_fwd(Tensor x, Tensor w, Tensor? bias) -> Tensor");
  m.def("linear_out1_bwd(Tensor dy, Tensor x, Tensor w, Tensor(a!) dw, Tensor(b!)? db, bool need_dx) -> Tensor");
}

TORCH_LIBRARY_IMPL(trb200, CUDA, m) {
  m.impl("linear_small_k_fwd", &trb::linear_small_k_fwd);
  m.impl("linear_small_k_wgrad_acc", &trb::linear_small_k_wgrad_acc);
  m.impl("linear_out1_fwd", &trb::linear_out1_fwd);
  m.impl("linear_out1_bwd", &trb::linear_out1_bwd);
}
