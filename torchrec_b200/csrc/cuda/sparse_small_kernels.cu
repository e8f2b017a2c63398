// Small sparse-data kernels that the Python layer would otherwise compose from several library launches:
//
//   offsets_range     position of every element inside its segment (an arange that restarts at every segment start)
//   segment_sum_csr   sum of values over [csr[i] * batch, csr[i + 1] * batch): one warp per segment
//   vbe_expand        variable-batch pooled output -> full batch: every (feature, sample) copies the row that the inverse
//                     indices name, straight to its output column (replaces one index_select per feature plus a concat)
//
// The reference takes the first two from an external operator library and composes the third
// (torchrec/distributed/embeddingbag.py:385-440).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "common.cuh"

namespace trb {

template <typename T>
__global__ void __launch_bounds__(256) offsets_range_kernel(const T* __restrict__ starts, int64_t n_seg, T* __restrict__ out, int64_t total) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  // last segment whose start is <= i
  int64_t lo = 0, hi = n_seg;
  while (hi - lo > 1) {
    const int64_t mid = (lo + hi) >> 1;
    if (int64_t(starts[mid]) <= i) lo = mid; else hi = mid;
  }
  out[i] = T(i - int64_t(starts[lo]));
}

template <typename V, typename I>
__global__ void __launch_bounds__(256) segment_sum_csr_kernel(const I* __restrict__ csr, int64_t batch, const V* __restrict__ values,
                                                              V* __restrict__ out, int64_t n_seg) {
  const int lane = threadIdx.x & 31;
  const int64_t seg = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (seg >= n_seg) return;
  const int64_t lo = int64_t(csr[seg]) * batch, hi = int64_t(csr[seg + 1]) * batch;
  double acc = 0.0;  // integer inputs stay exact up to 2^53, floats get a wider accumulator than their own type
  for (int64_t i = lo + lane; i < hi; i += 32) acc += double(values[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) out[seg] = V(acc);
}

// flat: the per-feature outputs [b_f, D_f] back to back; desc (int64 [F, 4]): flat offset, b_f, D_f, output column
template <typename V, typename I>
__global__ void __launch_bounds__(256) vbe_expand_kernel(const V* __restrict__ flat, const int64_t* __restrict__ desc, const I* __restrict__ inverse,
                                                         int64_t inv_stride, V* __restrict__ out, int64_t B, int64_t out_stride, int F, int* err) {
  const int lane = threadIdx.x & 31;
  const int64_t w = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (w >= int64_t(F) * B) return;
  const int f = int(w / B);
  const int64_t b = w - int64_t(f) * B;
  const int64_t base = desc[f * 4], rows = desc[f * 4 + 1], D = desc[f * 4 + 2], col = desc[f * 4 + 3];
  int64_t src = int64_t(inverse[f * inv_stride + b]);
  if (src < 0 || src >= rows) {  // never read outside the feature's block
    if (lane == 0) atomicExch(err, 1);
    src = 0;
    if (rows == 0) return;
  }
  const V* in = flat + base + src * D;
  V* o = out + b * out_stride + col;
  for (int64_t e = lane; e < D; e += 32) o[e] = in[e];
}

at::Tensor offsets_range(const at::Tensor& starts, int64_t total) {
  TORCH_CHECK(starts.is_cuda() && starts.dim() == 1 && starts.is_contiguous() && (starts.scalar_type() == at::kInt || starts.scalar_type() == at::kLong));
  c10::cuda::CUDAGuard guard(starts.device());
  at::Tensor out = at::empty({total}, starts.options());
  if (total == 0 || starts.numel() == 0) return out;
  auto stream = at::cuda::getCurrentCUDAStream();
  const int64_t blocks = (total + 255) / 256;
  if (starts.scalar_type() == at::kLong)
    offsets_range_kernel<int64_t><<<blocks, 256, 0, stream>>>(starts.data_ptr<int64_t>(), starts.numel(), out.data_ptr<int64_t>(), total);
  else
    offsets_range_kernel<int32_t><<<blocks, 256, 0, stream>>>(starts.data_ptr<int32_t>(), starts.numel(), out.data_ptr<int32_t>(), total);
  TRB_CUDA_CHECK(cudaGetLastError());
  return out;
}

at::Tensor segment_sum_csr(int64_t batch, const at::Tensor& csr, const at::Tensor& values) {
  TORCH_CHECK(csr.is_cuda() && values.is_cuda() && csr.is_contiguous() && values.is_contiguous());
  TORCH_CHECK(csr.scalar_type() == at::kInt || csr.scalar_type() == at::kLong, "csr offsets must be int32 or int64");
  c10::cuda::CUDAGuard guard(values.device());
  const int64_t n_seg = std::max<int64_t>(csr.numel() - 1, 0);
  at::Tensor out = at::empty({n_seg}, values.options());
  if (n_seg == 0) return out;
  auto stream = at::cuda::getCurrentCUDAStream();
  const int64_t blocks = (n_seg * 32 + 255) / 256;
  AT_DISPATCH_ALL_TYPES_AND2(at::kHalf, at::kBFloat16, values.scalar_type(), "segment_sum_csr", [&] {
    if (csr.scalar_type() == at::kLong)
      segment_sum_csr_kernel<scalar_t, int64_t><<<blocks, 256, 0, stream>>>(csr.data_ptr<int64_t>(), batch, values.data_ptr<scalar_t>(), out.data_ptr<scalar_t>(), n_seg);
    else
      segment_sum_csr_kernel<scalar_t, int32_t><<<blocks, 256, 0, stream>>>(csr.data_ptr<int32_t>(), batch, values.data_ptr<scalar_t>(), out.data_ptr<scalar_t>(), n_seg);
  });
  TRB_CUDA_CHECK(cudaGetLastError());
  return out;
}

at::Tensor vbe_expand(const at::Tensor& flat, const at::Tensor& desc, const at::Tensor& inverse, int64_t out_cols, at::Tensor err) {
  TORCH_CHECK(flat.is_cuda() && flat.dim() == 1 && flat.is_contiguous());
  TORCH_CHECK(desc.is_cuda() && desc.scalar_type() == at::kLong && desc.dim() == 2 && desc.size(1) == 4 && desc.is_contiguous());
  TORCH_CHECK(inverse.is_cuda() && inverse.dim() == 2 && inverse.stride(1) == 1 && inverse.size(0) == desc.size(0));
  TORCH_CHECK(inverse.scalar_type() == at::kInt || inverse.scalar_type() == at::kLong);
  c10::cuda::CUDAGuard guard(flat.device());
  const int F = int(desc.size(0));
  const int64_t B = inverse.size(1);
  at::Tensor out = at::empty({B, out_cols}, flat.options());
  if (F == 0 || B == 0) return out;
  auto stream = at::cuda::getCurrentCUDAStream();
  const int64_t blocks = (int64_t(F) * B * 32 + 255) / 256;
  AT_DISPATCH_FLOATING_TYPES_AND2(at::kHalf, at::kBFloat16, flat.scalar_type(), "vbe_expand", [&] {
    if (inverse.scalar_type() == at::kLong)
      vbe_expand_kernel<scalar_t, int64_t><<<blocks, 256, 0, stream>>>(flat.data_ptr<scalar_t>(), desc.data_ptr<int64_t>(), inverse.data_ptr<int64_t>(),
                                                                      inverse.stride(0), out.data_ptr<scalar_t>(), B, out_cols, F, err.data_ptr<int>());
    else
      vbe_expand_kernel<scalar_t, int32_t><<<blocks, 256, 0, stream>>>(flat.data_ptr<scalar_t>(), desc.data_ptr<int64_t>(), inverse.data_ptr<int32_t>(),
                                                                      inverse.stride(0), out.data_ptr<scalar_t>(), B, out_cols, F, err.data_ptr<int>());
  });
  TRB_CUDA_CHECK(cudaGetLastError());
  return out;
}

}  // namespace trb

TORCH_LIBRARY_FRAGMENT(trb200, m) {
  m.def("offsets_range(Tensor starts, int total) -> Tensor");
  m.def("segment_sum_csr(int batch, Tensor csr, Tensor values) -> Tensor");
  m.def("vbe_expand(Tensor flat, Tensor desc, Tensor inverse, int out_cols, Tensor(a!) err) -> Tensor");
}

TORCH_LIBRARY_IMPL(trb200, CUDA, m) {
  m.impl("offsets_range", &trb::offsets_range);
  m.impl("segment_sum_csr", &trb::segment_sum_csr);
  m.impl("vbe_expand", &trb::vbe_expand);
}
