// Small sparse-data kernels that the Python layer would otherwise compose from several library launches:
//
//   offsets_range     position of every element inside its segment (an arange that restarts at every segment start)
//   segment_sum_csr   sum of values over [csr[i] * batch, csr[i + 1] * batch): blocks over (segment, slice), then the slices in order
//   vbe_expand        variable-batch pooled output -> full batch: every (feature, sample) copies the row that the inverse
//                     indices name, straight to its output column (replaces one index_select per feature plus a concat)
//
//   jagged_unique_indices   per-feature deduplication of ids: linearize (id + base of the feature's table), radix-sort the
//                     (key, position) pairs, flag the first of every run, scan the flags into ranks, scatter: unique ids, the
//                     reverse index of every input id, and the number of distinct ids per feature
//
// The reference takes the first two and the last from an external operator library and composes the third
// (torchrec/distributed/embeddingbag.py:385-440, torchrec/distributed/embedding.py:1329-1370).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <cub/cub.cuh>

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

// pass 1: block (segment, slice) sums its slice of the segment in double; pass 2: one thread per segment adds the slices in order
// (deterministic; integer inputs stay exact up to 2^53, floats get a wider accumulator than their own type)
template <typename V, typename I>
__global__ void __launch_bounds__(256) segment_sum_csr_kernel(const I* __restrict__ csr, int64_t batch, const V* __restrict__ values,
                                                              double* __restrict__ partial, int slices) {
  __shared__ double red[8];
  const int64_t seg = blockIdx.x;
  const int sl = blockIdx.y;
  const int64_t lo = int64_t(csr[seg]) * batch, hi = int64_t(csr[seg + 1]) * batch;
  const int64_t per = (hi - lo + slices - 1) / slices;
  const int64_t a = lo + sl * per, b = a + per < hi ? a + per : hi;
  double acc = 0.0;
  for (int64_t i = a + threadIdx.x; i < b; i += blockDim.x) acc += double(values[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w];
    partial[seg * slices + sl] = t;
  }
}

template <typename V>
__global__ void segment_sum_finish_kernel(const double* __restrict__ partial, int slices, V* __restrict__ out, int64_t n_seg) {
  const int64_t seg = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (seg >= n_seg) return;
  double t = 0.0;
  for (int s = 0; s < slices; ++s) t += partial[seg * slices + s];
  out[seg] = V(t);
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
  // enough (segment, slice) blocks to fill the GPU, but no slice shorter than a few thousand elements
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const int64_t avg = std::max<int64_t>(values.numel() / n_seg, 1);
  const int slices = int(std::max<int64_t>(1, std::min<int64_t>({(int64_t(sms) * 4 + n_seg - 1) / n_seg, (avg + 4095) / 4096, int64_t(1024)})));
  TORCH_CHECK(n_seg <= 2147483647, "too many segments");
  at::Tensor partial = at::empty({n_seg * slices}, values.options().dtype(at::kDouble));
  const dim3 grid(static_cast<unsigned>(n_seg), static_cast<unsigned>(slices));
  AT_DISPATCH_ALL_TYPES_AND2(at::kHalf, at::kBFloat16, values.scalar_type(), "segment_sum_csr", [&] {
    if (csr.scalar_type() == at::kLong)
      segment_sum_csr_kernel<scalar_t, int64_t><<<grid, 256, 0, stream>>>(csr.data_ptr<int64_t>(), batch, values.data_ptr<scalar_t>(), partial.data_ptr<double>(), slices);
    else
      segment_sum_csr_kernel<scalar_t, int32_t><<<grid, 256, 0, stream>>>(csr.data_ptr<int32_t>(), batch, values.data_ptr<scalar_t>(), partial.data_ptr<double>(), slices);
    segment_sum_finish_kernel<scalar_t><<<unsigned((n_seg + 255) / 256), 256, 0, stream>>>(partial.data_ptr<double>(), slices, out.data_ptr<scalar_t>(), n_seg);
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

// ---- jagged_unique_indices ---------------------------------------------------------------------------------------------
// last index j in [0, n) with a[j] <= v (a ascending, a[0] <= v)
__device__ __forceinline__ int64_t last_not_above(const int64_t* __restrict__ a, int64_t n, int64_t v) {
  int64_t lo = 0, hi = n;
  while (hi - lo > 1) {
    const int64_t mid = (lo + hi) >> 1;
    if (a[mid] <= v) lo = mid; else hi = mid;
  }
  return lo;
}

// key[i] = indices[i] + base[table of the feature of i]; pos[i] = i.  offsets [F * B + 1] bound the bags (feature-major).
template <typename I>
__global__ void __launch_bounds__(256) unique_linearize_kernel(const I* __restrict__ indices, const int64_t* __restrict__ offsets, int64_t n_bags, int64_t B,
                                                               const int64_t* __restrict__ feat_base, int64_t N, int64_t* __restrict__ key,
                                                               int64_t* __restrict__ pos) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= N) return;
  const int64_t bag = last_not_above(offsets, n_bags + 1, i);  // offsets[bag] <= i < offsets[bag + 1] (empty bags are skipped by "last")
  key[i] = int64_t(indices[i]) + feat_base[bag / B];
  pos[i] = i;
}

__global__ void __launch_bounds__(256) unique_heads_kernel(const int64_t* __restrict__ key_sorted, int64_t N, int32_t* __restrict__ head) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= N) return;
  head[i] = (i == 0 || key_sorted[i] != key_sorted[i - 1]) ? 1 : 0;
}

template <typename I>
__global__ void __launch_bounds__(256) unique_scatter_kernel(const int64_t* __restrict__ key_sorted, const int64_t* __restrict__ pos_sorted,
                                                             const int32_t* __restrict__ head, const int64_t* __restrict__ rank, int64_t N,
                                                             const int64_t* __restrict__ feat_base, int64_t F, I* __restrict__ unique, I* __restrict__ reverse,
                                                             int64_t* __restrict__ unique_key) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= N) return;
  const int64_t r = rank[i] - 1;
  reverse[pos_sorted[i]] = I(r);
  if (head[i]) {
    const int64_t f = last_not_above(feat_base, F, key_sorted[i]);
    unique[r] = I(key_sorted[i] - feat_base[f]);
    unique_key[r] = key_sorted[i];
  }
}

// distinct ids per feature from the sorted unique keys: the keys of feature f lie in [base[f], base[f + 1]) (features that share a
// base: everything is counted under the last of them, the others get 0); one thread per feature, no atomics
__global__ void unique_count_kernel(const int64_t* __restrict__ unique_key, const int64_t* __restrict__ rank, int64_t N, const int64_t* __restrict__ feat_base,
                                    int64_t F, int64_t* __restrict__ per_feature) {
  const int64_t f = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (f >= F) return;
  const int64_t U = rank[N - 1];
  auto first_not_below = [&](int64_t v) {
    int64_t lo = 0, hi = U;
    while (lo < hi) {
      const int64_t mid = (lo + hi) >> 1;
      if (unique_key[mid] < v) lo = mid + 1; else hi = mid;
    }
    return lo;
  };
  const int64_t begin = first_not_below(feat_base[f]);
  const int64_t end = (f + 1 < F) ? first_not_below(feat_base[f + 1]) : U;
  per_feature[f] = end - begin;
}

// feat_base [F] ascending: the id base of every feature's table.  Returns (distinct ids per feature [F] int64, unique ids (feature-major,
// ascending inside a feature), reverse index [N]); one host read for the number of distinct ids.
std::tuple<at::Tensor, at::Tensor, at::Tensor> jagged_unique_indices(const at::Tensor& feat_base, const at::Tensor& offsets, const at::Tensor& indices,
                                                                    int64_t key_bits) {
  TORCH_CHECK(indices.is_cuda() && indices.dim() == 1 && indices.is_contiguous() && (indices.scalar_type() == at::kInt || indices.scalar_type() == at::kLong));
  TORCH_CHECK(offsets.is_cuda() && offsets.scalar_type() == at::kLong && offsets.is_contiguous() && offsets.numel() >= 1);
  TORCH_CHECK(feat_base.is_cuda() && feat_base.scalar_type() == at::kLong && feat_base.is_contiguous() && feat_base.numel() >= 1);
  c10::cuda::CUDAGuard guard(indices.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const int64_t N = indices.numel(), F = feat_base.numel(), n_bags = offsets.numel() - 1;
  TORCH_CHECK(n_bags % F == 0, "offsets must describe the same number of bags for every feature");
  const auto lopt = indices.options().dtype(at::kLong);
  at::Tensor per_feature = at::zeros({F}, lopt);
  if (N == 0) return {per_feature, at::empty({0}, indices.options()), at::empty({0}, indices.options())};
  at::Tensor key = at::empty({N}, lopt), pos = at::empty({N}, lopt), key_s = at::empty({N}, lopt), pos_s = at::empty({N}, lopt);
  at::Tensor head = at::empty({N}, indices.options().dtype(at::kInt)), rank = at::empty({N}, lopt);
  const int64_t blocks = (N + 255) / 256;
  AT_DISPATCH_INDEX_TYPES(indices.scalar_type(), "jagged_unique_linearize", [&] {
    unique_linearize_kernel<index_t><<<blocks, 256, 0, stream>>>(indices.data_ptr<index_t>(), offsets.data_ptr<int64_t>(), n_bags, std::max<int64_t>(n_bags / F, 1),
                                                                feat_base.data_ptr<int64_t>(), N, key.data_ptr<int64_t>(), pos.data_ptr<int64_t>());
  });
  const int end_bit = int(std::min<int64_t>(64, std::max<int64_t>(1, key_bits)));
  size_t bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, bytes, key.data_ptr<int64_t>(), key_s.data_ptr<int64_t>(), pos.data_ptr<int64_t>(), pos_s.data_ptr<int64_t>(), N, 0, end_bit,
                                  stream);
  at::Tensor tmp = at::empty({int64_t(bytes)}, indices.options().dtype(at::kByte));
  cub::DeviceRadixSort::SortPairs(tmp.data_ptr(), bytes, key.data_ptr<int64_t>(), key_s.data_ptr<int64_t>(), pos.data_ptr<int64_t>(), pos_s.data_ptr<int64_t>(), N, 0,
                                  end_bit, stream);
  unique_heads_kernel<<<blocks, 256, 0, stream>>>(key_s.data_ptr<int64_t>(), N, head.data_ptr<int32_t>());
  size_t sbytes = 0;
  cub::DeviceScan::InclusiveSum(nullptr, sbytes, head.data_ptr<int32_t>(), rank.data_ptr<int64_t>(), N, stream);
  at::Tensor stmp = at::empty({int64_t(sbytes)}, indices.options().dtype(at::kByte));
  cub::DeviceScan::InclusiveSum(stmp.data_ptr(), sbytes, head.data_ptr<int32_t>(), rank.data_ptr<int64_t>(), N, stream);
  at::Tensor unique = at::empty({N}, indices.options()), reverse = at::empty({N}, indices.options());
  at::Tensor unique_key = key;  // the unsorted keys are no longer needed: their buffer takes the sorted distinct keys
  AT_DISPATCH_INDEX_TYPES(indices.scalar_type(), "jagged_unique_scatter", [&] {
    unique_scatter_kernel<index_t><<<blocks, 256, 0, stream>>>(key_s.data_ptr<int64_t>(), pos_s.data_ptr<int64_t>(), head.data_ptr<int32_t>(), rank.data_ptr<int64_t>(), N,
                                                              feat_base.data_ptr<int64_t>(), F, unique.data_ptr<index_t>(), reverse.data_ptr<index_t>(),
                                                              unique_key.data_ptr<int64_t>());
  });
  unique_count_kernel<<<unsigned((F + 127) / 128), 128, 0, stream>>>(unique_key.data_ptr<int64_t>(), rank.data_ptr<int64_t>(), N, feat_base.data_ptr<int64_t>(), F,
                                                                    per_feature.data_ptr<int64_t>());
  TRB_CUDA_CHECK(cudaGetLastError());
  const int64_t distinct = rank[N - 1].item<int64_t>();  // the only host read: the output's size
  return {per_feature, unique.narrow(0, 0, distinct), reverse};
}

}  // namespace trb

TORCH_LIBRARY_FRAGMENT(trb200, m) {
  m.def("jagged_unique_indices(Tensor feat_base, Tensor offsets, Tensor indices, int key_bits) -> (Tensor, Tensor, Tensor)");
  m.def("offsets_range(Tensor starts, int total) -> Tensor");
  m.def("segment_sum_csr(int batch, Tensor csr, Tensor values) -> Tensor");
  m.def("vbe_expand(Tensor flat, Tensor desc, Tensor inverse, int out_cols, Tensor(a!) err) -> Tensor");
}

TORCH_LIBRARY_IMPL(trb200, CUDA, m) {
  m.impl("jagged_unique_indices", &trb::jagged_unique_indices);
  m.impl("offsets_range", &trb::offsets_range);
  m.impl("segment_sum_csr", &trb::segment_sum_csr);
  m.impl("vbe_expand", &trb::vbe_expand);
}
