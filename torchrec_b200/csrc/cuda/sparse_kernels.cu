// Jagged / sparse-input kernels for sm_100a: scans, KJT permute, row-wise bucketization and
// jagged <-> padded conversion.  All are HBM-bound integer kernels; none allocates per element and the
// only host round trip is the optional output-size query when the caller does not know it.
//
// The reference calls the equivalent operators of an external wheel
// (torchrec/sparse/jagged_tensor.py:80,2577; torchrec/distributed/embedding_sharding.py:263).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <cub/cub.cuh>

#include "common.cuh"

namespace trb {

// ---- complete cumsum: out[0] = 0, out[i+1] = sum(x[0..i]) ---------------------------------------
template <typename T>
__global__ void set_zero_first(T* out) { out[0] = T(0); }

at::Tensor complete_cumsum(const at::Tensor& x) {
  TORCH_CHECK(x.dim() == 1 && x.is_contiguous());
  c10::cuda::CUDAGuard guard(x.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const int64_t n = x.numel();
  at::Tensor out = at::empty({n + 1}, x.options());
  auto run = [&](auto tag) {
    using T = decltype(tag);
    set_zero_first<T><<<1, 1, 0, stream>>>(out.data_ptr<T>());
    if (n == 0) return;
    size_t bytes = 0;
    cub::DeviceScan::InclusiveSum(nullptr, bytes, x.data_ptr<T>(), out.data_ptr<T>() + 1, n, stream);
    at::Tensor tmp = at::empty({int64_t(bytes)}, x.options().dtype(at::kByte));
    cub::DeviceScan::InclusiveSum(tmp.data_ptr(), bytes, x.data_ptr<T>(), out.data_ptr<T>() + 1, n, stream);
  };
  if (x.scalar_type() == at::kLong) run(int64_t(0));
  else if (x.scalar_type() == at::kInt) run(int32_t(0));
  else if (x.scalar_type() == at::kFloat) run(float(0));
  else TORCH_CHECK(false, "complete_cumsum: unsupported dtype ", x.scalar_type());
  return out;
}

// ---- permute_2d_sparse_data ---------------------------------------------------------------------
template <typename len_t, typename pidx_t>
__global__ void permute_lengths_kernel(const pidx_t* __restrict__ permute, const len_t* __restrict__ lengths,
                                       len_t* __restrict__ out_lengths, int Tp, int B) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= int64_t(Tp) * B) return;
  const int t = int(i / B), b = int(i - int64_t(t) * B);
  out_lengths[i] = lengths[int64_t(permute[t]) * B + b];
}

// every output row (all B bags of one key) is one contiguous run in both layouts
template <typename val_t, typename off_t, typename pidx_t>
__global__ void permute_rows_copy_kernel(const pidx_t* __restrict__ permute, const off_t* __restrict__ in_off,
                                         const off_t* __restrict__ out_off, const val_t* __restrict__ in,
                                         val_t* __restrict__ out, const float* __restrict__ win,
                                         float* __restrict__ wout, int B) {
  const int t = blockIdx.y;
  const int64_t src0 = int64_t(in_off[int64_t(permute[t]) * B]);
  const int64_t dst0 = int64_t(out_off[int64_t(t) * B]);
  const int64_t n = int64_t(out_off[int64_t(t + 1) * B]) - dst0;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
    out[dst0 + i] = in[src0 + i];
    if (win) wout[dst0 + i] = win[src0 + i];
  }
}

std::tuple<at::Tensor, at::Tensor, c10::optional<at::Tensor>> permute_2d_sparse_data(
    const at::Tensor& permute, const at::Tensor& lengths, const at::Tensor& values,
    const c10::optional<at::Tensor>& weights, int64_t permuted_sum) {
  TORCH_CHECK(lengths.dim() == 2);
  c10::cuda::CUDAGuard guard(values.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const int B = int(lengths.size(1)), Tp = int(permute.numel());
  at::Tensor lengths_c = lengths.contiguous();
  at::Tensor out_lengths = at::empty({Tp, B}, lengths.options());
  at::Tensor perm = permute.scalar_type() == at::kInt ? permute.contiguous() : permute.to(at::kInt);
  const bool has_w = weights.has_value() && weights->defined();
  if (Tp == 0 || B == 0) {
    return {out_lengths, at::empty({0}, values.options()),
            has_w ? c10::optional<at::Tensor>(at::empty({0}, weights->options())) : c10::nullopt};
  }
  const int64_t nl = int64_t(Tp) * B;
  auto launch_len = [&](auto tag) {
    using L = decltype(tag);
    permute_lengths_kernel<L, int32_t><<<(nl + 255) / 256, 256, 0, stream>>>(
        perm.data_ptr<int32_t>(), lengths_c.data_ptr<L>(), out_lengths.data_ptr<L>(), Tp, B);
  };
  if (lengths.scalar_type() == at::kLong) launch_len(int64_t(0));
  else if (lengths.scalar_type() == at::kInt) launch_len(int32_t(0));
  else TORCH_CHECK(false, "lengths must be int32/int64");
  at::Tensor in_off = complete_cumsum(lengths_c.view({-1}));
  at::Tensor out_off = complete_cumsum(out_lengths.view({-1}));
  const int64_t total = permuted_sum >= 0 ? permuted_sum : out_off[-1].item<int64_t>();
  at::Tensor out_values = at::empty({total}, values.options());
  at::Tensor out_weights;
  if (has_w) out_weights = at::empty({total}, weights->options());
  if (total > 0) {
    const int64_t per_row = (total + Tp - 1) / Tp;
    dim3 grid(unsigned(std::max<int64_t>(1, std::min<int64_t>((per_row + 255) / 256, 1024))), Tp);
    auto launch = [&](auto vtag, auto otag) {
      using V = decltype(vtag);
      using O = decltype(otag);
      permute_rows_copy_kernel<V, O, int32_t><<<grid, 256, 0, stream>>>(
          perm.data_ptr<int32_t>(), in_off.data_ptr<O>(), out_off.data_ptr<O>(),
          reinterpret_cast<const V*>(values.data_ptr()), reinterpret_cast<V*>(out_values.data_ptr()),
          has_w ? weights->data_ptr<float>() : nullptr, has_w ? out_weights.data_ptr<float>() : nullptr, B);
    };
    const size_t es = values.element_size();
    const bool o64 = lengths.scalar_type() == at::kLong;
    if (es == 8) { if (o64) launch(int64_t(0), int64_t(0)); else launch(int64_t(0), int32_t(0)); }
    else if (es == 4) { if (o64) launch(int32_t(0), int64_t(0)); else launch(int32_t(0), int32_t(0)); }
    else TORCH_CHECK(false, "values must be 4 or 8 bytes wide");
    TRB_CUDA_CHECK(cudaGetLastError());
  }
  return {out_lengths, out_values, has_w ? c10::optional<at::Tensor>(out_weights) : c10::nullopt};
}

// ---- block bucketize ------------------------------------------------------------------------------
template <typename idx_t>
__device__ __forceinline__ void bucket_of(idx_t id, int64_t blk, int my_size, int& bucket, int64_t& local) {
  const int64_t v = int64_t(id);
  if (v < blk * my_size) {
    bucket = int(v / blk);
    local = v - int64_t(bucket) * blk;
  } else {
    bucket = int(v % my_size);
    local = v / my_size;
  }
}

template <typename idx_t, typename len_t>
__global__ void __launch_bounds__(256) bucketize_count_kernel(const len_t* __restrict__ offsets,
                                                              const idx_t* __restrict__ indices,
                                                              const int64_t* __restrict__ block_sizes, int F, int B,
                                                              int my_size, len_t* __restrict__ new_lengths) {
  const int lane = threadIdx.x & 31;
  const int64_t bag = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nbags = int64_t(F) * B;
  if (bag >= nbags) return;
  const int f = int(bag / B);
  const int64_t blk = max(int64_t(1), block_sizes[f]);
  const int64_t s = offsets[bag], e = offsets[bag + 1];
  int cnt_mine = 0;  // lane w counts bucket w
  for (int64_t i0 = s; i0 < e; i0 += 32) {
    int bucket = -1;
    int64_t local;
    if (i0 + lane < e) bucket_of(indices[i0 + lane], blk, my_size, bucket, local);
    for (int w = 0; w < my_size; ++w) {
      const unsigned m = __ballot_sync(0xffffffffu, bucket == w);
      if (lane == w) cnt_mine += __popc(m);
    }
  }
  if (lane < my_size) new_lengths[int64_t(lane) * nbags + bag] = len_t(cnt_mine);
}

template <typename idx_t, typename len_t>
__global__ void __launch_bounds__(256) bucketize_scatter_kernel(
    const len_t* __restrict__ offsets, const idx_t* __restrict__ indices, const float* __restrict__ weights,
    const int64_t* __restrict__ block_sizes, int F, int B, int my_size, const len_t* __restrict__ new_offsets,
    idx_t* __restrict__ new_indices, float* __restrict__ new_weights, idx_t* __restrict__ new_pos,
    idx_t* __restrict__ unbucketize, int keep_orig) {
  const int lane = threadIdx.x & 31;
  const int64_t bag = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nbags = int64_t(F) * B;
  if (bag >= nbags) return;
  const int f = int(bag / B);
  const int64_t blk = max(int64_t(1), block_sizes[f]);
  const int64_t s = offsets[bag], e = offsets[bag + 1];
  int64_t base_mine = lane < my_size ? int64_t(new_offsets[int64_t(lane) * nbags + bag]) : 0;  // next free slot of bucket `lane`
  for (int64_t i0 = s; i0 < e; i0 += 32) {
    int bucket = -1;
    int64_t local = 0;
    idx_t id = 0;
    const bool act = i0 + lane < e;
    if (act) {
      id = indices[i0 + lane];
      bucket_of(id, blk, my_size, bucket, local);
    }
    int64_t dst = 0;
    for (int w = 0; w < my_size; ++w) {
      const unsigned m = __ballot_sync(0xffffffffu, bucket == w);
      const int64_t base = __shfl_sync(0xffffffffu, base_mine, w);
      if (bucket == w) dst = base + __popc(m & ((1u << lane) - 1u));
      if (lane == w) base_mine += __popc(m);
    }
    if (act) {
      new_indices[dst] = keep_orig ? id : idx_t(local);
      if (weights) new_weights[dst] = weights[i0 + lane];
      if (new_pos) new_pos[dst] = idx_t(i0 + lane - s);
      if (unbucketize) unbucketize[i0 + lane] = idx_t(dst);
    }
  }
}

std::tuple<at::Tensor, at::Tensor, c10::optional<at::Tensor>, c10::optional<at::Tensor>, c10::optional<at::Tensor>>
block_bucketize(const at::Tensor& lengths, const at::Tensor& indices, bool bucketize_pos, bool sequence,
                const at::Tensor& block_sizes, int64_t my_size, const c10::optional<at::Tensor>& weights,
                bool keep_orig_idx) {
  c10::cuda::CUDAGuard guard(indices.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  TORCH_CHECK(my_size >= 1 && my_size <= 32, "block_bucketize supports up to 32 buckets");
  TORCH_CHECK(lengths.scalar_type() == indices.scalar_type(), "lengths and indices must share a dtype");
  const int F = int(block_sizes.numel());
  const int64_t nbags = lengths.numel();
  const int B = F > 0 ? int(nbags / F) : 0;
  const int64_t N = indices.numel();
  at::Tensor bs = block_sizes.to(at::kLong).contiguous();
  at::Tensor lengths_c = lengths.contiguous().view({-1});
  at::Tensor offsets = complete_cumsum(lengths_c);
  at::Tensor new_lengths = at::empty({my_size * nbags}, lengths.options());
  at::Tensor new_indices = at::empty({N}, indices.options());
  const bool has_w = weights.has_value() && weights->defined();
  at::Tensor new_weights, new_pos, unbucketize;
  if (has_w) new_weights = at::empty({N}, weights->options());
  if (bucketize_pos) new_pos = at::empty({N}, indices.options());
  if (sequence) unbucketize = at::empty({N}, indices.options());
  if (nbags > 0) {
    const int threads = 256;
    const int64_t blocks = (nbags * 32 + threads - 1) / threads;
    auto run = [&](auto tag) {
      using I = decltype(tag);
      bucketize_count_kernel<I, I><<<blocks, threads, 0, stream>>>(offsets.data_ptr<I>(), indices.data_ptr<I>(),
                                                                   bs.data_ptr<int64_t>(), F, B, int(my_size),
                                                                   new_lengths.data_ptr<I>());
      at::Tensor new_offsets = complete_cumsum(new_lengths);
      bucketize_scatter_kernel<I, I><<<blocks, threads, 0, stream>>>(
          offsets.data_ptr<I>(), indices.data_ptr<I>(), has_w ? weights->data_ptr<float>() : nullptr,
          bs.data_ptr<int64_t>(), F, B, int(my_size), new_offsets.data_ptr<I>(), new_indices.data_ptr<I>(),
          has_w ? new_weights.data_ptr<float>() : nullptr, bucketize_pos ? new_pos.data_ptr<I>() : nullptr,
          sequence ? unbucketize.data_ptr<I>() : nullptr, keep_orig_idx ? 1 : 0);
    };
    if (indices.scalar_type() == at::kLong) run(int64_t(0));
    else if (indices.scalar_type() == at::kInt) run(int32_t(0));
    else TORCH_CHECK(false, "indices must be int32/int64");
    TRB_CUDA_CHECK(cudaGetLastError());
  }
  return {new_lengths, new_indices, has_w ? c10::optional<at::Tensor>(new_weights) : c10::nullopt,
          bucketize_pos ? c10::optional<at::Tensor>(new_pos) : c10::nullopt,
          sequence ? c10::optional<at::Tensor>(unbucketize) : c10::nullopt};
}

// ---- jagged <-> padded ----------------------------------------------------------------------------
// one warp per (sample, position) row of D elements; rows are moved as raw bytes
template <typename off_t>
__global__ void __launch_bounds__(256) jagged_to_padded_kernel(const uint8_t* __restrict__ values,
                                                               const off_t* __restrict__ offsets,
                                                               uint8_t* __restrict__ out, int64_t Bn, int L,
                                                               int row_bytes, uint32_t pad_bits, int elem_size) {
  const int lane = threadIdx.x & 31;
  const int64_t r = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (r >= Bn * L) return;
  const int64_t b = r / L;
  const int l = int(r - b * L);
  const int64_t s = offsets[b], e = offsets[b + 1];
  uint8_t* dst = out + r * row_bytes;
  if (s + l < e) {
    const uint8_t* src = values + (s + l) * row_bytes;
    if ((row_bytes & 15) == 0) {
      for (int i = lane * 16; i < row_bytes; i += 512) *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
    } else {
      for (int i = lane; i < row_bytes; i += 32) dst[i] = src[i];
    }
  } else {
    if (elem_size == 4) {
      for (int i = lane * 4; i < row_bytes; i += 128) *reinterpret_cast<uint32_t*>(dst + i) = pad_bits;
    } else {
      for (int i = lane * 2; i < row_bytes; i += 64) *reinterpret_cast<uint16_t*>(dst + i) = uint16_t(pad_bits);
    }
  }
}

at::Tensor jagged_to_padded_dense(const at::Tensor& values, const at::Tensor& offsets, int64_t max_length,
                                  double padding_value) {
  TORCH_CHECK(values.dim() == 2 && values.is_contiguous());
  c10::cuda::CUDAGuard guard(values.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const int64_t Bn = offsets.numel() - 1;
  const int64_t D = values.size(1);
  at::Tensor out = at::empty({Bn, max_length, D}, values.options());
  if (Bn * max_length == 0) return out;
  const int es = int(values.element_size());
  TORCH_CHECK(es == 4 || es == 2, "jagged_to_padded_dense supports 2- and 4-byte element types");
  uint32_t pad_bits = 0;
  if (values.scalar_type() == at::kFloat) { float f = float(padding_value); memcpy(&pad_bits, &f, 4); }
  else if (values.scalar_type() == at::kHalf) { __half h = __float2half(float(padding_value)); uint16_t u; memcpy(&u, &h, 2); pad_bits = u; }
  else if (values.scalar_type() == at::kBFloat16) { __nv_bfloat16 h = __float2bfloat16(float(padding_value)); uint16_t u; memcpy(&u, &h, 2); pad_bits = u; }
  else if (values.scalar_type() == at::kInt) { int32_t v = int32_t(padding_value); memcpy(&pad_bits, &v, 4); }
  else TORCH_CHECK(false, "unsupported dtype");
  const int64_t rows = Bn * max_length;
  const int64_t blocks = (rows * 32 + 255) / 256;
  at::Tensor off = offsets.contiguous();
  if (off.scalar_type() == at::kLong) {
    jagged_to_padded_kernel<int64_t><<<blocks, 256, 0, stream>>>(
        reinterpret_cast<const uint8_t*>(values.data_ptr()), off.data_ptr<int64_t>(),
        reinterpret_cast<uint8_t*>(out.data_ptr()), Bn, int(max_length), int(D * es), pad_bits, es);
  } else {
    TORCH_CHECK(off.scalar_type() == at::kInt);
    jagged_to_padded_kernel<int32_t><<<blocks, 256, 0, stream>>>(
        reinterpret_cast<const uint8_t*>(values.data_ptr()), off.data_ptr<int32_t>(),
        reinterpret_cast<uint8_t*>(out.data_ptr()), Bn, int(max_length), int(D * es), pad_bits, es);
  }
  TRB_CUDA_CHECK(cudaGetLastError());
  return out;
}

template <typename off_t>
__global__ void __launch_bounds__(256) padded_to_jagged_kernel(const uint8_t* __restrict__ dense,
                                                               const off_t* __restrict__ offsets,
                                                               uint8_t* __restrict__ out, int64_t Bn, int L,
                                                               int row_bytes) {
  const int lane = threadIdx.x & 31;
  const int64_t r = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (r >= Bn * L) return;
  const int64_t b = r / L;
  const int l = int(r - b * L);
  const int64_t s = offsets[b], e = offsets[b + 1];
  if (s + l >= e) return;
  const uint8_t* src = dense + r * row_bytes;
  uint8_t* dst = out + (s + l) * row_bytes;
  if ((row_bytes & 15) == 0) {
    for (int i = lane * 16; i < row_bytes; i += 512) *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
  } else {
    for (int i = lane; i < row_bytes; i += 32) dst[i] = src[i];
  }
}

at::Tensor padded_dense_to_jagged(const at::Tensor& dense, const at::Tensor& offsets, int64_t total) {
  TORCH_CHECK(dense.dim() == 3 && dense.is_contiguous());
  c10::cuda::CUDAGuard guard(dense.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const int64_t Bn = dense.size(0), L = dense.size(1), D = dense.size(2);
  at::Tensor out = at::zeros({total, D}, dense.options());
  if (Bn * L == 0 || total == 0) return out;
  const int64_t rows = Bn * L;
  const int64_t blocks = (rows * 32 + 255) / 256;
  at::Tensor off = offsets.contiguous();
  const int rb = int(D * dense.element_size());
  if (off.scalar_type() == at::kLong) {
    padded_to_jagged_kernel<int64_t><<<blocks, 256, 0, stream>>>(
        reinterpret_cast<const uint8_t*>(dense.data_ptr()), off.data_ptr<int64_t>(),
        reinterpret_cast<uint8_t*>(out.data_ptr()), Bn, int(L), rb);
  } else {
    TORCH_CHECK(off.scalar_type() == at::kInt);
    padded_to_jagged_kernel<int32_t><<<blocks, 256, 0, stream>>>(
        reinterpret_cast<const uint8_t*>(dense.data_ptr()), off.data_ptr<int32_t>(),
        reinterpret_cast<uint8_t*>(out.data_ptr()), Bn, int(L), rb);
  }
  TRB_CUDA_CHECK(cudaGetLastError());
  return out;
}

}  // namespace trb

TORCH_LIBRARY_FRAGMENT(trb200, m) {
  m.def("complete_cumsum(Tensor x) -> Tensor");
  m.def("permute_2d_sparse_data(Tensor permute, Tensor lengths, Tensor values, Tensor? weights, int permuted_sum) -> (Tensor, Tensor, Tensor?)");
  m.def(
      "block_bucketize(Tensor lengths, Tensor indices, bool bucketize_pos, bool sequence, Tensor block_sizes, "
      "int my_size, Tensor? weights, bool keep_orig_idx) -> (Tensor, Tensor, Tensor?, Tensor?, Tensor?)");
  m.def("jagged_to_padded_dense(Tensor values, Tensor offsets, int max_length, float padding_value) -> Tensor");
  m.def("padded_dense_to_jagged(Tensor dense, Tensor offsets, int total) -> Tensor");
}

TORCH_LIBRARY_IMPL(trb200, CUDA, m) {
  m.impl("complete_cumsum", &trb::complete_cumsum);
  m.impl("permute_2d_sparse_data", &trb::permute_2d_sparse_data);
  m.impl("block_bucketize", &trb::block_bucketize);
  m.impl("jagged_to_padded_dense", &trb::jagged_to_padded_dense);
  m.impl("padded_dense_to_jagged", &trb::padded_dense_to_jagged);
}
