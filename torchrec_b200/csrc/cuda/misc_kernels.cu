// Smaller sm_100a kernels: row-wise N-bit quantization of embedding tables, fused binary cross entropy
// (loss and gradient in one pass), multi-probe zero-collision hash, in-training-pruning index remap and the
// keyed-tensor regroup (one launch for any number of inputs and groups).  All are HBM-bound streaming or
// random-access kernels; none waits on another thread block.
//
// The reference takes these from an external wheel: quantization torchrec/quant/embedding_modules.py:261-276,
// hash lookup torchrec/modules/hash_mc_modules.py:518, pruning remap torchrec/modules/itep_modules.py:533,
// regroup torchrec/modules/regroup.py:56.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "common.cuh"
#include "zch_hash.h"

namespace trb {

// ================================================================================================
// row-wise N-bit quantization: [R, D] fp32/fp16/bf16 -> [R, D*bits/8 + 4] bytes (payload, fp16 scale, fp16 bias)
// one warp per row; the row is read twice (min/max, then pack), the second time from L1/L2.
// ================================================================================================
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T, int BITS>
__global__ void __launch_bounds__(256) rowwise_quantize_kernel(const T* __restrict__ w, uint8_t* __restrict__ out, int64_t R, int D) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (row >= R) return;
  const T* src = w + row * D;
  float lo = INFINITY, hi = -INFINITY;
  for (int c = lane; c < D; c += 32) {
    const float v = to_f32(src[c]);
    lo = fminf(lo, v);
    hi = fmaxf(hi, v);
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) {
    lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, s));
    hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, s));
  }
  constexpr float qmax = float((1 << BITS) - 1);
  // scale and bias are stored in fp16: quantize against the values the lookup kernel will use
  const __half hs = __float2half_rn(__fdiv_rn(hi - lo, qmax));
  const __half hb = __float2half_rn(lo);
  float scale = __half2float(hs);
  if (scale == 0.f) scale = 1.f;
  const float bias = __half2float(hb);
  constexpr int PER = 8 / BITS;  // values per payload byte
  const int nbytes = D / PER;
  uint8_t* dst = out + row * (int64_t(nbytes) + 4);
  for (int b = lane; b < nbytes; b += 32) {
    uint32_t byte = 0;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const float v = to_f32(src[b * PER + j]);
      float q = rintf(__fdiv_rn(v - bias, scale));
      q = fminf(fmaxf(q, 0.f), qmax);
      byte |= uint32_t(q) << (j * BITS);
    }
    dst[b] = uint8_t(byte);
  }
  if (lane == 0) {
    const __half one = __float2half_rn(1.f);
    const __half stored = (__half2float(hs) == 0.f) ? one : hs;
    const uint16_t s16 = *reinterpret_cast<const uint16_t*>(&stored), b16 = *reinterpret_cast<const uint16_t*>(&hb);
    dst[nbytes + 0] = uint8_t(s16 & 0xff);
    dst[nbytes + 1] = uint8_t(s16 >> 8);
    dst[nbytes + 2] = uint8_t(b16 & 0xff);
    dst[nbytes + 3] = uint8_t(b16 >> 8);
  }
}

at::Tensor rowwise_quantize_nbit(const at::Tensor& w, int64_t bits) {
  TORCH_CHECK(w.is_cuda() && w.dim() == 2 && w.is_contiguous(), "rowwise_quantize_nbit: contiguous CUDA [R, D] expected");
  TORCH_CHECK(bits == 8 || bits == 4 || bits == 2, "rowwise_quantize_nbit: bits must be 8, 4 or 2");
  const int64_t R = w.size(0), D = w.size(1);
  TORCH_CHECK((D * bits) % 8 == 0, "rowwise_quantize_nbit: D*bits must be a whole number of bytes");
  c10::cuda::CUDAGuard guard(w.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  at::Tensor out = at::empty({R, D * bits / 8 + 4}, w.options().dtype(at::kByte));
  if (R == 0) return out;
  const int threads = 256;
  const int64_t blocks = (R * 32 + threads - 1) / threads;
  auto launch = [&](auto tag) {
    using T = decltype(tag);
    const T* p = reinterpret_cast<const T*>(w.data_ptr());
    if (bits == 8) rowwise_quantize_kernel<T, 8><<<blocks, threads, 0, stream>>>(p, out.data_ptr<uint8_t>(), R, int(D));
    else if (bits == 4) rowwise_quantize_kernel<T, 4><<<blocks, threads, 0, stream>>>(p, out.data_ptr<uint8_t>(), R, int(D));
    else rowwise_quantize_kernel<T, 2><<<blocks, threads, 0, stream>>>(p, out.data_ptr<uint8_t>(), R, int(D));
  };
  if (w.scalar_type() == at::kFloat) launch(float(0));
  else if (w.scalar_type() == at::kHalf) launch(__half());
  else if (w.scalar_type() == at::kBFloat16) launch(__nv_bfloat16());
  else TORCH_CHECK(false, "rowwise_quantize_nbit: unsupported dtype ", w.scalar_type());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

// ================================================================================================
// binary cross entropy with logits, mean reduction, loss and d(loss)/d(logit) in one pass.
// loss_i = w_i * (max(x,0) - x*y + log1p(exp(-|x|)));  grad_i = w_i * (sigmoid(x) - y) / N.
// Block partials are combined by the last block to finish (fixed order -> deterministic).
// ================================================================================================
template <typename T>
__global__ void __launch_bounds__(256) bce_fwd_bwd_kernel(const T* __restrict__ x, const float* __restrict__ y, const float* __restrict__ wt,
                                                          float* __restrict__ grad, float* __restrict__ partial, unsigned int* __restrict__ counter,
                                                          float* __restrict__ loss, int64_t N) {
  __shared__ float red[8];
  __shared__ bool last;
  const float inv_n = 1.f / float(N);
  float acc = 0.f;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < N; i += int64_t(gridDim.x) * blockDim.x) {
    const float xi = to_f32(x[i]), yi = y[i], wi = wt ? wt[i] : 1.f;
    const float e = expf(-fabsf(xi));
    acc += wi * (fmaxf(xi, 0.f) - xi * yi + log1pf(e));
    const float sig = xi >= 0.f ? __fdiv_rn(1.f, 1.f + e) : __fdiv_rn(e, 1.f + e);
    grad[i] = wi * (sig - yi) * inv_n;
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) s += red[i];
    partial[blockIdx.x] = s;
    __threadfence();
    last = atomicAdd(counter, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (last && threadIdx.x < 32) {
    float s = 0.f;
    for (int i = threadIdx.x; i < gridDim.x; i += 32) s += __ldcg(partial + i);
#pragma unroll
    for (int k = 16; k > 0; k >>= 1) s += __shfl_xor_sync(0xffffffffu, s, k);
    if (threadIdx.x == 0) {
      loss[0] = s * inv_n;
      *counter = 0;  // ready for the next launch that reuses the workspace
    }
  }
}

std::tuple<at::Tensor, at::Tensor> bce_with_logits_fwd_bwd(const at::Tensor& logits, const at::Tensor& labels, const c10::optional<at::Tensor>& weights) {
  TORCH_CHECK(logits.is_cuda() && logits.is_contiguous() && labels.is_contiguous() && labels.scalar_type() == at::kFloat);
  TORCH_CHECK(logits.numel() == labels.numel());
  const int64_t N = logits.numel();
  c10::cuda::CUDAGuard guard(logits.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  auto f32 = logits.options().dtype(at::kFloat);
  at::Tensor grad = at::empty(logits.sizes(), f32);
  at::Tensor loss = at::zeros({}, f32);
  if (N == 0) return {loss, grad};
  const int threads = 256;
  const int blocks = int(std::min<int64_t>((N + threads - 1) / threads, 148 * 4));
  at::Tensor ws = at::zeros({blocks + 1}, f32);  // partials + the arrival counter
  const float* wp = nullptr;
  if (weights.has_value() && weights->defined()) {
    TORCH_CHECK(weights->scalar_type() == at::kFloat && weights->is_contiguous() && weights->numel() == N);
    wp = weights->data_ptr<float>();
  }
  auto run = [&](auto tag) {
    using T = decltype(tag);
    bce_fwd_bwd_kernel<T><<<blocks, threads, 0, stream>>>(reinterpret_cast<const T*>(logits.data_ptr()), labels.data_ptr<float>(), wp, grad.data_ptr<float>(),
                                                         ws.data_ptr<float>(), reinterpret_cast<unsigned int*>(ws.data_ptr<float>() + blocks), loss.data_ptr<float>(), N);
  };
  if (logits.scalar_type() == at::kFloat) run(float(0));
  else if (logits.scalar_type() == at::kHalf) run(__half());
  else if (logits.scalar_type() == at::kBFloat16) run(__nv_bfloat16());
  else TORCH_CHECK(false, "bce_with_logits_fwd_bwd: unsupported dtype ", logits.scalar_type());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {loss, grad};
}

// ================================================================================================
// multi-probe zero-collision hash.
//
// ``identities[S]`` holds the id stored in every slot (-1 = empty); ``metadata[S]`` (optional) the eviction score of the
// slot: expiry hour (TTL policy) or last access (LRU policy); empty slots carry INT32_MAX so that a slot that has just been
// claimed but whose score has not been written yet can never be evicted.  The slots are cut into buckets by ``segments``
// (global boundaries, ``num_buckets + 1`` entries); this rank owns the slots ``[out_offset, out_offset + S)``.  An id probes
// only inside its bucket, linearly and circularly from ``mix(id) % bucket_size``, at most ``max_probe`` slots.
//
// Two launches: (1) lookup -- hits get their slot and refresh the slot's score; (2) insert -- the misses claim an empty slot
// (CAS on the identity) or evict an expired one (CAS on the score first: only the thread that wins the score owns the
// eviction).  Because every hit of the batch refreshed its score before any insertion starts, an id that occurs in the batch is
// never evicted by the same batch.  No loop waits on another thread: every loop is bounded by ``max_probe``.
// ================================================================================================
struct ZchArgs {
  const int64_t* ids;
  int64_t* identities;
  int32_t* metadata;          // may be null
  const int64_t* segments;    // [num_buckets + 1]
  const int32_t* input_meta;  // may be null: score to write for each id
  int64_t* slots;             // out: local slot, -1 = none
  int64_t* evicted;           // out: local slot whose previous id was evicted by this entry, else -1
  int64_t N, S, num_buckets, input_hash_size, out_offset;
  int64_t reserved;           // slots at the end of every bucket that are never claimed: the shared rows of ids that were not admitted
  int max_probe, policy, eviction_threshold;
  bool disable_fallback;
};

__device__ __forceinline__ bool zch_range(const ZchArgs& a, int64_t id, int64_t& lo, int64_t& size, int64_t& start) {
  const int64_t b = zch_bucket(id, a.input_hash_size, a.num_buckets);
  lo = a.segments[b] - a.out_offset;
  const int64_t hi = a.segments[b + 1] - a.out_offset;
  if (lo < 0 || hi > a.S || hi <= lo) return false;  // the bucket is not on this rank
  size = hi - lo;
  if (a.reserved > 0 && a.reserved < size) size -= a.reserved;  // ids probe (and claim) only the part in front of the reserved block
  start = int64_t(zch_mix(uint64_t(id)) % uint64_t(size));
  return true;
}

__global__ void __launch_bounds__(256) zch_lookup_kernel(ZchArgs a) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= a.N) return;
  const int64_t id = a.ids[i];
  int64_t lo, size, start, found = -1;
  if (zch_range(a, id, lo, size, start)) {
    const int probes = int(a.max_probe < size ? int64_t(a.max_probe) : size);
    for (int p = 0; p < probes; ++p) {
      int64_t s = start + p;
      if (s >= size) s -= size;
      const int64_t cur = __ldcg(a.identities + lo + s);
      if (cur == id) { found = lo + s; break; }
      if (cur == -1) break;
    }
    if (found >= 0 && a.metadata != nullptr && a.input_meta != nullptr) atomicMax(a.metadata + found, a.input_meta[i]);
  }
  a.slots[i] = found;
  a.evicted[i] = -1;
}

__global__ void __launch_bounds__(256) zch_insert_kernel(ZchArgs a) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= a.N || a.slots[i] >= 0) return;
  const int64_t id = a.ids[i];
  int64_t lo, size, start;
  if (!zch_range(a, id, lo, size, start)) return;
  using ull = unsigned long long;
  const int32_t fresh = a.input_meta ? a.input_meta[i] : 0;
  const int probes = int(a.max_probe < size ? int64_t(a.max_probe) : size);
  int64_t found = -1, victim = -1;
  int32_t lru_meta = INT32_MAX;
  int64_t lru_slot = -1;
  for (int p = 0; p < probes && found < 0; ++p) {
    int64_t s = start + p;
    if (s >= size) s -= size;
    s += lo;
    int64_t cur = __ldcg(a.identities + s);
    if (cur == -1) {
      const int64_t seen = int64_t(atomicCAS(reinterpret_cast<ull*>(a.identities + s), ull(-1ll), ull(id)));
      if (seen == -1) {
        found = s;
        if (a.metadata) atomicExch(a.metadata + s, fresh);
        break;
      }
      cur = seen;  // somebody else took it just now
    }
    if (cur == id) { found = s; break; }
    if (a.metadata == nullptr || a.policy == ZCH_NO_EVICT) continue;
    const int32_t m = __ldcg(a.metadata + s);
    if (a.policy == ZCH_TTL) {
      if (m < a.eviction_threshold && atomicCAS(a.metadata + s, m, fresh) == m) {
        atomicExch(reinterpret_cast<ull*>(a.identities + s), ull(id));
        found = s;
        victim = s;
      }
    } else if (m < lru_meta) {
      lru_meta = m;
      lru_slot = s;
    }
  }
  if (found < 0 && a.policy == ZCH_LRU && lru_slot >= 0 && lru_meta < fresh && atomicCAS(a.metadata + lru_slot, lru_meta, fresh) == lru_meta) {
    atomicExch(reinterpret_cast<ull*>(a.identities + lru_slot), ull(id));
    found = lru_slot;
    victim = lru_slot;
  }
  if (found >= 0 && victim < 0 && a.metadata && a.input_meta) atomicMax(a.metadata + found, fresh);
  a.slots[i] = found;
  a.evicted[i] = victim;
}

__global__ void __launch_bounds__(256) zch_fallback_kernel(ZchArgs a) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= a.N || a.slots[i] >= 0 || a.disable_fallback) return;
  int64_t lo, size, start;
  if (!zch_range(a, a.ids[i], lo, size, start)) return;
  const int64_t bucket = a.segments[zch_bucket(a.ids[i], a.input_hash_size, a.num_buckets) + 1] - a.out_offset - lo;
  if (a.reserved > 0 && a.reserved < bucket) a.slots[i] = lo + size + int64_t(zch_mix(uint64_t(a.ids[i])) % uint64_t(a.reserved));  // a reserved row
  else a.slots[i] = lo + start;  // shares the row of whoever lives there
}

std::tuple<at::Tensor, at::Tensor> zch_probe(const at::Tensor& ids, at::Tensor identities, c10::optional<at::Tensor> metadata, const at::Tensor& segments,
                                             int64_t input_hash_size, int64_t out_offset, int64_t max_probe, bool readonly, bool disable_fallback,
                                             const c10::optional<at::Tensor>& input_metadata, int64_t eviction_threshold, int64_t eviction_policy,
                                             int64_t reserved_slots) {
  TORCH_CHECK(ids.is_cuda() && ids.scalar_type() == at::kLong && ids.is_contiguous());
  TORCH_CHECK(identities.is_cuda() && identities.scalar_type() == at::kLong && identities.is_contiguous() && identities.dim() == 1);
  TORCH_CHECK(segments.is_cuda() && segments.scalar_type() == at::kLong && segments.numel() >= 2);
  c10::cuda::CUDAGuard guard(ids.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  ZchArgs a{};
  a.N = ids.numel();
  a.S = identities.numel();
  at::Tensor slots = at::empty({a.N}, ids.options()), evicted = at::empty({a.N}, ids.options());
  if (a.N == 0) return {slots, evicted};
  a.ids = ids.data_ptr<int64_t>();
  a.identities = identities.data_ptr<int64_t>();
  if (metadata.has_value() && metadata->defined()) {
    TORCH_CHECK(metadata->scalar_type() == at::kInt && metadata->numel() == a.S && metadata->is_contiguous());
    a.metadata = metadata->data_ptr<int32_t>();
  }
  if (input_metadata.has_value() && input_metadata->defined()) {
    TORCH_CHECK(input_metadata->scalar_type() == at::kInt && input_metadata->numel() == a.N && input_metadata->is_contiguous());
    a.input_meta = input_metadata->data_ptr<int32_t>();
  }
  a.segments = segments.data_ptr<int64_t>();
  a.slots = slots.data_ptr<int64_t>();
  a.evicted = evicted.data_ptr<int64_t>();
  a.num_buckets = segments.numel() - 1;
  a.input_hash_size = input_hash_size;
  a.out_offset = out_offset;
  a.max_probe = int(std::max<int64_t>(1, max_probe));
  a.policy = int(eviction_policy);
  a.eviction_threshold = int(eviction_threshold);
  a.disable_fallback = disable_fallback;
  a.reserved = std::max<int64_t>(0, reserved_slots);
  const int threads = 256;
  const int blocks = int((a.N + threads - 1) / threads);
  zch_lookup_kernel<<<blocks, threads, 0, stream>>>(a);
  if (!readonly) zch_insert_kernel<<<blocks, threads, 0, stream>>>(a);
  if (!disable_fallback) zch_fallback_kernel<<<blocks, threads, 0, stream>>>(a);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {slots, evicted};
}

// ================================================================================================
// in-training pruning: remap the ids of the pruned tables through ``address_lookup`` and count the accesses.
// ``feature_offsets[F+1]`` cuts ``values`` into features, ``feature_buffer[F]`` names the pruning buffer of the feature
// (-1 = the feature's table is not pruned), ``buffer_offsets`` locates each buffer in ``address_lookup`` / ``row_util``.
// An entry v of address_lookup is the row itself (v >= 0: the id owns that row) or -(row+1) (the id shares a row).
// ================================================================================================
__global__ void __launch_bounds__(256) itep_remap_kernel(const int64_t* __restrict__ values, int64_t N, const int64_t* __restrict__ feature_offsets,
                                                         const int32_t* __restrict__ feature_buffer, int F, const int64_t* __restrict__ address_lookup,
                                                         float* __restrict__ row_util, const int64_t* __restrict__ buffer_offsets, bool update_util,
                                                         int64_t* __restrict__ out) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= N) return;
  int lo = 0, hi = F;  // last feature whose offset is <= i
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (feature_offsets[mid] <= i) lo = mid; else hi = mid;
  }
  const int buf = feature_buffer[lo];
  const int64_t v = values[i];
  if (buf < 0) { out[i] = v; return; }
  const int64_t base = buffer_offsets[buf], size = buffer_offsets[buf + 1] - base;
  if (v < 0 || v >= size) { out[i] = v; return; }
  const int64_t e = address_lookup[base + v];
  out[i] = e >= 0 ? e : -(e + 1);
  if (update_util) atomicAdd(row_util + base + v, 1.f);
}

at::Tensor itep_remap(const at::Tensor& values, const at::Tensor& feature_offsets, const at::Tensor& feature_buffer, const at::Tensor& address_lookup,
                      at::Tensor row_util, const at::Tensor& buffer_offsets, bool update_util) {
  TORCH_CHECK(values.is_cuda() && values.scalar_type() == at::kLong && values.is_contiguous());
  TORCH_CHECK(feature_offsets.scalar_type() == at::kLong && feature_buffer.scalar_type() == at::kInt && feature_offsets.numel() == feature_buffer.numel() + 1);
  TORCH_CHECK(address_lookup.scalar_type() == at::kLong && row_util.scalar_type() == at::kFloat && buffer_offsets.scalar_type() == at::kLong);
  c10::cuda::CUDAGuard guard(values.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  at::Tensor out = at::empty_like(values);
  const int64_t N = values.numel();
  if (N == 0 || feature_buffer.numel() == 0) return values.clone();
  itep_remap_kernel<<<int((N + 255) / 256), 256, 0, stream>>>(values.data_ptr<int64_t>(), N, feature_offsets.data_ptr<int64_t>(), feature_buffer.data_ptr<int32_t>(),
                                                            int(feature_buffer.numel()), address_lookup.data_ptr<int64_t>(), row_util.data_ptr<float>(),
                                                            buffer_offsets.data_ptr<int64_t>(), update_util, out.data_ptr<int64_t>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

// ================================================================================================
// keyed-tensor regroup: every destination column block is the sum of ``n_src`` source column blocks.
// Forward: destinations are the groups, one source each.  Backward: destinations are the input gradients, sources are the
// blocks of the group gradients that read them (none -> zeros, several -> summed in a fixed order).
// One launch for any number of tensors: pointers and row strides travel in the kernel parameters.
// ================================================================================================
constexpr int kRegroupMaxTensors = 32;
struct RegroupPtrs {
  const void* src[kRegroupMaxTensors];
  void* dst[kRegroupMaxTensors];
  int64_t src_stride[kRegroupMaxTensors];
  int64_t dst_stride[kRegroupMaxTensors];
};

template <typename T>
__global__ void __launch_bounds__(256) regroup_kernel(RegroupPtrs p, const int32_t* __restrict__ desc, const int32_t* __restrict__ srcs, int64_t B, int rows_per_block) {
  const int32_t* d = desc + 5 * blockIdx.x;
  const int dst_t = d[0], dst_off = d[1], len = d[2], src_begin = d[3], n_src = d[4];
  const int64_t row0 = int64_t(blockIdx.y) * rows_per_block;
  const int64_t rows = (B - row0 < rows_per_block ? B - row0 : int64_t(rows_per_block));
  T* dst = reinterpret_cast<T*>(p.dst[dst_t]);
  const int64_t total = rows * len;
  for (int64_t e = threadIdx.x; e < total; e += blockDim.x) {
    const int64_t r = row0 + e / len;
    const int c = int(e % len);
    float acc = 0.f;
    T single = T(0);
    for (int s = 0; s < n_src; ++s) {
      const int st = srcs[2 * (src_begin + s)], so = srcs[2 * (src_begin + s) + 1];
      const T v = reinterpret_cast<const T*>(p.src[st])[r * p.src_stride[st] + so + c];
      single = v;
      acc += to_f32(v);
    }
    T o;
    if (n_src == 1) o = single;  // bit-exact copy
    else if constexpr (std::is_same<T, float>::value) o = acc;
    else if constexpr (std::is_same<T, __half>::value) o = __float2half_rn(acc);
    else o = __float2bfloat16_rn(acc);
    dst[r * p.dst_stride[dst_t] + dst_off + c] = o;
  }
}

// ``srcs_t``: source tensors [B, *]; ``dst_widths``: widths of the destination tensors; ``desc`` int32 [n, 5] and ``srcs`` int32 [m, 2] on the device.
std::vector<at::Tensor> kt_regroup(const std::vector<at::Tensor>& srcs_t, std::vector<int64_t> dst_widths, const at::Tensor& desc, const at::Tensor& srcs) {
  TORCH_CHECK(!srcs_t.empty() && srcs_t.size() <= size_t(kRegroupMaxTensors) && dst_widths.size() <= size_t(kRegroupMaxTensors), "kt_regroup: at most 32 tensors on each side");
  TORCH_CHECK(desc.is_cuda() && desc.scalar_type() == at::kInt && desc.dim() == 2 && desc.size(1) == 5 && desc.is_contiguous());
  TORCH_CHECK(srcs.scalar_type() == at::kInt && srcs.is_contiguous());
  const at::Tensor& first = srcs_t[0];
  c10::cuda::CUDAGuard guard(first.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const int64_t B = first.size(0);
  RegroupPtrs p{};
  for (size_t i = 0; i < srcs_t.size(); ++i) {
    const at::Tensor& t = srcs_t[i];
    TORCH_CHECK(t.is_cuda() && t.dim() == 2 && t.size(0) == B && t.stride(1) == 1 && t.scalar_type() == first.scalar_type(), "kt_regroup: inputs must be [B, *] with unit column stride and one dtype");
    p.src[i] = t.data_ptr();
    p.src_stride[i] = t.stride(0);
  }
  std::vector<at::Tensor> outs;
  for (size_t i = 0; i < dst_widths.size(); ++i) {
    outs.push_back(at::empty({B, dst_widths[i]}, first.options()));
    p.dst[i] = outs.back().data_ptr();
    p.dst_stride[i] = dst_widths[i];
  }
  const int n = int(desc.size(0));
  if (n == 0 || B == 0) return outs;
  const int rows_per_block = 32;
  dim3 grid(n, unsigned((B + rows_per_block - 1) / rows_per_block));
  TORCH_CHECK(grid.y <= 65535, "kt_regroup: batch too large for one launch");
  if (first.scalar_type() == at::kFloat) regroup_kernel<float><<<grid, 256, 0, stream>>>(p, desc.data_ptr<int32_t>(), srcs.data_ptr<int32_t>(), B, rows_per_block);
  else if (first.scalar_type() == at::kHalf) regroup_kernel<__half><<<grid, 256, 0, stream>>>(p, desc.data_ptr<int32_t>(), srcs.data_ptr<int32_t>(), B, rows_per_block);
  else if (first.scalar_type() == at::kBFloat16) regroup_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(p, desc.data_ptr<int32_t>(), srcs.data_ptr<int32_t>(), B, rows_per_block);
  else TORCH_CHECK(false, "kt_regroup: unsupported dtype ", first.scalar_type());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return outs;
}

}  // namespace trb

TORCH_LIBRARY_FRAGMENT(trb200, m) {
  m.def("rowwise_quantize_nbit(Tensor w, int bits) -> Tensor");
  m.def("bce_with_logits_fwd_bwd(Tensor logits, Tensor labels, Tensor? weights) -> (Tensor, Tensor)");
  m.def(
      "zch_probe(Tensor ids, Tensor(a!) identities, Tensor(b!)? metadata, Tensor segments, int input_hash_size, int out_offset, int max_probe, bool readonly, "
      "bool disable_fallback, Tensor? input_metadata, int eviction_threshold, int eviction_policy, int reserved_slots=0) -> (Tensor, Tensor)");
  m.def("itep_remap(Tensor values, Tensor feature_offsets, Tensor feature_buffer, Tensor address_lookup, Tensor(a!) row_util, Tensor buffer_offsets, bool update_util) -> Tensor");
  m.def("kt_regroup(Tensor[] srcs, int[] dst_widths, Tensor desc, Tensor src_list) -> Tensor[]");
}

TORCH_LIBRARY_IMPL(trb200, CUDA, m) {
  m.impl("rowwise_quantize_nbit", &trb::rowwise_quantize_nbit);
  m.impl("bce_with_logits_fwd_bwd", &trb::bce_with_logits_fwd_bwd);
  m.impl("zch_probe", &trb::zch_probe);
  m.impl("itep_remap", &trb::itep_remap);
  m.impl("kt_regroup", &trb::kt_regroup);
}
