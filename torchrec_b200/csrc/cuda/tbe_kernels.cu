// Table-batched embedding (TBE) kernels for sm_100a.
//
//   tbe_forward          pooled lookup (sum / mean / weighted), one warp per bag, 16-byte row slices
//                        per lane, fp32 accumulation.  The pooled bag is written straight into the
//                        buffer of the rank that owns the sample: `out[dst_rank][b_local, col]` where
//                        the buffers are peer-mapped (NVLink) pointers.  With one rank this is a plain
//                        local store.  In accumulate mode (row-wise sharding) the partial sum is added
//                        into the owner's fp32 buffer with a vector `red`, which is the reduce-scatter.
//   tbe_sequence_forward unpooled lookup, one warp per bag writing one row per id.
//   tbe_backward         gradient of either lookup fused with the optimizer update.  Ids are sorted by
//                        global row (cub radix sort), the sorted list is cut into fixed blocks of
//                        kBlk entries and one warp walks each block, summing the upstream gradient rows
//                        of equal ids in registers.  A row whose entries lie inside one block is
//                        updated immediately; rows that span blocks (hot ids of a Zipf distribution)
//                        leave partial sums in scratch that a second pass combines in a fixed order,
//                        so the update is deterministic.  No [ids, D] gradient tensor is materialised.
//
// The reference obtains these from an external wheel (call sites
// torchrec/distributed/batched_embedding_kernel.py:2561-2584, :3211-3231).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <torch/library.h>

#include <cub/cub.cuh>

#include "common.cuh"

namespace trb {

// per-feature metadata rows of the int64 [kMetaRows, F] tensor
enum MetaRow : int { M_WOFF = 0, M_HASHOFF = 1, M_ROWS = 2, M_DIM = 3, M_OUTOFF = 4, kMetaRows = 5 };

enum Pooling : int { POOL_SUM = 0, POOL_MEAN = 1, POOL_NONE = 2 };

enum OptType : int {
  OPT_SGD = 0,
  OPT_ROWWISE_ADAGRAD = 1,
  OPT_ADAGRAD = 2,
  OPT_ADAM = 3,
  OPT_PARTIAL_ROWWISE_ADAM = 4,
  OPT_LARS_SGD = 5,
  OPT_LAMB = 6,
  OPT_PARTIAL_ROWWISE_LAMB = 7,
  OPT_DENSE_GRAD = 100,  // write the summed gradient into a dense buffer instead of updating
};

struct FwdParams {
  const void* weights;
  const int64_t* meta;  // [kMetaRows, F]
  const void* indices;
  const void* offsets;
  const float* psw;  // per-sample weights or null
  PeerPtrs out;      // output buffer on every destination rank
  int out_dtype;
  int64_t out_stride;  // elements per output row
  int B;               // bags per feature handled here
  int B_local;         // bags per feature per destination rank
  int F;
  int pooling;
  int accumulate;  // 1: add fp32 partial sums into the destination (row-wise reduce-scatter)
  int skip_empty;  // 1: do not touch the destination for an empty bag (accumulate mode)
  int* err;
};

template <typename emb_t, typename idx_t, int kVecs>
__global__ void __launch_bounds__(256) tbe_fwd_kernel(FwdParams p) {
  constexpr int kUnroll = kVecs <= 2 ? 4 : (kVecs == 4 ? 2 : 1);
  const int lane = threadIdx.x & 31;
  const int64_t bag = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nbags = int64_t(p.F) * p.B;
  if (bag >= nbags) return;
  const int f = int(bag / p.B);
  const int b = int(bag - int64_t(f) * p.B);
  const idx_t* offsets = reinterpret_cast<const idx_t*>(p.offsets);
  const idx_t* indices = reinterpret_cast<const idx_t*>(p.indices);
  const int64_t start = offsets[bag], end = offsets[bag + 1];
  const int F = p.F;
  const int D = int(p.meta[M_DIM * F + f]);
  const int64_t rows = p.meta[M_ROWS * F + f];
  const emb_t* w = reinterpret_cast<const emb_t*>(p.weights) + p.meta[M_WOFF * F + f];
  const int out_off = int(p.meta[M_OUTOFF * F + f]);

  float4 acc[kVecs];
#pragma unroll
  for (int v = 0; v < kVecs; ++v) acc[v] = f4zero();

  for (int64_t i0 = start; i0 < end; i0 += 32) {
    const int cnt = int(min(int64_t(32), end - i0));
    int64_t my_idx = 0;
    float my_w = 0.f;
    if (lane < cnt) {
      my_idx = int64_t(indices[i0 + lane]);
      my_w = p.psw ? p.psw[i0 + lane] : 1.f;
      if (my_idx < 0 || my_idx >= rows) {
        atomicExch(p.err, 1);
        my_idx = 0;
        my_w = 0.f;
      }
    }
    for (int j = 0; j < cnt; j += kUnroll) {
      int64_t r[kUnroll];
      float ww[kUnroll];
      float4 v[kUnroll][kVecs];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int src = min(j + u, cnt - 1);
        r[u] = __shfl_sync(0xffffffffu, my_idx, src);
        ww[u] = __shfl_sync(0xffffffffu, my_w, src);
        if (j + u >= cnt) ww[u] = 0.f;
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
        for (int vv = 0; vv < kVecs; ++vv) {
          const int e = vv * 128 + lane * 4;
          v[u][vv] = (e < D) ? Vec4<emb_t>::load(w + r[u] * D + e) : f4zero();
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
        for (int vv = 0; vv < kVecs; ++vv) {
          acc[vv].x = fmaf(ww[u], v[u][vv].x, acc[vv].x);
          acc[vv].y = fmaf(ww[u], v[u][vv].y, acc[vv].y);
          acc[vv].z = fmaf(ww[u], v[u][vv].z, acc[vv].z);
          acc[vv].w = fmaf(ww[u], v[u][vv].w, acc[vv].w);
        }
      }
    }
  }
  if (p.pooling == POOL_MEAN && end > start) {
    const float s = 1.f / float(end - start);
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      acc[v].x *= s; acc[v].y *= s; acc[v].z *= s; acc[v].w *= s;
    }
  }
  if (p.accumulate && p.skip_empty && end == start) return;
  const int dst = b / p.B_local;
  const int bl = b - dst * p.B_local;
  void* base = p.out.p[dst];
  const int64_t row_e = int64_t(bl) * p.out_stride + out_off;
#pragma unroll
  for (int v = 0; v < kVecs; ++v) {
    const int e = v * 128 + lane * 4;
    if (e < D) {
      if (p.accumulate) {
        red_add_f32x4(reinterpret_cast<float*>(base) + row_e + e, acc[v]);
      } else {
        store4_dyn(base, row_e + e, acc[v], p.out_dtype);
      }
    }
  }
}

// unpooled: out[i, :] = W[idx_i].  One warp per group of kSeqPer consecutive ids, independent of how the ids are cut into
// bags (a single bag may hold most of a batch); the feature of an id is found by a search over the F+1 feature boundaries.
constexpr int kSeqPer = 8;
template <typename emb_t, typename idx_t, int kVecs>
__global__ void __launch_bounds__(256) tbe_seq_fwd_kernel(FwdParams p, int64_t N) {
  const int lane = threadIdx.x & 31;
  const int64_t i0 = ((int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5) * kSeqPer;
  if (i0 >= N) return;
  const idx_t* offsets = reinterpret_cast<const idx_t*>(p.offsets);
  const idx_t* indices = reinterpret_cast<const idx_t*>(p.indices);
  const int F = p.F;
  const int64_t B = p.B;
  const int cnt = int(min(int64_t(kSeqPer), N - i0));
  int64_t my_idx = lane < cnt ? int64_t(indices[i0 + lane]) : 0;
  // last feature whose first id is <= i0 (features may be empty)
  int lo = 0, hi = F;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (int64_t(offsets[int64_t(mid) * B]) <= i0) lo = mid; else hi = mid;
  }
  int f = lo;
  int64_t f_end = int64_t(offsets[int64_t(f + 1) * B]);
  void* base = p.out.p[0];
  for (int j = 0; j < cnt; ++j) {
    const int64_t i = i0 + j;
    while (i >= f_end && f + 1 < F) {
      ++f;
      f_end = int64_t(offsets[int64_t(f + 1) * B]);
    }
    const int D = int(p.meta[M_DIM * F + f]);
    const int64_t rows = p.meta[M_ROWS * F + f];
    const emb_t* w = reinterpret_cast<const emb_t*>(p.weights) + p.meta[M_WOFF * F + f];
    const int64_t r = __shfl_sync(0xffffffffu, my_idx, j);
    const bool rok = r >= 0 && r < rows;
    if (!rok && lane == 0) atomicExch(p.err, 1);
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      const int e = v * 128 + lane * 4;
      if (e < D) {
        float4 x = rok ? Vec4<emb_t>::load(w + r * D + e) : f4zero();
        store4_dyn(base, i * p.out_stride + e, x, p.out_dtype);
      }
    }
  }
}

// Unpooled lookup whose ids arrived through the fused input distribution: id k of the receive buffer carries a return
// address `ret[k]` = (requesting rank << 32 | position of the id in that rank's KJT), and its row is stored straight into
// row `position` of the requester's output buffer (peer-mapped), at this table's output column.  This is the sequence
// all-to-all folded into the lookup.  Only positions [offsets[0], offsets[F * B]) of the buffer belong to this module.
template <typename emb_t, typename idx_t, int kVecs>
__global__ void __launch_bounds__(256) tbe_seq_fwd_dist_kernel(FwdParams p, const int64_t* __restrict__ ret, int64_t out_rows, int nranks) {
  const int lane = threadIdx.x & 31;
  const idx_t* offsets = reinterpret_cast<const idx_t*>(p.offsets);
  const idx_t* indices = reinterpret_cast<const idx_t*>(p.indices);
  const int F = p.F;
  const int64_t B = p.B;
  const int64_t first = int64_t(offsets[0]), last = int64_t(offsets[int64_t(F) * B]);
  const int64_t i0 = first + ((int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5) * kSeqPer;
  if (i0 >= last) return;
  const int cnt = int(min(int64_t(kSeqPer), last - i0));
  int64_t my_idx = 0, my_ret = 0;
  if (lane < cnt) {
    my_idx = int64_t(indices[i0 + lane]);
    my_ret = ret[i0 + lane];
  }
  int lo = 0, hi = F;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (int64_t(offsets[int64_t(mid) * B]) <= i0) lo = mid; else hi = mid;
  }
  int f = lo;
  int64_t f_end = int64_t(offsets[int64_t(f + 1) * B]);
  for (int j = 0; j < cnt; ++j) {
    const int64_t i = i0 + j;
    while (i >= f_end && f + 1 < F) {
      ++f;
      f_end = int64_t(offsets[int64_t(f + 1) * B]);
    }
    const int D = int(p.meta[M_DIM * F + f]);
    const int64_t rows = p.meta[M_ROWS * F + f];
    const int64_t col = p.meta[M_OUTOFF * F + f];
    const emb_t* w = reinterpret_cast<const emb_t*>(p.weights) + p.meta[M_WOFF * F + f];
    const int64_t r = __shfl_sync(0xffffffffu, my_idx, j);
    const int64_t ra = __shfl_sync(0xffffffffu, my_ret, j);
    const bool rok = r >= 0 && r < rows;
    if (!rok && lane == 0) atomicExch(p.err, 1);
    const int64_t dst_rank = ra >> 32, dst_row = ra & 0xffffffffLL;
    if (dst_rank < 0 || dst_rank >= nranks || dst_row >= out_rows) {  // never store outside a peer's buffer
      if (lane == 0) atomicExch(p.err, 2);
      continue;
    }
    void* base = p.out.p[int(dst_rank)];
    const int64_t row_e = dst_row * p.out_stride + col;
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      const int e = v * 128 + lane * 4;
      if (e < D) {
        float4 x = rok ? Vec4<emb_t>::load(w + r * D + e) : f4zero();
        store4_dyn(base, row_e + e, x, p.out_dtype);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// backward
// ------------------------------------------------------------------------------------------------
struct OptParams {
  int type;
  int stochastic_rounding;  // fp16 / bf16 tables: round the updated weights up or down at random, unbiased in expectation
  const int64_t* sr_counter;  // device-side call counter that salts the random bits (a replayed CUDA graph keeps host values frozen)
  float lr, eps, beta1, beta2, weight_decay;
  float bias_corr1, bias_corr2;  // 1 - beta^t
  float max_grad;                // > 0: clamp the summed gradient elementwise
};

struct BwdParams {
  void* weights;
  float* mom1;
  float* mom2;
  float* dense_grad;    // OPT_DENSE_GRAD target (same layout as weights, fp32)
  const int64_t* meta;  // [kMetaRows, F]
  const int64_t* sorted_keys;  // [N] global row ids, ascending
  const int32_t* sorted_src;   // [N] pooled: bag id (f*B+b); unpooled: position of the id
  const float* sorted_w;       // [N] per-sample weights in sorted order, or null
  const int32_t* src_feature;  // unpooled only: feature of every position (null when pooled)
  const void* grad;            // upstream gradient rows
  int grad_dtype;
  int64_t grad_stride;
  const float* bag_scale;  // mean pooling: 1/len per bag, or null
  int64_t N;
  const int64_t* n_valid;  // device-side count of valid sorted entries (the tail holds padding keys), or null: all N are valid
  int B;
  int F;
  int pooled;
  float* partials;  // [2*nblocks, Dpad] fp32 scratch
  int32_t* flags;   // [2*nblocks]  slot state, see below
  int64_t* long_list;  // [2*cap] (head block, last block) of chains left to pass 3
  int* long_count;
  int Dpad;
  // pooled gradients that live on peer ranks (fused exchange): bag b of the global batch is row b % B_local of
  // rank b / B_local.  B_local == 0: all gradient rows are in `grad`.
  PeerPtrs grad_peers;
  const int64_t* ret;  // unpooled, fused exchange: return address of every received id (see tbe_seq_fwd_dist_kernel); gradient rows
                       // are pulled from row `position` of the requesting rank's gradient buffer
  int B_local;
  float grad_scale;  // factor on every gradient row (1 / world size when gradients are averaged over ranks)
  OptParams opt;
};

constexpr int kBlk = 64;        // sorted entries per warp
constexpr int FLAG_USED = 1;    // slot holds a partial sum
constexpr int FLAG_CONT = 2;    // (slot A only) the row continues into the next block

// ---- stochastic rounding of updated weights (16-bit tables) --------------------------------------------------------
// Rounding to nearest loses every update smaller than half a unit in the last place, which stalls training of fp16 / bf16
// tables with small learning rates.  Rounding up with probability equal to the discarded fraction keeps the expectation.
// The random bits come from a hash of (row, element, value, a call counter kept on the device): a host-side seed would be
// frozen by a replayed CUDA graph, and a hash of the value alone would give a weight that was rounded back to where it
// started the same bits again at the next step.
__device__ __forceinline__ uint32_t sr_hash(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}
__device__ __forceinline__ __nv_bfloat16 sr_bf16(float x, uint32_t salt) {
  const uint32_t bits = __float_as_uint(x);
  if ((bits & 0x7f800000u) == 0x7f800000u) return __float2bfloat16(x);  // inf / nan
  const uint32_t r = sr_hash(bits ^ salt) & 0xffffu;
  return __ushort_as_bfloat16((unsigned short)((bits + r) >> 16));
}
__device__ __forceinline__ __half sr_f16(float x, uint32_t salt) {
  const uint32_t bits = __float_as_uint(x);
  if ((bits & 0x7f800000u) == 0x7f800000u) return __float2half(x);
  const uint32_t r = sr_hash(bits ^ salt) & 0x1fffu;  // fp32 keeps 13 more mantissa bits than fp16
  return __float2half_rz(__uint_as_float(bits + r));
}
template <typename emb_t>
__device__ __forceinline__ void store4_stochastic(emb_t* p, float4 v, uint32_t salt) { Vec4<emb_t>::store(p, v); }
template <>
__device__ __forceinline__ void store4_stochastic<__nv_bfloat16>(__nv_bfloat16* p, float4 v, uint32_t salt) {
  p[0] = sr_bf16(v.x, salt); p[1] = sr_bf16(v.y, salt + 1); p[2] = sr_bf16(v.z, salt + 2); p[3] = sr_bf16(v.w, salt + 3);
}
template <>
__device__ __forceinline__ void store4_stochastic<__half>(__half* p, float4 v, uint32_t salt) {
  p[0] = sr_f16(v.x, salt); p[1] = sr_f16(v.y, salt + 1); p[2] = sr_f16(v.z, salt + 2); p[3] = sr_f16(v.w, salt + 3);
}

// Optimizer update of one table row.  `g` is the summed gradient of the row, `w` the row's current weights and
// `mpre` (lane 0) its row-wise Adagrad state, both already loaded by the caller so that their latency overlaps
// with the gradient gather.
template <typename emb_t, int kVecs>
__device__ __forceinline__ void apply_update_core(const BwdParams& p, int64_t key, int64_t woff, int D, float4 (&g)[kVecs],
                                                  float4 (&w)[kVecs], float mpre, int lane) {
  const OptParams& o = p.opt;
  if (o.max_grad > 0.f) {
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      g[v].x = fminf(fmaxf(g[v].x, -o.max_grad), o.max_grad);
      g[v].y = fminf(fmaxf(g[v].y, -o.max_grad), o.max_grad);
      g[v].z = fminf(fmaxf(g[v].z, -o.max_grad), o.max_grad);
      g[v].w = fminf(fmaxf(g[v].w, -o.max_grad), o.max_grad);
    }
  }
  if (o.type == OPT_DENSE_GRAD) {
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      const int e = v * 128 + lane * 4;
      if (e < D) Vec4<float>::store(p.dense_grad + woff + e, g[v]);
    }
    return;
  }
  emb_t* wp = reinterpret_cast<emb_t*>(p.weights) + woff;
  if (o.weight_decay != 0.f && o.type != OPT_LAMB && o.type != OPT_PARTIAL_ROWWISE_LAMB) {
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      g[v].x = fmaf(o.weight_decay, w[v].x, g[v].x);
      g[v].y = fmaf(o.weight_decay, w[v].y, g[v].y);
      g[v].z = fmaf(o.weight_decay, w[v].z, g[v].z);
      g[v].w = fmaf(o.weight_decay, w[v].w, g[v].w);
    }
  }
  auto sumsq = [&](float4 (&x)[kVecs]) {
    float s = 0.f;
#pragma unroll
    for (int v = 0; v < kVecs; ++v) s += x[v].x * x[v].x + x[v].y * x[v].y + x[v].z * x[v].z + x[v].w * x[v].w;
    return warp_sum(s);
  };
  switch (o.type) {
    case OPT_SGD: {
#pragma unroll
      for (int v = 0; v < kVecs; ++v) {
        w[v].x -= o.lr * g[v].x; w[v].y -= o.lr * g[v].y; w[v].z -= o.lr * g[v].z; w[v].w -= o.lr * g[v].w;
      }
      break;
    }
    case OPT_LARS_SGD: {
      const float wn = sqrtf(sumsq(w)), gn = sqrtf(sumsq(g));
      const float trust = (wn > 0.f && gn > 0.f) ? o.eps * wn / gn : 1.f;  // eps field carries eta
      const float s = o.lr * trust;
#pragma unroll
      for (int v = 0; v < kVecs; ++v) {
        w[v].x -= s * g[v].x; w[v].y -= s * g[v].y; w[v].z -= s * g[v].z; w[v].w -= s * g[v].w;
      }
      break;
    }
    case OPT_ROWWISE_ADAGRAD: {
      const float g2 = sumsq(g) / float(D);
      float m = 0.f;
      if (lane == 0) {
        m = mpre + g2;
        p.mom1[key] = m;
      }
      m = __shfl_sync(0xffffffffu, m, 0);
      const float s = o.lr / (sqrtf(m) + o.eps);
#pragma unroll
      for (int v = 0; v < kVecs; ++v) {
        w[v].x -= s * g[v].x; w[v].y -= s * g[v].y; w[v].z -= s * g[v].z; w[v].w -= s * g[v].w;
      }
      break;
    }
    case OPT_ADAGRAD: {
#pragma unroll
      for (int v = 0; v < kVecs; ++v) {
        const int e = v * 128 + lane * 4;
        if (e < D) {
          float4 m = Vec4<float>::load_plain(p.mom1 + woff + e);
          m.x += g[v].x * g[v].x; m.y += g[v].y * g[v].y; m.z += g[v].z * g[v].z; m.w += g[v].w * g[v].w;
          Vec4<float>::store(p.mom1 + woff + e, m);
          w[v].x -= o.lr * g[v].x / (sqrtf(m.x) + o.eps);
          w[v].y -= o.lr * g[v].y / (sqrtf(m.y) + o.eps);
          w[v].z -= o.lr * g[v].z / (sqrtf(m.z) + o.eps);
          w[v].w -= o.lr * g[v].w / (sqrtf(m.w) + o.eps);
        }
      }
      break;
    }
    case OPT_ADAM:
    case OPT_PARTIAL_ROWWISE_ADAM:
    case OPT_LAMB:
    case OPT_PARTIAL_ROWWISE_LAMB: {
      const bool rowwise2 = (o.type == OPT_PARTIAL_ROWWISE_ADAM || o.type == OPT_PARTIAL_ROWWISE_LAMB);
      const bool lamb = (o.type == OPT_LAMB || o.type == OPT_PARTIAL_ROWWISE_LAMB);
      float m2row = 0.f;
      if (rowwise2) {
        const float g2 = sumsq(g) / float(D);
        if (lane == 0) {
          m2row = o.beta2 * p.mom2[key] + (1.f - o.beta2) * g2;
          p.mom2[key] = m2row;
        }
        m2row = __shfl_sync(0xffffffffu, m2row, 0);
      }
      float4 upd[kVecs];
#pragma unroll
      for (int v = 0; v < kVecs; ++v) {
        const int e = v * 128 + lane * 4;
        upd[v] = f4zero();
        if (e < D) {
          float4 m1 = Vec4<float>::load_plain(p.mom1 + woff + e);
          m1.x = o.beta1 * m1.x + (1.f - o.beta1) * g[v].x;
          m1.y = o.beta1 * m1.y + (1.f - o.beta1) * g[v].y;
          m1.z = o.beta1 * m1.z + (1.f - o.beta1) * g[v].z;
          m1.w = o.beta1 * m1.w + (1.f - o.beta1) * g[v].w;
          Vec4<float>::store(p.mom1 + woff + e, m1);
          float4 m2;
          if (rowwise2) {
            m2 = make_float4(m2row, m2row, m2row, m2row);
          } else {
            m2 = Vec4<float>::load_plain(p.mom2 + woff + e);
            m2.x = o.beta2 * m2.x + (1.f - o.beta2) * g[v].x * g[v].x;
            m2.y = o.beta2 * m2.y + (1.f - o.beta2) * g[v].y * g[v].y;
            m2.z = o.beta2 * m2.z + (1.f - o.beta2) * g[v].z * g[v].z;
            m2.w = o.beta2 * m2.w + (1.f - o.beta2) * g[v].w * g[v].w;
            Vec4<float>::store(p.mom2 + woff + e, m2);
          }
          const float c1 = 1.f / o.bias_corr1, c2 = 1.f / o.bias_corr2;
          upd[v].x = (m1.x * c1) / (sqrtf(m2.x * c2) + o.eps);
          upd[v].y = (m1.y * c1) / (sqrtf(m2.y * c2) + o.eps);
          upd[v].z = (m1.z * c1) / (sqrtf(m2.z * c2) + o.eps);
          upd[v].w = (m1.w * c1) / (sqrtf(m2.w * c2) + o.eps);
          if (lamb && o.weight_decay != 0.f) {
            upd[v].x = fmaf(o.weight_decay, w[v].x, upd[v].x);
            upd[v].y = fmaf(o.weight_decay, w[v].y, upd[v].y);
            upd[v].z = fmaf(o.weight_decay, w[v].z, upd[v].z);
            upd[v].w = fmaf(o.weight_decay, w[v].w, upd[v].w);
          }
        }
      }
      float s = o.lr;
      if (lamb) {
        const float wn = sqrtf(sumsq(w)), un = sqrtf(sumsq(upd));
        if (wn > 0.f && un > 0.f) s = o.lr * wn / un;
      }
#pragma unroll
      for (int v = 0; v < kVecs; ++v) {
        w[v].x -= s * upd[v].x; w[v].y -= s * upd[v].y; w[v].z -= s * upd[v].z; w[v].w -= s * upd[v].w;
      }
      break;
    }
    default:
      break;
  }
#pragma unroll
  for (int v = 0; v < kVecs; ++v) {
    const int e = v * 128 + lane * 4;
    if (e < D) {
      if (o.stochastic_rounding) store4_stochastic(wp + e, w[v], (uint32_t(key) * 2654435761u + uint32_t(e)) ^ (uint32_t(*o.sr_counter) * 0x9e3779b9u));
      else Vec4<emb_t>::store(wp + e, w[v]);
    }
  }
}

// Loads the row state of the row at element offset `woff` and applies the update.
template <typename emb_t, int kVecs>
__device__ __forceinline__ void apply_update_at(const BwdParams& p, int64_t key, int64_t woff, int D, float4 (&g)[kVecs], int lane) {
  float4 w[kVecs];
  float mpre = 0.f;
  if (p.opt.type != OPT_DENSE_GRAD) {
    const emb_t* wp = reinterpret_cast<const emb_t*>(p.weights) + woff;
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      const int e = v * 128 + lane * 4;
      w[v] = (e < D) ? Vec4<emb_t>::load_plain(wp + e) : f4zero();
    }
    if (p.opt.type == OPT_ROWWISE_ADAGRAD && lane == 0) mpre = p.mom1[key];
  }
  apply_update_core<emb_t, kVecs>(p, key, woff, D, g, w, mpre, lane);
}

template <typename emb_t, int kVecs>
__device__ __forceinline__ void apply_update(const BwdParams& p, int64_t key, int f, float4 (&g)[kVecs], int lane) {
  const int F = p.F;
  const int D = int(p.meta[M_DIM * F + f]);
  const int64_t woff = p.meta[M_WOFF * F + f] + (key - p.meta[M_HASHOFF * F + f]) * D;
  apply_update_at<emb_t, kVecs>(p, key, woff, D, g, lane);
}

template <int kVecs>
__device__ __forceinline__ void store_partial(const BwdParams& p, int64_t slot, float4 (&g)[kVecs], int lane) {
  float* dst = p.partials + slot * p.Dpad;
#pragma unroll
  for (int v = 0; v < kVecs; ++v) {
    const int e = v * 128 + lane * 4;
    if (e < p.Dpad) Vec4<float>::store(dst + e, g[v]);
  }
}

constexpr int kSmemF = 256;  // per-feature metadata is staged in shared memory up to this many features

__device__ __forceinline__ void prefetch_l2_range(const void* ptr, int bytes) {
  const uintptr_t lo = reinterpret_cast<uintptr_t>(ptr) & ~uintptr_t(127);
  const uintptr_t hi = reinterpret_cast<uintptr_t>(ptr) + bytes;
  for (uintptr_t a = lo; a < hi; a += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
}

// pass 1: one warp per block of kBlk sorted entries.
//
// Preamble, one or two entries per lane: everything that depends on one entry only (feature, address of its
// gradient row slice, weight row offset, whether the table row ends at this entry) is computed once and parked in
// shared memory, and the gradient row of every entry plus the weight row (and row-wise state) of every row that
// ends in the block are requested into L2 with prefetches.  That puts the whole block's DRAM traffic in flight at
// once without holding registers.  The walk itself then costs per entry one 16-byte shared-memory broadcast, the
// gradient load (an L2 hit by then) and the multiply-adds.
template <typename emb_t, typename grad_t, int kVecs>
__global__ void __launch_bounds__(256, kVecs == 1 ? 4 : 2) tbe_bwd_block_kernel(BwdParams p) {
  const int64_t N_ = p.n_valid ? min(p.N, *p.n_valid) : p.N;
  __shared__ int64_t s_meta[kMetaRows * kSmemF];
  __shared__ uint4 s_rec[8][kBlk];     // {gradient byte offset lo, hi, weight bits, ctl}; ctl = end | D << 1 | f << 16
  __shared__ int64_t s_woff[8][kBlk];  // element offset of the entry's table row in the weights
  __shared__ int64_t s_key[8][kBlk];
  const int F = p.F;
  const int64_t* __restrict__ meta = p.meta;
  if (F <= kSmemF) {
    for (int i = threadIdx.x; i < kMetaRows * F; i += blockDim.x) s_meta[i] = p.meta[i];
    __syncthreads();
    meta = s_meta;
  }
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const int64_t blk = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t start = blk * kBlk;
  if (start >= N_) return;
  const int n = int(min(int64_t(kBlk), N_ - start));
  const int opt_type = p.opt.type;
  const char* __restrict__ gbase = reinterpret_cast<const char*>(p.grad);

  if (lane == 0) {
    p.flags[2 * blk] = 0;
    p.flags[2 * blk + 1] = 0;
  }
#pragma unroll
  for (int t = 0; t < kBlk / 32; ++t) {
    const int k = t * 32 + lane;
    if (k < n) {
      const int64_t i = start + k;
      const int64_t key = p.sorted_keys[i];
      const int64_t nxt = (i + 1 < N_) ? p.sorted_keys[i + 1] : int64_t(-1);
      int src = p.sorted_src[i];
      float w = p.sorted_w ? p.sorted_w[i] : 1.f;
      if (src < 0) {  // id outside its table: no gradient, no state change (matches the forward, which skipped it)
        src = -src - 1;
        w = 0.f;
      }
      int f;
      int64_t goff;
      const char* gsrc = gbase;
      bool local_grad = true;
      if (p.pooled) {
        f = src / p.B;
        int b = src - f * p.B;
        if (p.B_local > 0) {
          const int owner = b / p.B_local;
          b -= owner * p.B_local;
          gsrc = reinterpret_cast<const char*>(p.grad_peers.p[owner]);
          local_grad = gsrc == gbase;
        }
        goff = int64_t(b) * p.grad_stride + meta[M_OUTOFF * F + f];
        if (p.bag_scale) w *= p.bag_scale[src];
      } else {
        f = p.src_feature[src];
        if (p.ret != nullptr) {
          const int64_t ra = p.ret[src];
          gsrc = reinterpret_cast<const char*>(p.grad_peers.p[int(ra >> 32)]);
          local_grad = gsrc == gbase;
          goff = (ra & 0xffffffffLL) * p.grad_stride + meta[M_OUTOFF * F + f];
        } else {
          goff = int64_t(src) * p.grad_stride;
        }
      }
      w *= p.grad_scale;
      const int D = int(meta[M_DIM * F + f]);
      const int64_t woff = meta[M_WOFF * F + f] + (key - meta[M_HASHOFF * F + f]) * D;
      const bool is_end = key != nxt;
      // the record holds the address of the row slice relative to the local gradient base (peer bases included)
      const int64_t gbyte = (gsrc - gbase) + goff * int64_t(sizeof(grad_t));
      s_rec[wib][k] = make_uint4(uint32_t(uint64_t(gbyte)), uint32_t(uint64_t(gbyte) >> 32), __float_as_uint(w),
                                 uint32_t(is_end ? 1 : 0) | (uint32_t(D) << 1) | (uint32_t(f) << 16));
      s_woff[wib][k] = woff;
      s_key[wib][k] = key;
      if (local_grad) prefetch_l2_range(gbase + gbyte, D * int(sizeof(grad_t)));
      if (is_end && opt_type != OPT_DENSE_GRAD) {
        prefetch_l2_range(reinterpret_cast<const emb_t*>(p.weights) + woff, D * int(sizeof(emb_t)));
        if (opt_type == OPT_ROWWISE_ADAGRAD) prefetch_l2_range(p.mom1 + key, 4);
      }
    }
  }
  __syncwarp();

  float4 acc[kVecs];
#pragma unroll
  for (int v = 0; v < kVecs; ++v) acc[v] = f4zero();
  // does the first row of this block begin in an earlier block?
  bool started_before = (start > 0) && (p.sorted_keys[start - 1] == s_key[wib][0]);
  bool open = false;  // entries accumulated since the last row end
  int cur_f = 0;

  constexpr int kUnroll = kVecs == 1 ? 4 : (kVecs == 2 ? 2 : 1);
  for (int j = 0; j < n; j += kUnroll) {
    uint4 r[kUnroll];
    float4 gv[kUnroll][kVecs];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      r[u] = s_rec[wib][min(j + u, n - 1)];
      const grad_t* gp = reinterpret_cast<const grad_t*>(gbase + (uint64_t(r[u].x) | (uint64_t(r[u].y) << 32)));
      const int D = int(r[u].w >> 1) & 0x7fff;
#pragma unroll
      for (int v = 0; v < kVecs; ++v) {
        const int e = v * 128 + lane * 4;
        gv[u][v] = (e < D) ? Vec4<grad_t>::load_plain(gp + e) : f4zero();
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (j + u < n) {
        const float ww = __uint_as_float(r[u].z);
#pragma unroll
        for (int v = 0; v < kVecs; ++v) {
          acc[v].x = fmaf(ww, gv[u][v].x, acc[v].x);
          acc[v].y = fmaf(ww, gv[u][v].y, acc[v].y);
          acc[v].z = fmaf(ww, gv[u][v].z, acc[v].z);
          acc[v].w = fmaf(ww, gv[u][v].w, acc[v].w);
        }
        open = true;
        cur_f = int(r[u].w >> 16);
        if (r[u].w & 1u) {
          // the row ends here
          if (!started_before) {
            apply_update_at<emb_t, kVecs>(p, s_key[wib][j + u], s_woff[wib][j + u], int(r[u].w >> 1) & 0x7fff, acc, lane);
          } else {
            store_partial<kVecs>(p, 2 * blk, acc, lane);
            if (lane == 0) p.flags[2 * blk] = FLAG_USED;
          }
#pragma unroll
          for (int v = 0; v < kVecs; ++v) acc[v] = f4zero();
          started_before = false;
          open = false;
        }
      }
    }
  }
  if (!open) return;
  // the last row continues in the next block
  if (started_before) {
    // middle of a long row: slot A
    store_partial<kVecs>(p, 2 * blk, acc, lane);
    if (lane == 0) p.flags[2 * blk] = FLAG_USED | FLAG_CONT;
  } else {
    // head of a long row: slot B; remember the feature for the second pass
    store_partial<kVecs>(p, 2 * blk + 1, acc, lane);
    if (lane == 0) p.flags[2 * blk + 1] = FLAG_USED | (cur_f << 8);
  }
}

constexpr int kSerialChain = 16;  // chains of at most this many slots are folded by one warp

__device__ __forceinline__ int64_t upper_bound_key(const int64_t* __restrict__ keys, int64_t lo, int64_t hi, int64_t key) {
  // first position in [lo, hi) whose key is greater than `key` (keys ascending)
  while (lo < hi) {
    const int64_t mid = lo + ((hi - lo) >> 1);
    if (keys[mid] <= key) lo = mid + 1;
    else hi = mid;
  }
  return lo;
}

// pass 2: the head block of every row that spans blocks folds the chain of partial sums.  Short chains are folded
// by the head's warp; long chains (hot rows of a skewed id distribution) are queued for pass 3.
template <typename emb_t, int kVecs>
__global__ void __launch_bounds__(256) tbe_bwd_long_kernel(BwdParams p) {
  const int64_t N_ = p.n_valid ? min(p.N, *p.n_valid) : p.N;
  const int lane = threadIdx.x & 31;
  const int64_t blk = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t nblocks = (N_ + kBlk - 1) / kBlk;
  if (blk >= nblocks) return;
  const int fl = p.flags[2 * blk + 1];
  if (!(fl & FLAG_USED)) return;
  const int f = fl >> 8;
  const int64_t end = min(N_, (blk + 1) * kBlk);
  const int64_t key = p.sorted_keys[end - 1];
  int64_t last_blk = 0;
  if (lane == 0) last_blk = (upper_bound_key(p.sorted_keys, end, N_, key) - 1) / kBlk;
  last_blk = __shfl_sync(0xffffffffu, last_blk, 0);
  if (last_blk - blk > kSerialChain) {
    if (lane == 0) {
      const int slot = atomicAdd(p.long_count, 1);
      p.long_list[2 * slot] = blk;
      p.long_list[2 * slot + 1] = last_blk;
    }
    return;
  }
  float4 acc[kVecs];
  {
    const float* src = p.partials + (2 * blk + 1) * p.Dpad;
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      const int e = v * 128 + lane * 4;
      acc[v] = (e < p.Dpad) ? Vec4<float>::load_plain(src + e) : f4zero();
    }
  }
  for (int64_t j = blk + 1; j <= last_blk; ++j) {
    const float* src = p.partials + (2 * j) * p.Dpad;
#pragma unroll
    for (int v = 0; v < kVecs; ++v) {
      const int e = v * 128 + lane * 4;
      if (e < p.Dpad) {
        float4 x = Vec4<float>::load_plain(src + e);
        acc[v].x += x.x; acc[v].y += x.y; acc[v].z += x.z; acc[v].w += x.w;
      }
    }
  }
  apply_update<emb_t, kVecs>(p, key, f, acc, lane);
}

// pass 3: one CTA per queued long chain.  Warp w sums slots blk+1+w, blk+1+w+8, ... (fixed assignment, so the result
// is deterministic), the eight sums are combined in shared memory in warp order, and warp 0 applies the update.
template <typename emb_t, int kVecs>
__global__ void __launch_bounds__(256) tbe_bwd_verylong_kernel(BwdParams p) {
  const int64_t N_ = p.n_valid ? min(p.N, *p.n_valid) : p.N;
  __shared__ float4 red[8][kVecs][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int count = *p.long_count;
  for (int i = blockIdx.x; i < count; i += gridDim.x) {
    const int64_t blk = p.long_list[2 * i], last_blk = p.long_list[2 * i + 1];
    float4 acc[kVecs];
#pragma unroll
    for (int v = 0; v < kVecs; ++v) acc[v] = f4zero();
    for (int64_t j0 = blk + 1 + warp; j0 <= last_blk; j0 += 32) {
      float4 x[4][kVecs];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t j = j0 + 8 * u;
        const float* src = p.partials + (2 * min(j, last_blk)) * p.Dpad;
#pragma unroll
        for (int v = 0; v < kVecs; ++v) {
          const int e = v * 128 + lane * 4;
          x[u][v] = (j <= last_blk && e < p.Dpad) ? Vec4<float>::load_plain(src + e) : f4zero();
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
#pragma unroll
        for (int v = 0; v < kVecs; ++v) {
          acc[v].x += x[u][v].x; acc[v].y += x[u][v].y; acc[v].z += x[u][v].z; acc[v].w += x[u][v].w;
        }
      }
    }
#pragma unroll
    for (int v = 0; v < kVecs; ++v) red[warp][v][lane] = acc[v];
    __syncthreads();
    if (warp == 0) {
      const float* src = p.partials + (2 * blk + 1) * p.Dpad;  // the head's own partial
#pragma unroll
      for (int v = 0; v < kVecs; ++v) {
        const int e = v * 128 + lane * 4;
        float4 t = (e < p.Dpad) ? Vec4<float>::load_plain(src + e) : f4zero();
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float4 y = red[k][v][lane];
          t.x += y.x; t.y += y.y; t.z += y.z; t.w += y.w;
        }
        acc[v] = t;
      }
      const int f = p.flags[2 * blk + 1] >> 8;
      const int64_t end = min(N_, (blk + 1) * kBlk);
      apply_update<emb_t, kVecs>(p, p.sorted_keys[end - 1], f, acc, lane);
    }
    __syncthreads();
  }
}

// keys: global row id of every id; src: bag id (pooled) or position (unpooled).  kLanes lanes share one bag (32: a warp per bag,
// for long bags; 8: four bags per warp, for the common bags of a handful of ids, where a whole warp would leave most lanes idle)
template <typename idx_t, int kLanes>
__global__ void __launch_bounds__(256) tbe_linearize_kernel(
    const idx_t* __restrict__ indices, const idx_t* __restrict__ offsets, const int64_t* __restrict__ meta, int F, int B,
    int pooled, int64_t* __restrict__ keys, int32_t* __restrict__ src, int32_t* __restrict__ src_feature,
    float* __restrict__ bag_scale, int* err) {
  const int lane = threadIdx.x & (kLanes - 1);
  const int64_t bag = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) / kLanes;
  if (bag >= int64_t(F) * B) return;
  const int f = int(bag / B);
  const int64_t start = offsets[bag], end = offsets[bag + 1];
  const int64_t hoff = meta[M_HASHOFF * F + f];
  const int64_t rows = meta[M_ROWS * F + f];
  if (bag_scale && lane == 0) bag_scale[bag] = end > start ? 1.f / float(end - start) : 0.f;
  for (int64_t i = start + lane; i < end; i += kLanes) {
    int64_t r = int64_t(indices[i]);
    const bool bad = r < 0 || r >= rows;
    if (bad) {
      atomicExch(err, 1);
      r = 0;
    }
    keys[i] = hoff + r;
    // an id outside its table contributed nothing to the forward; a negative source tells the backward to give it weight 0
    const int32_t s = pooled ? int32_t(bag) : int32_t(i);
    src[i] = bad ? -s - 1 : s;
    if (src_feature) src_feature[i] = f;
  }
}

// Unpooled variant: one thread per id, whatever the bag sizes (a single bag may hold most of the ids, e.g. a candidate list), the
// feature of a position found by a search over the F + 1 feature boundaries.
template <typename idx_t>
__global__ void __launch_bounds__(256) tbe_linearize_seq_kernel(const idx_t* __restrict__ indices, const idx_t* __restrict__ offsets,
                                                                const int64_t* __restrict__ meta, int F, int B, int64_t* __restrict__ keys,
                                                                int32_t* __restrict__ src, int32_t* __restrict__ src_feature, int* err) {
  const int64_t first = int64_t(offsets[0]), last = int64_t(offsets[int64_t(F) * B]);
  const int64_t i = first + int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= last) return;
  int lo = 0, hi = F;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (int64_t(offsets[int64_t(mid) * B]) <= i) lo = mid; else hi = mid;
  }
  // features without ids share a boundary: take the last feature that starts at or before i and still has ids there
  int f = lo;
  while (f + 1 < F && int64_t(offsets[int64_t(f + 1) * B]) <= i) ++f;
  int64_t r = int64_t(indices[i]);
  const bool bad = r < 0 || r >= meta[M_ROWS * F + f];
  if (bad) {
    atomicExch(err, 1);
    r = 0;
  }
  keys[i] = meta[M_HASHOFF * F + f] + r;
  src[i] = bad ? -int32_t(i) - 1 : int32_t(i);
  src_feature[i] = f;
}

__global__ void tbe_bump_counter_kernel(int64_t* counter) { counter[0] += 1; }

template <typename idx_t>
__global__ void tbe_count_valid_kernel(const idx_t* __restrict__ offsets, int64_t nbags, int64_t* __restrict__ out) {
  out[0] = int64_t(offsets[nbags]) - int64_t(offsets[0]);
}

__global__ void gather_sorted_weights_kernel(const float* __restrict__ psw, const int32_t* __restrict__ sorted_pos,
                                             const int32_t* __restrict__ bag_of_pos, float* __restrict__ out_w,
                                             int32_t* __restrict__ out_src, int64_t N) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= N) return;
  const int32_t pos = sorted_pos[i];
  out_w[i] = psw[pos];
  out_src[i] = bag_of_pos ? bag_of_pos[pos] : pos;
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
static int out_dtype_code(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return OUT_F32;
    case at::kHalf: return OUT_F16;
    case at::kBFloat16: return OUT_BF16;
    default: TORCH_CHECK(false, "unsupported dtype ", t);
  }
}

static int vecs_for_dim(int64_t max_D) {
  TORCH_CHECK(max_D % 4 == 0, "embedding dims must be multiples of 4");
  if (max_D <= 128) return 1;
  if (max_D <= 256) return 2;
  if (max_D <= 512) return 4;
  TORCH_CHECK(max_D <= 1024, "embedding dims above 1024 are not supported");
  return 8;
}

#define TRB_DISPATCH_EMB(TYPE, ...)                                   \
  [&] {                                                               \
    if (TYPE == at::kFloat) { using emb_t = float; __VA_ARGS__(); }   \
    else if (TYPE == at::kHalf) { using emb_t = __half; __VA_ARGS__(); } \
    else if (TYPE == at::kBFloat16) { using emb_t = __nv_bfloat16; __VA_ARGS__(); } \
    else TORCH_CHECK(false, "unsupported weights dtype");             \
  }()

#define TRB_DISPATCH_VECS(NV, ...)                                    \
  [&] {                                                               \
    if (NV == 1) { constexpr int kVecs = 1; __VA_ARGS__(); }          \
    else if (NV == 2) { constexpr int kVecs = 2; __VA_ARGS__(); }     \
    else if (NV == 4) { constexpr int kVecs = 4; __VA_ARGS__(); }     \
    else { constexpr int kVecs = 8; __VA_ARGS__(); }                  \
  }()

// out_ptrs: int64 CPU tensor [W] of device pointers (one per destination rank), or empty -> `out`.
void tbe_forward_impl(const at::Tensor& weights, const at::Tensor& meta, const at::Tensor& indices,
                      const at::Tensor& offsets, const c10::optional<at::Tensor>& psw, at::Tensor& out,
                      const std::vector<int64_t>& out_ptrs, int64_t out_dtype, int64_t out_stride, int64_t B,
                      int64_t B_local, int64_t max_D, int64_t pooling, bool accumulate, bool skip_empty,
                      at::Tensor& err) {
  const int F = int(meta.size(1));
  TORCH_CHECK(meta.size(0) == kMetaRows && meta.scalar_type() == at::kLong && meta.is_contiguous());
  TORCH_CHECK(indices.scalar_type() == offsets.scalar_type(), "indices and offsets must share a dtype");
  TORCH_CHECK(offsets.numel() == int64_t(F) * B + 1, "offsets must have F*B+1 entries");
  if (F == 0 || B == 0) return;
  c10::cuda::CUDAGuard guard(weights.device());
  FwdParams p;
  p.weights = weights.data_ptr();
  p.meta = meta.data_ptr<int64_t>();
  p.indices = indices.data_ptr();
  p.offsets = offsets.data_ptr();
  p.psw = psw.has_value() && psw->defined() ? psw->data_ptr<float>() : nullptr;
  if (out_ptrs.empty()) {
    p.out.p[0] = out.data_ptr();
    TORCH_CHECK(B_local == B);
  } else {
    TORCH_CHECK(out_ptrs.size() <= size_t(kMaxPeers));
    TORCH_CHECK(int64_t(out_ptrs.size()) * B_local >= B);
    for (size_t i = 0; i < out_ptrs.size(); ++i) p.out.p[i] = reinterpret_cast<void*>(out_ptrs[i]);
  }
  p.out_dtype = int(out_dtype);
  p.out_stride = out_stride;
  p.B = int(B);
  p.B_local = int(B_local);
  p.F = F;
  p.pooling = int(pooling);
  p.accumulate = accumulate ? 1 : 0;
  p.skip_empty = skip_empty ? 1 : 0;
  p.err = err.data_ptr<int>();
  TORCH_CHECK(!accumulate || out_dtype == OUT_F32, "accumulate mode needs an fp32 destination");
  const int64_t nbags = int64_t(F) * B;
  const int threads = 256;
  const int64_t blocks = (nbags * 32 + threads - 1) / threads;
  auto stream = at::cuda::getCurrentCUDAStream();
  const int nv = vecs_for_dim(max_D);
  const bool i64 = indices.scalar_type() == at::kLong;
  TORCH_CHECK(i64 || indices.scalar_type() == at::kInt, "indices must be int32 or int64");
  TRB_DISPATCH_EMB(weights.scalar_type(), [&] {
    TRB_DISPATCH_VECS(nv, [&] {
      if (pooling == POOL_NONE) {
        const int64_t n_ids = indices.numel();
        const int64_t seq_blocks = ((n_ids + kSeqPer - 1) / kSeqPer * 32 + threads - 1) / threads;
        if (n_ids == 0) return;
        if (i64) tbe_seq_fwd_kernel<emb_t, int64_t, kVecs><<<seq_blocks, threads, 0, stream>>>(p, n_ids);
        else tbe_seq_fwd_kernel<emb_t, int32_t, kVecs><<<seq_blocks, threads, 0, stream>>>(p, n_ids);
      } else {
        if (i64) tbe_fwd_kernel<emb_t, int64_t, kVecs><<<blocks, threads, 0, stream>>>(p);
        else tbe_fwd_kernel<emb_t, int32_t, kVecs><<<blocks, threads, 0, stream>>>(p);
      }
    });
  });
  TRB_CUDA_CHECK(cudaGetLastError());
}

at::Tensor tbe_forward(const at::Tensor& weights, const at::Tensor& meta, const at::Tensor& indices,
                       const at::Tensor& offsets, const c10::optional<at::Tensor>& psw, int64_t B, int64_t total_D,
                       int64_t max_D, int64_t pooling, int64_t out_dtype, at::Tensor err) {
  auto dt = out_dtype == OUT_F32 ? at::kFloat : (out_dtype == OUT_F16 ? at::kHalf : at::kBFloat16);
  at::Tensor out;
  if (pooling == POOL_NONE) {
    out = at::empty({indices.numel(), max_D}, weights.options().dtype(dt));
    tbe_forward_impl(weights, meta, indices, offsets, psw, out, {}, out_dtype, max_D, B, B, max_D, pooling, false,
                     false, err);
  } else {
    out = at::empty({B, total_D}, weights.options().dtype(dt));
    tbe_forward_impl(weights, meta, indices, offsets, psw, out, {}, out_dtype, total_D, B, B, max_D, pooling, false,
                     false, err);
  }
  return out;
}

// Pooled forward whose destination rows live on peer ranks (fused lookup + all-to-all / reduce-scatter).
void tbe_forward_dist(const at::Tensor& weights, const at::Tensor& meta, const at::Tensor& indices,
                      const at::Tensor& offsets, const c10::optional<at::Tensor>& psw, std::vector<int64_t> out_ptrs,
                      int64_t out_dtype, int64_t out_stride, int64_t B, int64_t B_local, int64_t max_D,
                      int64_t pooling, bool accumulate, bool skip_empty, at::Tensor err) {
  at::Tensor dummy;
  tbe_forward_impl(weights, meta, indices, offsets, psw, dummy, out_ptrs, out_dtype, out_stride, B, B_local, max_D,
                   pooling, accumulate, skip_empty, err);
}

struct SortedPlan {
  at::Tensor keys, src, w, src_feature, bag_scale;
};

// Build the sorted (row -> contributing bags) plan for one batch.  It depends on the ids only, so a
// pipeline may run it on a side stream while the dense towers of the previous step are still busy.
std::vector<at::Tensor> tbe_build_plan(const at::Tensor& meta, const at::Tensor& indices, const at::Tensor& offsets,
                                       const c10::optional<at::Tensor>& psw, int64_t B, int64_t total_rows,
                                       bool pooled, bool mean_pooling, bool padded, at::Tensor err) {
  const int F = int(meta.size(1));
  const int64_t N = indices.numel();
  c10::cuda::CUDAGuard guard(indices.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  auto opts_i64 = indices.options().dtype(at::kLong);
  auto opts_i32 = indices.options().dtype(at::kInt);
  auto opts_f32 = indices.options().dtype(at::kFloat);
  // padded: `indices` is a buffer of fixed capacity of which only [offsets[0], offsets[F*B]) holds ids of these tables.
  // Every other position gets a key past the last table row, sorts to the tail and is skipped by the backward kernels,
  // which read the number of real entries from `n_valid` on the device: no size ever travels to the host.
  at::Tensor keys = padded ? at::full({N}, total_rows, opts_i64) : at::empty({N}, opts_i64), src = at::empty({N}, opts_i32);
  at::Tensor n_valid = padded ? at::empty({1}, opts_i64) : at::Tensor();
  at::Tensor src_feature = pooled ? at::Tensor() : at::empty({N}, opts_i32);
  at::Tensor bag_scale = (pooled && mean_pooling) ? at::empty({int64_t(F) * B}, opts_f32) : at::Tensor();
  const bool weighted = psw.has_value() && psw->defined();
  at::Tensor pos;  // weighted: sort positions, then gather weights
  if (N > 0 && F > 0 && B > 0) {
    const int threads = 256;
    const int64_t blocks = (int64_t(F) * B * 32 + threads - 1) / threads;
    const bool i64 = indices.scalar_type() == at::kLong;
    // weighted path keeps bag ids aside and sorts positions instead
    at::Tensor bag_of_pos;
    int32_t* src_ptr = src.data_ptr<int32_t>();
    if (weighted && pooled) {
      bag_of_pos = at::empty({N}, opts_i32);
      src_ptr = bag_of_pos.data_ptr<int32_t>();
    }
    if (!pooled && !weighted) {
      // positions [offsets[0], offsets[F*B]) hold this module's ids; the grid covers the whole buffer and idle threads return
      const int64_t seq_blocks = (N + threads - 1) / threads;
      if (i64) tbe_linearize_seq_kernel<int64_t><<<seq_blocks, threads, 0, stream>>>(indices.data_ptr<int64_t>(), offsets.data_ptr<int64_t>(), meta.data_ptr<int64_t>(), F, int(B), keys.data_ptr<int64_t>(), src_ptr, src_feature.data_ptr<int32_t>(), err.data_ptr<int>());
      else tbe_linearize_seq_kernel<int32_t><<<seq_blocks, threads, 0, stream>>>(indices.data_ptr<int32_t>(), offsets.data_ptr<int32_t>(), meta.data_ptr<int64_t>(), F, int(B), keys.data_ptr<int64_t>(), src_ptr, src_feature.data_ptr<int32_t>(), err.data_ptr<int>());
    } else {
      // short bags (up to 16 ids on average): eight lanes per bag
      const bool narrow = N <= int64_t(F) * B * 16;
      const int64_t lin_blocks = narrow ? (int64_t(F) * B * 8 + threads - 1) / threads : blocks;
      auto launch = [&](auto tag, auto lanes) {
        using T = decltype(tag);
        constexpr int kL = decltype(lanes)::value;
        tbe_linearize_kernel<T, kL><<<lin_blocks, threads, 0, stream>>>(
            indices.data_ptr<T>(), offsets.data_ptr<T>(), meta.data_ptr<int64_t>(), F, int(B), pooled ? 1 : 0, keys.data_ptr<int64_t>(), src_ptr,
            pooled ? nullptr : src_feature.data_ptr<int32_t>(), bag_scale.defined() ? bag_scale.data_ptr<float>() : nullptr, err.data_ptr<int>());
      };
      if (i64) {
        if (narrow) launch(int64_t(0), std::integral_constant<int, 8>()); else launch(int64_t(0), std::integral_constant<int, 32>());
      } else {
        if (narrow) launch(int32_t(0), std::integral_constant<int, 8>()); else launch(int32_t(0), std::integral_constant<int, 32>());
      }
    }
    if (padded) {
      if (i64) tbe_count_valid_kernel<int64_t><<<1, 1, 0, stream>>>(offsets.data_ptr<int64_t>(), int64_t(F) * B, n_valid.data_ptr<int64_t>());
      else tbe_count_valid_kernel<int32_t><<<1, 1, 0, stream>>>(offsets.data_ptr<int32_t>(), int64_t(F) * B, n_valid.data_ptr<int64_t>());
    }
    TRB_CUDA_CHECK(cudaGetLastError());
    at::Tensor vals_in = src;
    if (weighted) {
      vals_in = at::arange(N, opts_i32);
    }
    at::Tensor keys_out = at::empty({N}, opts_i64), vals_out = at::empty({N}, opts_i32);
    int end_bit = 1;
    while ((int64_t(1) << end_bit) < total_rows + (padded ? 1 : 0) && end_bit < 63) ++end_bit;
    size_t tmp_bytes = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, tmp_bytes, keys.data_ptr<int64_t>(), keys_out.data_ptr<int64_t>(),
                                    vals_in.data_ptr<int32_t>(), vals_out.data_ptr<int32_t>(), N, 0, end_bit, stream);
    at::Tensor tmp = at::empty({int64_t(tmp_bytes)}, indices.options().dtype(at::kByte));
    cub::DeviceRadixSort::SortPairs(tmp.data_ptr(), tmp_bytes, keys.data_ptr<int64_t>(), keys_out.data_ptr<int64_t>(),
                                    vals_in.data_ptr<int32_t>(), vals_out.data_ptr<int32_t>(), N, 0, end_bit, stream);
    keys = keys_out;
    at::Tensor w_sorted;
    if (weighted) {
      w_sorted = at::empty({N}, opts_f32);
      at::Tensor src_sorted = at::empty({N}, opts_i32);
      const int64_t gb = (N + 255) / 256;
      gather_sorted_weights_kernel<<<gb, 256, 0, stream>>>(
          psw->data_ptr<float>(), vals_out.data_ptr<int32_t>(), pooled ? bag_of_pos.data_ptr<int32_t>() : nullptr,
          w_sorted.data_ptr<float>(), src_sorted.data_ptr<int32_t>(), N);
      TRB_CUDA_CHECK(cudaGetLastError());
      src = src_sorted;
    } else {
      src = vals_out;
    }
    std::vector<at::Tensor> res = {keys, src, w_sorted.defined() ? w_sorted : at::empty({0}, opts_f32),
                                   src_feature.defined() ? src_feature : at::empty({0}, opts_i32),
                                   bag_scale.defined() ? bag_scale : at::empty({0}, opts_f32)};
    if (padded) res.push_back(n_valid);
    return res;
  }
  std::vector<at::Tensor> res = {keys, src, at::empty({0}, opts_f32), src_feature.defined() ? src_feature : at::empty({0}, opts_i32),
                                 bag_scale.defined() ? bag_scale : at::empty({0}, opts_f32)};
  if (padded) res.push_back(at::zeros({1}, opts_i64));
  return res;
}

// Apply the sorted plan: segment-reduce upstream gradient rows per table row and update in place.
static void tbe_backward_apply_impl(at::Tensor weights, c10::optional<at::Tensor> mom1, c10::optional<at::Tensor> mom2,
                                    c10::optional<at::Tensor> dense_grad, const at::Tensor& meta, const at::Tensor& sorted_keys,
                                    const at::Tensor& sorted_src, const at::Tensor& sorted_w, const at::Tensor& src_feature,
                                    const at::Tensor& bag_scale, const at::Tensor& grad, int64_t grad_stride, int64_t B,
                                    int64_t max_D, bool pooled, int64_t opt_type, double lr, double eps, double beta1,
                                    double beta2, double weight_decay, int64_t step, double max_grad,
                                    const std::vector<int64_t>& grad_ptrs, int64_t B_local, double grad_scale,
                                    const c10::optional<at::Tensor>& n_valid = c10::nullopt,
                                    const c10::optional<at::Tensor>& sr_counter = c10::nullopt,
                                    const c10::optional<at::Tensor>& ret = c10::nullopt) {
  const int64_t N = sorted_keys.numel();
  if (N == 0) return;
  c10::cuda::CUDAGuard guard(weights.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const int F = int(meta.size(1));
  const int nv = vecs_for_dim(max_D);
  const int Dpad = int(max_D);
  const int64_t nblocks = (N + kBlk - 1) / kBlk;
  at::Tensor partials = at::empty({2 * nblocks * Dpad}, weights.options().dtype(at::kFloat));
  at::Tensor flags = at::empty({2 * nblocks}, weights.options().dtype(at::kInt));
  at::Tensor long_list = at::empty({2 * (nblocks / kSerialChain + 1)}, weights.options().dtype(at::kLong));
  at::Tensor long_count = at::zeros({1}, weights.options().dtype(at::kInt));
  BwdParams p;
  p.weights = weights.data_ptr();
  p.mom1 = mom1.has_value() && mom1->defined() ? mom1->data_ptr<float>() : nullptr;
  p.mom2 = mom2.has_value() && mom2->defined() ? mom2->data_ptr<float>() : nullptr;
  p.dense_grad = dense_grad.has_value() && dense_grad->defined() ? dense_grad->data_ptr<float>() : nullptr;
  p.meta = meta.data_ptr<int64_t>();
  p.sorted_keys = sorted_keys.data_ptr<int64_t>();
  p.sorted_src = sorted_src.data_ptr<int32_t>();
  p.sorted_w = sorted_w.numel() > 0 ? sorted_w.data_ptr<float>() : nullptr;
  p.src_feature = src_feature.numel() > 0 ? src_feature.data_ptr<int32_t>() : nullptr;
  p.grad = grad.data_ptr();
  p.grad_dtype = out_dtype_code(grad.scalar_type());
  p.grad_stride = grad_stride;
  p.bag_scale = bag_scale.numel() > 0 ? bag_scale.data_ptr<float>() : nullptr;
  p.N = N;
  p.n_valid = n_valid.has_value() && n_valid->defined() ? n_valid->data_ptr<int64_t>() : nullptr;
  p.B = int(B);
  p.F = F;
  p.pooled = pooled ? 1 : 0;
  p.partials = partials.data_ptr<float>();
  p.flags = flags.data_ptr<int32_t>();
  p.long_list = long_list.data_ptr<int64_t>();
  p.long_count = long_count.data_ptr<int>();
  p.Dpad = Dpad;
  p.B_local = 0;
  p.grad_scale = float(grad_scale);
  for (int i = 0; i < kMaxPeers; ++i) p.grad_peers.p[i] = nullptr;
  p.ret = nullptr;
  if (ret.has_value() && ret->defined()) {
    TORCH_CHECK(!pooled && !grad_ptrs.empty() && grad_ptrs.size() <= size_t(kMaxPeers), "return addresses serve the unpooled peer backward");
    TORCH_CHECK(ret->scalar_type() == at::kLong && ret->is_contiguous() && ret->numel() >= N);
    p.ret = ret->data_ptr<int64_t>();
    for (size_t i = 0; i < grad_ptrs.size(); ++i) p.grad_peers.p[i] = reinterpret_cast<void*>(grad_ptrs[i]);
  } else if (!grad_ptrs.empty()) {
    TORCH_CHECK(pooled && B_local > 0 && int64_t(grad_ptrs.size()) * B_local == B && grad_ptrs.size() <= size_t(kMaxPeers),
                "peer gradients: B must be world * B_local");
    p.B_local = int(B_local);
    bool has_local = false;
    for (size_t i = 0; i < grad_ptrs.size(); ++i) {
      p.grad_peers.p[i] = reinterpret_cast<void*>(grad_ptrs[i]);
      has_local = has_local || p.grad_peers.p[i] == grad.data_ptr();
    }
    TORCH_CHECK(has_local, "grad must be this rank's own buffer among grad_ptrs");
  }
  p.opt.type = int(opt_type);
  p.opt.lr = float(lr);
  p.opt.eps = float(eps);
  p.opt.beta1 = float(beta1);
  p.opt.beta2 = float(beta2);
  p.opt.weight_decay = float(weight_decay);
  p.opt.bias_corr1 = float(1.0 - std::pow(beta1, double(std::max<int64_t>(step, 1))));
  p.opt.bias_corr2 = float(1.0 - std::pow(beta2, double(std::max<int64_t>(step, 1))));
  p.opt.max_grad = float(max_grad);
  const bool sr = sr_counter.has_value() && sr_counter->defined() && weights.scalar_type() != at::kFloat;
  if (sr) TORCH_CHECK(sr_counter->is_cuda() && sr_counter->scalar_type() == at::kLong && sr_counter->numel() >= 1);
  p.opt.stochastic_rounding = sr ? 1 : 0;
  p.opt.sr_counter = sr ? sr_counter->data_ptr<int64_t>() : nullptr;
  TORCH_CHECK(pooled || p.src_feature != nullptr, "unpooled backward needs src_feature");
  if (opt_type == OPT_DENSE_GRAD) TORCH_CHECK(p.dense_grad != nullptr);
  const int threads = 256;
  const int64_t blocks = (nblocks * 32 + threads - 1) / threads;
  TRB_DISPATCH_EMB(weights.scalar_type(), [&] {
    TRB_DISPATCH_VECS(nv, [&] {
      if (p.grad_dtype == OUT_F32) tbe_bwd_block_kernel<emb_t, float, kVecs><<<blocks, threads, 0, stream>>>(p);
      else if (p.grad_dtype == OUT_F16) tbe_bwd_block_kernel<emb_t, __half, kVecs><<<blocks, threads, 0, stream>>>(p);
      else tbe_bwd_block_kernel<emb_t, __nv_bfloat16, kVecs><<<blocks, threads, 0, stream>>>(p);
      tbe_bwd_long_kernel<emb_t, kVecs><<<blocks, threads, 0, stream>>>(p);
      tbe_bwd_verylong_kernel<emb_t, kVecs><<<296, 256, 0, stream>>>(p);
    });
  });
  if (sr) tbe_bump_counter_kernel<<<1, 1, 0, stream>>>(sr_counter->data_ptr<int64_t>());
  TRB_CUDA_CHECK(cudaGetLastError());
}

void tbe_backward_apply(at::Tensor weights, c10::optional<at::Tensor> mom1, c10::optional<at::Tensor> mom2,
                        c10::optional<at::Tensor> dense_grad, const at::Tensor& meta, const at::Tensor& sorted_keys,
                        const at::Tensor& sorted_src, const at::Tensor& sorted_w, const at::Tensor& src_feature,
                        const at::Tensor& bag_scale, const at::Tensor& grad, int64_t grad_stride, int64_t B,
                        int64_t max_D, bool pooled, int64_t opt_type, double lr, double eps, double beta1,
                        double beta2, double weight_decay, int64_t step, double max_grad, c10::optional<at::Tensor> n_valid,
                        c10::optional<at::Tensor> sr_counter) {
  tbe_backward_apply_impl(weights, mom1, mom2, dense_grad, meta, sorted_keys, sorted_src, sorted_w, src_feature, bag_scale, grad,
                          grad_stride, B, max_D, pooled, opt_type, lr, eps, beta1, beta2, weight_decay, step, max_grad, {}, 0, 1.0,
                          n_valid, sr_counter);
}

// Backward of the fused lookup + exchange: the pooled gradient of bag b (of the global batch) is read from the
// buffer of the rank that owns sample b (`grad_ptrs[b / B_local]`, peer-mapped), scaled by `grad_scale`.
void tbe_backward_apply_dist(at::Tensor weights, c10::optional<at::Tensor> mom1, c10::optional<at::Tensor> mom2,
                             c10::optional<at::Tensor> dense_grad, const at::Tensor& meta, const at::Tensor& sorted_keys,
                             const at::Tensor& sorted_src, const at::Tensor& sorted_w, const at::Tensor& src_feature,
                             const at::Tensor& bag_scale, const at::Tensor& grad, int64_t grad_stride, int64_t B,
                             int64_t max_D, bool pooled, int64_t opt_type, double lr, double eps, double beta1,
                             double beta2, double weight_decay, int64_t step, double max_grad,
                             std::vector<int64_t> grad_ptrs, int64_t B_local, double grad_scale,
                             c10::optional<at::Tensor> n_valid, c10::optional<at::Tensor> ret,
                             c10::optional<at::Tensor> sr_counter) {
  tbe_backward_apply_impl(weights, mom1, mom2, dense_grad, meta, sorted_keys, sorted_src, sorted_w, src_feature, bag_scale, grad,
                          grad_stride, B, max_D, pooled, opt_type, lr, eps, beta1, beta2, weight_decay, step, max_grad, grad_ptrs,
                          B_local, grad_scale, n_valid, sr_counter, ret);
}

// Unpooled forward of the fused exchange: row of id k goes to row (ret[k] & 0xffffffff) of the output buffer of rank
// ret[k] >> 32, at the table's output column.  `indices` / `ret` are receive buffers of fixed capacity; `offsets` (F*B+1
// entries, absolute positions in them) delimits this module's ids.
void tbe_seq_forward_dist(const at::Tensor& weights, const at::Tensor& meta, const at::Tensor& indices, const at::Tensor& offsets,
                          const at::Tensor& ret, std::vector<int64_t> out_ptrs, int64_t out_rows, int64_t out_dtype, int64_t out_stride,
                          int64_t B, int64_t max_D, at::Tensor err) {
  const int F = int(meta.size(1));
  TORCH_CHECK(meta.size(0) == kMetaRows && meta.scalar_type() == at::kLong && meta.is_contiguous());
  TORCH_CHECK(indices.scalar_type() == offsets.scalar_type(), "indices and offsets must share a dtype");
  TORCH_CHECK(offsets.numel() == int64_t(F) * B + 1, "offsets must have F*B+1 entries");
  TORCH_CHECK(ret.scalar_type() == at::kLong && ret.numel() >= indices.numel());
  TORCH_CHECK(!out_ptrs.empty() && out_ptrs.size() <= size_t(kMaxPeers));
  const int64_t cap = indices.numel();
  if (F == 0 || B == 0 || cap == 0) return;
  c10::cuda::CUDAGuard guard(weights.device());
  FwdParams p;
  p.weights = weights.data_ptr();
  p.meta = meta.data_ptr<int64_t>();
  p.indices = indices.data_ptr();
  p.offsets = offsets.data_ptr();
  p.psw = nullptr;
  for (size_t i = 0; i < out_ptrs.size(); ++i) p.out.p[i] = reinterpret_cast<void*>(out_ptrs[i]);
  p.out_dtype = int(out_dtype);
  p.out_stride = out_stride;
  p.B = int(B);
  p.B_local = int(B);
  p.F = F;
  p.pooling = POOL_NONE;
  p.accumulate = 0;
  p.skip_empty = 0;
  p.err = err.data_ptr<int>();
  const int threads = 256;
  const int64_t blocks = ((cap + kSeqPer - 1) / kSeqPer * 32 + threads - 1) / threads;
  auto stream = at::cuda::getCurrentCUDAStream();
  const int nv = vecs_for_dim(max_D);
  const bool i64 = indices.scalar_type() == at::kLong;
  const int64_t* rp = ret.data_ptr<int64_t>();
  TRB_DISPATCH_EMB(weights.scalar_type(), [&] {
    TRB_DISPATCH_VECS(nv, [&] {
      if (i64) tbe_seq_fwd_dist_kernel<emb_t, int64_t, kVecs><<<blocks, threads, 0, stream>>>(p, rp, out_rows, int(out_ptrs.size()));
      else tbe_seq_fwd_dist_kernel<emb_t, int32_t, kVecs><<<blocks, threads, 0, stream>>>(p, rp, out_rows, int(out_ptrs.size()));
    });
  });
  TRB_CUDA_CHECK(cudaGetLastError());
}

}  // namespace trb

// ---------------------------------------------------------------------------------------------------------------
// Allocation-free C entry point (declared and documented in tbe_noalloc.h).  The scratch that the operator above
// takes from the caching allocator lives here in a fixed device array; the host reaches it through the address
// that cudaGetSymbolAddress reports, looked up once per device.
// ---------------------------------------------------------------------------------------------------------------
#include "tbe_noalloc.h"

#include <cstdarg>
#include <cstdio>
#include <mutex>

namespace {

constexpr size_t kNaMaxBlocks = TRB_NOALLOC_MAX_ENTRIES / trb::kBlk;                               // 4096
constexpr size_t kNaPartialBytes = size_t(2) * TRB_NOALLOC_MAX_BLOCK_DIM * sizeof(float);          // 4 MiB
constexpr size_t kNaFlagBytes = size_t(2) * kNaMaxBlocks * sizeof(int32_t);                        // 32 KiB
constexpr size_t kNaLongListBytes = ((2 * (kNaMaxBlocks / trb::kSerialChain + 1) * sizeof(int64_t)) + 255) / 256 * 256;
constexpr size_t kNaCountBytes = 256;
constexpr size_t kNaOffFlags = kNaPartialBytes;
constexpr size_t kNaOffLongList = kNaOffFlags + kNaFlagBytes;
constexpr size_t kNaOffCount = kNaOffLongList + kNaLongListBytes;
constexpr size_t kNaScratchBytes = kNaOffCount + kNaCountBytes;

static __device__ __align__(256) unsigned char g_tbe_noalloc_scratch[kNaScratchBytes];

constexpr int kNaMaxDevices = 64;
std::mutex g_na_mutex;
unsigned char* g_na_scratch_ptr[kNaMaxDevices] = {};  // device address of the array, per device

int na_fail(int code, char* errbuf, size_t errbuf_len, const char* fmt, ...) {
  if (errbuf != nullptr && errbuf_len > 0) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(errbuf, errbuf_len, fmt, ap);
    va_end(ap);
  }
  return code;
}

template <typename emb_t>
void na_launch(int nv, int64_t blocks, int threads, cudaStream_t stream, const trb::BwdParams& p) {
  TRB_DISPATCH_VECS(nv, [&] {
    if (p.grad_dtype == trb::OUT_F32) trb::tbe_bwd_block_kernel<emb_t, float, kVecs><<<blocks, threads, 0, stream>>>(p);
    else if (p.grad_dtype == trb::OUT_F16) trb::tbe_bwd_block_kernel<emb_t, __half, kVecs><<<blocks, threads, 0, stream>>>(p);
    else trb::tbe_bwd_block_kernel<emb_t, __nv_bfloat16, kVecs><<<blocks, threads, 0, stream>>>(p);
    trb::tbe_bwd_long_kernel<emb_t, kVecs><<<blocks, threads, 0, stream>>>(p);
    trb::tbe_bwd_verylong_kernel<emb_t, kVecs><<<296, 256, 0, stream>>>(p);
  });
}

}  // namespace

extern "C" int trb_tbe_backward_apply_noalloc(const trb_tbe_bwd_noalloc_args* a, void* stream_v, char* errbuf,
                                              size_t errbuf_len) {
  if (a == nullptr) return na_fail(TRB_NOALLOC_E_BAD_ARG, errbuf, errbuf_len, "args is null");
  if (a->N == 0) return TRB_NOALLOC_OK;
  if (a->N < 0 || a->weights == nullptr || a->meta == nullptr || a->sorted_keys == nullptr || a->sorted_src == nullptr ||
      a->grad == nullptr)
    return na_fail(TRB_NOALLOC_E_BAD_ARG, errbuf, errbuf_len, "weights, meta, sorted_keys, sorted_src and grad must be set and N >= 0");
  if (a->weights_dtype < 0 || a->weights_dtype > 2 || a->grad_dtype < 0 || a->grad_dtype > 2)
    return na_fail(TRB_NOALLOC_E_BAD_ARG, errbuf, errbuf_len, "dtype codes are 0 (fp32), 1 (fp16), 2 (bf16)");
  if (a->max_D <= 0 || a->max_D % 4 != 0 || a->max_D > 1024)
    return na_fail(TRB_NOALLOC_E_BAD_ARG, errbuf, errbuf_len, "max_D=%d must be a positive multiple of 4, at most 1024", a->max_D);
  if (a->F <= 0 || a->B <= 0) return na_fail(TRB_NOALLOC_E_BAD_ARG, errbuf, errbuf_len, "F and B must be positive");
  if (!a->pooled && a->src_feature == nullptr)
    return na_fail(TRB_NOALLOC_E_BAD_ARG, errbuf, errbuf_len, "the unpooled backward needs src_feature");
  if (a->opt_type == trb::OPT_DENSE_GRAD && a->dense_grad == nullptr)
    return na_fail(TRB_NOALLOC_E_BAD_ARG, errbuf, errbuf_len, "opt_type 100 needs dense_grad");
  const int64_t nblocks = (a->N + trb::kBlk - 1) / trb::kBlk;
  if (a->N > TRB_NOALLOC_MAX_ENTRIES || nblocks * int64_t(a->max_D) > TRB_NOALLOC_MAX_BLOCK_DIM)
    return na_fail(TRB_NOALLOC_E_TOO_LARGE, errbuf, errbuf_len,
                   "N=%lld entries with max_D=%d is beyond the fixed scratch: N <= %d and ceil(N/64)*max_D <= %d; "
                   "use trb200::tbe_backward_apply for larger batches",
                   (long long)a->N, a->max_D, TRB_NOALLOC_MAX_ENTRIES, TRB_NOALLOC_MAX_BLOCK_DIM);

  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return na_fail(TRB_NOALLOC_E_CUDA, errbuf, errbuf_len, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kNaMaxDevices) return na_fail(TRB_NOALLOC_E_DEVICE, errbuf, errbuf_len, "device %d out of range", dev);
  cudaPointerAttributes attr;
  e = cudaPointerGetAttributes(&attr, a->weights);
  if (e != cudaSuccess) return na_fail(TRB_NOALLOC_E_CUDA, errbuf, errbuf_len, "cudaPointerGetAttributes: %s", cudaGetErrorString(e));
  if (attr.type != cudaMemoryTypeDevice || attr.device != dev)
    return na_fail(TRB_NOALLOC_E_DEVICE, errbuf, errbuf_len, "weights are not device memory of the current device %d", dev);

  // set-up, once per device with that device current: the device address of the scratch array
  unsigned char* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_na_mutex);
    if (g_na_scratch_ptr[dev] == nullptr) {
      void* ptr = nullptr;
      e = cudaGetSymbolAddress((void**)&ptr, g_tbe_noalloc_scratch);
      if (e != cudaSuccess || ptr == nullptr)
        return na_fail(TRB_NOALLOC_E_CUDA, errbuf, errbuf_len, "cudaGetSymbolAddress(scratch) on device %d: %s", dev,
                       cudaGetErrorString(e));
      g_na_scratch_ptr[dev] = static_cast<unsigned char*>(ptr);
    }
    scratch = g_na_scratch_ptr[dev];
  }

  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  trb::BwdParams p;
  p.weights = a->weights;
  p.mom1 = a->mom1;
  p.mom2 = a->mom2;
  p.dense_grad = a->dense_grad;
  p.meta = a->meta;
  p.sorted_keys = a->sorted_keys;
  p.sorted_src = a->sorted_src;
  p.sorted_w = a->sorted_w;
  p.src_feature = a->src_feature;
  p.grad = a->grad;
  p.grad_dtype = a->grad_dtype;
  p.grad_stride = a->grad_stride;
  p.bag_scale = a->bag_scale;
  p.N = a->N;
  p.n_valid = nullptr;
  p.ret = nullptr;
  p.B = a->B;
  p.F = a->F;
  p.pooled = a->pooled ? 1 : 0;
  p.partials = reinterpret_cast<float*>(scratch);
  p.flags = reinterpret_cast<int32_t*>(scratch + kNaOffFlags);
  p.long_list = reinterpret_cast<int64_t*>(scratch + kNaOffLongList);
  p.long_count = reinterpret_cast<int*>(scratch + kNaOffCount);
  p.Dpad = a->max_D;
  p.B_local = 0;
  p.grad_scale = 1.f;
  for (int i = 0; i < trb::kMaxPeers; ++i) p.grad_peers.p[i] = nullptr;
  p.opt.type = a->opt_type;
  p.opt.lr = a->lr;
  p.opt.eps = a->eps;
  p.opt.beta1 = a->beta1;
  p.opt.beta2 = a->beta2;
  p.opt.weight_decay = a->weight_decay;
  const int64_t step = a->step > 1 ? a->step : 1;
  p.opt.bias_corr1 = float(1.0 - std::pow(double(a->beta1), double(step)));
  p.opt.bias_corr2 = float(1.0 - std::pow(double(a->beta2), double(step)));
  p.opt.max_grad = a->max_grad;
  p.opt.stochastic_rounding = 0;
  p.opt.sr_counter = nullptr;

  // the only word that must start at zero: the queue length of long chains (pass 1 writes every flag it covers)
  e = cudaMemsetAsync(p.long_count, 0, sizeof(int), stream);
  if (e != cudaSuccess) return na_fail(TRB_NOALLOC_E_CUDA, errbuf, errbuf_len, "cudaMemsetAsync: %s", cudaGetErrorString(e));
  const int nv = a->max_D <= 128 ? 1 : (a->max_D <= 256 ? 2 : (a->max_D <= 512 ? 4 : 8));
  const int threads = 256;
  const int64_t blocks = (nblocks * 32 + threads - 1) / threads;
  if (a->weights_dtype == trb::OUT_F32) na_launch<float>(nv, blocks, threads, stream, p);
  else if (a->weights_dtype == trb::OUT_F16) na_launch<__half>(nv, blocks, threads, stream, p);
  else na_launch<__nv_bfloat16>(nv, blocks, threads, stream, p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return na_fail(TRB_NOALLOC_E_CUDA, errbuf, errbuf_len, "kernel launch: %s", cudaGetErrorString(e));
  return TRB_NOALLOC_OK;
}

TORCH_LIBRARY_FRAGMENT(trb200, m) {
  m.def(
      "tbe_forward(Tensor weights, Tensor meta, Tensor indices, Tensor offsets, Tensor? psw, int B, int total_D, "
      "int max_D, int pooling, int out_dtype, Tensor(a!) err) -> Tensor");
  m.def(
      "tbe_forward_dist(Tensor weights, Tensor meta, Tensor indices, Tensor offsets, Tensor? psw, int[] out_ptrs, "
      "int out_dtype, int out_stride, int B, int B_local, int max_D, int pooling, bool accumulate, bool skip_empty, "
      "Tensor(a!) err) -> ()");
  m.def(
      "tbe_build_plan(Tensor meta, Tensor indices, Tensor offsets, Tensor? psw, int B, int total_rows, bool pooled, "
      "bool mean_pooling, bool padded, Tensor(a!) err) -> Tensor[]");
  m.def(
      "tbe_backward_apply(Tensor(a!) weights, Tensor(b!)? mom1, Tensor(c!)? mom2, Tensor(d!)? dense_grad, Tensor meta, "
      "Tensor sorted_keys, Tensor sorted_src, Tensor sorted_w, Tensor src_feature, Tensor bag_scale, Tensor grad, "
      "int grad_stride, int B, int max_D, bool pooled, int opt_type, float lr, float eps, float beta1, float beta2, "
      "float weight_decay, int step, float max_grad, Tensor? n_valid, Tensor(e!)? sr_counter=None) -> ()");
  m.def(
      "tbe_backward_apply_dist(Tensor(a!) weights, Tensor(b!)? mom1, Tensor(c!)? mom2, Tensor(d!)? dense_grad, Tensor meta, "
      "Tensor sorted_keys, Tensor sorted_src, Tensor sorted_w, Tensor src_feature, Tensor bag_scale, Tensor grad, "
      "int grad_stride, int B, int max_D, bool pooled, int opt_type, float lr, float eps, float beta1, float beta2, "
      "float weight_decay, int step, float max_grad, int[] grad_ptrs, int B_local, float grad_scale, Tensor? n_valid, "
      "Tensor? ret=None, Tensor(e!)? sr_counter=None) -> ()");
  m.def(
      "tbe_seq_forward_dist(Tensor weights, Tensor meta, Tensor indices, Tensor offsets, Tensor ret, int[] out_ptrs, "
      "int out_rows, int out_dtype, int out_stride, int B, int max_D, Tensor(a!) err) -> ()");
}

TORCH_LIBRARY_IMPL(trb200, CUDA, m) {
  m.impl("tbe_forward", &trb::tbe_forward);
  m.impl("tbe_build_plan", &trb::tbe_build_plan);
  m.impl("tbe_backward_apply", &trb::tbe_backward_apply);
  m.impl("tbe_backward_apply_dist", &trb::tbe_backward_apply_dist);
  m.impl("tbe_seq_forward_dist", &trb::tbe_seq_forward_dist);
}

TORCH_LIBRARY_IMPL(trb200, CompositeExplicitAutograd, m) { m.impl("tbe_forward_dist", &trb::tbe_forward_dist); }
