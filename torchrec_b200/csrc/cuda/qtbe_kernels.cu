// Quantized table-batched embedding lookup for inference (int8 / int4 / int2 rows, fp16 or fp32 rows too).
//
// Row format (row-wise N-bit quantization): D * bits / 8 payload bytes, then an fp16 scale and an fp16 bias:
//   value[j] = scale * q[j] + bias.    Rows of one table are contiguous; different tables may use different bits.
// One warp per bag; lane l owns elements [4l, 4l+4) (+128 per extra vector).  For int8 that is one 4-byte load per
// row, for int4 a 2-byte load, for int2 a 1-byte load; accumulation in fp32; output fp16 / bf16 / fp32 written
// straight into the [B, total_D] result.  The same kernel serves pooled (sum / mean / per-sample weights) and
// unpooled lookups (pooling = 2: one output row per id).
//
// The reference gets this from an external kernel wheel (IntNBitTableBatchedEmbeddingBagsCodegen, call sites
// torchrec/quant/embedding_modules.py:332-560).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <ATen/cuda/PeerToPeerAccess.h>

#include "common.cuh"

namespace trb {

// per-feature metadata rows of the int64 [kQMetaRows, F] tensor
enum QMetaRow : int { QM_WOFF = 0 /*byte offset of the table*/, QM_ROWS = 1, QM_DIM = 2, QM_OUTOFF = 3, QM_BITS = 4 /*32,16,8,4,2*/, kQMetaRows = 5 };

struct QFwdParams {
  const uint8_t* weights;
  const int64_t* meta;
  const void* indices;
  const void* offsets;
  const float* psw;
  void* out;
  int out_dtype;
  int64_t out_stride;
  int B, F, pooling;  // 0 sum, 1 mean, 2 none
  int* err;
};

__device__ __forceinline__ int64_t qrow_bytes(int D, int bits) { return bits >= 16 ? int64_t(D) * bits / 8 : int64_t(D) * bits / 8 + 4; }

// elements [e, e+4) of one row as fp32; BITS is a compile-time constant so that the loads of several rows can be issued
// back to back without a branch between them
template <int BITS>
__device__ __forceinline__ float4 qload4(const uint8_t* row, int D, int e) {
  if (BITS == 32) return __ldg(reinterpret_cast<const float4*>(row + int64_t(e) * 4));
  if (BITS == 16) return Vec4<__half>::load(reinterpret_cast<const __half*>(row) + e);
  const __half2 sb = *reinterpret_cast<const __half2*>(row + int64_t(D) * BITS / 8);
  const float scale = __low2float(sb), bias = __high2float(sb);
  uint32_t q0, q1, q2, q3;
  if (BITS == 8) {
    const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(row + e));
    q0 = w & 0xff; q1 = (w >> 8) & 0xff; q2 = (w >> 16) & 0xff; q3 = w >> 24;
  } else if (BITS == 4) {
    const uint32_t w = __ldg(reinterpret_cast<const uint16_t*>(row + e / 2));
    q0 = w & 0xf; q1 = (w >> 4) & 0xf; q2 = (w >> 8) & 0xf; q3 = (w >> 12) & 0xf;
  } else {  // 2 bits
    const uint32_t w = __ldg(row + e / 4);
    q0 = w & 3; q1 = (w >> 2) & 3; q2 = (w >> 4) & 3; q3 = (w >> 6) & 3;
  }
  return make_float4(fmaf(scale, float(q0), bias), fmaf(scale, float(q1), bias), fmaf(scale, float(q2), bias), fmaf(scale, float(q3), bias));
}


// One bag (ids [start, end)) of one table.  Ids and weights are fetched 32 at a time, one per lane, and handed round by
// shuffles; rows are then read kQUnroll at a time so that a warp keeps several DRAM requests in flight instead of one.
template <int BITS, typename idx_t, int kVecs>
__device__ __forceinline__ void qbag(const QFwdParams& p, const uint8_t* table, int64_t rb, int D, int64_t rows, int64_t start,
                                     int64_t end, int lane, float4 (&acc)[kVecs]) {
  constexpr int kQUnroll = kVecs >= 4 ? 2 : 4;  // rows whose loads are in flight together per warp (bounded by registers)
  const idx_t* indices = reinterpret_cast<const idx_t*>(p.indices);
  const bool unpooled = p.pooling == 2;
  for (int64_t c = start; c < end; c += 32) {
    const int n = int(min(int64_t(32), end - c));
    int64_t my_r = 0;
    float my_w = 0.f;
    if (lane < n) {
      my_r = int64_t(indices[c + lane]);
      my_w = p.psw ? p.psw[c + lane] : 1.f;
      if (my_r < 0 || my_r >= rows) {
        atomicExch(p.err, 1);
        my_r = 0;
        my_w = 0.f;
      }
    }
    for (int j0 = 0; j0 < n; j0 += kQUnroll) {
      float4 x[kQUnroll][kVecs];
      float w[kQUnroll];
#pragma unroll
      for (int u = 0; u < kQUnroll; ++u) {
        const int j = min(j0 + u, n - 1);  // the tail re-reads the last row (weight 0 below)
        const int64_t r = __shfl_sync(0xffffffffu, my_r, j);
        w[u] = (j0 + u < n) ? __shfl_sync(0xffffffffu, my_w, j) : 0.f;
        const uint8_t* row = table + r * rb;
#pragma unroll
        for (int v = 0; v < kVecs; ++v) {
          const int e = v * 128 + lane * 4;
          x[u][v] = e < D ? qload4<BITS>(row, D, e) : f4zero();
        }
      }
#pragma unroll
      for (int u = 0; u < kQUnroll; ++u) {
        if (unpooled) {
          if (j0 + u < n) {
#pragma unroll
            for (int v = 0; v < kVecs; ++v) {
              const int e = v * 128 + lane * 4;
              if (e < D) {
                float4 y = x[u][v];
                if (w[u] == 0.f) y = f4zero();  // an id outside the table yields a zero row
                store4_dyn(p.out, (c + j0 + u) * p.out_stride + e, y, p.out_dtype);
              }
            }
          }
        } else {
#pragma unroll
          for (int v = 0; v < kVecs; ++v) {
            acc[v].x = fmaf(w[u], x[u][v].x, acc[v].x); acc[v].y = fmaf(w[u], x[u][v].y, acc[v].y);
            acc[v].z = fmaf(w[u], x[u][v].z, acc[v].z); acc[v].w = fmaf(w[u], x[u][v].w, acc[v].w);
          }
        }
      }
    }
  }
}

// ---- low-bit rows, several rows per load instruction -------------------------------------------------------------------
// A row of D int8 / int4 values is only D or D / 2 payload bytes: with one row per warp a load instruction moves 128 bytes or
// less and a warp has a handful of requests in flight.  Here kLanes = payload / 16 lanes cover one row with a 16-byte load each
// and the 32 / kLanes groups of a warp work on DIFFERENT ids of the bag at the same time (two rounds unrolled), so one load
// instruction fetches up to eight rows.  Partial sums of the groups are combined by shuffles at the end of the bag.
template <int BITS>
__device__ __forceinline__ void qdequant16(const uint4& raw, float scale, float bias, float w, float* acc) {
  const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
  constexpr int kPerByte = 8 / BITS;
  constexpr uint32_t kMask = (1u << BITS) - 1u;
  const float ws = w * scale, wb = w * bias;
#pragma unroll
  for (int k = 0; k < 16; ++k) {
    const uint32_t byte = (words[k >> 2] >> (8 * (k & 3))) & 0xffu;
#pragma unroll
    for (int q = 0; q < kPerByte; ++q) acc[k * kPerByte + q] += fmaf(ws, float((byte >> (BITS * q)) & kMask), wb);
  }
}

template <int BITS, int kLanes, typename idx_t>
__global__ void __launch_bounds__(256) qtbe_fwd_sub_kernel(QFwdParams p) {
  constexpr int kGroups = 32 / kLanes;
  constexpr int kElems = 16 * 8 / BITS;  // elements per lane
  const int lane = threadIdx.x & 31;
  const int64_t bag = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (bag >= int64_t(p.F) * p.B) return;
  const int f = int(bag / p.B), b = int(bag - int64_t(f) * p.B);
  const int F = p.F;
  const idx_t* offsets = reinterpret_cast<const idx_t*>(p.offsets);
  const idx_t* indices = reinterpret_cast<const idx_t*>(p.indices);
  const int64_t start = offsets[bag], end = offsets[bag + 1];
  const int D = int(p.meta[QM_DIM * F + f]);
  const int64_t rows = p.meta[QM_ROWS * F + f];
  const uint8_t* table = p.weights + p.meta[QM_WOFF * F + f];
  const int payload = D * BITS / 8;
  const int64_t rb = payload + 4;
  const int out_off = int(p.meta[QM_OUTOFF * F + f]);
  const int grp = lane / kLanes, lig = lane - grp * kLanes;
  const bool unpooled = p.pooling == 2;
  float acc[kElems];
#pragma unroll
  for (int e = 0; e < kElems; ++e) acc[e] = 0.f;
  for (int64_t c = start; c < end; c += 32) {
    const int n = int(min(int64_t(32), end - c));
    int64_t my_r = 0;
    float my_w = 0.f;
    if (lane < n) {
      my_r = int64_t(indices[c + lane]);
      my_w = p.psw ? p.psw[c + lane] : 1.f;
      if (my_r < 0 || my_r >= rows) {
        atomicExch(p.err, 1);
        my_r = 0;
        my_w = 0.f;
      }
    }
    for (int j0 = 0; j0 < n; j0 += 2 * kGroups) {
      uint4 raw[2];
      __half2 sb[2];
      float w[2];
      int jj[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        jj[u] = j0 + u * kGroups + grp;
        const int src = min(jj[u], n - 1);  // groups past the end re-read the last row with weight 0
        const int64_t r = __shfl_sync(0xffffffffu, my_r, src);
        const float ww = __shfl_sync(0xffffffffu, my_w, src);
        w[u] = jj[u] < n ? ww : 0.f;
        const uint8_t* row = table + r * rb;
        // rows start at multiples of (payload + 4) bytes: 4-byte aligned only, so the 16 bytes arrive as four words
        const uint32_t* q = reinterpret_cast<const uint32_t*>(row + lig * 16);
        raw[u] = make_uint4(__ldg(q), __ldg(q + 1), __ldg(q + 2), __ldg(q + 3));
        sb[u] = *reinterpret_cast<const __half2*>(row + payload);
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const float scale = __low2float(sb[u]), bias = __high2float(sb[u]);
        if (unpooled) {
          if (jj[u] < n) {
            float rowv[kElems];
#pragma unroll
            for (int e = 0; e < kElems; ++e) rowv[e] = 0.f;
            qdequant16<BITS>(raw[u], scale, bias, w[u] == 0.f ? 0.f : 1.f, rowv);
#pragma unroll
            for (int e = 0; e < kElems; e += 4)
              store4_dyn(p.out, (c + jj[u]) * p.out_stride + lig * kElems + e, make_float4(rowv[e], rowv[e + 1], rowv[e + 2], rowv[e + 3]), p.out_dtype);
          }
        } else {
          qdequant16<BITS>(raw[u], scale, bias, w[u], acc);
        }
      }
    }
  }
  if (unpooled) return;
#pragma unroll
  for (int o = kLanes; o < 32; o <<= 1)
#pragma unroll
    for (int e = 0; e < kElems; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], o);
  if (grp != 0) return;
  const float s = (p.pooling == 1 && end > start) ? 1.f / float(end - start) : 1.f;
#pragma unroll
  for (int e = 0; e < kElems; e += 4)
    store4_dyn(p.out, int64_t(b) * p.out_stride + out_off + lig * kElems + e,
               make_float4(acc[e] * s, acc[e + 1] * s, acc[e + 2] * s, acc[e + 3] * s), p.out_dtype);
}

template <typename idx_t, int kVecs>
__global__ void __launch_bounds__(256) qtbe_fwd_kernel(QFwdParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t bag = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (bag >= int64_t(p.F) * p.B) return;
  const int f = int(bag / p.B), b = int(bag - int64_t(f) * p.B);
  const int F = p.F;
  const idx_t* offsets = reinterpret_cast<const idx_t*>(p.offsets);
  const int64_t start = offsets[bag], end = offsets[bag + 1];
  const int D = int(p.meta[QM_DIM * F + f]), bits = int(p.meta[QM_BITS * F + f]);
  const int64_t rows = p.meta[QM_ROWS * F + f];
  const uint8_t* table = p.weights + p.meta[QM_WOFF * F + f];
  const int64_t rb = qrow_bytes(D, bits);
  const int out_off = int(p.meta[QM_OUTOFF * F + f]);
  float4 acc[kVecs];
#pragma unroll
  for (int v = 0; v < kVecs; ++v) acc[v] = f4zero();
  switch (bits) {
    case 8: qbag<8, idx_t, kVecs>(p, table, rb, D, rows, start, end, lane, acc); break;
    case 4: qbag<4, idx_t, kVecs>(p, table, rb, D, rows, start, end, lane, acc); break;
    case 2: qbag<2, idx_t, kVecs>(p, table, rb, D, rows, start, end, lane, acc); break;
    case 16: qbag<16, idx_t, kVecs>(p, table, rb, D, rows, start, end, lane, acc); break;
    default: qbag<32, idx_t, kVecs>(p, table, rb, D, rows, start, end, lane, acc); break;
  }
  if (p.pooling == 2) return;
  if (p.pooling == 1 && end > start) {
    const float s = 1.f / float(end - start);
#pragma unroll
    for (int v = 0; v < kVecs; ++v) { acc[v].x *= s; acc[v].y *= s; acc[v].z *= s; acc[v].w *= s; }
  }
#pragma unroll
  for (int v = 0; v < kVecs; ++v) {
    const int e = v * 128 + lane * 4;
    if (e < D) store4_dyn(p.out, int64_t(b) * p.out_stride + out_off + e, acc[v], p.out_dtype);
  }
}

static void qtbe_launch(const at::Tensor& weights, const at::Tensor& meta, const at::Tensor& indices, const at::Tensor& offsets,
                        const c10::optional<at::Tensor>& psw, void* out, int64_t out_dtype, int64_t stride, int64_t B, int64_t max_D,
                        int64_t pooling, at::Tensor& err, int64_t sub_bits) {
  const int F = int(meta.size(1));
  QFwdParams p;
  p.weights = weights.data_ptr<uint8_t>();
  p.meta = meta.data_ptr<int64_t>();
  p.indices = indices.data_ptr();
  p.offsets = offsets.data_ptr();
  p.psw = psw.has_value() && psw->defined() ? psw->data_ptr<float>() : nullptr;
  p.out = out;
  p.out_dtype = int(out_dtype);
  p.out_stride = stride;
  p.B = int(B);
  p.F = F;
  p.pooling = int(pooling);
  p.err = err.data_ptr<int>();
  const int64_t nbags = int64_t(F) * B;
  const int64_t blocks = (nbags * 32 + 255) / 256;
  auto stream = at::cuda::getCurrentCUDAStream();
  const bool i64 = indices.scalar_type() == at::kLong;
  if (sub_bits > 0) {
    // every feature of the module has the same low-bit row format: rows shared out over lane groups
    const int lanes = int(max_D) * int(sub_bits) / 8 / 16;
#define TRB_QSUB(BITS_, LANES_)                                                                                   \
  if (sub_bits == BITS_ && lanes == LANES_) {                                                                     \
    if (i64) qtbe_fwd_sub_kernel<BITS_, LANES_, int64_t><<<blocks, 256, 0, stream>>>(p);                          \
    else qtbe_fwd_sub_kernel<BITS_, LANES_, int32_t><<<blocks, 256, 0, stream>>>(p);                              \
    TRB_CUDA_CHECK(cudaGetLastError());                                                                           \
    return;                                                                                                       \
  }
    TRB_QSUB(8, 2) TRB_QSUB(8, 4) TRB_QSUB(8, 8) TRB_QSUB(8, 16)
    TRB_QSUB(4, 1) TRB_QSUB(4, 2) TRB_QSUB(4, 4) TRB_QSUB(4, 8)
#undef TRB_QSUB
  }
  const int nv = max_D <= 128 ? 1 : (max_D <= 256 ? 2 : (max_D <= 512 ? 4 : 8));
#define TRB_Q_LAUNCH(NV)                                                                          \
  if (i64) qtbe_fwd_kernel<int64_t, NV><<<blocks, 256, 0, stream>>>(p);                             \
  else qtbe_fwd_kernel<int32_t, NV><<<blocks, 256, 0, stream>>>(p);
  if (nv == 1) { TRB_Q_LAUNCH(1) } else if (nv == 2) { TRB_Q_LAUNCH(2) } else if (nv == 4) { TRB_Q_LAUNCH(4) } else { TRB_Q_LAUNCH(8) }
#undef TRB_Q_LAUNCH
  TRB_CUDA_CHECK(cudaGetLastError());
}

static void qtbe_check(const at::Tensor& weights, const at::Tensor& meta, const at::Tensor& indices, const at::Tensor& offsets, int64_t max_D) {
  TORCH_CHECK(weights.is_cuda() && weights.scalar_type() == at::kByte && weights.is_contiguous());
  TORCH_CHECK(meta.size(0) == kQMetaRows && meta.scalar_type() == at::kLong && meta.is_contiguous());
  TORCH_CHECK(indices.scalar_type() == offsets.scalar_type(), "indices and offsets must share a dtype");
  TORCH_CHECK(max_D % 4 == 0 && max_D <= 1024, "embedding dims must be multiples of 4, at most 1024");
}

at::Tensor qtbe_forward(const at::Tensor& weights, const at::Tensor& meta, const at::Tensor& indices, const at::Tensor& offsets,
                        const c10::optional<at::Tensor>& psw, int64_t B, int64_t total_D, int64_t max_D, int64_t pooling,
                        int64_t out_dtype, at::Tensor err, int64_t uniform_bits) {
  qtbe_check(weights, meta, indices, offsets, max_D);
  const int F = int(meta.size(1));
  c10::cuda::CUDAGuard guard(weights.device());
  auto dt = out_dtype == OUT_F32 ? at::kFloat : (out_dtype == OUT_F16 ? at::kHalf : at::kBFloat16);
  at::Tensor out;
  int64_t stride;
  if (pooling == 2) {
    out = at::empty({indices.numel(), max_D}, weights.options().dtype(dt));
    stride = max_D;
  } else {
    out = at::empty({B, total_D}, weights.options().dtype(dt));
    stride = total_D;
  }
  if (F == 0 || B == 0) return out;
  qtbe_launch(weights, meta, indices, offsets, psw, out.data_ptr(), out_dtype, stride, B, max_D, pooling, err, uniform_bits);
  return out;
}

// Pooled lookup stored into an existing [B, stride] buffer at the per-feature columns of `meta` (row QM_OUTOFF).  The buffer
// may live on ANOTHER device of this process (the serving GPU that assembles the request's result): peer access is switched
// on for the pair and the rows travel over NVLink as plain stores from this kernel; no copy kernel, no concatenation.
void qtbe_forward_into(const at::Tensor& weights, const at::Tensor& meta, const at::Tensor& indices, const at::Tensor& offsets,
                       const c10::optional<at::Tensor>& psw, at::Tensor out, int64_t B, int64_t max_D, int64_t pooling, at::Tensor err,
                       int64_t uniform_bits) {
  qtbe_check(weights, meta, indices, offsets, max_D);
  TORCH_CHECK(pooling != 2, "pooled lookups only");
  TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.stride(1) == 1 && out.size(0) >= B);
  TORCH_CHECK(out.stride(0) % 4 == 0 && reinterpret_cast<uintptr_t>(out.data_ptr()) % 16 == 0,
              "rows of the output buffer must start on 16-byte boundaries (the kernel stores four elements at a time)");
  const int F = int(meta.size(1));
  if (F == 0 || B == 0) return;
  if (out.device() != weights.device()) {
    TORCH_CHECK(at::cuda::get_p2p_access(weights.device().index(), out.device().index()),
                "no peer access from device ", int(weights.device().index()), " to device ", int(out.device().index()));
  }
  c10::cuda::CUDAGuard guard(weights.device());
  const int64_t code = out.scalar_type() == at::kFloat ? OUT_F32 : (out.scalar_type() == at::kHalf ? OUT_F16 : OUT_BF16);
  TORCH_CHECK(code != OUT_BF16 || out.scalar_type() == at::kBFloat16, "output must be fp32, fp16 or bf16");
  qtbe_launch(weights, meta, indices, offsets, psw, out.data_ptr(), code, out.stride(0), B, max_D, pooling, err, uniform_bits);
}

}  // namespace trb

TORCH_LIBRARY_FRAGMENT(trb200, m) {
  m.def(
      "qtbe_forward(Tensor weights, Tensor meta, Tensor indices, Tensor offsets, Tensor? psw, int B, int total_D, int max_D, "
      "int pooling, int out_dtype, Tensor(a!) err, int uniform_bits=0) -> Tensor");
  m.def(
      "qtbe_forward_into(Tensor weights, Tensor meta, Tensor indices, Tensor offsets, Tensor? psw, Tensor(a!) out, int B, int max_D, "
      "int pooling, Tensor(b!) err, int uniform_bits=0) -> ()");
}

TORCH_LIBRARY_IMPL(trb200, CUDA, m) { m.impl("qtbe_forward", &trb::qtbe_forward); }

// dispatched by hand: `out` may sit on another device than the tables
TORCH_LIBRARY_IMPL(trb200, CompositeExplicitAutograd, m) { m.impl("qtbe_forward_into", &trb::qtbe_forward_into); }
