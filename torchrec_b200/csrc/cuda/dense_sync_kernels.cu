// Data-parallel side of the dense towers on one node, sm_100a:
//
//   peer_allreduce      two-shot all-reduce (reduce-scatter then all-gather) of a flat fp32 gradient buffer that lives
//                       in peer-mapped memory on every rank.  Rank r sums slice r of all ranks' buffers with plain peer
//                       loads in a fixed order (deterministic), scales it, and stores the result into slice r of every
//                       rank's buffer with plain peer stores.  Slice r of any buffer is only ever touched by rank r, so
//                       the reduction happens in place.  Entry and exit are flag handshakes with bounded waits; the
//                       kernel is persistent (one CTA per SM) so that every CTA is resident while it waits.
//   dense_optimizer     one launch updates ALL dense parameters (flat fp32 master buffer, flat gradient, flat state):
//                       Adagrad / SGD / Adam, and writes the bf16 copy the tensor-core GEMMs read plus, for matrices,
//                       the transposed bf16 copy the input-gradient GEMMs read.  This replaces one optimizer launch
//                       group and ~40 cast / transpose launches per step.
//
// The reference leaves both to libraries: DistributedDataParallel's bucketed NCCL all-reduce
// (torchrec/distributed/model_parallel.py:104-145) and torch.optim.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "common.cuh"
#include "peer_sync.cuh"

namespace trb {

struct ArParams {
  PeerPtrs buf;    // float [n] on every rank
  PeerPtrs flags;  // int32 [nslots, W]
  int rank, W, slot_in, slot_out;
  int* epochs;
  int* counter;
  int64_t n;
  float scale;
  long long wait_cycles;
  int* err;
  int signal_inside;
};

__global__ void __launch_bounds__(512) peer_allreduce_kernel(ArParams p) {
  __shared__ int s_ok, s_last, s_e_in, s_e_out;
  const int tid = threadIdx.x;
  if (tid == 0) {
    s_ok = 1;
    s_e_in = p.epochs[p.slot_in] + (p.signal_inside ? 1 : 0);
    s_e_out = p.epochs[p.slot_out] + 1;
  }
  __syncthreads();
  const int e_in = s_e_in, e_out = s_e_out;
  // entry: everybody's gradients are complete (this kernel follows the backward in stream order on every rank)
  if (p.signal_inside && blockIdx.x == 0 && tid < p.W) peer_signal_one(p.flags, tid, p.rank, p.W, p.slot_in, e_in);
  if (tid < p.W && !peer_wait_one(p.flags, tid, p.rank, p.W, p.slot_in, e_in, p.wait_cycles, p.err, 400)) s_ok = 0;
  __syncthreads();
  if (s_ok) {
    const int64_t nvec = (p.n + 3) / 4;
    const int64_t per = (nvec + p.W - 1) / p.W;
    const int64_t v0 = per * p.rank, v1 = min(nvec, v0 + per);
    for (int64_t v = v0 + int64_t(blockIdx.x) * blockDim.x + tid; v < v1; v += int64_t(gridDim.x) * blockDim.x) {
      float4 acc = f4zero();
      for (int r = 0; r < p.W; ++r) {
        const float4 x = *(reinterpret_cast<const float4*>(p.buf.p[r]) + v);
        acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
      }
      acc.x *= p.scale; acc.y *= p.scale; acc.z *= p.scale; acc.w *= p.scale;
      for (int r = 0; r < p.W; ++r) *(reinterpret_cast<float4*>(p.buf.p[r]) + v) = acc;
    }
  }
  // exit: the CTA that finishes last tells every rank that slice `rank` is in place
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    const int t = atomicAdd(p.counter, 1);
    s_last = (t == int(gridDim.x) - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence_system();
  if (tid < p.W) peer_signal_one(p.flags, tid, p.rank, p.W, p.slot_out, e_out);
  if (tid == 0) {
    if (p.signal_inside) p.epochs[p.slot_in] = e_in;
    p.epochs[p.slot_out] = e_out;
    *p.counter = 0;
  }
}

// buf_ptrs[r]: rank r's flat buffer (padded to a multiple of 4 floats).  The caller waits on `slot_out` (peer_sync)
// before reading the reduced values.
void peer_allreduce(std::vector<int64_t> buf_ptrs, int64_t n, double scale, std::vector<int64_t> flag_ptrs, int64_t rank,
                    int64_t slot_in, int64_t slot_out, at::Tensor epochs, at::Tensor counter, bool signal_inside,
                    int64_t wait_cycles, at::Tensor err) {
  const int world = int(buf_ptrs.size());
  TORCH_CHECK(world >= 1 && world <= kMaxPeers && int(flag_ptrs.size()) == world);
  TORCH_CHECK(epochs.is_cuda() && epochs.scalar_type() == at::kInt && counter.is_cuda() && counter.scalar_type() == at::kInt);
  c10::cuda::CUDAGuard guard(err.device());
  ArParams p;
  for (int i = 0; i < kMaxPeers; ++i) {
    p.buf.p[i] = i < world ? reinterpret_cast<void*>(buf_ptrs[i]) : nullptr;
    p.flags.p[i] = i < world ? reinterpret_cast<void*>(flag_ptrs[i]) : nullptr;
    TORCH_CHECK(i >= world || buf_ptrs[i] % 16 == 0, "buffers must be 16-byte aligned");
  }
  p.rank = int(rank);
  p.W = world;
  p.slot_in = int(slot_in);
  p.slot_out = int(slot_out);
  p.epochs = epochs.data_ptr<int>();
  p.counter = counter.data_ptr<int>();
  p.n = n;
  p.scale = float(scale);
  p.wait_cycles = (long long)wait_cycles;
  p.err = err.data_ptr<int>();
  p.signal_inside = signal_inside ? 1 : 0;
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  peer_allreduce_kernel<<<sms, 512, 0, at::cuda::getCurrentCUDAStream()>>>(p);
  TRB_CUDA_CHECK(cudaGetLastError());
}

// ---- fused multi-tensor optimizer ------------------------------------------------------------------------------------
// descriptor rows of the int64 [T, kDescCols] table; parameters are [rows, cols] row-major slices of the flat buffers
enum DescCol : int { DC_OFF = 0, DC_ROWS = 1, DC_COLS = 2, DC_TILE0 = 3, DC_TRANSPOSED = 4, kDescCols = 5 };
enum DenseOpt : int { DOPT_ADAGRAD = 0, DOPT_SGD = 1, DOPT_ADAM = 2 };

struct DenseOptParams {
  float* w;             // master weights
  const float* g;       // gradients
  float* s1;            // Adagrad sum / Adam m
  float* s2;            // Adam v
  __nv_bfloat16* w16;   // bf16 copy, same layout
  __nv_bfloat16* wT16;  // bf16 copy of the transposed matrices (same offsets), or null
  const int64_t* desc;
  int T;
  int opt;
  float lr, eps, beta1, beta2, weight_decay;
  const int64_t* step;  // Adam: device-side step counter (already incremented for this step)
};

__global__ void __launch_bounds__(256) dense_optimizer_kernel(DenseOptParams p) {
  __shared__ float tile[32][33];
  __shared__ int s_t;
  __shared__ float s_bc[2];
  // which tensor does this tile belong to (T is small: linear search by one thread)
  if (threadIdx.x == 0 && threadIdx.y == 0) {
    int t = 0;
    while (t + 1 < p.T && p.desc[(t + 1) * kDescCols + DC_TILE0] <= int64_t(blockIdx.x)) ++t;
    s_t = t;
    if (p.opt == DOPT_ADAM) {
      // bias corrections in double: the fast-math single-precision power is too coarse for 1 - beta^t at small t
      const double st = double(p.step[0]);
      s_bc[0] = float(1.0 - pow(double(p.beta1), st));
      s_bc[1] = float(1.0 - pow(double(p.beta2), st));
    }
  }
  __syncthreads();
  const int64_t* d = p.desc + s_t * kDescCols;
  const int64_t off = d[DC_OFF];
  const int rows = int(d[DC_ROWS]), cols = int(d[DC_COLS]);
  const int tiles_x = (cols + 31) / 32;
  const int lt = int(int64_t(blockIdx.x) - d[DC_TILE0]);
  const int ty = lt / tiles_x, tx = lt - ty * tiles_x;
  float bc1 = 1.f, bc2 = 1.f;
  if (p.opt == DOPT_ADAM) {
    bc1 = s_bc[0];
    bc2 = s_bc[1];
  }
  const int c = tx * 32 + threadIdx.x;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int rl = threadIdx.y + i * 8;
    const int r = ty * 32 + rl;
    float wn = 0.f;
    if (r < rows && c < cols) {
      const int64_t e = off + int64_t(r) * cols + c;
      float w = p.w[e], g = p.g[e];
      if (p.weight_decay != 0.f) g += p.weight_decay * w;
      if (p.opt == DOPT_ADAGRAD) {
        const float h = p.s1[e] + g * g;
        p.s1[e] = h;
        w -= p.lr * g / (sqrtf(h) + p.eps);
      } else if (p.opt == DOPT_SGD) {
        w -= p.lr * g;
      } else {
        const float m = p.beta1 * p.s1[e] + (1.f - p.beta1) * g;
        const float v = p.beta2 * p.s2[e] + (1.f - p.beta2) * g * g;
        p.s1[e] = m;
        p.s2[e] = v;
        w -= p.lr * (m / bc1) / (sqrtf(v / bc2) + p.eps);
      }
      p.w[e] = w;
      p.w16[e] = __float2bfloat16(w);
      wn = w;
    }
    tile[rl][threadIdx.x] = wn;
  }
  if (p.wT16 == nullptr || d[DC_TRANSPOSED] == 0) return;
  __syncthreads();
  // transposed copy: element (r, c) goes to [c, r] of a [cols, rows] matrix at the same offset
  const int r2 = ty * 32 + threadIdx.x;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int cl = threadIdx.y + i * 8;
    const int c2 = tx * 32 + cl;
    if (r2 < rows && c2 < cols) p.wT16[off + int64_t(c2) * rows + r2] = __float2bfloat16(tile[threadIdx.x][cl]);
  }
}

void dense_optimizer_step(at::Tensor w, const at::Tensor& g, c10::optional<at::Tensor> s1, c10::optional<at::Tensor> s2, at::Tensor w16,
                          c10::optional<at::Tensor> wT16, const at::Tensor& desc, int64_t total_tiles, int64_t opt, double lr, double eps,
                          double beta1, double beta2, double weight_decay, c10::optional<at::Tensor> step) {
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == at::kFloat && g.scalar_type() == at::kFloat && w16.scalar_type() == at::kBFloat16);
  TORCH_CHECK(g.numel() >= w.numel() && w16.numel() >= w.numel());
  TORCH_CHECK(desc.is_cuda() && desc.scalar_type() == at::kLong && desc.dim() == 2 && desc.size(1) == kDescCols && desc.is_contiguous());
  if (total_tiles == 0) return;
  c10::cuda::CUDAGuard guard(w.device());
  DenseOptParams p;
  p.w = w.data_ptr<float>();
  p.g = g.data_ptr<float>();
  p.s1 = s1.has_value() && s1->defined() ? s1->data_ptr<float>() : nullptr;
  p.s2 = s2.has_value() && s2->defined() ? s2->data_ptr<float>() : nullptr;
  p.w16 = reinterpret_cast<__nv_bfloat16*>(w16.data_ptr());
  p.wT16 = wT16.has_value() && wT16->defined() ? reinterpret_cast<__nv_bfloat16*>(wT16->data_ptr()) : nullptr;
  p.desc = desc.data_ptr<int64_t>();
  p.T = int(desc.size(0));
  p.opt = int(opt);
  p.lr = float(lr);
  p.eps = float(eps);
  p.beta1 = float(beta1);
  p.beta2 = float(beta2);
  p.weight_decay = float(weight_decay);
  p.step = step.has_value() && step->defined() ? step->data_ptr<int64_t>() : nullptr;
  TORCH_CHECK(opt != DOPT_ADAGRAD || p.s1 != nullptr, "Adagrad needs its sum buffer");
  TORCH_CHECK(opt != DOPT_ADAM || (p.s1 != nullptr && p.s2 != nullptr && p.step != nullptr), "Adam needs m, v and the step counter");
  dense_optimizer_kernel<<<unsigned(total_tiles), dim3(32, 8), 0, at::cuda::getCurrentCUDAStream()>>>(p);
  TRB_CUDA_CHECK(cudaGetLastError());
}

}  // namespace trb

TORCH_LIBRARY_FRAGMENT(trb200, m) {
  m.def(
      "peer_allreduce(int[] buf_ptrs, int n, float scale, int[] flag_ptrs, int rank, int slot_in, int slot_out, Tensor(a!) epochs, "
      "Tensor(b!) counter, bool signal_inside, int wait_cycles, Tensor(c!) err) -> ()");
  m.def(
      "dense_optimizer_step(Tensor(a!) w, Tensor g, Tensor(b!)? s1, Tensor(c!)? s2, Tensor(d!) w16, Tensor(e!)? wT16, Tensor desc, "
      "int total_tiles, int opt, float lr, float eps, float beta1, float beta2, float weight_decay, Tensor? step) -> ()");
}

TORCH_LIBRARY_IMPL(trb200, CompositeExplicitAutograd, m) {
  m.impl("peer_allreduce", &trb::peer_allreduce);
  m.impl("dense_optimizer_step", &trb::dense_optimizer_step);
}
