// Throughput probes used by the kernel benchmark to put a ceiling next to a measured figure.
//
//   mma_sync_probe   every warp issues `iters` rounds of `chains` independent mma.sync.m16n8k16 (bf16 in, fp32 accumulate) on
//                    register operands: the rate at which the warp-level tensor instruction can be issued on this GPU, with no
//                    memory traffic at all.  The packed-attention and dot-interaction kernels use that instruction.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "common.cuh"

namespace trb {

template <int CHAINS>
__global__ void __launch_bounds__(256) mma_sync_probe_kernel(float* __restrict__ sink, int iters) {
  float c[CHAINS][4];
#pragma unroll
  for (int i = 0; i < CHAINS; ++i)
#pragma unroll
    for (int k = 0; k < 4; ++k) c[i][k] = 0.f;
  uint32_t a0 = 0x3f803f80u + threadIdx.x, a1 = 0x3f803f80u, a2 = 0x3c003c00u, a3 = 0x3f803f80u, b0 = 0x3f803f80u ^ blockIdx.x, b1 = 0x3c003c00u;
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int i = 0; i < CHAINS; ++i)
      asm volatile(
          "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
          : "+f"(c[i][0]), "+f"(c[i][1]), "+f"(c[i][2]), "+f"(c[i][3])
          : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < CHAINS; ++i) s += c[i][0] + c[i][1] + c[i][2] + c[i][3];
  if (s == 12345.678f) sink[0] = s;  // keeps the products alive without a store in practice
}

// returns the number of floating-point operations the launch performs (2 * 16 * 8 * 16 per instruction)
double mma_sync_probe(at::Tensor sink, int64_t iters, int64_t chains, int64_t blocks_per_sm) {
  TORCH_CHECK(sink.is_cuda() && sink.scalar_type() == at::kFloat && sink.numel() >= 1);
  TORCH_CHECK(iters > 0 && (chains == 1 || chains == 4 || chains == 8) && blocks_per_sm >= 1 && blocks_per_sm <= 8);
  c10::cuda::CUDAGuard guard(sink.device());
  const int blocks = at::cuda::getCurrentDeviceProperties()->multiProcessorCount * int(blocks_per_sm);
  auto stream = at::cuda::getCurrentCUDAStream();
  if (chains == 1) mma_sync_probe_kernel<1><<<blocks, 256, 0, stream>>>(sink.data_ptr<float>(), int(iters));
  else if (chains == 4) mma_sync_probe_kernel<4><<<blocks, 256, 0, stream>>>(sink.data_ptr<float>(), int(iters));
  else mma_sync_probe_kernel<8><<<blocks, 256, 0, stream>>>(sink.data_ptr<float>(), int(iters));
  TRB_CUDA_CHECK(cudaGetLastError());
  return double(blocks) * 8.0 * double(iters) * double(chains) * 2.0 * 16 * 8 * 16;
}

}  // namespace trb

TORCH_LIBRARY_FRAGMENT(trb200, m) { m.def("mma_sync_probe(Tensor(a!) sink, int iters, int chains, int blocks_per_sm) -> float"); }

TORCH_LIBRARY_IMPL(trb200, CUDA, m) { m.impl("mma_sync_probe", &trb::mma_sync_probe); }
