// Cross-GPU synchronisation over peer-mapped memory (NVLink / NVSwitch) for the fused lookup + exchange path.
//
// Every rank owns an int32 flag array `flags[world]` in its own memory, mapped into all peers.  Barrier number `e`
// (e grows by one per call, the same on all ranks): rank r publishes everything it has written to peer memory
// (`__threadfence_system`), stores `e` into flags[r] of every peer, then waits until its own flags[p] >= e for
// every peer p.  A stream that runs "push kernel, barrier" therefore sees the pushes of all peers after the
// barrier.  The wait is bounded (about one second of SM clock): on expiry the kernel records an error code and
// returns, it never traps and never spins for ever.  One kernel per rank and GPU; ranks never share a GPU.
//
// The reference has no counterpart: it exchanges pooled embeddings with library all-to-all / reduce-scatter calls
// (torchrec/distributed/comm_ops.py:574-1073).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <cstring>

#include "common.cuh"

namespace trb {

constexpr long long kBarrierWaitCycles = 2000000000LL;

__global__ void peer_barrier_kernel(PeerPtrs flags, int rank, int world, int epoch, int* err) {
  const int p = threadIdx.x;
  if (p >= world) return;
  __threadfence_system();
  volatile int* remote = reinterpret_cast<volatile int*>(flags.p[p]) + rank;
  *remote = epoch;
  __threadfence_system();
  volatile int* mine = reinterpret_cast<volatile int*>(flags.p[rank]) + p;
  const long long t0 = clock64();
  while (*mine < epoch) {
    if (clock64() - t0 > kBarrierWaitCycles) {
      atomicCAS(err, 0, 100 + p);  // which peer never arrived
      return;
    }
  }
  __threadfence_system();
}

void peer_barrier(std::vector<int64_t> flag_ptrs, int64_t rank, int64_t epoch, at::Tensor err) {
  const int world = int(flag_ptrs.size());
  TORCH_CHECK(world >= 1 && world <= kMaxPeers, "peer_barrier supports up to ", kMaxPeers, " ranks");
  TORCH_CHECK(err.is_cuda() && err.scalar_type() == at::kInt && err.numel() >= 1);
  c10::cuda::CUDAGuard guard(err.device());
  PeerPtrs f;
  for (int i = 0; i < kMaxPeers; ++i) f.p[i] = i < world ? reinterpret_cast<void*>(flag_ptrs[i]) : nullptr;
  peer_barrier_kernel<<<1, 32, 0, at::cuda::getCurrentCUDAStream()>>>(f, int(rank), world, int(epoch), err.data_ptr<int>());
  TRB_CUDA_CHECK(cudaGetLastError());
}

// ---- buffers that other processes of the node can map ----------------------------------------------------------
// The buffer comes from cudaMalloc directly (not from the tensor library's caching allocator): an inter-process
// handle names a whole allocation, and a peer maps it with cudaIpcOpenMemHandle while ITS OWN device is current
// and with lazy peer access, so that the driver sets up the NVLink mapping for exactly the device whose kernels
// will touch the memory.

at::Tensor peer_alloc(int64_t nbytes, at::Device device) {
  TORCH_CHECK(device.is_cuda() && nbytes > 0);
  c10::cuda::CUDAGuard guard(device);
  void* ptr = nullptr;
  const int64_t padded = (nbytes + 255) / 256 * 256;
  TRB_CUDA_CHECK(cudaMalloc(&ptr, size_t(padded)));
  TRB_CUDA_CHECK(cudaMemset(ptr, 0, size_t(padded)));
  TRB_CUDA_CHECK(cudaDeviceSynchronize());
  return at::from_blob(ptr, {nbytes}, [](void* p) { cudaFree(p); }, at::TensorOptions().dtype(at::kByte).device(device));
}

// 64-byte inter-process handle of a buffer made by peer_alloc (a CPU uint8 tensor, safe to pickle)
at::Tensor peer_handle(const at::Tensor& buf) {
  TORCH_CHECK(buf.is_cuda());
  c10::cuda::CUDAGuard guard(buf.device());
  cudaIpcMemHandle_t h;
  TRB_CUDA_CHECK(cudaIpcGetMemHandle(&h, buf.data_ptr()));
  at::Tensor out = at::empty({int64_t(sizeof(h))}, at::TensorOptions().dtype(at::kByte));
  std::memcpy(out.data_ptr(), &h, sizeof(h));
  return out;
}

// Map a peer's buffer for kernels of `device`; returns the device address in this process.
int64_t peer_open(const at::Tensor& handle, at::Device device) {
  TORCH_CHECK(!handle.is_cuda() && handle.scalar_type() == at::kByte && handle.numel() == int64_t(sizeof(cudaIpcMemHandle_t)));
  c10::cuda::CUDAGuard guard(device);
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle.data_ptr(), sizeof(h));
  void* ptr = nullptr;
  TRB_CUDA_CHECK(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return reinterpret_cast<int64_t>(ptr);
}

void peer_close(int64_t ptr, at::Device device) {
  c10::cuda::CUDAGuard guard(device);
  cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr));
}

// Host-driven check that `nbytes` at a mapped peer address can be read from `device`: an asynchronous device-to-device
// copy into a fresh local tensor, which the caller compares with what the peer wrote.  A copy that the driver
// refuses comes back as an error code, not as a fault.
at::Tensor peer_read(int64_t ptr, int64_t nbytes, at::Device device) {
  c10::cuda::CUDAGuard guard(device);
  at::Tensor out = at::empty({nbytes}, at::TensorOptions().dtype(at::kByte).device(device));
  auto stream = at::cuda::getCurrentCUDAStream();
  TRB_CUDA_CHECK(cudaMemcpyAsync(out.data_ptr(), reinterpret_cast<const void*>(ptr), size_t(nbytes), cudaMemcpyDeviceToDevice, stream));
  TRB_CUDA_CHECK(cudaStreamSynchronize(stream));
  return out;
}

}  // namespace trb

TORCH_LIBRARY_FRAGMENT(trb200, m) {
  m.def("peer_barrier(int[] flag_ptrs, int rank, int epoch, Tensor(a!) err) -> ()");
  m.def("peer_alloc(int nbytes, Device device) -> Tensor");
  m.def("peer_handle(Tensor buf) -> Tensor");
  m.def("peer_open(Tensor handle, Device device) -> int");
  m.def("peer_close(int ptr, Device device) -> ()");
  m.def("peer_read(int ptr, int nbytes, Device device) -> Tensor");
}

TORCH_LIBRARY_IMPL(trb200, CompositeExplicitAutograd, m) {
  m.impl("peer_barrier", &trb::peer_barrier);
  m.impl("peer_alloc", &trb::peer_alloc);
  m.impl("peer_handle", &trb::peer_handle);
  m.impl("peer_open", &trb::peer_open);
  m.impl("peer_close", &trb::peer_close);
  m.impl("peer_read", &trb::peer_read);
}
