// Cross-GPU synchronisation over peer-mapped memory (NVLink / NVSwitch) for the fused exchange paths.
//
// Every rank owns an int32 flag array `flags[nslots][world]` in its own memory, mapped into all peers, and a local
// (unshared) counter `epochs[nslots]`.  A slot is one synchronisation point of a step (split sizes published, ids
// delivered, pooled rows delivered, gradients published, ...).  Signalling slot s: the rank takes the next epoch
// e = epochs[s] + 1, publishes everything it wrote to peer memory (`__threadfence_system`), raises flags[s][rank]
// of every peer to e with a system-scope atomic max (so a flag never moves backwards, whatever the order in which
// two signals land) and stores e back.  Waiting on slot s: spin until flags[s][p] >= epochs[s] for every peer p.
// Epochs live on the device, so the same launches can be replayed from a CUDA graph: the host passes no counter.
// All ranks run the same sequence of signals, hence agree on the epoch numbers without talking.
//
// Waits are bounded by a caller-given number of SM clock cycles: on expiry the kernel stores an error code
// (100 + peer for a plain wait) in `err` and returns; it never traps and never spins for ever.  The host reads `err`
// (PeerGroup.poll_error) and raises.  One waiting kernel per rank and GPU at a time; ranks never share a GPU.
//
// The reference has no counterpart: it synchronises through library collectives
// (torchrec/distributed/comm_ops.py:574-1073).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <cstring>

#include "common.cuh"
#include "peer_sync.cuh"

namespace trb {

__global__ void peer_sync_kernel(PeerPtrs flags, int rank, int world, int slot, int* epochs, int do_signal, int do_wait,
                                 long long wait_cycles, int* err) {
  const int p = threadIdx.x;
  __shared__ int s_epoch;
  if (p == 0) s_epoch = epochs[slot] + (do_signal ? 1 : 0);
  __syncthreads();
  const int epoch = s_epoch;
  if (do_signal && p < world) peer_signal_one(flags, p, rank, world, slot, epoch);
  if (do_wait && p < world) peer_wait_one(flags, p, rank, world, slot, epoch, wait_cycles, err, 100);
  __syncthreads();
  if (do_signal && p == 0) epochs[slot] = epoch;
}

void peer_sync(std::vector<int64_t> flag_ptrs, int64_t rank, int64_t slot, at::Tensor epochs, bool signal, bool wait,
               int64_t wait_cycles, at::Tensor err) {
  const int world = int(flag_ptrs.size());
  TORCH_CHECK(world >= 1 && world <= kMaxPeers, "peer_sync supports up to ", kMaxPeers, " ranks");
  TORCH_CHECK(err.is_cuda() && err.scalar_type() == at::kInt && err.numel() >= 1);
  TORCH_CHECK(epochs.is_cuda() && epochs.scalar_type() == at::kInt && slot >= 0 && slot < epochs.numel());
  c10::cuda::CUDAGuard guard(err.device());
  PeerPtrs f;
  for (int i = 0; i < kMaxPeers; ++i) f.p[i] = i < world ? reinterpret_cast<void*>(flag_ptrs[i]) : nullptr;
  peer_sync_kernel<<<1, 32, 0, at::cuda::getCurrentCUDAStream()>>>(f, int(rank), world, int(slot), epochs.data_ptr<int>(),
                                                                   signal ? 1 : 0, wait ? 1 : 0, (long long)wait_cycles,
                                                                   err.data_ptr<int>());
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
  m.def("peer_sync(int[] flag_ptrs, int rank, int slot, Tensor(a!) epochs, bool signal, bool wait, int wait_cycles, Tensor(b!) err) -> ()");
  m.def("peer_alloc(int nbytes, Device device) -> Tensor");
  m.def("peer_handle(Tensor buf) -> Tensor");
  m.def("peer_open(Tensor handle, Device device) -> int");
  m.def("peer_close(int ptr, Device device) -> ()");
  m.def("peer_read(int ptr, int nbytes, Device device) -> Tensor");
}

TORCH_LIBRARY_IMPL(trb200, CompositeExplicitAutograd, m) {
  m.impl("peer_sync", &trb::peer_sync);
  m.impl("peer_alloc", &trb::peer_alloc);
  m.impl("peer_handle", &trb::peer_handle);
  m.impl("peer_open", &trb::peer_open);
  m.impl("peer_close", &trb::peer_close);
  m.impl("peer_read", &trb::peer_read);
}
