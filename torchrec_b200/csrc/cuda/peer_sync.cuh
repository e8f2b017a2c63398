// Device-side pieces of the flag protocol over peer-mapped memory (see peer_kernels.cu for the protocol).
#pragma once

#include "common.cuh"

namespace trb {

// raise flags[slot][rank] on peer `p` to `epoch`
__device__ __forceinline__ void peer_signal_one(const PeerPtrs& flags, int p, int rank, int world, int slot, int epoch) {
  __threadfence_system();
  int* remote = reinterpret_cast<int*>(flags.p[p]) + slot * world + rank;
  atomicMax_system(remote, epoch);
}

// wait until peer `p` has signalled `epoch` on `slot`; returns false (and records err_base + p) when the wait ran out
__device__ __forceinline__ bool peer_wait_one(const PeerPtrs& flags, int p, int rank, int world, int slot, int epoch,
                                              long long wait_cycles, int* err, int err_base) {
  volatile int* mine = reinterpret_cast<volatile int*>(flags.p[rank]) + slot * world + p;
  const long long t0 = clock64();
  while (*mine < epoch) {
    if (clock64() - t0 > wait_cycles) {
      atomicCAS(err, 0, err_base + p);
      return false;
    }
    __nanosleep(64);
  }
  __threadfence_system();
  return true;
}

}  // namespace trb
