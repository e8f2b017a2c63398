// Hash and bucket arithmetic shared by the device and the host implementation of the multi-probe
// zero-collision hash, so that both place an id in the same slot.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define TRB_HD __host__ __device__ __forceinline__
#else
#define TRB_HD inline
#endif

namespace trb {

// 64-bit finalizer (splitmix64): every input bit influences every output bit.
TRB_HD uint64_t zch_mix(uint64_t x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}

// Bucket of an id: ids are dealt round-robin over the buckets when the id space is unbounded
// (input_hash_size == 0), otherwise the id space is cut into equal contiguous blocks -- the same rule the
// row-wise input distribution uses, so an id always lands on the rank that owns its bucket.
TRB_HD int64_t zch_bucket(int64_t id, int64_t input_hash_size, int64_t num_buckets) {
  if (input_hash_size == 0) {
    int64_t b = id % num_buckets;
    return b < 0 ? b + num_buckets : b;
  }
  const int64_t blk = (input_hash_size + num_buckets - 1) / num_buckets;
  int64_t b = id / blk;
  return b < 0 ? 0 : (b >= num_buckets ? num_buckets - 1 : b);
}

enum ZchPolicy : int { ZCH_NO_EVICT = 0, ZCH_TTL = 1, ZCH_LRU = 2 };

}  // namespace trb
