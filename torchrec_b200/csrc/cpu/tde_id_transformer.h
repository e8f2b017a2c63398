// Maps unbounded global ids to a bounded range of cache slots [0, num_embeddings).
//
// transform(): for every global id returns its slot; an id not seen before takes a free slot (lowest first) and is
// reported as (global id, slot) so that the caller can fetch its row from the parameter server.  When no slot is
// free the call stops and reports how many ids it handled; the caller evicts and retries with the rest.
// evict(n): removes the n entries the mixed LFU/LRU strategy ranks lowest and returns them as (global id, slot).
//
// The table is open-addressing with linear probing over a power-of-two array; a slot stack provides the free cache
// ids.  Counterpart of torchrec/csrc/dynamic_embedding/details/naive_id_transformer.h and id_transformer_wrapper.h.
#pragma once

#include <cstdint>
#include <utility>
#include <vector>

#include "tde_lxu_strategy.h"

namespace trb {
namespace tde {

class IdTransformer {
 public:
  explicit IdTransformer(int64_t num_embeddings, uint16_t min_used_freq_power = 5);

  struct Result {
    bool success;            // false: ran out of slots after `num_transformed` ids
    int64_t num_transformed;
    std::vector<std::pair<int64_t, int64_t>> fetch;  // (global id, slot) of ids seen for the first time
  };

  Result transform(const int64_t* global_ids, int64_t n, int64_t* cache_ids, uint32_t time);
  std::vector<std::pair<int64_t, int64_t>> evict(int64_t num_to_evict);
  std::vector<std::pair<int64_t, int64_t>> save() const;  // every (global id, slot) currently held
  int64_t size() const { return size_; }
  int64_t capacity() const { return num_embeddings_; }

 private:
  struct Entry {
    int64_t global_id;
    int64_t cache_id;
    LxuRecord record;
    uint8_t state;  // 0 empty, 1 used, 2 tombstone
  };
  size_t probe(int64_t global_id, bool* found) const;
  void rehash();

  int64_t num_embeddings_;
  int64_t size_ = 0;
  size_t tombstones_ = 0;
  std::vector<Entry> table_;
  size_t mask_;
  std::vector<int64_t> free_slots_;  // stack, lowest slot on top
  MixedLfuLruStrategy strategy_;
};

}  // namespace tde
}  // namespace trb
