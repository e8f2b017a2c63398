// Maps unbounded global ids to a bounded range of cache slots [0, num_embeddings).
//
// transform(): for every global id returns its slot; an id not seen before takes a free slot (lowest first) and is
// reported as (global id, slot) so that the caller can fetch its row from the parameter server.  When no slot is
// free the call stops and reports how many ids it handled; the caller evicts and retries with the rest.
// evict(n): removes the n entries the mixed LFU/LRU strategy ranks lowest and returns them as (global id, slot).
//
// Two table layouts behind one interface (`make_id_transformer("naive" | "cacheline", ...)`):
//   naive      open addressing with linear probing over a power-of-two array of 24-byte entries;
//   cacheline  the same idea over 64-byte lines of four 16-byte entries: a probe reads one line and decides hit / miss /
//              next line from it, so a lookup touches one cache line in the common case.
// A slot stack provides the free cache ids.  Counterpart of torchrec/csrc/dynamic_embedding/details/naive_id_transformer.h,
// cacheline_id_transformer.h and id_transformer_variant.h.
#pragma once

#include <cstdint>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "tde_lxu_strategy.h"

namespace trb {
namespace tde {

struct TransformOutcome {
  bool success;            // false: ran out of slots after `num_transformed` ids
  int64_t num_transformed;
  std::vector<std::pair<int64_t, int64_t>> fetch;  // (global id, slot) of ids seen for the first time
};

class IdTransformerBase {
 public:
  virtual ~IdTransformerBase() = default;
  virtual TransformOutcome transform(const int64_t* global_ids, int64_t n, int64_t* cache_ids, uint32_t time) = 0;
  virtual std::vector<std::pair<int64_t, int64_t>> evict(int64_t num_to_evict) = 0;
  virtual std::vector<std::pair<int64_t, int64_t>> save() const = 0;  // every (global id, slot) currently held
  virtual int64_t size() const = 0;
  virtual int64_t capacity() const = 0;
};

// "naive" or "cacheline"; throws std::invalid_argument for anything else
std::unique_ptr<IdTransformerBase> make_id_transformer(const std::string& variant, int64_t num_embeddings, uint16_t min_used_freq_power = 5);

class IdTransformer : public IdTransformerBase {
 public:
  explicit IdTransformer(int64_t num_embeddings, uint16_t min_used_freq_power = 5);

  using Result = TransformOutcome;

  Result transform(const int64_t* global_ids, int64_t n, int64_t* cache_ids, uint32_t time) override;
  std::vector<std::pair<int64_t, int64_t>> evict(int64_t num_to_evict) override;
  std::vector<std::pair<int64_t, int64_t>> save() const override;
  int64_t size() const override { return size_; }
  int64_t capacity() const override { return num_embeddings_; }

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

class CachelineIdTransformer : public IdTransformerBase {
 public:
  explicit CachelineIdTransformer(int64_t num_embeddings, uint16_t min_used_freq_power = 5);

  TransformOutcome transform(const int64_t* global_ids, int64_t n, int64_t* cache_ids, uint32_t time) override;
  std::vector<std::pair<int64_t, int64_t>> evict(int64_t num_to_evict) override;
  std::vector<std::pair<int64_t, int64_t>> save() const override;
  int64_t size() const override { return size_; }
  int64_t capacity() const override { return num_embeddings_; }

 private:
  static constexpr uint32_t kEmpty = 0xFFFFFFFFu, kTombstone = 0xFFFFFFFEu;  // cache_id values that mark a free entry
  static constexpr int kWays = 4;
  struct Entry {
    int64_t global_id;
    uint32_t cache_id;
    uint32_t record;  // LxuRecord bits
  };
  struct alignas(64) Line {
    Entry way[kWays];
  };
  // entry index (line * kWays + way) of the id, or of the free entry where it would go; SIZE_MAX when the table has no room
  size_t probe(int64_t global_id, bool* found) const;
  Entry& at(size_t i) { return lines_[i / kWays].way[i % kWays]; }
  const Entry& at(size_t i) const { return lines_[i / kWays].way[i % kWays]; }
  void rehash();

  int64_t num_embeddings_;
  int64_t size_ = 0;
  size_t tombstones_ = 0;
  std::vector<Line> lines_;
  size_t line_mask_;
  std::vector<int64_t> free_slots_;
  MixedLfuLruStrategy strategy_;
};

}  // namespace tde
}  // namespace trb
