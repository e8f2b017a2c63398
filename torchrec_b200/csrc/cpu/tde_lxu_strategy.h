// Mixed LFU/LRU eviction records for the dynamic-embedding id transformer.
//
// A record packs, in 32 bits, the last access time (27 bits, caller-supplied logical clock) and the base-2
// logarithm of the access frequency (5 bits).  The frequency is a probabilistic counter: a hit at level f raises
// the level with probability 2^-f, so that level f stands for about 2^f accesses.  Eviction order: lowest
// frequency level first, oldest access first inside a level.
//
// Plays the role of torchrec/csrc/dynamic_embedding/details/mixed_lfu_lru_strategy.h (record layout :30-52) with a
// xorshift generator instead of a shared bit reservoir.
#pragma once

#include <algorithm>
#include <cstdint>
#include <queue>
#include <vector>

namespace trb {
namespace tde {

struct LxuRecord {
  uint32_t bits = 0;
  static constexpr uint32_t kTimeBits = 27;
  static constexpr uint32_t kFreqBits = 5;
  static constexpr uint32_t kTimeMask = (1u << kTimeBits) - 1;
  static constexpr uint32_t kMaxFreq = (1u << kFreqBits) - 1;

  uint32_t time() const { return bits & kTimeMask; }
  uint32_t freq_power() const { return bits >> kTimeBits; }
  void set(uint32_t time, uint32_t freq_power) { bits = (time & kTimeMask) | (std::min(freq_power, kMaxFreq) << kTimeBits); }
  // eviction priority: smaller is evicted first
  uint64_t priority() const { return (uint64_t(freq_power()) << kTimeBits) | time(); }
};

class MixedLfuLruStrategy {
 public:
  explicit MixedLfuLruStrategy(uint16_t min_used_freq_power = 5, uint64_t seed = 0x9E3779B97F4A7C15ull)
      : min_used_freq_power_(min_used_freq_power), state_(seed ? seed : 1) {}

  void update_time(uint32_t time) { time_ = time; }

  // record of an id seen for the first time / seen again
  LxuRecord first_seen() const {
    LxuRecord r;
    r.set(time_, min_used_freq_power_);
    return r;
  }
  LxuRecord touched(LxuRecord old) {
    uint32_t f = old.freq_power();
    if (f < LxuRecord::kMaxFreq && coin(f)) ++f;
    LxuRecord r;
    r.set(time_, f);
    return r;
  }

  // indices (into `records`) of the `n` entries to evict, best candidates first
  template <typename GetRecord>
  std::vector<size_t> select_evictions(size_t count, size_t n, GetRecord get) const {
    using Item = std::pair<uint64_t, size_t>;
    std::priority_queue<Item> heap;  // max-heap keeps the n smallest priorities
    for (size_t i = 0; i < count; ++i) {
      LxuRecord r;
      if (!get(i, &r)) continue;
      const uint64_t pr = r.priority();
      if (heap.size() < n) heap.emplace(pr, i);
      else if (pr < heap.top().first) {
        heap.pop();
        heap.emplace(pr, i);
      }
    }
    std::vector<size_t> out(heap.size());
    for (size_t k = heap.size(); k-- > 0;) {
      out[k] = heap.top().second;
      heap.pop();
    }
    return out;
  }

 private:
  bool coin(uint32_t power) {  // true with probability 2^-power
    if (power == 0) return true;
    state_ ^= state_ << 13;
    state_ ^= state_ >> 7;
    state_ ^= state_ << 17;
    return (state_ & ((uint64_t(1) << power) - 1)) == 0;
  }
  uint16_t min_used_freq_power_;
  uint32_t time_ = 0;
  uint64_t state_;
};

}  // namespace tde
}  // namespace trb
