#include "tde_id_transformer.h"

#include <stdexcept>

namespace trb {
namespace tde {

static inline uint64_t mix(uint64_t x) {
  x ^= x >> 33;
  x *= 0xff51afd7ed558ccdull;
  x ^= x >> 33;
  x *= 0xc4ceb9fe1a85ec53ull;
  x ^= x >> 33;
  return x;
}

IdTransformer::IdTransformer(int64_t num_embeddings, uint16_t min_used_freq_power)
    : num_embeddings_(num_embeddings), strategy_(min_used_freq_power) {
  if (num_embeddings <= 0) throw std::invalid_argument("num_embeddings must be positive");
  size_t cap = 16;
  while (cap < size_t(num_embeddings) * 2) cap <<= 1;  // load factor <= 0.5
  table_.assign(cap, Entry{0, 0, LxuRecord{}, 0});
  mask_ = cap - 1;
  free_slots_.reserve(num_embeddings);
  for (int64_t s = num_embeddings - 1; s >= 0; --s) free_slots_.push_back(s);
}

size_t IdTransformer::probe(int64_t global_id, bool* found) const {
  size_t i = mix(uint64_t(global_id)) & mask_;
  size_t first_free = SIZE_MAX;
  for (size_t step = 0; step <= mask_; ++step, i = (i + 1) & mask_) {
    const Entry& e = table_[i];
    if (e.state == 1 && e.global_id == global_id) {
      *found = true;
      return i;
    }
    if (e.state == 2 && first_free == SIZE_MAX) first_free = i;
    if (e.state == 0) {
      *found = false;
      return first_free != SIZE_MAX ? first_free : i;
    }
  }
  *found = false;
  return first_free;
}

void IdTransformer::rehash() {
  std::vector<Entry> old;
  old.swap(table_);
  table_.assign(old.size(), Entry{0, 0, LxuRecord{}, 0});
  tombstones_ = 0;
  for (const Entry& e : old) {
    if (e.state != 1) continue;
    bool found;
    table_[probe(e.global_id, &found)] = e;
  }
}

IdTransformer::Result IdTransformer::transform(const int64_t* global_ids, int64_t n, int64_t* cache_ids, uint32_t time) {
  strategy_.update_time(time);
  Result res{true, 0, {}};
  for (int64_t k = 0; k < n; ++k) {
    const int64_t gid = global_ids[k];
    bool found;
    size_t pos = probe(gid, &found);
    if (found) {
      Entry& e = table_[pos];
      e.record = strategy_.touched(e.record);
      cache_ids[k] = e.cache_id;
    } else {
      if (free_slots_.empty()) {
        res.success = false;
        return res;
      }
      const int64_t slot = free_slots_.back();
      free_slots_.pop_back();
      if (table_[pos].state == 2) --tombstones_;
      table_[pos] = Entry{gid, slot, strategy_.first_seen(), 1};
      ++size_;
      cache_ids[k] = slot;
      res.fetch.emplace_back(gid, slot);
    }
    ++res.num_transformed;
  }
  return res;
}

std::vector<std::pair<int64_t, int64_t>> IdTransformer::evict(int64_t num_to_evict) {
  std::vector<std::pair<int64_t, int64_t>> out;
  if (num_to_evict <= 0 || size_ == 0) return out;
  auto picks = strategy_.select_evictions(table_.size(), size_t(num_to_evict), [&](size_t i, LxuRecord* r) {
    if (table_[i].state != 1) return false;
    *r = table_[i].record;
    return true;
  });
  out.reserve(picks.size());
  for (size_t i : picks) {
    Entry& e = table_[i];
    out.emplace_back(e.global_id, e.cache_id);
    free_slots_.push_back(e.cache_id);
    e.state = 2;
    ++tombstones_;
    --size_;
  }
  if (tombstones_ > table_.size() / 4) rehash();
  return out;
}

std::vector<std::pair<int64_t, int64_t>> IdTransformer::save() const {
  std::vector<std::pair<int64_t, int64_t>> out;
  out.reserve(size_);
  for (const Entry& e : table_)
    if (e.state == 1) out.emplace_back(e.global_id, e.cache_id);
  return out;
}

// ---- the cache-line layout ------------------------------------------------------------------------------------------------
CachelineIdTransformer::CachelineIdTransformer(int64_t num_embeddings, uint16_t min_used_freq_power)
    : num_embeddings_(num_embeddings), strategy_(min_used_freq_power) {
  if (num_embeddings <= 0) throw std::invalid_argument("num_embeddings must be positive");
  if (uint64_t(num_embeddings) >= uint64_t(kTombstone)) throw std::invalid_argument("the cache-line layout stores 32-bit slots");
  size_t lines = 4;
  while (lines * kWays < size_t(num_embeddings) * 2) lines <<= 1;  // load factor <= 0.5
  Line blank;
  for (auto& e : blank.way) e = Entry{0, kEmpty, 0};
  lines_.assign(lines, blank);
  line_mask_ = lines - 1;
  free_slots_.reserve(num_embeddings);
  for (int64_t s = num_embeddings - 1; s >= 0; --s) free_slots_.push_back(s);
}

size_t CachelineIdTransformer::probe(int64_t global_id, bool* found) const {
  size_t line = mix(uint64_t(global_id)) & line_mask_;
  size_t first_free = SIZE_MAX;
  for (size_t step = 0; step <= line_mask_; ++step, line = (line + 1) & line_mask_) {
    const Line& l = lines_[line];
    bool saw_empty = false;
    for (int w = 0; w < kWays; ++w) {
      const Entry& e = l.way[w];
      if (e.cache_id < kTombstone) {
        if (e.global_id == global_id) {
          *found = true;
          return line * kWays + w;
        }
        continue;
      }
      if (first_free == SIZE_MAX) first_free = line * kWays + w;
      if (e.cache_id == kEmpty) saw_empty = true;
    }
    if (saw_empty) break;  // an id is never stored past a line that still had a never-used entry
  }
  *found = false;
  return first_free;
}

void CachelineIdTransformer::rehash() {
  std::vector<Line> old;
  old.swap(lines_);
  Line blank;
  for (auto& e : blank.way) e = Entry{0, kEmpty, 0};
  lines_.assign(old.size(), blank);
  tombstones_ = 0;
  for (const Line& l : old)
    for (const Entry& e : l.way) {
      if (e.cache_id >= kTombstone) continue;
      bool found;
      at(probe(e.global_id, &found)) = e;
    }
}

TransformOutcome CachelineIdTransformer::transform(const int64_t* global_ids, int64_t n, int64_t* cache_ids, uint32_t time) {
  strategy_.update_time(time);
  TransformOutcome res{true, 0, {}};
  for (int64_t k = 0; k < n; ++k) {
    const int64_t gid = global_ids[k];
    bool found;
    const size_t pos = probe(gid, &found);
    if (found) {
      Entry& e = at(pos);
      LxuRecord r;
      r.bits = e.record;
      e.record = strategy_.touched(r).bits;
      cache_ids[k] = int64_t(e.cache_id);
    } else {
      if (free_slots_.empty() || pos == SIZE_MAX) {
        res.success = false;
        return res;
      }
      const int64_t slot = free_slots_.back();
      free_slots_.pop_back();
      if (at(pos).cache_id == kTombstone) --tombstones_;
      at(pos) = Entry{gid, uint32_t(slot), strategy_.first_seen().bits};
      ++size_;
      cache_ids[k] = slot;
      res.fetch.emplace_back(gid, slot);
    }
    ++res.num_transformed;
  }
  return res;
}

std::vector<std::pair<int64_t, int64_t>> CachelineIdTransformer::evict(int64_t num_to_evict) {
  std::vector<std::pair<int64_t, int64_t>> out;
  if (num_to_evict <= 0 || size_ == 0) return out;
  auto picks = strategy_.select_evictions(lines_.size() * kWays, size_t(num_to_evict), [&](size_t i, LxuRecord* r) {
    const Entry& e = at(i);
    if (e.cache_id >= kTombstone) return false;
    r->bits = e.record;
    return true;
  });
  out.reserve(picks.size());
  for (size_t i : picks) {
    Entry& e = at(i);
    out.emplace_back(e.global_id, int64_t(e.cache_id));
    free_slots_.push_back(int64_t(e.cache_id));
    e.cache_id = kTombstone;
    ++tombstones_;
    --size_;
  }
  if (tombstones_ > lines_.size() * kWays / 4) rehash();
  return out;
}

std::vector<std::pair<int64_t, int64_t>> CachelineIdTransformer::save() const {
  std::vector<std::pair<int64_t, int64_t>> out;
  out.reserve(size_);
  for (const Line& l : lines_)
    for (const Entry& e : l.way)
      if (e.cache_id < kTombstone) out.emplace_back(e.global_id, int64_t(e.cache_id));
  return out;
}

std::unique_ptr<IdTransformerBase> make_id_transformer(const std::string& variant, int64_t num_embeddings, uint16_t min_used_freq_power) {
  if (variant == "naive") return std::make_unique<IdTransformer>(num_embeddings, min_used_freq_power);
  if (variant == "cacheline") return std::make_unique<CachelineIdTransformer>(num_embeddings, min_used_freq_power);
  throw std::invalid_argument("unknown id transformer variant '" + variant + "' (naive | cacheline)");
}

}  // namespace tde
}  // namespace trb
