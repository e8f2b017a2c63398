#include "tde_ps.h"

#include <algorithm>

namespace trb {
namespace tde {

PS::PS(const std::string& table_name, c10::intrusive_ptr<LocalShardList> shards, int64_t col_size, int64_t num_optimizer_states,
       const std::string& io_url, int64_t chunk_size)
    : table_name_(table_name), shards_(std::move(shards)), col_size_(col_size), num_states_(num_optimizer_states + 1),
      chunk_size_(std::max<int64_t>(chunk_size, 1)), io_(new IO(io_url)) {
  for (const LocalShard& s : shards_->shards()) {
    TORCH_CHECK(int64_t(s.tensors.size()) == num_states_, "every shard needs the weight and ", num_optimizer_states, " optimizer state tensors");
    if (std::find(col_ids_.begin(), col_ids_.end(), s.col_start) == col_ids_.end()) col_ids_.push_back(s.col_start);
  }
  std::sort(col_ids_.begin(), col_ids_.end());
}

// per state: the pieces (one per column shard, ascending columns) of the row held in slot `cache_id`
std::vector<torch::Tensor> PS::rows_of(int64_t cache_id) {
  std::vector<torch::Tensor> out;
  for (int64_t st = 0; st < num_states_; ++st)
    for (int64_t col : col_ids_)
      for (const LocalShard& s : shards_->shards())
        if (s.col_start == col && cache_id >= s.row_start && cache_id < s.row_start + s.row_size) {
          torch::Tensor t = s.tensors[st];
          out.push_back(t.dim() >= 2 ? t.select(0, cache_id - s.row_start) : t.narrow(0, cache_id - s.row_start, 1));
        }
  return out;
}

c10::intrusive_ptr<FetchHandle> PS::fetch(torch::Tensor ids_to_fetch, int64_t time, bool reinit, double weight_init_min, double weight_init_max) {
  TORCH_CHECK(ids_to_fetch.dim() == 2 && ids_to_fetch.size(1) == 2 && ids_to_fetch.scalar_type() == torch::kLong, "ids_to_fetch must be int64 [n, 2]");
  ids_to_fetch = ids_to_fetch.contiguous().cpu();
  const int64_t n = ids_to_fetch.size(0);
  auto state = std::make_shared<FetchHandle::State>();
  if (n == 0) return c10::make_intrusive<FetchHandle>(state);
  const int64_t* p = ids_to_fetch.data_ptr<int64_t>();
  const int64_t chunks = (n + chunk_size_ - 1) / chunk_size_;
  {
    std::lock_guard<std::mutex> lock(state->mu);
    state->pending = int(chunks);
  }
  for (int64_t c = 0; c < chunks; ++c) {
    const int64_t lo = c * chunk_size_, hi = std::min(n, lo + chunk_size_);
    std::vector<int64_t> gids(hi - lo), slots(hi - lo);
    for (int64_t i = lo; i < hi; ++i) {
      gids[i - lo] = p[2 * i];
      slots[i - lo] = p[2 * i + 1];
    }
    io_->fetch(table_name_, gids, col_ids_, uint32_t(num_states_), [this, state, slots, reinit, weight_init_min, weight_init_max](IO::Fetched f) {
      torch::NoGradGuard guard;
      for (size_t i = 0; i < slots.size(); ++i) {
        auto rows = rows_of(slots[i]);
        const size_t ncols = col_ids_.size();
        for (int64_t st = 0; st < num_states_; ++st) {
          const std::vector<float>& v = f.data[i * num_states_ + st];
          size_t off = 0;
          for (size_t c = 0; c < ncols; ++c) {
            torch::Tensor dst = rows[st * ncols + c];
            if (!v.empty()) {
              const int64_t len = dst.numel();
              TORCH_CHECK(off + len <= v.size(), "stored row is shorter than the local row");
              dst.copy_(torch::from_blob(const_cast<float*>(v.data() + off), {len}, torch::kFloat).view(dst.sizes()));
              off += len;
            } else if (reinit) {
              if (st == 0) dst.uniform_(weight_init_min, weight_init_max);
              else dst.zero_();
            }
          }
        }
      }
      std::lock_guard<std::mutex> lock(state->mu);
      if (--state->pending == 0) state->cv.notify_all();
    });
  }
  (void)time;
  return c10::make_intrusive<FetchHandle>(state);
}

void PS::evict(torch::Tensor ids_to_evict) {
  TORCH_CHECK(ids_to_evict.dim() == 2 && ids_to_evict.size(1) == 2 && ids_to_evict.scalar_type() == torch::kLong, "ids_to_evict must be int64 [n, 2]");
  ids_to_evict = ids_to_evict.contiguous().cpu();
  const int64_t n = ids_to_evict.size(0);
  if (n == 0) return;
  const int64_t* p = ids_to_evict.data_ptr<int64_t>();
  std::vector<uint32_t> state_ids(num_states_);
  for (int64_t s = 0; s < num_states_; ++s) state_ids[s] = uint32_t(s);
  auto state = std::make_shared<FetchHandle::State>();
  const int64_t chunks = (n + chunk_size_ - 1) / chunk_size_;
  state->pending = int(chunks);
  for (int64_t c = 0; c < chunks; ++c) {
    const int64_t lo = c * chunk_size_, hi = std::min(n, lo + chunk_size_);
    std::vector<int64_t> gids;
    std::vector<float> data;
    std::vector<uint64_t> offsets{0};
    for (int64_t i = lo; i < hi; ++i) {
      gids.push_back(p[2 * i]);
      auto rows = rows_of(p[2 * i + 1]);
      const size_t ncols = col_ids_.size();
      for (int64_t st = 0; st < num_states_; ++st) {
        for (size_t cc = 0; cc < ncols; ++cc) {
          torch::Tensor r = rows[st * ncols + cc].detach().to(torch::kCPU, torch::kFloat).contiguous().view(-1);
          data.insert(data.end(), r.data_ptr<float>(), r.data_ptr<float>() + r.numel());
        }
        offsets.push_back(data.size());
      }
    }
    io_->push(table_name_, gids, col_ids_, state_ids, data, offsets, [state] {
      std::lock_guard<std::mutex> lock(state->mu);
      if (--state->pending == 0) state->cv.notify_all();
    });
  }
  std::unique_lock<std::mutex> lock(state->mu);
  state->cv.wait(lock, [&] { return state->pending == 0; });
}

}  // namespace tde
}  // namespace trb
