// Parameter-server client of one embedding table: moves rows (and their optimizer states) between a remote
// key-value store and the local shard tensors that back the HBM cache.
//
//   fetch(ids_to_fetch [n,2] = (global id, cache slot), ...) -> FetchHandle   asynchronous; rows found in the store are
//        copied into the local shard that owns the slot; rows not found are (optionally) re-initialised uniformly.
//   evict(ids_to_evict [n,2])                                                  synchronous; rows are read from the shards
//        and pushed to the store in chunks.
//
// `LocalShardList` describes the local shards: per shard its row / column range and the tensors (weight, optimizer
// states) holding them.  Counterpart of torchrec/csrc/dynamic_embedding/ps.{h,cpp}.
#pragma once

#include <torch/custom_class.h>
#include <torch/torch.h>

#include <condition_variable>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "tde_io.h"

namespace trb {
namespace tde {

struct LocalShard {
  int64_t row_start, col_start, row_size, col_size;
  std::vector<torch::Tensor> tensors;  // [weight, optimizer state 0, ...], each [row_size, col_size]-shaped (or [row_size])
};

class LocalShardList : public torch::CustomClassHolder {
 public:
  void emplace_back(int64_t row_start, int64_t col_start, int64_t row_size, int64_t col_size, std::vector<torch::Tensor> tensors) {
    shards_.push_back(LocalShard{row_start, col_start, row_size, col_size, std::move(tensors)});
  }
  const std::vector<LocalShard>& shards() const { return shards_; }
  int64_t size() const { return int64_t(shards_.size()); }

 private:
  std::vector<LocalShard> shards_;
};

class FetchHandle : public torch::CustomClassHolder {
 public:
  struct State {
    std::mutex mu;
    std::condition_variable cv;
    int pending = 0;
  };
  explicit FetchHandle(std::shared_ptr<State> s) : state_(std::move(s)) {}
  void wait() {
    if (!state_) return;
    std::unique_lock<std::mutex> lock(state_->mu);
    state_->cv.wait(lock, [&] { return state_->pending == 0; });
  }

 private:
  std::shared_ptr<State> state_;
};

class PS : public torch::CustomClassHolder {
 public:
  PS(const std::string& table_name, c10::intrusive_ptr<LocalShardList> shards, int64_t col_size, int64_t num_optimizer_states,
     const std::string& io_url, int64_t chunk_size);

  c10::intrusive_ptr<FetchHandle> fetch(torch::Tensor ids_to_fetch, int64_t time, bool reinit, double weight_init_min, double weight_init_max);
  void evict(torch::Tensor ids_to_evict);

 private:
  std::vector<torch::Tensor> rows_of(int64_t cache_id);  // views of the slot's row in every state tensor, column shards in order
  std::string table_name_;
  c10::intrusive_ptr<LocalShardList> shards_;
  int64_t col_size_;
  int64_t num_states_;  // weight + optimizer states
  std::vector<int64_t> col_ids_;
  int64_t chunk_size_;
  std::unique_ptr<IO> io_;
};

}  // namespace tde
}  // namespace trb
