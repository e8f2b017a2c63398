// Serving runtime, shared declarations: the dynamic batching queue (see inference_batching_queue.cpp for the flow) that the
// executor threads of inference_executor.cpp consume.
#pragma once

#include <torch/custom_class.h>
#include <torch/library.h>
#include <torch/torch.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <mutex>
#include <thread>
#include <unordered_map>

namespace trb {
namespace inference {

struct Request {
  int64_t id;
  torch::Tensor dense, lengths, values;
  int64_t batch_size;
  std::chrono::steady_clock::time_point arrival;
};

struct Batch {
  torch::Tensor dense, lengths, values, request_ids, request_sizes;
  std::chrono::steady_clock::time_point formed_at;
  bool empty() const { return !request_ids.defined() || request_ids.numel() == 0; }
};

class BatchingQueue : public torch::CustomClassHolder {
 public:
  BatchingQueue(int64_t max_batch_size, int64_t batching_timeout_ms, int64_t num_queues, int64_t num_features, bool pin_memory)
      : max_batch_size_(max_batch_size), timeout_ms_(batching_timeout_ms), num_features_(num_features),
        pin_(pin_memory && torch::cuda::is_available()), queues_(size_t(std::max<int64_t>(num_queues, 1))) {
    worker_ = std::thread([this] { run(); });
  }
  ~BatchingQueue() override { stop(); }

  int64_t add_request(torch::Tensor dense, torch::Tensor lengths, torch::Tensor values) {
    TORCH_CHECK(dense.dim() == 2, "dense must be [b, D]");
    const int64_t b = dense.size(0);
    TORCH_CHECK(lengths.numel() == num_features_ * b, "lengths must hold num_features * b entries (feature-major)");
    TORCH_CHECK(lengths.sum().item<int64_t>() == values.numel(), "values must hold sum(lengths) ids");
    const int64_t id = next_id_.fetch_add(1);  // the id this call returns: concurrent callers must not read the counter again
    Request r{id, dense.contiguous(), lengths.contiguous().view({num_features_, b}), values.contiguous(), b,
              std::chrono::steady_clock::now()};
    {
      std::lock_guard<std::mutex> lock(mu_);
      TORCH_CHECK(!stopped_, "the queue was stopped");
      pending_.push_back(std::move(r));
      pending_samples_ += b;
    }
    cv_.notify_all();
    return id;
  }

  // (dense, lengths, values, request_ids, request_sizes); all empty when nothing arrived within the timeout
  std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor> get_batch(int64_t queue, int64_t timeout_ms) {
    TORCH_CHECK(queue >= 0 && queue < int64_t(queues_.size()));
    std::unique_lock<std::mutex> lock(mu_);
    auto& q = queues_[size_t(queue)];
    out_cv_.wait_for(lock, std::chrono::milliseconds(timeout_ms), [&] { return !q.empty() || stopped_; });
    if (q.empty()) {
      auto e = torch::empty({0});
      return {e, e, e, e, e};
    }
    Batch b = std::move(q.front());
    q.pop_front();
    return {b.dense, b.lengths, b.values, b.request_ids, b.request_sizes};
  }

  // executor side: the next batch of `queue`, or an empty Batch when none arrived within the timeout
  Batch pop_batch(int64_t queue, int64_t timeout_ms) {
    TORCH_CHECK(queue >= 0 && queue < int64_t(queues_.size()));
    std::unique_lock<std::mutex> lock(mu_);
    auto& q = queues_[size_t(queue)];
    out_cv_.wait_for(lock, std::chrono::milliseconds(timeout_ms), [&] { return !q.empty() || stopped_; });
    if (q.empty()) return Batch{};
    Batch b = std::move(q.front());
    q.pop_front();
    return b;
  }

  // fail the requests of a batch (rejected after waiting too long, or the model raised): wait_result rethrows the message
  void set_error(torch::Tensor request_ids, const std::string& message) {
    auto ids = request_ids.cpu().contiguous();
    std::lock_guard<std::mutex> lock(res_mu_);
    for (int64_t i = 0; i < ids.numel(); ++i) errors_[ids.data_ptr<int64_t>()[i]] = message;
    res_cv_.notify_all();
  }

  // results that were already cut per request (a result-split function did it)
  void set_split_results(torch::Tensor request_ids, const std::vector<torch::Tensor>& per_request) {
    auto ids = request_ids.cpu().contiguous();
    TORCH_CHECK(int64_t(per_request.size()) == ids.numel());
    std::lock_guard<std::mutex> lock(res_mu_);
    for (int64_t i = 0; i < ids.numel(); ++i) results_[ids.data_ptr<int64_t>()[i]] = per_request[size_t(i)];
    res_cv_.notify_all();
  }

  // split `output` (first dim = samples of the batch, in request order) back to the requests
  void set_results(torch::Tensor request_ids, torch::Tensor request_sizes, torch::Tensor output) {
    auto ids = request_ids.cpu().contiguous();
    auto sizes = request_sizes.cpu().contiguous();
    output = output.detach().cpu();
    int64_t off = 0;
    std::lock_guard<std::mutex> lock(res_mu_);
    for (int64_t i = 0; i < ids.numel(); ++i) {
      const int64_t n = sizes.data_ptr<int64_t>()[i];
      results_[ids.data_ptr<int64_t>()[i]] = output.narrow(0, off, n).clone();
      off += n;
    }
    res_cv_.notify_all();
  }

  torch::Tensor wait_result(int64_t request_id, int64_t timeout_ms) {
    std::unique_lock<std::mutex> lock(res_mu_);
    const bool ok = res_cv_.wait_for(lock, std::chrono::milliseconds(timeout_ms),
                                     [&] { return results_.count(request_id) > 0 || errors_.count(request_id) > 0; });
    TORCH_CHECK(ok, "request ", request_id, " produced no result within ", timeout_ms, " ms");
    if (errors_.count(request_id) > 0) {
      const std::string msg = errors_[request_id];
      errors_.erase(request_id);
      TORCH_CHECK(false, "request ", request_id, " failed: ", msg);
    }
    torch::Tensor t = results_[request_id];
    results_.erase(request_id);
    return t;
  }

  void stop() {
    {
      std::lock_guard<std::mutex> lock(mu_);
      if (stopped_) return;
      stopped_ = true;
    }
    cv_.notify_all();
    out_cv_.notify_all();
    if (worker_.joinable()) worker_.join();
  }

  int64_t batches_formed() { return batches_formed_.load(); }

 private:
  torch::Tensor maybe_pin(torch::Tensor t) { return pin_ ? t.pin_memory() : t; }

  void run() {
    size_t next_queue = 0;
    std::unique_lock<std::mutex> lock(mu_);
    while (!stopped_) {
      if (pending_.empty()) {
        cv_.wait_for(lock, std::chrono::milliseconds(50));
        continue;
      }
      const auto deadline = pending_.front().arrival + std::chrono::milliseconds(timeout_ms_);
      if (pending_samples_ < max_batch_size_ && std::chrono::steady_clock::now() < deadline) {
        cv_.wait_until(lock, deadline);
        continue;
      }
      // take requests while they fit (always at least one)
      std::vector<Request> take;
      int64_t n = 0;
      while (!pending_.empty() && (take.empty() || n + pending_.front().batch_size <= max_batch_size_)) {
        n += pending_.front().batch_size;
        pending_samples_ -= pending_.front().batch_size;
        take.push_back(std::move(pending_.front()));
        pending_.pop_front();
      }
      lock.unlock();
      Batch b = combine(take);
      b.formed_at = std::chrono::steady_clock::now();
      lock.lock();
      queues_[next_queue].push_back(std::move(b));
      next_queue = (next_queue + 1) % queues_.size();
      ++batches_formed_;
      out_cv_.notify_all();
    }
  }

  Batch combine(const std::vector<Request>& reqs) {
    std::vector<torch::Tensor> dense, ids, sizes;
    for (const auto& r : reqs) dense.push_back(r.dense);
    // sparse, feature-major: for feature f the columns of every request in turn
    std::vector<torch::Tensor> len_cols, val_parts;
    std::vector<std::vector<torch::Tensor>> per_req_vals;
    for (const auto& r : reqs) {
      auto per_feature = r.lengths.sum(1).cpu();
      std::vector<int64_t> splits(per_feature.data_ptr<int64_t>(), per_feature.data_ptr<int64_t>() + per_feature.numel());
      per_req_vals.push_back(r.values.split_with_sizes(splits));
    }
    for (int64_t f = 0; f < num_features_; ++f)
      for (size_t i = 0; i < reqs.size(); ++i) {
        len_cols.push_back(reqs[i].lengths.select(0, f));
        val_parts.push_back(per_req_vals[i][size_t(f)]);
      }
    Batch b;
    b.dense = maybe_pin(torch::cat(dense, 0));
    b.lengths = maybe_pin(torch::cat(len_cols, 0));
    b.values = maybe_pin(torch::cat(val_parts, 0));
    b.request_ids = torch::empty({int64_t(reqs.size())}, torch::kLong);
    b.request_sizes = torch::empty({int64_t(reqs.size())}, torch::kLong);
    for (size_t i = 0; i < reqs.size(); ++i) {
      b.request_ids.data_ptr<int64_t>()[i] = reqs[i].id;
      b.request_sizes.data_ptr<int64_t>()[i] = reqs[i].batch_size;
    }
    return b;
  }

  const int64_t max_batch_size_, timeout_ms_, num_features_;
  const bool pin_;
  std::mutex mu_;
  std::condition_variable cv_, out_cv_;
  std::deque<Request> pending_;
  int64_t pending_samples_ = 0;
  std::vector<std::deque<Batch>> queues_;
  bool stopped_ = false;
  std::atomic<int64_t> next_id_{0};
  std::atomic<int64_t> batches_formed_{0};
  std::thread worker_;
  std::mutex res_mu_;
  std::condition_variable res_cv_;
  std::unordered_map<int64_t, torch::Tensor> results_;
  std::unordered_map<int64_t, std::string> errors_;
};

}  // namespace inference
}  // namespace trb

