// Serving runtime, execution side (C++, no interpreter in the request path):
//
//   Validation       cheap structural checks of a request before it is queued (sparse: lengths non-negative and summing to the
//                    number of ids, weights as long as the ids; dense: batch x features elements).
//   batching funcs   a registry name -> function that merges the tensors of several requests into one batch: "dense" (rows
//                    concatenated), "sparse" (feature-major merge of lengths / ids / optional weights, the layout a
//                    KeyedJaggedTensor wants), "embedding" (pre-computed embedding rows concatenated).
//   result split     name -> function that cuts a batched model output back into per-request results: "dict_of_tensor" (every
//                    value is [B, ...] and is cut along dim 0), "dict_of_tensors" (every value is a list of such tensors),
//                    "dict_with_mask_tensor" (a value tensor plus a [B] mask: a request gets the rows whose mask is set).
//   GPUExecutor      worker threads of one device: take a batch from the batching queue, reject it when it waited longer than
//                    the queue time-out, move it to the device on the thread's own stream, run a TorchScript module, bring the
//                    output back and hand the per-request pieces to the waiting clients.  Counters (batches, requests, rejects,
//                    failures, microseconds per stage) play the role of the reference's observers.
//
// Counterpart of torchrec/inference/inference_legacy/src/{Validation,Batching,ResultSplit,GPUExecutor}.cpp; the model is a
// TorchScript module instead of a torch::deploy interpreter session.
#include <torch/script.h>

#include <c10/core/StreamGuard.h>
#include <c10/core/impl/VirtualGuardImpl.h>

#include "inference_runtime.h"

namespace trb {
namespace inference {

// ---- validation ---------------------------------------------------------------------------------------------------------
std::string validate_sparse(const torch::Tensor& values, const torch::Tensor& lengths, const c10::optional<torch::Tensor>& weights) {
  if (lengths.numel() > 0 && lengths.min().item<int64_t>() < 0) return "lengths must be non-negative";
  const int64_t total = lengths.numel() > 0 ? lengths.sum().item<int64_t>() : 0;
  if (total != values.numel()) return "sum of lengths (" + std::to_string(total) + ") differs from the number of ids (" + std::to_string(values.numel()) + ")";
  if (weights.has_value() && weights->defined() && weights->numel() != values.numel()) return "weights must be as long as the ids";
  return "";
}

std::string validate_dense(const torch::Tensor& dense, int64_t batch_size, int64_t num_features) {
  if (dense.numel() != batch_size * num_features)
    return "dense features hold " + std::to_string(dense.numel()) + " elements, expected " + std::to_string(batch_size * num_features);
  return "";
}

// ---- batching functions -------------------------------------------------------------------------------------------------
using TensorList = std::vector<torch::Tensor>;
using BatchingFn = std::function<TensorList(const std::vector<TensorList>&, int64_t)>;

static TensorList batch_rows(const std::vector<TensorList>& reqs, int64_t) {
  TensorList parts;
  for (const auto& r : reqs) {
    TORCH_CHECK(r.size() == 1, "one tensor per request expected");
    parts.push_back(r[0]);
  }
  return {torch::cat(parts, 0)};
}

// per request: lengths [F * b] (feature-major), ids, optionally weights -> merged feature-major lengths, ids, (weights)
static TensorList batch_sparse(const std::vector<TensorList>& reqs, int64_t num_features) {
  TORCH_CHECK(!reqs.empty());
  const bool weighted = reqs[0].size() == 3;
  std::vector<std::vector<torch::Tensor>> ids(reqs.size()), wts(reqs.size());
  std::vector<torch::Tensor> len2d(reqs.size());
  for (size_t i = 0; i < reqs.size(); ++i) {
    TORCH_CHECK(reqs[i].size() == (weighted ? 3u : 2u), "requests disagree on whether they carry weights");
    const auto& lengths = reqs[i][0];
    TORCH_CHECK(num_features > 0 && lengths.numel() % num_features == 0, "lengths must hold num_features * b entries");
    len2d[i] = lengths.view({num_features, -1});
    auto per_feature = len2d[i].sum(1).to(torch::kLong).cpu().contiguous();
    std::vector<int64_t> splits(per_feature.data_ptr<int64_t>(), per_feature.data_ptr<int64_t>() + per_feature.numel());
    ids[i] = reqs[i][1].split_with_sizes(splits);
    if (weighted) wts[i] = reqs[i][2].split_with_sizes(splits);
  }
  TensorList len_parts, id_parts, w_parts;
  for (int64_t f = 0; f < num_features; ++f)
    for (size_t i = 0; i < reqs.size(); ++i) {
      len_parts.push_back(len2d[i].select(0, f));
      id_parts.push_back(ids[i][size_t(f)]);
      if (weighted) w_parts.push_back(wts[i][size_t(f)]);
    }
  TensorList out = {torch::cat(len_parts, 0), torch::cat(id_parts, 0)};
  if (weighted) out.push_back(torch::cat(w_parts, 0));
  return out;
}

static std::mutex g_registry_mu;
static std::unordered_map<std::string, BatchingFn>& batching_registry() {
  static std::unordered_map<std::string, BatchingFn> reg = {{"dense", batch_rows}, {"embedding", batch_rows}, {"sparse", batch_sparse}};
  return reg;
}

void register_batching_fn(const std::string& name, BatchingFn fn) {
  std::lock_guard<std::mutex> lock(g_registry_mu);
  batching_registry()[name] = std::move(fn);
}

TensorList run_batching_fn(const std::string& name, const std::vector<TensorList>& reqs, int64_t num_features) {
  BatchingFn fn;
  {
    std::lock_guard<std::mutex> lock(g_registry_mu);
    auto it = batching_registry().find(name);
    TORCH_CHECK(it != batching_registry().end(), "no batching function named '", name, "'");
    fn = it->second;
  }
  return fn(reqs, num_features);
}

// ---- result split -------------------------------------------------------------------------------------------------------
using TensorDict = c10::Dict<std::string, torch::Tensor>;

static std::vector<int64_t> to_vec(const torch::Tensor& sizes) {
  auto s = sizes.to(torch::kLong).cpu().contiguous();
  return std::vector<int64_t>(s.data_ptr<int64_t>(), s.data_ptr<int64_t>() + s.numel());
}

std::vector<TensorDict> split_dict_of_tensor(const TensorDict& out, const torch::Tensor& sizes) {
  const auto n = to_vec(sizes);
  std::vector<TensorDict> res(n.size());
  for (const auto& kv : out) {
    int64_t off = 0;
    for (size_t i = 0; i < n.size(); ++i) {
      res[i].insert(kv.key(), kv.value().narrow(0, off, n[i]));
      off += n[i];
    }
    TORCH_CHECK(off == kv.value().size(0), "output '", kv.key(), "' has ", kv.value().size(0), " rows for ", off, " samples");
  }
  return res;
}

std::vector<c10::Dict<std::string, TensorList>> split_dict_of_tensors(const c10::Dict<std::string, TensorList>& out, const torch::Tensor& sizes) {
  const auto n = to_vec(sizes);
  std::vector<c10::Dict<std::string, TensorList>> res(n.size());
  for (const auto& kv : out) {
    std::vector<TensorList> per(n.size());
    for (const auto& t : kv.value()) {
      int64_t off = 0;
      for (size_t i = 0; i < n.size(); ++i) {
        per[i].push_back(t.narrow(0, off, n[i]));
        off += n[i];
      }
    }
    for (size_t i = 0; i < n.size(); ++i) res[i].insert(kv.key(), per[i]);
  }
  return res;
}

// values[name] is [B, ...], masks[name] is [B] (bool or 0/1): a request gets the rows of its samples whose mask is set
std::vector<TensorDict> split_dict_with_mask_tensor(const TensorDict& values, const TensorDict& masks, const torch::Tensor& sizes) {
  const auto n = to_vec(sizes);
  std::vector<TensorDict> res(n.size());
  for (const auto& kv : values) {
    TORCH_CHECK(masks.contains(kv.key()), "no mask for output '", kv.key(), "'");
    const auto mask = masks.at(kv.key()).to(torch::kBool);
    int64_t off = 0;
    for (size_t i = 0; i < n.size(); ++i) {
      auto rows = mask.narrow(0, off, n[i]).nonzero().view({-1});
      res[i].insert(kv.key(), kv.value().narrow(0, off, n[i]).index_select(0, rows));
      off += n[i];
    }
  }
  return res;
}

// ---- executor -------------------------------------------------------------------------------------------------------------
class GPUExecutor : public torch::CustomClassHolder {
 public:
  GPUExecutor(c10::intrusive_ptr<BatchingQueue> queue, std::string module_path, int64_t device_index, int64_t queue_index,
              int64_t num_threads, int64_t queue_timeout_ms, std::string output_key)
      : queue_(std::move(queue)), device_(device_index < 0 ? torch::Device(torch::kCPU) : torch::Device(torch::kCUDA, c10::DeviceIndex(device_index))),
        queue_index_(queue_index), queue_timeout_ms_(queue_timeout_ms), output_key_(std::move(output_key)) {
    TORCH_CHECK(num_threads >= 1 && num_threads <= 64);
    for (int64_t i = 0; i < num_threads; ++i) {
      modules_.push_back(torch::jit::load(module_path, device_));
      modules_.back().eval();
    }
    for (int64_t i = 0; i < num_threads; ++i) workers_.emplace_back([this, i] { run(size_t(i)); });
  }
  ~GPUExecutor() override { stop(); }

  void stop() {
    if (stopped_.exchange(true)) return;
    for (auto& t : workers_)
      if (t.joinable()) t.join();
  }

  c10::Dict<std::string, int64_t> stats() {
    c10::Dict<std::string, int64_t> d;
    d.insert("batches", batches_.load());
    d.insert("requests", requests_.load());
    d.insert("rejected_batches", rejected_.load());
    d.insert("failed_batches", failed_.load());
    d.insert("queue_us", queue_us_.load());
    d.insert("copy_in_us", copy_in_us_.load());
    d.insert("forward_us", forward_us_.load());
    d.insert("copy_out_us", copy_out_us_.load());
    return d;
  }

 private:
  static int64_t us_since(std::chrono::steady_clock::time_point t0) {
    return std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
  }

  void run(size_t worker) {
    torch::NoGradGuard no_grad;
    // every worker issues on its own stream so that copies and kernels of different batches overlap on the device
    c10::optional<c10::Stream> stream;
    if (device_.is_cuda()) stream = c10::impl::VirtualGuardImpl(device_.type()).getStreamFromGlobalPool(device_, /*isHighPriority=*/false);
    while (!stopped_.load()) {
      Batch b = queue_->pop_batch(queue_index_, 20);
      if (b.empty()) continue;
      const int64_t waited = us_since(b.formed_at);
      queue_us_ += waited;
      if (queue_timeout_ms_ > 0 && waited > queue_timeout_ms_ * 1000) {
        ++rejected_;
        queue_->set_error(b.request_ids, "rejected: the batch waited " + std::to_string(waited / 1000) + " ms in the executor queue");
        continue;
      }
      try {
        c10::OptionalStreamGuard guard(stream);
        auto t0 = std::chrono::steady_clock::now();
        auto dense = b.dense.to(device_, /*non_blocking=*/true);
        auto lengths = b.lengths.to(device_, /*non_blocking=*/true);
        auto values = b.values.to(device_, /*non_blocking=*/true);
        copy_in_us_ += us_since(t0);
        t0 = std::chrono::steady_clock::now();
        auto out = modules_[worker].forward({dense, lengths, values});
        forward_us_ += us_since(t0);
        t0 = std::chrono::steady_clock::now();
        torch::Tensor result;
        if (out.isTensor()) {
          result = out.toTensor();
        } else if (out.isGenericDict()) {
          auto dict = out.toGenericDict();
          auto it = output_key_.empty() ? dict.begin() : dict.find(output_key_);
          TORCH_CHECK(it != dict.end(), "the model output has no entry '", output_key_, "'");
          result = it->value().toTensor();
        } else {
          TORCH_CHECK(false, "the model must return a tensor or a dict of tensors");
        }
        result = result.to(torch::kCPU);  // synchronises this worker's stream only
        copy_out_us_ += us_since(t0);
        queue_->set_results(b.request_ids, b.request_sizes, result);
        ++batches_;
        requests_ += b.request_ids.numel();
      } catch (const std::exception& e) {
        ++failed_;
        queue_->set_error(b.request_ids, std::string("the model raised: ") + e.what());
      }
    }
  }

  c10::intrusive_ptr<BatchingQueue> queue_;
  torch::Device device_;
  const int64_t queue_index_, queue_timeout_ms_;
  const std::string output_key_;
  std::vector<torch::jit::Module> modules_;
  std::vector<std::thread> workers_;
  std::atomic<bool> stopped_{false};
  std::atomic<int64_t> batches_{0}, requests_{0}, rejected_{0}, failed_{0}, queue_us_{0}, copy_in_us_{0}, forward_us_{0}, copy_out_us_{0};
};

}  // namespace inference
}  // namespace trb

TORCH_LIBRARY_FRAGMENT(trb_inference, m) {
  using namespace trb::inference;
  m.class_<GPUExecutor>("GPUExecutor")
      .def(torch::init<c10::intrusive_ptr<BatchingQueue>, std::string, int64_t, int64_t, int64_t, int64_t, std::string>())
      .def("stats", &GPUExecutor::stats)
      .def("stop", &GPUExecutor::stop);
  m.def("validate_sparse(Tensor values, Tensor lengths, Tensor? weights) -> str", &validate_sparse);
  m.def("validate_dense(Tensor dense, int batch_size, int num_features) -> str", &validate_dense);
  m.def("batch_requests(str kind, Tensor[][] requests, int num_features) -> Tensor[]",
        [](std::string kind, std::vector<std::vector<torch::Tensor>> reqs, int64_t num_features) { return run_batching_fn(kind, reqs, num_features); });
  m.def("split_dict_of_tensor(Dict(str, Tensor) output, Tensor sizes) -> Dict(str, Tensor)[]", &split_dict_of_tensor);
  m.def("split_dict_of_tensors(Dict(str, Tensor[]) output, Tensor sizes) -> Dict(str, Tensor[])[]", &split_dict_of_tensors);
  m.def("split_dict_with_mask_tensor(Dict(str, Tensor) values, Dict(str, Tensor) masks, Tensor sizes) -> Dict(str, Tensor)[]", &split_dict_with_mask_tensor);
}
