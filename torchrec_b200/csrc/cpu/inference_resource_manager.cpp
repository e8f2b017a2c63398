// Bounds the number of batches in flight per device of a serving process: an executor asks for a slot before it launches a
// batch and gives it back when the results are out.  `occupy(device, timeout_ms)` waits at most the given time and reports
// failure instead of queueing without bound, so an overloaded server rejects work early.
// Counterpart of the reference's legacy runtime (torchrec/inference/include/torchrec/inference/ResourceManager.h).
#include <torch/custom_class.h>
#include <torch/library.h>

#include <chrono>
#include <condition_variable>
#include <mutex>
#include <vector>

namespace trb {
namespace inference {

class ResourceManager : public torch::CustomClassHolder {
 public:
  ResourceManager(int64_t num_devices, int64_t max_outstanding_batches)
      : max_(max_outstanding_batches), in_flight_(size_t(num_devices), 0), peak_(size_t(num_devices), 0), rejected_(0) {
    TORCH_CHECK(num_devices > 0 && max_outstanding_batches > 0);
  }

  bool occupy(int64_t device, int64_t timeout_ms) {
    TORCH_CHECK(device >= 0 && size_t(device) < in_flight_.size(), "device out of range");
    std::unique_lock<std::mutex> lock(mu_);
    const bool ok = cv_.wait_for(lock, std::chrono::milliseconds(timeout_ms), [&] { return in_flight_[size_t(device)] < max_; });
    if (!ok) {
      ++rejected_;
      return false;
    }
    const int64_t now = ++in_flight_[size_t(device)];
    if (now > peak_[size_t(device)]) peak_[size_t(device)] = now;
    return true;
  }

  void release(int64_t device) {
    {
      std::lock_guard<std::mutex> lock(mu_);
      TORCH_CHECK(device >= 0 && size_t(device) < in_flight_.size() && in_flight_[size_t(device)] > 0, "release without occupy");
      --in_flight_[size_t(device)];
    }
    cv_.notify_all();
  }

  int64_t outstanding(int64_t device) {
    std::lock_guard<std::mutex> lock(mu_);
    return in_flight_.at(size_t(device));
  }
  int64_t peak(int64_t device) {
    std::lock_guard<std::mutex> lock(mu_);
    return peak_.at(size_t(device));
  }
  int64_t rejected() {
    std::lock_guard<std::mutex> lock(mu_);
    return rejected_;
  }

 private:
  const int64_t max_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::vector<int64_t> in_flight_, peak_;
  int64_t rejected_;
};

}  // namespace inference
}  // namespace trb

TORCH_LIBRARY_FRAGMENT(trb_inference, m) {
  using trb::inference::ResourceManager;
  m.class_<ResourceManager>("ResourceManager")
      .def(torch::init<int64_t, int64_t>())
      .def("occupy", &ResourceManager::occupy)
      .def("release", &ResourceManager::release)
      .def("outstanding", &ResourceManager::outstanding)
      .def("peak", &ResourceManager::peak)
      .def("rejected", &ResourceManager::rejected);
}
