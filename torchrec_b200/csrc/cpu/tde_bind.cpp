// torch.classes.trb_tde.{TransformResult, IDTransformer, LocalShardList, FetchHandle, PS} and torch.ops.trb_tde.register_io
// (cf. torchrec/csrc/dynamic_embedding/bind.cpp:16-48).
#include <torch/custom_class.h>
#include <torch/library.h>
#include <torch/torch.h>

#include "tde_id_transformer.h"
#include "tde_io.h"
#include "tde_ps.h"

namespace trb {
namespace tde {

struct TransformResult : public torch::CustomClassHolder {
  TransformResult(bool s, int64_t n, torch::Tensor f) : success(s), num_transformed(n), ids_to_fetch(std::move(f)) {}
  bool success;
  int64_t num_transformed;
  torch::Tensor ids_to_fetch;  // int64 [n, 2] (global id, cache slot)
};

static torch::Tensor pairs_to_tensor(const std::vector<std::pair<int64_t, int64_t>>& v) {
  torch::Tensor t = torch::empty({int64_t(v.size()), 2}, torch::kLong);
  int64_t* p = t.data_ptr<int64_t>();
  for (size_t i = 0; i < v.size(); ++i) {
    p[2 * i] = v[i].first;
    p[2 * i + 1] = v[i].second;
  }
  return t;
}

class IDTransformerWrapper : public torch::CustomClassHolder {
 public:
  explicit IDTransformerWrapper(int64_t num_embeddings, int64_t min_used_freq_power = 5, const std::string& variant = "naive")
      : impl_(make_id_transformer(variant, num_embeddings, uint16_t(min_used_freq_power))) {}

  c10::intrusive_ptr<TransformResult> transform(torch::Tensor global_ids, torch::Tensor cache_ids, int64_t time) {
    TORCH_CHECK(global_ids.scalar_type() == torch::kLong && cache_ids.scalar_type() == torch::kLong);
    TORCH_CHECK(global_ids.is_contiguous() && cache_ids.is_contiguous() && global_ids.numel() == cache_ids.numel());
    TORCH_CHECK(!global_ids.is_cuda() && !cache_ids.is_cuda(), "the id transformer runs on host tensors");
    auto r = impl_->transform(global_ids.data_ptr<int64_t>(), global_ids.numel(), cache_ids.data_ptr<int64_t>(), uint32_t(time));
    return c10::make_intrusive<TransformResult>(r.success, r.num_transformed, pairs_to_tensor(r.fetch));
  }
  torch::Tensor evict(int64_t num_to_evict) { return pairs_to_tensor(impl_->evict(num_to_evict)); }
  torch::Tensor save() { return pairs_to_tensor(impl_->save()); }
  int64_t size() { return impl_->size(); }

 private:
  std::unique_ptr<IdTransformerBase> impl_;
};

}  // namespace tde
}  // namespace trb

TORCH_LIBRARY(trb_tde, m) {
  using namespace trb::tde;
  register_memory_io_provider();
  m.def("register_io(str plugin_path) -> ()", [](const std::string& path) { IORegistry::instance().load(path); });
  m.class_<TransformResult>("TransformResult")
      .def_readonly("success", &TransformResult::success)
      .def_readonly("num_transformed", &TransformResult::num_transformed)
      .def_readonly("ids_to_fetch", &TransformResult::ids_to_fetch);
  m.class_<IDTransformerWrapper>("IDTransformer")
      .def(torch::init<int64_t, int64_t, const std::string&>())
      .def("transform", &IDTransformerWrapper::transform)
      .def("evict", &IDTransformerWrapper::evict)
      .def("save", &IDTransformerWrapper::save)
      .def("size", &IDTransformerWrapper::size);
  m.class_<LocalShardList>("LocalShardList")
      .def(torch::init([]() { return c10::make_intrusive<LocalShardList>(); }))
      .def("append", [](const c10::intrusive_ptr<LocalShardList>& self, int64_t row_start, int64_t col_start, int64_t row_size, int64_t col_size,
                        std::vector<torch::Tensor> tensors) { self->emplace_back(row_start, col_start, row_size, col_size, std::move(tensors)); })
      .def("__len__", [](const c10::intrusive_ptr<LocalShardList>& self) { return self->size(); });
  m.class_<FetchHandle>("FetchHandle").def("wait", &FetchHandle::wait);
  m.class_<PS>("PS")
      .def(torch::init<const std::string&, c10::intrusive_ptr<LocalShardList>, int64_t, int64_t, const std::string&, int64_t>())
      .def("fetch", &PS::fetch)
      .def("evict", &PS::evict);
}
