#include "tde_io.h"

#include <dlfcn.h>

#include <map>
#include <stdexcept>
#include <tuple>

namespace trb {
namespace tde {

IORegistry& IORegistry::instance() {
  static IORegistry r;
  return r;
}

void IORegistry::register_provider(IOProvider provider) {
  std::lock_guard<std::mutex> lock(mu_);
  providers_[provider.type] = provider;
}

void IORegistry::load(const std::string& path) {
  void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
  if (h == nullptr) throw std::runtime_error(std::string("cannot load IO plugin ") + path + ": " + dlerror());
  using Fn = IOProvider (*)();
  Fn fn = reinterpret_cast<Fn>(dlsym(h, "trb_tde_io_provider"));
  if (fn == nullptr) {
    dlclose(h);
    throw std::runtime_error("IO plugin " + path + " does not export trb_tde_io_provider");
  }
  register_provider(fn());
  std::lock_guard<std::mutex> lock(mu_);
  handles_.push_back(h);
}

IOProvider IORegistry::resolve(const std::string& type) const {
  std::lock_guard<std::mutex> lock(mu_);
  auto it = providers_.find(type);
  if (it == providers_.end()) throw std::runtime_error("no IO provider registered for type '" + type + "'");
  return it->second;
}

IO::IO(const std::string& url) {
  const auto pos = url.find("://");
  if (pos == std::string::npos) throw std::invalid_argument("IO url must look like type://config, got " + url);
  provider_ = IORegistry::instance().resolve(url.substr(0, pos));
  instance_ = provider_.initialize(url.substr(pos + 3).c_str());
}

IO::~IO() {
  if (instance_ != nullptr) provider_.finalize(instance_);
}

namespace {
struct FetchCtx {
  IO::Fetched result;
  std::function<void(IO::Fetched)> done;
  uint32_t num_states;
  std::vector<int64_t> gids, cols;  // keep the request alive for the provider
  std::string table;
};
struct PushCtx {
  std::function<void()> done;
  std::vector<int64_t> gids, cols;
  std::vector<uint32_t> state_ids;
  std::vector<float> data;
  std::vector<uint64_t> offsets;
  std::string table;
};
}  // namespace

void IO::fetch(const std::string& table, const std::vector<int64_t>& global_ids, const std::vector<int64_t>& col_ids,
               uint32_t num_optimizer_states, std::function<void(Fetched)> done) {
  auto* ctx = new FetchCtx{{}, std::move(done), num_optimizer_states, global_ids, col_ids, table};
  ctx->result.data.resize(global_ids.size() * num_optimizer_states);
  IOFetchParameter p{};
  p.table_name = ctx->table.c_str();
  p.num_cols = uint32_t(ctx->cols.size());
  p.num_global_ids = uint32_t(ctx->gids.size());
  p.col_ids = ctx->cols.data();
  p.global_ids = ctx->gids.data();
  p.num_optimizer_states = num_optimizer_states;
  p.on_complete_context = ctx;
  p.on_global_id_fetched = +[](void* c, uint32_t offset, uint32_t state, const float* data, uint32_t len) {
    auto* fc = static_cast<FetchCtx*>(c);
    if (data != nullptr) fc->result.data[size_t(offset) * fc->num_states + state].assign(data, data + len);
  };
  p.on_all_fetched = +[](void* c) {
    auto* fc = static_cast<FetchCtx*>(c);
    fc->done(std::move(fc->result));
    delete fc;
  };
  provider_.fetch(instance_, p);
}

void IO::push(const std::string& table, const std::vector<int64_t>& global_ids, const std::vector<int64_t>& col_ids,
              const std::vector<uint32_t>& optimizer_state_ids, const std::vector<float>& data,
              const std::vector<uint64_t>& offsets, std::function<void()> done) {
  auto* ctx = new PushCtx{std::move(done), global_ids, col_ids, optimizer_state_ids, data, offsets, table};
  IOPushParameter p{};
  p.table_name = ctx->table.c_str();
  p.num_cols = uint32_t(ctx->cols.size());
  p.num_global_ids = uint32_t(ctx->gids.size());
  p.col_ids = ctx->cols.data();
  p.global_ids = ctx->gids.data();
  p.num_optimizer_states = uint32_t(ctx->state_ids.size());
  p.optimizer_state_ids = ctx->state_ids.data();
  p.num_offsets = uint32_t(ctx->offsets.size());
  p.offsets = ctx->offsets.data();
  p.data = ctx->data.data();
  p.on_complete_context = ctx;
  p.on_push_complete = +[](void* c) {
    auto* pc = static_cast<PushCtx*>(c);
    pc->done();
    delete pc;
  };
  provider_.push(instance_, p);
}

// ---- built-in provider: an in-process map (table, global id, col, state) -> vector<float> -------------------------
namespace {
struct MemoryStore {
  std::mutex mu;
  std::map<std::tuple<std::string, int64_t, int64_t, uint32_t>, std::vector<float>> kv;
};
// stores are shared by config name so that two clients of "memory://x" see the same data
std::mutex g_stores_mu;
std::unordered_map<std::string, std::shared_ptr<MemoryStore>> g_stores;
struct MemoryInstance {
  std::shared_ptr<MemoryStore> store;
};
}  // namespace

void register_memory_io_provider() {
  IOProvider p{};
  p.type = "memory";
  p.initialize = +[](const char* config) -> void* {
    std::lock_guard<std::mutex> lock(g_stores_mu);
    auto& s = g_stores[config ? config : ""];
    if (!s) s = std::make_shared<MemoryStore>();
    return new MemoryInstance{s};
  };
  p.fetch = +[](void* inst, IOFetchParameter q) {
    auto* m = static_cast<MemoryInstance*>(inst);
    {
      std::lock_guard<std::mutex> lock(m->store->mu);
      const uint32_t ncols = q.num_cols == 0 ? 1 : q.num_cols;
      for (uint32_t i = 0; i < q.num_global_ids; ++i)
        for (uint32_t s = 0; s < q.num_optimizer_states; ++s) {
          // the row of one id is the concatenation of its column shards
          std::vector<float> row;
          bool missing = false;
          for (uint32_t c = 0; c < ncols && !missing; ++c) {
            auto it = m->store->kv.find({q.table_name, q.global_ids[i], q.num_cols ? q.col_ids[c] : 0, s});
            if (it == m->store->kv.end()) missing = true;
            else row.insert(row.end(), it->second.begin(), it->second.end());
          }
          q.on_global_id_fetched(q.on_complete_context, i, s, missing ? nullptr : row.data(), uint32_t(row.size()));
        }
    }
    q.on_all_fetched(q.on_complete_context);
  };
  p.push = +[](void* inst, IOPushParameter q) {
    auto* m = static_cast<MemoryInstance*>(inst);
    {
      std::lock_guard<std::mutex> lock(m->store->mu);
      const uint32_t ncols = q.num_cols == 0 ? 1 : q.num_cols;
      for (uint32_t i = 0; i < q.num_global_ids; ++i)
        for (uint32_t s = 0; s < q.num_optimizer_states; ++s) {
          const size_t k = size_t(i) * q.num_optimizer_states + s;
          const float* b = q.data + q.offsets[k];
          const size_t len = size_t(q.offsets[k + 1] - q.offsets[k]);
          const size_t per = len / ncols;
          for (uint32_t c = 0; c < ncols; ++c)
            m->store->kv[{q.table_name, q.global_ids[i], q.num_cols ? q.col_ids[c] : 0, q.optimizer_state_ids[s]}] =
                std::vector<float>(b + c * per, b + (c + 1) * per);
        }
    }
    q.on_push_complete(q.on_complete_context);
  };
  p.finalize = +[](void* inst) { delete static_cast<MemoryInstance*>(inst); };
  IORegistry::instance().register_provider(p);
}

}  // namespace tde
}  // namespace trb
