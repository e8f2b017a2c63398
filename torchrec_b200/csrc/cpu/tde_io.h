// Storage back ends of the parameter-server client.
//
// A back end is a table of C functions (`IOProvider`), found by its type name in a process-wide registry.  Providers
// come from shared libraries loaded at run time (`IORegistry::load`, which calls the library's exported
// `trb_tde_io_provider()`), or are registered in process (the built-in "memory" provider, used by tests and as a
// host-memory parameter store).  `IO` is the client-side façade: it parses "type://config", initialises the
// provider and forwards fetch / push requests.
//
// fetch: for every (global id) deliver `num_optimizer_states + 1` float vectors (row, then states) or "missing".
// push : store those vectors.  Both are asynchronous for the provider; the callbacks run on provider threads.
//
// Counterpart of torchrec/csrc/dynamic_embedding/details/io.h, io_registry.h and io_parameter.h.
#pragma once

#include <cstdint>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

namespace trb {
namespace tde {

struct IOFetchParameter {
  const char* table_name;
  uint32_t num_cols;
  uint32_t num_global_ids;
  const int64_t* col_ids;
  const int64_t* global_ids;
  uint32_t num_optimizer_states;
  void* on_complete_context;
  // called once per (global id index, optimizer state index); data == nullptr: not stored (caller initialises)
  void (*on_global_id_fetched)(void* ctx, uint32_t offset, uint32_t optimizer_state, const float* data, uint32_t data_len);
  void (*on_all_fetched)(void* ctx);
};

struct IOPushParameter {
  const char* table_name;
  uint32_t num_cols;
  uint32_t num_global_ids;
  const int64_t* col_ids;
  const int64_t* global_ids;
  uint32_t num_optimizer_states;
  const uint32_t* optimizer_state_ids;
  uint32_t num_offsets;      // num_global_ids * num_optimizer_states + 1
  const uint64_t* offsets;   // element offsets into `data`
  const float* data;
  void* on_complete_context;
  void (*on_push_complete)(void* ctx);
};

struct IOProvider {
  const char* type;
  void* (*initialize)(const char* config);
  void (*fetch)(void* instance, IOFetchParameter param);
  void (*push)(void* instance, IOPushParameter param);
  void (*finalize)(void* instance);
};

class IORegistry {
 public:
  static IORegistry& instance();
  void register_provider(IOProvider provider);
  void load(const std::string& shared_library_path);  // dlopen + trb_tde_io_provider()
  IOProvider resolve(const std::string& type) const;

 private:
  mutable std::mutex mu_;
  std::unordered_map<std::string, IOProvider> providers_;
  std::vector<void*> handles_;
};

class IO {
 public:
  explicit IO(const std::string& url);  // "type://config"
  ~IO();
  IO(const IO&) = delete;
  IO& operator=(const IO&) = delete;

  struct Fetched {
    std::vector<std::vector<float>> data;  // [num_global_ids * num_optimizer_states]; empty vector = missing
  };
  // asynchronous; `done` runs on a provider thread
  void fetch(const std::string& table, const std::vector<int64_t>& global_ids, const std::vector<int64_t>& col_ids,
             uint32_t num_optimizer_states, std::function<void(Fetched)> done);
  void push(const std::string& table, const std::vector<int64_t>& global_ids, const std::vector<int64_t>& col_ids,
            const std::vector<uint32_t>& optimizer_state_ids, const std::vector<float>& data,
            const std::vector<uint64_t>& offsets, std::function<void()> done);

 private:
  IOProvider provider_;
  void* instance_ = nullptr;
};

void register_memory_io_provider();  // built-in "memory://" provider

}  // namespace tde
}  // namespace trb
