// Unit tests and a micro-benchmark of the dynamic-embedding library that need no tensor library: the eviction record, the id
// transformer and the in-process store through the provider ABI.  Built and run by tests/test_native_cpp.py:
//   g++ -std=c++17 -O2 -pthread -I.. test_tde.cpp ../tde_id_transformer.cpp ../tde_io.cpp -ldl -o test_tde && ./test_tde [--bench]
// Counterpart of test/cpp/dynamic_embedding/*.cpp and benchmarks/cpp/dynamic_embedding/*.cpp of the reference.
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <random>
#include <set>
#include <string>
#include <vector>

#include "../tde_id_transformer.h"
#include "../tde_io.h"

using namespace trb::tde;

static int g_failed = 0;
#define CHECK(cond)                                                        \
  do {                                                                     \
    if (!(cond)) {                                                         \
      std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);      \
      ++g_failed;                                                          \
    }                                                                      \
  } while (0)

static void test_record() {
  LxuRecord r;
  r.set(123456, 7);
  CHECK(r.time() == 123456 && r.freq_power() == 7);
  r.set((1u << 27) + 5, 99);  // time wraps into 27 bits, frequency saturates at 31
  CHECK(r.time() == 5 && r.freq_power() == 31);
  LxuRecord older, newer;
  older.set(10, 3);
  newer.set(11, 3);
  CHECK(older.priority() < newer.priority());
  LxuRecord hot;
  hot.set(1, 4);
  CHECK(hot.priority() > newer.priority());  // frequency dominates recency
}

template <class Table>
static void test_transformer_basic() {
  Table t(4);
  int64_t ids[] = {100, 7, 100, 42};
  int64_t slots[4];
  auto r = t.transform(ids, 4, slots, 1);
  CHECK(r.success && r.num_transformed == 4 && r.fetch.size() == 3);
  CHECK(slots[0] == slots[2] && slots[0] == 0 && slots[1] == 1 && slots[3] == 2);
  CHECK(t.size() == 3);
  int64_t more[] = {1, 2, 3};
  auto r2 = t.transform(more, 3, slots, 2);
  CHECK(!r2.success && r2.num_transformed == 1);  // one free slot left
  auto ev = t.evict(2);
  CHECK(ev.size() == 2 && t.size() == 2);
  auto r3 = t.transform(more + 1, 2, slots, 3);
  CHECK(r3.success && r3.num_transformed == 2);
  std::set<int64_t> used;
  for (auto& p : t.save()) used.insert(p.second);
  CHECK(used.size() == 4);  // every slot is held by exactly one id
}

template <class Table>
static void test_transformer_eviction_order() {
  Table t(8);
  int64_t slots[8];
  int64_t a[] = {10, 11, 12, 13};
  t.transform(a, 4, slots, 1);
  int64_t b[] = {12, 13};
  for (uint32_t time = 2; time < 200; ++time) t.transform(b, 2, slots, time);  // 12 and 13 become frequent
  auto ev = t.evict(2);
  std::set<int64_t> gone{ev[0].first, ev[1].first};
  CHECK(gone.count(10) && gone.count(11));
}

template <class Table>
static void test_transformer_many_ids() {
  const int64_t cap = 1 << 14;
  Table t(cap);
  std::mt19937_64 rng(3);
  std::vector<int64_t> ids(cap), slots(cap);
  std::set<int64_t> uniq;
  for (auto& v : ids) {
    do v = int64_t(rng() >> 1); while (!uniq.insert(v).second);
  }
  auto r = t.transform(ids.data(), cap, slots.data(), 1);
  CHECK(r.success && int64_t(r.fetch.size()) == cap);
  std::set<int64_t> s(slots.begin(), slots.end());
  CHECK(int64_t(s.size()) == cap && *s.begin() == 0 && *s.rbegin() == cap - 1);
  std::vector<int64_t> again(cap);
  t.transform(ids.data(), cap, again.data(), 2);
  CHECK(again == slots);
  // churn: evict half, insert new ids, the table stays consistent through tombstones and rehash
  for (int round = 0; round < 6; ++round) {
    auto ev = t.evict(cap / 2);
    CHECK(int64_t(ev.size()) == cap / 2);
    std::vector<int64_t> fresh(cap / 2), fs(cap / 2);
    for (auto& v : fresh) v = int64_t(rng() >> 1);
    auto rr = t.transform(fresh.data(), cap / 2, fs.data(), 3 + round);
    CHECK(rr.success);
  }
  CHECK(t.size() <= cap);
}

struct FetchSink {
  std::mutex mu;
  std::condition_variable cv;
  bool done = false;
  std::vector<std::vector<float>> rows;
  std::vector<bool> missing;
};

static void test_memory_store() {
  register_memory_io_provider();
  IO io("memory://cpp_test");
  std::vector<int64_t> ids{5, 9}, cols{0};
  std::vector<uint32_t> states{0, 1};
  std::vector<float> data{1, 2, 3, 4, /*state of 5*/ 0.5f, /*row 9*/ 5, 6, 7, 8, /*state of 9*/ 0.25f};
  std::vector<uint64_t> offsets{0, 4, 5, 9, 10};
  std::mutex mu;
  std::condition_variable cv;
  bool pushed = false;
  io.push("tbl", ids, cols, states, data, offsets, [&] { std::lock_guard<std::mutex> l(mu); pushed = true; cv.notify_all(); });
  {
    std::unique_lock<std::mutex> l(mu);
    cv.wait(l, [&] { return pushed; });
  }
  bool fetched = false;
  IO::Fetched got;
  io.fetch("tbl", {9, 77, 5}, cols, 2, [&](IO::Fetched f) { std::lock_guard<std::mutex> l(mu); got = std::move(f); fetched = true; cv.notify_all(); });
  {
    std::unique_lock<std::mutex> l(mu);
    cv.wait(l, [&] { return fetched; });
  }
  CHECK(got.data.size() == 6);
  CHECK(got.data[0] == std::vector<float>({5, 6, 7, 8}) && got.data[1] == std::vector<float>({0.25f}));
  CHECK(got.data[2].empty() && got.data[3].empty());  // id 77 was never stored
  CHECK(got.data[4] == std::vector<float>({1, 2, 3, 4}) && got.data[5] == std::vector<float>({0.5f}));
  bool threw = false;
  try {
    IO bad("nosuchtype://x");
  } catch (const std::exception&) {
    threw = true;
  }
  CHECK(threw);
}

template <class Table>
static void bench(const char* name) {
  const int64_t cap = 1 << 20, batch = 1 << 16;
  Table t(cap);
  std::mt19937_64 rng(1);
  std::vector<int64_t> ids(batch), slots(batch);
  auto t0 = std::chrono::steady_clock::now();
  int64_t total = 0;
  for (int it = 0; it < 64; ++it) {
    for (auto& v : ids) v = int64_t(rng() % (4 * cap));
    auto r = t.transform(ids.data(), batch, slots.data(), uint32_t(it + 1));
    total += r.num_transformed;
    if (!r.success) t.evict(cap / 4);
  }
  const double s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  std::printf("BENCH id_transformer %s: %.1f M ids/s (%lld ids, capacity %lld)\n", name, total / s / 1e6, (long long)total, (long long)cap);
}

int main(int argc, char** argv) {
  test_record();
  test_transformer_basic<IdTransformer>();
  test_transformer_eviction_order<IdTransformer>();
  test_transformer_many_ids<IdTransformer>();
  test_transformer_basic<CachelineIdTransformer>();
  test_transformer_eviction_order<CachelineIdTransformer>();
  test_transformer_many_ids<CachelineIdTransformer>();
  {  // the factory knows both layouts and nothing else
    auto a = make_id_transformer("naive", 8), b = make_id_transformer("cacheline", 8);
    int64_t ids[] = {5, 6, 5}, sa[3], sb[3];
    CHECK(a->transform(ids, 3, sa, 1).fetch.size() == 2 && b->transform(ids, 3, sb, 1).fetch.size() == 2);
    CHECK(sa[0] == sb[0] && sa[1] == sb[1] && sa[2] == sb[2] && a->capacity() == 8 && b->size() == 2);
    bool threw = false;
    try {
      make_id_transformer("other", 8);
    } catch (const std::exception&) {
      threw = true;
    }
    CHECK(threw);
  }
  test_memory_store();
  if (argc > 1 && std::strcmp(argv[1], "--bench") == 0) {
    bench<IdTransformer>("naive");
    bench<CachelineIdTransformer>("cacheline");
  }
  if (g_failed) {
    std::printf("%d checks failed\n", g_failed);
    return 1;
  }
  std::printf("all native checks passed\n");
  return 0;
}
