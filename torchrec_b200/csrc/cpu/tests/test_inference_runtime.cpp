// Unit tests (and a small throughput figure with --bench) of the serving runtime's dynamic batching queue: how requests are merged
// into a batch (dense rows, feature-major sparse lengths and ids), how results and errors find their way back to the request that
// waits for them, the size limit and the time limit of a batch, and several producer threads against several consumer queues.
// Counterpart of the reference's gtests under torchrec/inference/inference_legacy/tests (BatchingQueueTest.cpp, ...).
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <string>

#include "../inference_runtime.h"

using trb::inference::Batch;
using trb::inference::BatchingQueue;

static int g_checks = 0;
#define EXPECT(cond)                                                              \
  do {                                                                            \
    ++g_checks;                                                                   \
    if (!(cond)) {                                                                \
      std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);      \
      std::exit(1);                                                               \
    }                                                                             \
  } while (0)

static torch::Tensor longs(std::initializer_list<int64_t> v) { return torch::tensor(std::vector<int64_t>(v), torch::kLong); }

static void test_requests_merge_feature_major() {
  BatchingQueue q(/*max_batch_size=*/6, /*timeout_ms=*/500, /*num_queues=*/1, /*num_features=*/2, /*pin=*/false);
  // request A: 2 samples; feature 0 lengths [1, 2] ids 10 11 12; feature 1 lengths [0, 1] ids 20
  const int64_t a = q.add_request(torch::ones({2, 3}), longs({1, 2, 0, 1}), longs({10, 11, 12, 20}));
  // request B: 4 samples; feature 0 lengths [1, 0, 0, 1] ids 30 31; feature 1 lengths [2, 0, 0, 0] ids 40 41
  const int64_t b = q.add_request(torch::full({4, 3}, 2.0), longs({1, 0, 0, 1, 2, 0, 0, 0}), longs({30, 31, 40, 41}));
  Batch batch = q.pop_batch(0, 2000);  // formed at once: 6 samples reach the size limit
  EXPECT(!batch.empty());
  EXPECT(batch.dense.size(0) == 6 && batch.dense[0][0].item<float>() == 1.f && batch.dense[5][2].item<float>() == 2.f);
  EXPECT(torch::equal(batch.lengths, longs({1, 2, 1, 0, 0, 1, 0, 1, 2, 0, 0, 0})));
  EXPECT(torch::equal(batch.values, longs({10, 11, 12, 30, 31, 20, 40, 41})));
  EXPECT(torch::equal(batch.request_ids, longs({a, b})) && torch::equal(batch.request_sizes, longs({2, 4})));
  // results are cut back by request size, errors are delivered as exceptions
  q.set_results(batch.request_ids, batch.request_sizes, torch::arange(6).to(torch::kFloat).view({6, 1}));
  EXPECT(torch::equal(q.wait_result(a, 1000).view({-1}), torch::tensor({0.f, 1.f})));
  EXPECT(torch::equal(q.wait_result(b, 1000).view({-1}), torch::tensor({2.f, 3.f, 4.f, 5.f})));
  const int64_t c = q.add_request(torch::ones({1, 3}), longs({0, 0}), torch::empty({0}, torch::kLong));
  Batch second = q.pop_batch(0, 3000);  // formed by the time limit
  EXPECT(!second.empty() && second.dense.size(0) == 1);
  q.set_error(second.request_ids, "model raised");
  bool threw = false;
  try {
    q.wait_result(c, 1000);
  } catch (const std::exception& e) {
    threw = std::strstr(e.what(), "model raised") != nullptr;
  }
  EXPECT(threw);
  EXPECT(q.batches_formed() == 2);
  q.stop();
}

static void test_limits_and_rejections() {
  BatchingQueue q(4, 20, 1, 1, false);
  // a request larger than the limit still travels, alone
  q.add_request(torch::zeros({7, 2}), torch::zeros({7}, torch::kLong), torch::empty({0}, torch::kLong));
  q.add_request(torch::zeros({1, 2}), torch::zeros({1}, torch::kLong), torch::empty({0}, torch::kLong));
  Batch big = q.pop_batch(0, 2000);
  EXPECT(big.dense.size(0) == 7 && big.request_ids.numel() == 1);
  Batch small = q.pop_batch(0, 2000);
  EXPECT(small.dense.size(0) == 1);
  EXPECT(q.pop_batch(0, 30).empty());  // nothing left: an empty batch after the timeout
  bool threw = false;
  try {
    q.add_request(torch::zeros({2, 2}), torch::zeros({3}, torch::kLong), torch::empty({0}, torch::kLong));  // lengths do not match the batch
  } catch (const std::exception&) {
    threw = true;
  }
  EXPECT(threw);
  threw = false;
  try {
    q.wait_result(12345, 20);  // nobody produces this
  } catch (const std::exception&) {
    threw = true;
  }
  EXPECT(threw);
  q.stop();
  threw = false;
  try {
    q.add_request(torch::zeros({1, 2}), torch::zeros({1}, torch::kLong), torch::empty({0}, torch::kLong));
  } catch (const std::exception&) {
    threw = true;
  }
  EXPECT(threw);
}

static double test_producers_and_consumers(int producers, int per_producer, bool report) {
  BatchingQueue q(64, 2, /*num_queues=*/2, 1, false);
  std::atomic<int64_t> answered{0};
  std::atomic<bool> done{false};
  std::vector<std::thread> consumers;
  for (int c = 0; c < 2; ++c)
    consumers.emplace_back([&, c] {
      while (!done.load()) {
        Batch b = q.pop_batch(c, 20);
        if (b.empty()) continue;
        q.set_results(b.request_ids, b.request_sizes, b.dense.sum(1, true));  // the "model": row sums
      }
    });
  const auto t0 = std::chrono::steady_clock::now();
  std::vector<std::thread> threads;
  for (int p = 0; p < producers; ++p)
    threads.emplace_back([&, p] {
      for (int i = 0; i < per_producer; ++i) {
        const float v = float(p * 1000 + i);
        const int64_t id = q.add_request(torch::full({2, 4}, v), longs({1, 1}), longs({p, i}));
        torch::Tensor r = q.wait_result(id, 10000);
        if (r.size(0) == 2 && r[0][0].item<float>() == 4 * v && r[1][0].item<float>() == 4 * v) answered.fetch_add(1);
      }
    });
  for (auto& t : threads) t.join();
  const double secs = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  done.store(true);
  for (auto& t : consumers) t.join();
  EXPECT(answered.load() == int64_t(producers) * per_producer);  // every request got its own rows back
  EXPECT(q.batches_formed() <= int64_t(producers) * per_producer);
  q.stop();
  if (report) std::printf("BENCH batching_queue %d producers x %d requests: %.0f requests/s, %lld batches\n", producers, per_producer,
                          producers * per_producer / secs, (long long)q.batches_formed());
  return secs;
}

int main(int argc, char** argv) {
  const bool bench = argc > 1 && std::string(argv[1]) == "--bench";
  test_requests_merge_feature_major();
  test_limits_and_rejections();
  test_producers_and_consumers(4, 50, false);
  if (bench) test_producers_and_consumers(8, 400, true);
  std::printf("all serving-runtime checks passed (%d checks)\n", g_checks);
  return 0;
}
