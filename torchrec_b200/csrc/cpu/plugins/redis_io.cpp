// Redis storage back end of the parameter-server client, as a run-time plugin (`trb_tde_io_provider`).
//
// Talks RESP2 over a TCP socket directly (no client library): fetch is one MGET over the keys of the request, push is one MSET.
// Keys are "<prefix><table>_<global id>_<col id>_<optimizer state>", values the raw little-endian floats of that column shard
// of that row.  Requests are queued to a small pool of worker threads, each with its own connection, so the callbacks run off the
// caller's thread like every provider's.
//
// URL: redis://host:port[/?prefix=<p>&db=<n>&num_threads=<n>&timeout_ms=<n>]
//
// Counterpart of torchrec/csrc/dynamic_embedding/details/redis/redis_io.{h,cpp} and url.h (which sit on hiredis).
#include <arpa/inet.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <unistd.h>

#include <condition_variable>
#include <cstring>
#include <deque>
#include <functional>
#include <mutex>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "../tde_io.h"

namespace {
using trb::tde::IOFetchParameter;
using trb::tde::IOProvider;
using trb::tde::IOPushParameter;

struct Options {
  std::string host = "127.0.0.1";
  int port = 6379;
  std::string prefix;
  int db = 0;
  int num_threads = 1;
  int timeout_ms = 5000;
};

Options parse_url(const std::string& config) {
  Options o;
  std::string rest = config;
  std::string query;
  const auto q = rest.find('?');
  if (q != std::string::npos) {
    query = rest.substr(q + 1);
    rest = rest.substr(0, q);
  }
  while (!rest.empty() && rest.back() == '/') rest.pop_back();
  const auto colon = rest.rfind(':');
  if (colon != std::string::npos) {
    o.host = rest.substr(0, colon);
    o.port = std::stoi(rest.substr(colon + 1));
  } else if (!rest.empty()) {
    o.host = rest;
  }
  size_t pos = 0;
  while (pos < query.size()) {
    auto amp = query.find('&', pos);
    if (amp == std::string::npos) amp = query.size();
    const std::string kv = query.substr(pos, amp - pos);
    const auto eq = kv.find('=');
    if (eq != std::string::npos) {
      const std::string k = kv.substr(0, eq), v = kv.substr(eq + 1);
      if (k == "prefix") o.prefix = v;
      else if (k == "db") o.db = std::stoi(v);
      else if (k == "num_threads") o.num_threads = std::max(1, std::stoi(v));
      else if (k == "timeout_ms") o.timeout_ms = std::max(1, std::stoi(v));
      else throw std::invalid_argument("redis io: unknown option " + k);
    }
    pos = amp + 1;
  }
  return o;
}

// One blocking RESP connection with send / receive time-outs.
class Connection {
 public:
  explicit Connection(const Options& o) {
    addrinfo hints{}, *res = nullptr;
    hints.ai_family = AF_UNSPEC;
    hints.ai_socktype = SOCK_STREAM;
    if (getaddrinfo(o.host.c_str(), std::to_string(o.port).c_str(), &hints, &res) != 0 || res == nullptr)
      throw std::runtime_error("redis io: cannot resolve " + o.host);
    for (addrinfo* p = res; p != nullptr; p = p->ai_next) {
      fd_ = ::socket(p->ai_family, p->ai_socktype, p->ai_protocol);
      if (fd_ < 0) continue;
      timeval tv{o.timeout_ms / 1000, (o.timeout_ms % 1000) * 1000};
      setsockopt(fd_, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
      setsockopt(fd_, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
      int one = 1;
      setsockopt(fd_, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
      if (::connect(fd_, p->ai_addr, p->ai_addrlen) == 0) break;
      ::close(fd_);
      fd_ = -1;
    }
    freeaddrinfo(res);
    if (fd_ < 0) throw std::runtime_error("redis io: cannot connect to " + o.host + ":" + std::to_string(o.port));
    if (o.db != 0) {
      command({"SELECT", std::to_string(o.db)});
      expect_simple();
    }
  }
  ~Connection() {
    if (fd_ >= 0) ::close(fd_);
  }
  Connection(const Connection&) = delete;
  Connection& operator=(const Connection&) = delete;

  void command(const std::vector<std::string>& args) {
    std::string out = "*" + std::to_string(args.size()) + "\r\n";
    for (const auto& a : args) {
      out += "$" + std::to_string(a.size()) + "\r\n";
      out += a;
      out += "\r\n";
    }
    size_t sent = 0;
    while (sent < out.size()) {
      const ssize_t n = ::send(fd_, out.data() + sent, out.size() - sent, MSG_NOSIGNAL);
      if (n <= 0) throw std::runtime_error("redis io: send failed");
      sent += size_t(n);
    }
  }

  void expect_simple() {
    const std::string line = read_line();
    if (line.empty() || line[0] == '-') throw std::runtime_error("redis io: server error: " + line);
  }

  // array of bulk strings; `present[i]` false for nil
  void read_bulk_array(std::vector<std::string>& values, std::vector<bool>& present) {
    const std::string head = read_line();
    if (head.empty() || head[0] != '*') throw std::runtime_error("redis io: expected an array, got: " + head);
    const long n = std::stol(head.substr(1));
    values.assign(size_t(std::max(0l, n)), std::string());
    present.assign(values.size(), false);
    for (long i = 0; i < n; ++i) {
      const std::string h = read_line();
      if (h.empty() || h[0] != '$') throw std::runtime_error("redis io: expected a bulk string, got: " + h);
      const long len = std::stol(h.substr(1));
      if (len < 0) continue;
      values[size_t(i)] = read_exact(size_t(len));
      read_exact(2);
      present[size_t(i)] = true;
    }
  }

 private:
  void fill() {
    char tmp[65536];
    const ssize_t n = ::recv(fd_, tmp, sizeof(tmp), 0);
    if (n <= 0) throw std::runtime_error("redis io: connection closed or timed out");
    buf_.append(tmp, size_t(n));
  }
  std::string read_line() {
    for (;;) {
      const auto p = buf_.find("\r\n", pos_);
      if (p != std::string::npos) {
        std::string line = buf_.substr(pos_, p - pos_);
        pos_ = p + 2;
        compact();
        return line;
      }
      fill();
    }
  }
  std::string read_exact(size_t n) {
    while (buf_.size() - pos_ < n) fill();
    std::string out = buf_.substr(pos_, n);
    pos_ += n;
    compact();
    return out;
  }
  void compact() {
    if (pos_ > (1u << 20)) {
      buf_.erase(0, pos_);
      pos_ = 0;
    }
  }
  int fd_ = -1;
  std::string buf_;
  size_t pos_ = 0;
};

class RedisIO {
 public:
  explicit RedisIO(const std::string& config) : opt_(parse_url(config)) {
    { Connection probe(opt_); }  // fail at construction, not at the first request
    for (int i = 0; i < opt_.num_threads; ++i) workers_.emplace_back([this] { run(); });
  }
  ~RedisIO() {
    {
      std::lock_guard<std::mutex> lock(mu_);
      stop_ = true;
    }
    cv_.notify_all();
    for (auto& t : workers_) t.join();
  }

  std::string key(const char* table, int64_t gid, int64_t col, uint32_t state) const {
    return opt_.prefix + table + "_" + std::to_string(gid) + "_" + std::to_string(col) + "_" + std::to_string(state);
  }

  void submit(std::function<void(Connection&)> job) {
    {
      std::lock_guard<std::mutex> lock(mu_);
      jobs_.push_back(std::move(job));
    }
    cv_.notify_one();
  }

 private:
  void run() {
    std::unique_ptr<Connection> conn;
    for (;;) {
      std::function<void(Connection&)> job;
      {
        std::unique_lock<std::mutex> lock(mu_);
        cv_.wait(lock, [this] { return stop_ || !jobs_.empty(); });
        if (jobs_.empty()) return;
        job = std::move(jobs_.front());
        jobs_.pop_front();
      }
      try {
        if (!conn) conn = std::make_unique<Connection>(opt_);
        job(*conn);
      } catch (...) {
        conn.reset();  // the job reports its own failure; the next one reconnects
      }
    }
  }
  Options opt_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<std::function<void(Connection&)>> jobs_;
  std::vector<std::thread> workers_;
  bool stop_ = false;
};

void* redis_initialize(const char* config) { return new RedisIO(config ? config : ""); }
void redis_finalize(void* inst) { delete static_cast<RedisIO*>(inst); }

void redis_fetch(void* inst, IOFetchParameter q) {
  auto* io = static_cast<RedisIO*>(inst);
  const uint32_t ncols = q.num_cols == 0 ? 1 : q.num_cols;
  std::vector<std::string> cmd{"MGET"};
  cmd.reserve(size_t(q.num_global_ids) * q.num_optimizer_states * ncols + 1);
  for (uint32_t i = 0; i < q.num_global_ids; ++i)
    for (uint32_t s = 0; s < q.num_optimizer_states; ++s)
      for (uint32_t c = 0; c < ncols; ++c) cmd.push_back(io->key(q.table_name, q.global_ids[i], q.num_cols ? q.col_ids[c] : 0, s));
  io->submit([q, ncols, cmd = std::move(cmd)](Connection& conn) {
    std::vector<std::string> values;
    std::vector<bool> present;
    bool ok = true;
    try {
      if (cmd.size() > 1) {
        conn.command(cmd);
        conn.read_bulk_array(values, present);
      }
    } catch (...) {
      ok = false;  // report every id as missing: the caller re-initialises the rows
    }
    size_t k = 0;
    std::vector<float> row;
    for (uint32_t i = 0; i < q.num_global_ids; ++i)
      for (uint32_t s = 0; s < q.num_optimizer_states; ++s) {
        row.clear();
        bool missing = !ok;
        for (uint32_t c = 0; c < ncols; ++c, ++k) {
          if (missing || k >= values.size() || !present[k] || values[k].size() % sizeof(float) != 0) {
            missing = true;
            continue;
          }
          const size_t n = values[k].size() / sizeof(float);
          const size_t at = row.size();
          row.resize(at + n);
          std::memcpy(row.data() + at, values[k].data(), values[k].size());
        }
        q.on_global_id_fetched(q.on_complete_context, i, s, missing ? nullptr : row.data(), uint32_t(row.size()));
      }
    q.on_all_fetched(q.on_complete_context);
    if (!ok) throw std::runtime_error("redis io: fetch failed");
  });
}

void redis_push(void* inst, IOPushParameter q) {
  auto* io = static_cast<RedisIO*>(inst);
  const uint32_t ncols = q.num_cols == 0 ? 1 : q.num_cols;
  std::vector<std::string> cmd{"MSET"};
  for (uint32_t i = 0; i < q.num_global_ids; ++i)
    for (uint32_t s = 0; s < q.num_optimizer_states; ++s) {
      const size_t k = size_t(i) * q.num_optimizer_states + s;
      const float* b = q.data + q.offsets[k];
      const size_t len = size_t(q.offsets[k + 1] - q.offsets[k]);
      const size_t per = len / ncols;
      for (uint32_t c = 0; c < ncols; ++c) {
        cmd.push_back(io->key(q.table_name, q.global_ids[i], q.num_cols ? q.col_ids[c] : 0, q.optimizer_state_ids[s]));
        cmd.emplace_back(reinterpret_cast<const char*>(b + c * per), per * sizeof(float));
      }
    }
  io->submit([q, cmd = std::move(cmd)](Connection& conn) {
    bool ok = true;
    try {
      if (cmd.size() > 1) {
        conn.command(cmd);
        conn.expect_simple();
      }
    } catch (...) {
      ok = false;
    }
    q.on_push_complete(q.on_complete_context);
    if (!ok) throw std::runtime_error("redis io: push failed");
  });
}
}  // namespace

extern "C" trb::tde::IOProvider trb_tde_io_provider() {
  IOProvider p{};
  p.type = "redis";
  p.initialize = &redis_initialize;
  p.fetch = &redis_fetch;
  p.push = &redis_push;
  p.finalize = &redis_finalize;
  return p;
}
