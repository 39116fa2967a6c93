// Host-runtime basics: assertions that throw, levelled logging, wall-clock helpers, a compact binary
// serializer (the wire format of control messages) and the range recorder used for tracing.
//
// Reference behaviour covered: csrc/include/constants.h:13-53 (ASSERT), csrc/include/logging.h:53-57 (DMOE_LOG),
// csrc/include/utils.hpp:17-22,150-184 (clocks, cerealize/decerealize), csrc/include/profiler.hpp:19-139 (Recorder).
#pragma once
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <iostream>
#include <map>
#include <memory>
#include <mutex>
#include <shared_mutex>
#include <sstream>
#include <stdexcept>
#include <string>
#include <thread>
#include <type_traits>
#include <unordered_map>
#include <vector>

namespace dmoe {

// ------------------------------------------------------------------------------------------- errors, logs
struct RuntimeError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

#define DMOE_STR2(x) #x
#define DMOE_STR(x) DMOE_STR2(x)
#define DMOE_CHECK(cond, msg)                                                                         \
  do {                                                                                                \
    if (!(cond)) {                                                                                    \
      std::ostringstream _os;                                                                         \
      _os << "check failed: " #cond " at " __FILE__ ":" DMOE_STR(__LINE__) " " << msg;                \
      throw ::dmoe::RuntimeError(_os.str());                                                          \
    }                                                                                                 \
  } while (0)
#define DMOE_ASSERT(cond) DMOE_CHECK(cond, "")

enum LogLevel { LOG_DEBUG = 0, LOG_INFO = 1, LOG_WARN = 2, LOG_ERROR = 3 };
inline int& log_threshold() {
  static int lvl = [] {
    const char* e = std::getenv("DMOE_LOG_LEVEL");
    if (e == nullptr) return (int)LOG_WARN;
    std::string s(e);
    if (s == "DEBUG") return (int)LOG_DEBUG;
    if (s == "INFO") return (int)LOG_INFO;
    if (s == "ERROR") return (int)LOG_ERROR;
    return (int)LOG_WARN;
  }();
  return lvl;
}
struct LogLine {
  std::ostringstream os;
  bool on;
  LogLine(int lvl, const char* file, int line) : on(lvl >= log_threshold()) {
    if (on) {
      static const char* names[] = {"D", "I", "W", "E"};
      os << "[dmoe " << names[lvl] << " t" << std::this_thread::get_id() << " " << file << ":" << line << "] ";
    }
  }
  ~LogLine() {
    if (on) {
      os << "\n";
      std::cerr << os.str();
    }
  }
  template <class T>
  LogLine& operator<<(const T& v) {
    if (on) os << v;
    return *this;
  }
};
#define DMOE_LOG(level) ::dmoe::LogLine(::dmoe::LOG_##level, __FILE__, __LINE__)

// ------------------------------------------------------------------------------------------- clocks
inline double now_ms() {
  using namespace std::chrono;
  return duration<double, std::milli>(steady_clock::now().time_since_epoch()).count();
}
// Wall-clock microseconds since the epoch: the unit of SloStat timestamps (CPS = 1e6 ticks per second).
inline int64_t wall_us() {
  using namespace std::chrono;
  return duration_cast<microseconds>(system_clock::now().time_since_epoch()).count();
}

// ------------------------------------------------------------------------------------------- serializer
// Little-endian, length-prefixed. Supports arithmetic types, strings, vectors, pairs and any struct that
// provides `template <class A> void io(A& a)` listing its fields with a(field...).
class Writer {
 public:
  std::string buf;
  static constexpr bool reading = false;
  template <class... Ts>
  void operator()(Ts&... vs) {
    (put(vs), ...);
  }
  template <class T>
  void put(const T& v) {
    if constexpr (std::is_arithmetic_v<T> || std::is_enum_v<T>) {
      buf.append(reinterpret_cast<const char*>(&v), sizeof(T));
    } else {
      put_obj(v);
    }
  }

 private:
  void put_obj(const std::string& s) {
    uint64_t n = s.size();
    put(n);
    buf.append(s);
  }
  template <class T>
  void put_obj(const std::vector<T>& v) {
    uint64_t n = v.size();
    put(n);
    if constexpr (std::is_arithmetic_v<T>) {
      buf.append(reinterpret_cast<const char*>(v.data()), n * sizeof(T));
    } else {
      for (const auto& x : v) put(x);
    }
  }
  template <class A, class B>
  void put_obj(const std::pair<A, B>& p) {
    put(p.first);
    put(p.second);
  }
  template <class T>
  void put_obj(const T& obj) {
    const_cast<T&>(obj).io(*this);
  }
};

class Reader {
 public:
  static constexpr bool reading = true;
  Reader(const char* data, size_t size) : p_(data), end_(data + size) {}
  explicit Reader(const std::string& s) : Reader(s.data(), s.size()) {}
  template <class... Ts>
  void operator()(Ts&... vs) {
    (get(vs), ...);
  }
  template <class T>
  void get(T& v) {
    if constexpr (std::is_arithmetic_v<T> || std::is_enum_v<T>) {
      need(sizeof(T));
      std::memcpy(&v, p_, sizeof(T));
      p_ += sizeof(T);
    } else {
      get_obj(v);
    }
  }
  bool done() const { return p_ == end_; }

 private:
  const char* p_;
  const char* end_;
  void need(size_t n) {
    if (static_cast<size_t>(end_ - p_) < n) throw RuntimeError("truncated message");
  }
  void get_obj(std::string& s) {
    uint64_t n;
    get(n);
    need(n);
    s.assign(p_, n);
    p_ += n;
  }
  template <class T>
  void get_obj(std::vector<T>& v) {
    uint64_t n;
    get(n);
    if constexpr (std::is_arithmetic_v<T>) {
      need(n * sizeof(T));
      v.resize(n);
      std::memcpy(v.data(), p_, n * sizeof(T));
      p_ += n * sizeof(T);
    } else {
      v.clear();
      v.reserve(n);
      for (uint64_t i = 0; i < n; ++i) {
        T x;
        get(x);
        v.emplace_back(std::move(x));
      }
    }
  }
  template <class A, class B>
  void get_obj(std::pair<A, B>& p) {
    get(p.first);
    get(p.second);
  }
  template <class T>
  void get_obj(T& obj) {
    obj.io(*this);
  }
};

template <class T>
std::string to_bytes(const T& obj) {
  Writer w;
  w.put(obj);
  return std::move(w.buf);
}
template <class T>
void from_bytes(const std::string& s, T& obj) {
  Reader r(s);
  r.get(obj);
}

// ------------------------------------------------------------------------------------------- recorder
struct TraceContext {
  std::string msg;
  double t_start = 0;  // ms, wall clock
  double t_dur = 0;    // ms
  int track_id = 0;    // nesting depth of the range on its thread
};

// Per-thread stacks of open ranges and lists of finished ranges. Off unless ENABLE_NVTX=1 (or enable(true)).
class Recorder {
 public:
  static Recorder& instance() {
    static Recorder r;
    return r;
  }
  void enable(bool on) { enabled_.store(on); }
  bool enabled() const { return enabled_.load(); }
  // Registers the calling thread under a readable name (otherwise the name is the thread id).
  void create(const std::string& name = "") {
    std::unique_lock<std::shared_mutex> lk(mu_);
    auto& t = threads_[std::this_thread::get_id()];
    if (!t) t = std::make_shared<PerThread>();
    if (!name.empty()) t->name = name;
  }
  void push(const std::string& msg) {
    if (!enabled()) return;
    auto t = mine();
    t->open.emplace_back(wall_ms(), msg);
  }
  void pop() {
    if (!enabled()) return;
    auto t = mine();
    if (t->open.empty()) return;
    auto [t0, msg] = t->open.back();
    t->open.pop_back();
    const double dur = wall_ms() - t0;
    if (dur > 0.01) {  // ranges under 10 us are dropped
      std::lock_guard<std::mutex> lk(t->mu);
      t->done.push_back(TraceContext{msg, t0, dur, static_cast<int>(t->open.size())});
    }
  }
  // Moves out everything recorded so far: thread name -> finished ranges.
  std::map<std::string, std::vector<TraceContext>> output() {
    std::map<std::string, std::vector<TraceContext>> out;
    std::shared_lock<std::shared_mutex> lk(mu_);
    for (auto& [id, t] : threads_) {
      std::ostringstream os;
      if (t->name.empty()) os << id; else os << t->name;
      std::lock_guard<std::mutex> tl(t->mu);
      auto& dst = out[os.str()];
      dst.insert(dst.end(), t->done.begin(), t->done.end());
      t->done.clear();
    }
    return out;
  }

 private:
  struct PerThread {
    std::string name;
    std::vector<std::pair<double, std::string>> open;
    std::vector<TraceContext> done;
    std::mutex mu;
  };
  Recorder() {
    const char* e = std::getenv("ENABLE_NVTX");
    enabled_.store(e != nullptr && std::string(e) == "1");
  }
  static double wall_ms() { return static_cast<double>(wall_us()) / 1000.0; }
  std::shared_ptr<PerThread> mine() {
    const auto id = std::this_thread::get_id();
    {
      std::shared_lock<std::shared_mutex> lk(mu_);
      auto it = threads_.find(id);
      if (it != threads_.end()) return it->second;
    }
    std::unique_lock<std::shared_mutex> lk(mu_);
    auto& t = threads_[id];
    if (!t) t = std::make_shared<PerThread>();
    return t;
  }
  std::atomic<bool> enabled_{false};
  std::shared_mutex mu_;
  std::map<std::thread::id, std::shared_ptr<PerThread>> threads_;
};

struct ScopedRange {
  explicit ScopedRange(const std::string& msg) { Recorder::instance().push(msg); }
  ~ScopedRange() { Recorder::instance().pop(); }
};
#define DMOE_RANGE(name) ::dmoe::ScopedRange _dmoe_range_##__LINE__(name)
#define DMOE_AUTO_RANGE ::dmoe::ScopedRange _dmoe_range_fn(__func__)

}  // namespace dmoe
