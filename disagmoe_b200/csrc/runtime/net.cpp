#include "net.h"
#include <chrono>
#include <thread>
#include <atomic>

#include <arpa/inet.h>
#include <fcntl.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <fstream>

namespace dmoe {

namespace {
std::mutex g_mu;
std::map<std::string, std::shared_ptr<InprocQueue>> g_inproc;
std::map<int, std::string> g_hosts;
bool g_inproc_transport = false;
int g_port_shift = 0;

std::shared_ptr<InprocQueue> inproc_queue(const std::string& name) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto& q = g_inproc[name];
  if (!q) q = std::make_shared<InprocQueue>();
  return q;
}

bool parse_tcp(const std::string& addr, std::string& host, int& port) {
  const std::string pre = "tcp://";
  if (addr.compare(0, pre.size(), pre) != 0) return false;
  const auto colon = addr.rfind(':');
  if (colon == std::string::npos || colon < pre.size()) return false;
  host = addr.substr(pre.size(), colon - pre.size());
  port = std::stoi(addr.substr(colon + 1));
  return true;
}

void write_all(int fd, const char* p, size_t n) {
  while (n > 0) {
    const ssize_t w = ::send(fd, p, n, MSG_NOSIGNAL);
    if (w < 0) {
      if (errno == EINTR) continue;
      throw RuntimeError(std::string("socket send failed: ") + std::strerror(errno));
    }
    p += w;
    n -= static_cast<size_t>(w);
  }
}

bool read_all(int fd, char* p, size_t n) {
  while (n > 0) {
    const ssize_t r = ::recv(fd, p, n, 0);
    if (r == 0) return false;
    if (r < 0) {
      if (errno == EINTR) continue;
      return false;
    }
    p += r;
    n -= static_cast<size_t>(r);
  }
  return true;
}
}  // namespace

// ------------------------------------------------------------------------------------------------ PullSocket
PullSocket::~PullSocket() { close(); }

void PullSocket::bind(const std::string& addr) {
  addr_ = addr;
  std::string host;
  int port;
  if (!parse_tcp(addr, host, port)) {
    inproc_ = inproc_queue(addr);
    return;
  }
  listen_fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
  DMOE_CHECK(listen_fd_ >= 0, "socket()");
  int one = 1;
  ::setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in sa{};
  sa.sin_family = AF_INET;
  sa.sin_port = htons(static_cast<uint16_t>(port));
  sa.sin_addr.s_addr = htonl(INADDR_ANY);
  DMOE_CHECK(::bind(listen_fd_, reinterpret_cast<sockaddr*>(&sa), sizeof(sa)) == 0,
             "bind " << addr << ": " << std::strerror(errno));
  DMOE_CHECK(::listen(listen_fd_, 128) == 0, "listen " << addr);
}

bool PullSocket::read_ready(int fd, Frames& out) {
  uint32_t nframes = 0;
  if (!read_all(fd, reinterpret_cast<char*>(&nframes), sizeof(nframes))) return false;
  out.resize(nframes);
  for (uint32_t i = 0; i < nframes; ++i) {
    uint64_t len = 0;
    if (!read_all(fd, reinterpret_cast<char*>(&len), sizeof(len))) return false;
    out[i].resize(len);
    if (len > 0 && !read_all(fd, out[i].data(), len)) return false;
  }
  return true;
}

bool PullSocket::recv(Frames& out, int timeout_ms) {
  if (inproc_) {
    std::unique_lock<std::mutex> lk(inproc_->mu);
    auto ready = [&] { return !inproc_->q.empty(); };
    if (timeout_ms < 0) {
      inproc_->cv.wait(lk, ready);
    } else if (!inproc_->cv.wait_for(lk, std::chrono::milliseconds(timeout_ms), ready)) {
      return false;
    }
    out = std::move(inproc_->q.front());
    inproc_->q.pop_front();
    return true;
  }
  DMOE_CHECK(listen_fd_ >= 0, "recv on an unbound socket");
  const double deadline = timeout_ms < 0 ? -1 : now_ms() + timeout_ms;
  for (;;) {
    std::vector<pollfd> fds;
    fds.push_back({listen_fd_, POLLIN, 0});
    for (int c : conns_) fds.push_back({c, POLLIN, 0});
    int wait = -1;
    if (deadline >= 0) {
      wait = static_cast<int>(std::max(0.0, deadline - now_ms()));
    }
    const int rc = ::poll(fds.data(), fds.size(), wait);
    if (rc < 0 && errno == EINTR) continue;
    if (rc <= 0) return false;
    if (fds[0].revents & POLLIN) {
      const int c = ::accept(listen_fd_, nullptr, nullptr);
      if (c >= 0) {
        int one = 1;
        ::setsockopt(c, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
        conns_.push_back(c);
      }
    }
    for (size_t i = 1; i < fds.size(); ++i) {
      if (fds[i].revents & (POLLIN | POLLHUP | POLLERR)) {
        if (read_ready(fds[i].fd, out)) return true;
        ::close(fds[i].fd);  // peer went away
        conns_.erase(std::find(conns_.begin(), conns_.end(), fds[i].fd));
        break;
      }
    }
    if (deadline >= 0 && now_ms() >= deadline) return false;
  }
}

void PullSocket::close() {
  for (int c : conns_) ::close(c);
  conns_.clear();
  if (listen_fd_ >= 0) ::close(listen_fd_);
  listen_fd_ = -1;
  inproc_.reset();
}

// ------------------------------------------------------------------------------------------------ PushSocket
PushSocket::~PushSocket() { close(); }

void PushSocket::connect(const std::string& addr, int timeout_ms) {
  std::string host;
  int port;
  if (!parse_tcp(addr, host, port)) {
    inproc_ = inproc_queue(addr);
    return;
  }
  const double deadline = now_ms() + timeout_ms;
  for (;;) {
    addrinfo hints{}, *res = nullptr;
    hints.ai_family = AF_INET;
    hints.ai_socktype = SOCK_STREAM;
    if (::getaddrinfo(host.c_str(), std::to_string(port).c_str(), &hints, &res) == 0 && res != nullptr) {
      const int fd = ::socket(res->ai_family, res->ai_socktype, res->ai_protocol);
      if (fd >= 0 && ::connect(fd, res->ai_addr, res->ai_addrlen) == 0) {
        int one = 1;
        ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
        ::freeaddrinfo(res);
        fd_ = fd;
        return;
      }
      if (fd >= 0) ::close(fd);
      ::freeaddrinfo(res);
    }
    DMOE_CHECK(now_ms() < deadline, "connect to " << addr << " timed out");
    std::this_thread::sleep_for(std::chrono::milliseconds(20));
  }
}

namespace {
std::mutex g_fault_mu;
int g_fault_kind = SEND_FAULT_NONE, g_fault_countdown = 0, g_fault_delay_ms = 0, g_faults_fired = 0;
std::atomic<uint64_t> g_msg_seq{0};

// Which fault (if any) applies to the message being sent now.
int take_send_fault(int* delay_ms) {
  std::lock_guard<std::mutex> lk(g_fault_mu);
  if (g_fault_kind == SEND_FAULT_NONE || --g_fault_countdown > 0) return SEND_FAULT_NONE;
  const int k = g_fault_kind;
  *delay_ms = g_fault_delay_ms;
  g_fault_kind = SEND_FAULT_NONE;
  ++g_faults_fired;
  return k;
}
}  // namespace

void set_send_fault(int kind, int nth, int delay_ms) {
  std::lock_guard<std::mutex> lk(g_fault_mu);
  g_fault_kind = kind;
  g_fault_countdown = nth < 1 ? 1 : nth;
  g_fault_delay_ms = delay_ms;
}

int send_faults_fired() {
  std::lock_guard<std::mutex> lk(g_fault_mu);
  return g_faults_fired;
}

uint64_t next_message_seq() { return ++g_msg_seq; }

bool SeqFilter::seen(int sender, uint64_t seq) {
  if (seq == 0) return false;
  auto& p = s_[sender];
  if (p.have.count(seq)) {
    ++dups_;
    return true;
  }
  p.have.insert(seq);
  p.order.push_back(seq);
  if (p.order.size() > kWindow) {
    p.have.erase(p.order.front());
    p.order.pop_front();
  }
  return false;
}

void PushSocket::send(const Frames& frames) {
  int delay_ms = 0;
  const int fault = take_send_fault(&delay_ms);
  if (fault == SEND_FAULT_DROP) return;
  if (fault == SEND_FAULT_DELAY) std::this_thread::sleep_for(std::chrono::milliseconds(delay_ms));
  send_now(frames);
  if (fault == SEND_FAULT_DUPLICATE) send_now(frames);
}

void PushSocket::send_now(const Frames& frames) {
  if (inproc_) {
    {
      std::lock_guard<std::mutex> lk(inproc_->mu);
      inproc_->q.push_back(frames);
    }
    inproc_->cv.notify_one();
    return;
  }
  DMOE_CHECK(fd_ >= 0, "send on an unconnected socket");
  std::lock_guard<std::mutex> lk(mu_);
  // header and small frames are coalesced into one write
  std::string head;
  const uint32_t n = static_cast<uint32_t>(frames.size());
  head.append(reinterpret_cast<const char*>(&n), sizeof(n));
  for (const auto& f : frames) {
    const uint64_t len = f.size();
    head.append(reinterpret_cast<const char*>(&len), sizeof(len));
    if (len <= 4096) {
      head.append(f);
    } else {
      write_all(fd_, head.data(), head.size());
      head.clear();
      write_all(fd_, f.data(), f.size());
    }
  }
  if (!head.empty()) write_all(fd_, head.data(), head.size());
}

void PushSocket::close() {
  if (fd_ >= 0) ::close(fd_);
  fd_ = -1;
  inproc_.reset();
}

// ------------------------------------------------------------------------------------------------ addressing
void set_hosts(int pid_tag, const std::map<int, std::string>& device_ip) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_hosts = device_ip;
  // persisted so that tools attached to the same job can resolve devices
  const std::string dir = "/tmp/disagmoe_b200";
  (void)::system(("mkdir -p " + dir).c_str());
  std::ofstream f(dir + "/hostfile_" + std::to_string(pid_tag));
  for (auto& [d, ip] : device_ip) f << d << " " << ip << "\n";
}

std::string get_ip_of_device(int device_id) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_hosts.find(device_id);
  return it == g_hosts.end() ? "127.0.0.1" : it->second;
}

void set_inproc_transport(bool on) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_inproc_transport = on;
}
bool inproc_transport() {
  std::lock_guard<std::mutex> lk(g_mu);
  return g_inproc_transport;
}
void set_port_base(int shift) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_port_shift = shift;
}

std::string get_zmq_addr(int device_id, bool is_gpu, int offset, int group_hash) {
  DMOE_CHECK(offset >= 0 && offset < 16, "socket offset " << offset);
  int base = is_gpu ? 24000 : 35000;
  if (group_hash > 0) base = 46000 + (group_hash % 997) * 16;
  int shift;
  bool inproc;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    shift = g_port_shift;
    inproc = g_inproc_transport;
  }
  const int port = base + shift + device_id * 16 + offset;
  if (inproc) return "inproc://dev" + std::to_string(device_id) + "/" + std::to_string(port);
  return "tcp://" + get_ip_of_device(device_id) + ":" + std::to_string(port);
}

}  // namespace dmoe
