// Control-plane transport: PUSH/PULL message sockets with multi-frame messages.
//
// It plays the role ZeroMQ plays in the reference (csrc/muhelper/muhelper.cpp:93-94,388-401,
// csrc/muhelper/comm.cpp:122-211) without depending on libzmq: "tcp://host:port" endpoints are plain TCP
// streams carrying length-prefixed frames, "inproc://name" endpoints are in-process queues. A PullSocket accepts
// any number of pushers. Receives take a timeout so that a helper thread can always be stopped (the reference
// joins threads that are blocked in recv). Port scheme of get_zmq_addr (csrc/include/distributed.hpp:52-59).
#pragma once
#include <map>
#include <set>
#include <condition_variable>
#include <deque>

#include "core.h"

namespace dmoe {

using Frames = std::vector<std::string>;

struct InprocQueue {
  std::mutex mu;
  std::condition_variable cv;
  std::deque<Frames> q;
};

class PullSocket {
 public:
  PullSocket() = default;
  ~PullSocket();
  PullSocket(const PullSocket&) = delete;
  void bind(const std::string& addr);
  // false on timeout (timeout_ms < 0 waits forever)
  bool recv(Frames& out, int timeout_ms);
  void close();
  const std::string& addr() const { return addr_; }

 private:
  bool read_ready(int fd, Frames& out);
  std::string addr_;
  int listen_fd_ = -1;
  std::vector<int> conns_;
  std::shared_ptr<InprocQueue> inproc_;
};

class PushSocket {
 public:
  PushSocket() = default;
  ~PushSocket();
  PushSocket(const PushSocket&) = delete;
  // Retries for up to timeout_ms until the peer has bound.
  void connect(const std::string& addr, int timeout_ms = 30000);
  void send(const Frames& frames);
  void close();
  bool connected() const { return fd_ >= 0 || inproc_ != nullptr; }

 private:
  void send_now(const Frames& frames);
  std::mutex mu_;
  int fd_ = -1;
  std::shared_ptr<InprocQueue> inproc_;
};

// Host-side fault injection for tests of the failure paths (no GPU is involved): the `nth` message sent by this
// process from now on (1 = the next one) is dropped, sent twice, or held back for `delay_ms`. One shot.
enum SendFault { SEND_FAULT_NONE = 0, SEND_FAULT_DROP = 1, SEND_FAULT_DUPLICATE = 2, SEND_FAULT_DELAY = 3 };
void set_send_fault(int kind, int nth, int delay_ms = 0);
int send_faults_fired();

// Receiver-side duplicate filter: remembers the last `window` sequence numbers seen per sender.
class SeqFilter {
 public:
  // True when (sender, seq) was seen before (the caller then drops the message). seq 0 = unnumbered, never a duplicate.
  bool seen(int sender, uint64_t seq);
  uint64_t duplicates() const { return dups_; }

 private:
  struct PerSender {
    std::deque<uint64_t> order;
    std::set<uint64_t> have;
  };
  std::map<int, PerSender> s_;
  uint64_t dups_ = 0;
  static constexpr size_t kWindow = 8192;
};
// Process-wide message numbering (strictly increasing, never 0).
uint64_t next_message_seq();

// device id -> ip table (persisted so that helper processes of the same job can read it)
void set_hosts(int pid_tag, const std::map<int, std::string>& device_ip);
std::string get_ip_of_device(int device_id);
// Address of the mailbox of `device_id`. offset selects one of 16 sockets of the device; group_hash > 0 selects
// the port range of group channels.
std::string get_zmq_addr(int device_id, bool is_gpu = true, int offset = 0, int group_hash = 0);
// All sockets use in-process queues instead of TCP (single-process tests and colocated workers).
void set_inproc_transport(bool on);
bool inproc_transport();
void set_port_base(int base_shift);

}  // namespace dmoe
