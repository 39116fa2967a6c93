// Tensor transports between workers.
//
//   Channel           abstract point-to-point edge (instantiate / send / recv / sync)
//   LocalChannel      same process: the tensor handle itself is queued (no copy)
//   SocketChannel     any two processes: bytes over the PUSH/PULL transport (CPU tensors; device tensors are staged
//                     through host memory) -- the data-carrying stand-in for the reference's ZmqChannel
//   NcclChannel       two GPUs: a 2-rank NCCL communicator, ncclSend / ncclRecv on a private stream
//   NcclGroupChannel  N GPUs (a TP group): broadcast, object broadcast, bf16 sum all-reduce, barrier
//
// NCCL and the CUDA runtime are resolved at run time from the libraries PyTorch has already loaded, so this
// module imports (and its CPU paths work) on a machine without a GPU.
//
// Reference behaviour covered: csrc/include/comm.h:17-177, csrc/muhelper/comm.cpp:9-476.
#pragma once
#include <torch/torch.h>

#include "net.h"
#include "types.h"

namespace dmoe {

torch::ScalarType dtype_from_string(const std::string& s);
std::string dtype_to_string(torch::ScalarType t);
// Serialises the rows of a tensor (moved to host memory if needed) / rebuilds a CPU tensor from bytes.
std::string tensor_to_bytes(const torch::Tensor& t);
torch::Tensor tensor_from_bytes(const std::string& bytes, const Metadata& meta);

class Channel {
 public:
  Channel(int local, int other) : local_(local), other_(other) {}
  virtual ~Channel() = default;
  virtual void instantiate() = 0;
  virtual void send(const torch::Tensor& t, const Metadata& meta) = 0;
  // Receives into `t` (pre-allocated by the caller from `meta`) or replaces it.
  virtual void recv(torch::Tensor& t, const Metadata& meta) = 0;
  virtual void sync() {}
  // True when the tensor bytes travel inside the mailbox message that carries the metadata.
  virtual bool inline_payload() const { return false; }
  // Same-process edges: the tensor is parked under a ticket that travels in the mailbox message, so that several
  // sender threads cannot mix up each other's tensors. 0 = tickets not supported.
  virtual uint64_t stash(const torch::Tensor& t) { (void)t; return 0; }
  virtual torch::Tensor claim(uint64_t ticket) { (void)ticket; return torch::Tensor(); }
  int local() const { return local_; }
  int other() const { return other_; }
  bool is_sender() const { return local_ < other_ || role_sender_; }
  void set_role(bool sender) { role_sender_ = sender; role_set_ = true; }
  std::mutex& send_mutex() { return send_mu_; }

 protected:
  int local_, other_;
  bool role_sender_ = false, role_set_ = false;
  std::mutex send_mu_;   // keeps (mailbox message, tensor) pairs of concurrent senders in the same order
};
using channel_t = std::shared_ptr<Channel>;

class LocalChannel : public Channel {
 public:
  using Channel::Channel;
  void instantiate() override {}
  void send(const torch::Tensor& t, const Metadata& meta) override;
  void recv(torch::Tensor& t, const Metadata& meta) override;
  uint64_t stash(const torch::Tensor& t) override;
  torch::Tensor claim(uint64_t ticket) override;

 private:
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<torch::Tensor> q_;
  std::map<uint64_t, torch::Tensor> parked_;
  uint64_t next_ticket_ = 1;
};

class SocketChannel : public Channel {
 public:
  // rank_offset selects one of the 16 sockets of the receiving device, so several channels can end on it.
  SocketChannel(int local, int other, bool is_sender, int rank_offset = 1);
  void instantiate() override;
  void send(const torch::Tensor& t, const Metadata& meta) override;
  void recv(torch::Tensor& t, const Metadata& meta) override;
  bool inline_payload() const override { return true; }

 private:
  bool sender_;
  int offset_;
  PushSocket push_;
  PullSocket pull_;
};

struct NcclId {
  char internal[128];
};

// Functions of libnccl / libcudart resolved with dlsym.
struct GpuApi {
  static GpuApi& get();
  bool available() const { return ok_; }
  const std::string& why_not() const { return why_; }
  // nccl
  int (*ncclGetUniqueId)(void*) = nullptr;
  int (*ncclCommInitRank)(void**, int, NcclId /*by value*/, int) = nullptr;
  int (*ncclCommDestroy)(void*) = nullptr;
  int (*ncclSend)(const void*, size_t, int, int, void*, void*) = nullptr;
  int (*ncclRecv)(void*, size_t, int, int, void*, void*) = nullptr;
  int (*ncclBroadcast)(const void*, void*, size_t, int, int, void*, void*) = nullptr;
  int (*ncclAllReduce)(const void*, void*, size_t, int, int, void*, void*) = nullptr;
  const char* (*ncclGetErrorString)(int) = nullptr;
  // cuda runtime
  int (*cudaStreamCreateWithFlags)(void**, unsigned) = nullptr;
  int (*cudaStreamSynchronize)(void*) = nullptr;
  int (*cudaStreamDestroy)(void*) = nullptr;
  int (*cudaMemcpyAsync)(void*, const void*, size_t, int, void*) = nullptr;
  int (*cudaSetDevice)(int) = nullptr;
  int (*cudaEventCreateWithFlags)(void**, unsigned) = nullptr;
  int (*cudaEventRecord)(void*, void*) = nullptr;
  int (*cudaStreamWaitEvent)(void*, void*, unsigned) = nullptr;
  int (*cudaEventDestroy)(void*) = nullptr;
  static void set_library_paths(const std::string& nccl, const std::string& cudart);

 private:
  GpuApi();
  bool ok_ = false;
  std::string why_;
};
std::string get_nccl_unique_id();  // 128 raw bytes

class NcclChannel : public Channel {
 public:
  NcclChannel(int local, int other, const std::string& uid);
  ~NcclChannel() override;
  void instantiate() override;
  void send(const torch::Tensor& t, const Metadata& meta) override;
  void recv(torch::Tensor& t, const Metadata& meta) override;
  void sync() override;

 private:
  int rank() const { return local_ < other_ ? 0 : 1; }
  void wait_for_compute();   // orders stream_ after everything enqueued so far on the default (compute) stream
  NcclId uid_;
  void* comm_ = nullptr;
  void* stream_ = nullptr;
  void* fence_ = nullptr;    // CUDA event reused by wait_for_compute
};

class NcclGroupChannel : public Channel {
 public:
  NcclGroupChannel(int local_rank, int world_size, const std::string& uid);
  ~NcclGroupChannel() override;
  void instantiate() override;
  void send(const torch::Tensor& t, const Metadata& meta) override;   // root side of a broadcast
  void recv(torch::Tensor& t, const Metadata& meta) override;         // non-root side of a broadcast
  void sync() override;
  bool is_root() const { return local_ == 0; }
  void broadcast(const void* send_buf, void* recv_buf, size_t count, int nccl_dtype, int root = 0);
  // Broadcasts an opaque byte string from rank 0 (size first, then bytes through a device staging buffer).
  void bcast_obj(std::string& bytes);
  void send_metadata(const Metadata& meta);
  void recv_metadata(Metadata& meta);
  void all_reduce(torch::Tensor& t);   // in-place sum
  void barrier();

 private:
  void wait_for_compute();  // orders stream_ after everything enqueued so far on the default (compute) stream
  int world_;
  NcclId uid_;
  void* comm_ = nullptr;
  void* stream_ = nullptr;
  void* fence_ = nullptr;
  torch::Tensor staging_;   // device buffer for object broadcasts
};

channel_t create_channel(int local, int other, const std::string& nccl_uid);
channel_t create_local_channel(int local);
channel_t create_socket_channel(int local, int other, bool is_sender, int rank_offset = 1);
std::shared_ptr<NcclGroupChannel> create_nccl_group_channel(int local_rank, int world, const std::string& uid);
// Instantiates every channel on its own thread (both ends of an NCCL edge must call at the same time).
void instantiate_channels(const std::vector<channel_t>& channels);

}  // namespace dmoe
