#include "channel.h"

#include <dlfcn.h>

namespace dmoe {

torch::ScalarType dtype_from_string(const std::string& s) {
  if (s == "bf16") return torch::kBFloat16;
  if (s == "fp16") return torch::kFloat16;
  if (s == "fp32") return torch::kFloat32;
  throw RuntimeError("unknown dtype " + s);
}
std::string dtype_to_string(torch::ScalarType t) {
  if (t == torch::kBFloat16) return "bf16";
  if (t == torch::kFloat16) return "fp16";
  if (t == torch::kFloat32) return "fp32";
  throw RuntimeError("unsupported tensor dtype");
}

std::string tensor_to_bytes(const torch::Tensor& t) {
  auto c = t.contiguous().cpu();
  return std::string(static_cast<const char*>(c.data_ptr()), c.nbytes());
}

torch::Tensor tensor_from_bytes(const std::string& bytes, const Metadata& meta) {
  auto t = torch::empty(meta.shape, torch::TensorOptions().dtype(dtype_from_string(meta.dtype)));
  DMOE_CHECK(t.nbytes() == bytes.size(), "payload of " << bytes.size() << " bytes for " << meta.str());
  std::memcpy(t.data_ptr(), bytes.data(), bytes.size());
  return t;
}

// ------------------------------------------------------------------------------------------------ local
void LocalChannel::send(const torch::Tensor& t, const Metadata&) {
  {
    std::lock_guard<std::mutex> lk(mu_);
    q_.push_back(t);
  }
  cv_.notify_one();
}
void LocalChannel::recv(torch::Tensor& t, const Metadata&) {
  std::unique_lock<std::mutex> lk(mu_);
  DMOE_CHECK(cv_.wait_for(lk, std::chrono::seconds(30), [&] { return !q_.empty(); }), "local channel recv timed out");
  t = q_.front();
  q_.pop_front();
}

uint64_t LocalChannel::stash(const torch::Tensor& t) {
  std::lock_guard<std::mutex> lk(mu_);
  const uint64_t id = next_ticket_++;
  parked_[id] = t;
  return id;
}
torch::Tensor LocalChannel::claim(uint64_t ticket) {
  std::lock_guard<std::mutex> lk(mu_);
  auto it = parked_.find(ticket);
  DMOE_CHECK(it != parked_.end(), "unknown local ticket " << ticket);
  auto t = it->second;
  parked_.erase(it);
  return t;
}

// ------------------------------------------------------------------------------------------------ socket
SocketChannel::SocketChannel(int local, int other, bool is_sender, int rank_offset)
    : Channel(local, other), sender_(is_sender), offset_(rank_offset) {
  set_role(is_sender);
}
void SocketChannel::instantiate() {
  // the receiving side owns the address
  const int owner = sender_ ? other_ : local_;
  const std::string addr = get_zmq_addr(owner, !is_embedding_node(owner), offset_);
  if (sender_) push_.connect(addr); else pull_.bind(addr);
}
void SocketChannel::send(const torch::Tensor& t, const Metadata& meta) {
  push_.send({to_bytes(meta), tensor_to_bytes(t)});
}
void SocketChannel::recv(torch::Tensor& t, const Metadata& meta) {
  Frames f;
  DMOE_CHECK(pull_.recv(f, 30000) && f.size() == 2, "socket channel recv timed out");
  Metadata m;
  from_bytes(f[0], m);
  auto host = tensor_from_bytes(f[1], m);
  if (t.defined() && t.numel() == host.numel()) t.copy_(host); else t = host;
}

// ------------------------------------------------------------------------------------------------ GPU api
namespace {
std::string g_nccl_path, g_cudart_path;
void* sym(void* h, const char* name) { return h != nullptr ? dlsym(h, name) : nullptr; }
void* open_lib(const std::string& path, const char* const* fallbacks) {
  if (!path.empty()) {
    if (void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_GLOBAL)) return h;
  }
  for (const char* const* f = fallbacks; *f != nullptr; ++f) {
    if (void* h = dlopen(*f, RTLD_NOW | RTLD_NOLOAD)) return h;   // already loaded by PyTorch
    if (void* h = dlopen(*f, RTLD_NOW | RTLD_GLOBAL)) return h;
  }
  return nullptr;
}
}  // namespace

void GpuApi::set_library_paths(const std::string& nccl, const std::string& cudart) {
  g_nccl_path = nccl;
  g_cudart_path = cudart;
}

GpuApi::GpuApi() {
  static const char* nccl_names[] = {"libnccl.so.2", "libnccl.so", nullptr};
  static const char* rt_names[] = {"libcudart.so.12", "libcudart.so", nullptr};
  void* hn = open_lib(g_nccl_path, nccl_names);
  void* hr = open_lib(g_cudart_path, rt_names);
  if (hn == nullptr || hr == nullptr) {
    why_ = std::string("could not load ") + (hn == nullptr ? "libnccl" : "libcudart");
    return;
  }
#define LOAD(h, name) name = reinterpret_cast<decltype(name)>(sym(h, #name)); if (name == nullptr) { why_ = "missing symbol " #name; return; }
  LOAD(hn, ncclGetUniqueId) LOAD(hn, ncclCommInitRank) LOAD(hn, ncclCommDestroy) LOAD(hn, ncclSend) LOAD(hn, ncclRecv)
  LOAD(hn, ncclBroadcast) LOAD(hn, ncclAllReduce) LOAD(hn, ncclGetErrorString)
  LOAD(hr, cudaStreamCreateWithFlags) LOAD(hr, cudaStreamSynchronize) LOAD(hr, cudaStreamDestroy)
  LOAD(hr, cudaMemcpyAsync) LOAD(hr, cudaSetDevice)
  LOAD(hr, cudaEventCreateWithFlags) LOAD(hr, cudaEventRecord) LOAD(hr, cudaStreamWaitEvent) LOAD(hr, cudaEventDestroy)
#undef LOAD
  ok_ = true;
}

GpuApi& GpuApi::get() {
  static GpuApi api;
  return api;
}

#define NCCL_OK(expr)                                                                                   \
  do {                                                                                                  \
    const int _r = (expr);                                                                              \
    DMOE_CHECK(_r == 0, "NCCL error " << _r << " (" << GpuApi::get().ncclGetErrorString(_r) << ") in " #expr); \
  } while (0)
#define CUDA_OK(expr)                                       \
  do {                                                      \
    const int _r = (expr);                                  \
    DMOE_CHECK(_r == 0, "CUDA error " << _r << " in " #expr); \
  } while (0)

static GpuApi& gpu_or_throw() {
  auto& a = GpuApi::get();
  DMOE_CHECK(a.available(), "NCCL transport unavailable: " << a.why_not());
  return a;
}

std::string get_nccl_unique_id() {
  NcclId id;
  NCCL_OK(gpu_or_throw().ncclGetUniqueId(&id));
  return std::string(id.internal, sizeof(id.internal));
}

static NcclId uid_from_string(const std::string& s) {
  DMOE_CHECK(s.size() == sizeof(NcclId), "an NCCL unique id has 128 bytes, got " << s.size());
  NcclId id;
  std::memcpy(id.internal, s.data(), sizeof(id.internal));
  return id;
}

static int nccl_dtype_of(const torch::Tensor& t) {
  // ncclDataType_t: int8 0, uint8 1, int32 2, int64 4, fp16 6, fp32 7, bf16 9
  switch (t.scalar_type()) {
    case torch::kBFloat16: return 9;
    case torch::kFloat16: return 6;
    case torch::kFloat32: return 7;
    case torch::kInt32: return 2;
    case torch::kInt64: return 4;
    case torch::kInt8: return 0;
    case torch::kUInt8: return 1;
    default: throw RuntimeError("dtype not supported by the NCCL channel");
  }
}

// ------------------------------------------------------------------------------------------------ NcclChannel
NcclChannel::NcclChannel(int local, int other, const std::string& uid) : Channel(local, other), uid_(uid_from_string(uid)) {}

NcclChannel::~NcclChannel() {
  auto& a = GpuApi::get();
  if (comm_ != nullptr && a.available()) a.ncclCommDestroy(comm_);
  if (stream_ != nullptr && a.available()) a.cudaStreamDestroy(stream_);
  if (fence_ != nullptr && a.available()) a.cudaEventDestroy(fence_);
}

void NcclChannel::instantiate() {
  auto& a = gpu_or_throw();
  CUDA_OK(a.cudaStreamCreateWithFlags(&stream_, 1 /*cudaStreamNonBlocking*/));
  CUDA_OK(a.cudaEventCreateWithFlags(&fence_, 2 /*cudaEventDisableTiming*/));
  NCCL_OK(a.ncclCommInitRank(&comm_, 2, uid_, rank()));
}

// The rows of a batch are produced by kernels on the default stream of the engine thread, and a freshly allocated
// receive buffer may be a cached block that kernels still queued there read. The channel's own stream is
// non-blocking, so both directions order themselves behind the default stream explicitly.
void NcclChannel::wait_for_compute() {
  auto& a = gpu_or_throw();
  CUDA_OK(a.cudaEventRecord(fence_, nullptr));
  CUDA_OK(a.cudaStreamWaitEvent(stream_, fence_, 0));
}

void NcclChannel::send(const torch::Tensor& t, const Metadata&) {
  auto& a = gpu_or_throw();
  DMOE_CHECK(t.is_cuda() && t.is_contiguous(), "NCCL send needs a contiguous CUDA tensor");
  wait_for_compute();
  NCCL_OK(a.ncclSend(t.data_ptr(), t.numel(), nccl_dtype_of(t), 1 - rank(), comm_, stream_));
  // the caller may drop its reference as soon as this returns, and the caching allocator would hand the block to the
  // next compute-stream allocation: the send has to be complete first
  CUDA_OK(a.cudaStreamSynchronize(stream_));
}

void NcclChannel::recv(torch::Tensor& t, const Metadata& meta) {
  auto& a = gpu_or_throw();
  if (!t.defined()) {
    t = torch::empty(meta.shape, torch::TensorOptions().dtype(dtype_from_string(meta.dtype)).device(torch::kCUDA));
  }
  wait_for_compute();
  NCCL_OK(a.ncclRecv(t.data_ptr(), t.numel(), nccl_dtype_of(t), 1 - rank(), comm_, stream_));
}

void NcclChannel::sync() { CUDA_OK(gpu_or_throw().cudaStreamSynchronize(stream_)); }

// ------------------------------------------------------------------------------------------------ NcclGroupChannel
NcclGroupChannel::NcclGroupChannel(int local_rank, int world, const std::string& uid)
    : Channel(local_rank, 0), world_(world), uid_(uid_from_string(uid)) {}

NcclGroupChannel::~NcclGroupChannel() {
  auto& a = GpuApi::get();
  if (comm_ != nullptr && a.available()) a.ncclCommDestroy(comm_);
  if (stream_ != nullptr && a.available()) a.cudaStreamDestroy(stream_);
  if (fence_ != nullptr && a.available()) a.cudaEventDestroy(fence_);
}

// Tensors handed to this channel are produced (or were last used) on the default stream, and the channel's stream
// is non-blocking: every collective first waits for an event recorded on the default stream.
void NcclGroupChannel::wait_for_compute() {
  auto& a = gpu_or_throw();
  CUDA_OK(a.cudaEventRecord(fence_, nullptr));
  CUDA_OK(a.cudaStreamWaitEvent(stream_, fence_, 0));
}

void NcclGroupChannel::instantiate() {
  auto& a = gpu_or_throw();
  CUDA_OK(a.cudaStreamCreateWithFlags(&stream_, 1));
  CUDA_OK(a.cudaEventCreateWithFlags(&fence_, 2 /*cudaEventDisableTiming*/));
  NCCL_OK(a.ncclCommInitRank(&comm_, world_, uid_, local_));
  staging_ = torch::empty({1 << 16}, torch::TensorOptions().dtype(torch::kUInt8).device(torch::kCUDA));
  barrier();
}

void NcclGroupChannel::broadcast(const void* send_buf, void* recv_buf, size_t count, int dtype, int root) {
  wait_for_compute();
  NCCL_OK(gpu_or_throw().ncclBroadcast(send_buf, recv_buf, count, dtype, root, comm_, stream_));
  sync();
}

void NcclGroupChannel::send(const torch::Tensor& t, const Metadata&) {
  broadcast(t.data_ptr(), t.data_ptr(), t.numel(), nccl_dtype_of(t), 0);
}
void NcclGroupChannel::recv(torch::Tensor& t, const Metadata& meta) {
  if (!t.defined())
    t = torch::empty(meta.shape, torch::TensorOptions().dtype(dtype_from_string(meta.dtype)).device(torch::kCUDA));
  broadcast(t.data_ptr(), t.data_ptr(), t.numel(), nccl_dtype_of(t), 0);
}
void NcclGroupChannel::sync() { CUDA_OK(gpu_or_throw().cudaStreamSynchronize(stream_)); }

void NcclGroupChannel::bcast_obj(std::string& bytes) {
  auto& a = gpu_or_throw();
  // 1. size, 2. bytes; both through the device staging buffer
  auto size_dev = torch::empty({1}, torch::TensorOptions().dtype(torch::kInt64).device(torch::kCUDA));
  if (is_root()) size_dev.fill_(static_cast<int64_t>(bytes.size()));
  broadcast(size_dev.data_ptr(), size_dev.data_ptr(), 1, 4, 0);
  const int64_t n = size_dev.cpu().item<int64_t>();
  if (n > staging_.numel()) staging_ = torch::empty({n}, staging_.options());
  if (is_root()) {
    CUDA_OK(a.cudaMemcpyAsync(staging_.data_ptr(), bytes.data(), n, 1 /*H2D*/, stream_));
  }
  broadcast(staging_.data_ptr(), staging_.data_ptr(), n, 1, 0);
  if (!is_root()) {
    bytes.resize(n);
    CUDA_OK(a.cudaMemcpyAsync(bytes.data(), staging_.data_ptr(), n, 2 /*D2H*/, stream_));
    sync();
  }
}

void NcclGroupChannel::send_metadata(const Metadata& meta) {
  std::string b = to_bytes(meta);
  bcast_obj(b);
}
void NcclGroupChannel::recv_metadata(Metadata& meta) {
  std::string b;
  bcast_obj(b);
  from_bytes(b, meta);
}

void NcclGroupChannel::all_reduce(torch::Tensor& t) {
  DMOE_CHECK(t.is_cuda() && t.is_contiguous(), "all_reduce needs a contiguous CUDA tensor");
  wait_for_compute();
  NCCL_OK(gpu_or_throw().ncclAllReduce(t.data_ptr(), t.data_ptr(), t.numel(), nccl_dtype_of(t), 0 /*sum*/, comm_, stream_));
}

void NcclGroupChannel::barrier() {
  auto one = torch::ones({1}, torch::TensorOptions().dtype(torch::kInt32).device(torch::kCUDA));
  wait_for_compute();
  NCCL_OK(gpu_or_throw().ncclAllReduce(one.data_ptr(), one.data_ptr(), 1, 2, 0, comm_, stream_));
  sync();
}

// ------------------------------------------------------------------------------------------------ factories
channel_t create_channel(int local, int other, const std::string& uid) {
  return std::make_shared<NcclChannel>(local, other, uid);
}
channel_t create_local_channel(int local) { return std::make_shared<LocalChannel>(local, local); }
channel_t create_socket_channel(int local, int other, bool is_sender, int rank_offset) {
  return std::make_shared<SocketChannel>(local, other, is_sender, rank_offset);
}
std::shared_ptr<NcclGroupChannel> create_nccl_group_channel(int local_rank, int world, const std::string& uid) {
  return std::make_shared<NcclGroupChannel>(local_rank, world, uid);
}

void instantiate_channels(const std::vector<channel_t>& channels) {
  std::vector<std::thread> ts;
  std::vector<std::string> errors(channels.size());
  for (size_t i = 0; i < channels.size(); ++i) {
    ts.emplace_back([&, i] {
      try {
        channels[i]->instantiate();
      } catch (const std::exception& e) {
        errors[i] = e.what();
      }
    });
  }
  for (auto& t : ts) t.join();
  for (auto& e : errors) DMOE_CHECK(e.empty(), "channel instantiate failed: " << e);
}

}  // namespace dmoe
