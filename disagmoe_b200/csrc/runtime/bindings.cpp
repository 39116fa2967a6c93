// pybind11 module `disagmoe_c`: the native host runtime exposed to Python.
// Reference surface covered: csrc/bindings.cpp:24-221 (class and function names kept where the concept exists here).
#include <chrono>

#include <pybind11/functional.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "engine.h"
#include "fused_scheduler.h"

namespace py = pybind11;
using namespace dmoe;

namespace {

// ---- in-module self tests (the reference compiles its tests into the extension too, binding_tests.hpp) ----
// Two socket channels in one process: a tensor goes 0 -> 1 and must arrive bit-exact.
bool test_socket_p2p(int n, int hidden) {
  auto rx = create_socket_channel(1, 0, false, 3);
  auto tx = create_socket_channel(0, 1, true, 3);
  rx->instantiate();
  tx->instantiate();
  auto t = torch::randn({n, hidden});
  Metadata m;
  m.shape = {n, hidden};
  m.dtype = "fp32";
  tx->send(t, m);
  torch::Tensor out;
  rx->recv(out, m);
  return torch::equal(t, out);
}

// A TP driver and `n_workers` workers whose pools were filled with the same tokens must pick identical batches.
bool test_parallel_attn_scheduler(int n_workers, int n_tokens) {
  const std::vector<int> layers{0, 1};
  std::map<int, int> need{{0, 1}, {1, 1}};
  std::vector<std::shared_ptr<MuAttentionPool>> pools;
  std::mutex mu;
  std::condition_variable cv;
  ScheduleDecision shared;
  int version = 0;
  for (int r = 0; r <= n_workers; ++r) {
    pools.push_back(std::make_shared<MuAttentionPool>(layers, 900 + r, std::map<int, channel_t>{}, need));
    auto meta = std::make_shared<Metadata>();
    meta->shape = {n_tokens, 8};
    meta->dtype = "fp32";
    meta->layer_id = 1;
    for (int i = 0; i < n_tokens; ++i) {
      meta->tok.req_ids.push_back(100 + i);
      meta->tok.positions.push_back(i % 3);
      meta->tok.init_prefill_lens.push_back(-1);
      meta->tok.attn_dp_ranks.push_back(0);
      meta->tok.topk_slots.push_back(0);
    }
    pools.back()->process_batch(torch::ones({n_tokens, 8}) * r, meta, MSG_TOKENS);
  }
  auto root_bcast = [&](ScheduleDecision& d) {
    std::lock_guard<std::mutex> lk(mu);
    shared = d;
    ++version;
    cv.notify_all();
  };
  AttentionDriverScheduler driver(pools[0], layers, root_bcast);
  std::vector<std::vector<int>> got(n_workers);
  std::vector<std::thread> ts;
  for (int r = 0; r < n_workers; ++r) {
    ts.emplace_back([&, r] {
      auto recv = [&](ScheduleDecision& d) {
        std::unique_lock<std::mutex> lk(mu);
        cv.wait_for(lk, std::chrono::seconds(5), [&] { return version > 0; });
        d = shared;
      };
      AttentionWorkerScheduler w(pools[r + 1], layers, recv);
      auto b = w.schedule();
      if (b.metadata) got[r] = b.metadata->seq_ids;
    });
  }
  auto b = driver.schedule();
  for (auto& t : ts) t.join();
  if (!b.metadata || static_cast<int>(b.metadata->seq_ids.size()) != n_tokens) return false;
  for (auto& g : got)
    if (g != b.metadata->seq_ids) return false;
  return true;
}

// Ten threads record nested ranges concurrently; every thread must end up with its own ranges.
int test_recorder_threads(int n_threads) {
  auto& r = Recorder::instance();
  const bool was = r.enabled();
  r.enable(true);
  r.output();
  std::vector<std::thread> ts;
  for (int i = 0; i < n_threads; ++i)
    ts.emplace_back([i] {
      Recorder::instance().create("t" + std::to_string(i));
      for (int k = 0; k < 3; ++k) {
        ScopedRange outer("outer");
        std::this_thread::sleep_for(std::chrono::milliseconds(1));
        ScopedRange inner("inner");
        std::this_thread::sleep_for(std::chrono::milliseconds(1));
      }
    });
  for (auto& t : ts) t.join();
  auto out = r.output();
  r.enable(was);
  int ok = 0;
  for (auto& [name, v] : out)
    if (name.rfind("t", 0) == 0 && v.size() == 6) ++ok;
  return ok;
}

// 2-rank NCCL channel in one process on two devices (GPU only).
bool test_nccl_p2p(int dev_a, int dev_b, int n, int hidden) {
  const std::string uid = get_nccl_unique_id();
  auto a = create_channel(0, 1, uid), b = create_channel(1, 0, uid);
  auto& api = GpuApi::get();
  std::thread ta([&] { api.cudaSetDevice(dev_a); a->instantiate(); });
  std::thread tb([&] { api.cudaSetDevice(dev_b); b->instantiate(); });
  ta.join();
  tb.join();
  auto src = torch::randn({n, hidden}, torch::TensorOptions().dtype(torch::kBFloat16).device(torch::kCUDA, dev_a));
  Metadata m;
  m.shape = {n, hidden};
  torch::Tensor dst = torch::empty({n, hidden}, torch::TensorOptions().dtype(torch::kBFloat16).device(torch::kCUDA, dev_b));
  std::thread ts([&] { api.cudaSetDevice(dev_a); a->send(src, m); a->sync(); });
  std::thread tr([&] { api.cudaSetDevice(dev_b); b->recv(dst, m); b->sync(); });
  ts.join();
  tr.join();
  return torch::equal(src.cpu(), dst.cpu());
}

// N ranks of one NCCL group channel in one process (one thread per device): barrier, tensor broadcast from rank 0,
// object broadcast, in-place all-reduce. True when every rank saw the expected values.
bool test_nccl_group(std::vector<int> devices) {
  const int world = static_cast<int>(devices.size());
  const std::string uid = get_nccl_unique_id();
  auto& api = GpuApi::get();
  std::vector<int> ok(world, 0);
  std::vector<std::thread> ts;
  for (int r = 0; r < world; ++r) {
    ts.emplace_back([&, r] {
      const int dev = devices[r];
      api.cudaSetDevice(dev);
      auto ch = create_nccl_group_channel(r, world, uid);
      ch->instantiate();
      ch->barrier();
      const auto opts = torch::TensorOptions().dtype(torch::kBFloat16).device(torch::kCUDA, dev);
      Metadata m;
      m.shape = {8, 64};
      auto want = torch::arange(8 * 64, torch::TensorOptions().dtype(torch::kFloat32)).reshape({8, 64}).to(torch::kBFloat16);
      torch::Tensor t = r == 0 ? want.to(opts.device()) : torch::zeros({8, 64}, opts);
      if (r == 0) ch->send(t, m); else ch->recv(t, m);
      ch->sync();
      bool good = torch::equal(t.cpu(), want);
      std::string obj = r == 0 ? std::string("schedule: layer 3, sequences 5 9 11") : std::string();
      ch->bcast_obj(obj);
      good = good && obj == "schedule: layer 3, sequences 5 9 11";
      auto x = torch::full({4, 32}, static_cast<float>(r + 1), opts);
      ch->all_reduce(x);
      ch->sync();
      good = good && torch::allclose(x.cpu().to(torch::kFloat32), torch::full({4, 32}, world * (world + 1) / 2.0f));
      ch->barrier();
      ok[r] = good ? 1 : 0;
    });
  }
  for (auto& t : ts) t.join();
  for (int v : ok)
    if (!v) return false;
  return true;
}

typedef int (*add_one_fn)(const float*, float*, long long, void*);

// Many small launches of the debug kernel on two streams at once, each stream a dependent chain x -> x + 1 -> ...;
// true when both chains end at `launches` (launch ordering inside a stream, independence between streams).
bool test_multi_launch(int device, int launches, int n) {
  auto fn = reinterpret_cast<add_one_fn>(kernel_library_symbol("dmoe_add_one"));
  DMOE_CHECK(fn != nullptr, "the kernel library (lib/libdmoe_kernels.so) is not built");
  auto& api = GpuApi::get();
  api.cudaSetDevice(device);
  const auto opts = torch::TensorOptions().dtype(torch::kFloat32).device(torch::kCUDA, device);
  void* streams[2] = {nullptr, nullptr};
  torch::Tensor buf[2][2];
  for (int s = 0; s < 2; ++s) {
    DMOE_CHECK(api.cudaStreamCreateWithFlags(&streams[s], 1) == 0, "cudaStreamCreateWithFlags failed");
    buf[s][0] = torch::zeros({n}, opts);
    buf[s][1] = torch::zeros({n}, opts);
  }
  api.cudaStreamSynchronize(nullptr);   // the zero fills ran on the default stream
  bool ok = true;
  for (int i = 0; i < launches; ++i)
    for (int s = 0; s < 2; ++s)
      ok = ok && fn(buf[s][i & 1].data_ptr<float>(), buf[s][(i + 1) & 1].data_ptr<float>(), n, streams[s]) == 0;
  for (int s = 0; s < 2; ++s) {
    api.cudaStreamSynchronize(streams[s]);
    ok = ok && torch::allclose(buf[s][launches & 1].cpu(), torch::full({n}, static_cast<float>(launches)));
    api.cudaStreamDestroy(streams[s]);
  }
  return ok;
}

// Does a collective on the group channel's stream overlap with kernels on a compute stream? Two ranks (one thread per
// device) time, on the host, a run of broadcasts alone, a run of debug-kernel launches alone, and both together.
// Returns rank 0's {broadcast ms, kernels ms, both ms}; overlap shows as both < broadcast + kernels.
std::vector<double> test_op_overlap(int dev_a, int dev_b, int mbytes, int launches) {
  auto fn = reinterpret_cast<add_one_fn>(kernel_library_symbol("dmoe_add_one"));
  DMOE_CHECK(fn != nullptr, "the kernel library (lib/libdmoe_kernels.so) is not built");
  const std::string uid = get_nccl_unique_id();
  auto& api = GpuApi::get();
  std::vector<double> out(3, 0.0);
  const int devs[2] = {dev_a, dev_b};
  auto worker = [&](int r) {
    const int dev = devs[r];
    api.cudaSetDevice(dev);
    auto ch = create_nccl_group_channel(r, 2, uid);
    ch->instantiate();
    const int64_t n = static_cast<int64_t>(mbytes) << 18;   // fp32 elements
    const auto opts = torch::TensorOptions().dtype(torch::kFloat32).device(torch::kCUDA, dev);
    auto payload = torch::ones({n}, opts), a = torch::zeros({n}, opts), b = torch::zeros({n}, opts);
    void* compute = nullptr;
    DMOE_CHECK(api.cudaStreamCreateWithFlags(&compute, 1) == 0, "cudaStreamCreateWithFlags failed");
    api.cudaStreamSynchronize(nullptr);
    auto bcasts = [&] { for (int i = 0; i < 4; ++i) ch->broadcast(payload.data_ptr(), payload.data_ptr(), n, 7 /*float*/, 0); };
    auto kernels = [&] { for (int i = 0; i < launches; ++i) fn(a.data_ptr<float>(), b.data_ptr<float>(), n, compute); };
    auto wait_all = [&] { ch->sync(); api.cudaStreamSynchronize(compute); };
    auto timed = [&](bool do_b, bool do_k) {
      ch->barrier();
      const auto t0 = std::chrono::steady_clock::now();
      if (do_b) bcasts();
      if (do_k) kernels();
      wait_all();
      return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    };
    timed(true, true);   // warm-up
    const double tb = timed(true, false), tk = timed(false, true), tboth = timed(true, true);
    ch->barrier();
    api.cudaStreamDestroy(compute);
    if (r == 0) { out[0] = tb; out[1] = tk; out[2] = tboth; }
  };
  std::thread t0(worker, 0), t1(worker, 1);
  t0.join();
  t1.join();
  return out;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "disagmoe_b200 native host runtime";
  py::register_exception<RuntimeError>(m, "RuntimeError", PyExc_RuntimeError);

  // ---- data types ------------------------------------------------------------------------------------
  py::class_<ChannelInfo>(m, "ChannelInfo")
      .def(py::init<>())
      .def(py::init<std::vector<ExpertId>, std::vector<int>, int>(), py::arg("expert_ids"), py::arg("attn_layer_ids"),
           py::arg("attn_dp_rank") = 0)
      .def_readwrite("expert_ids", &ChannelInfo::expert_ids)
      .def_readwrite("attn_layer_ids", &ChannelInfo::attn_layer_ids)
      .def_readwrite("attn_dp_rank", &ChannelInfo::attn_dp_rank)
      .def("is_sampler_channel", &ChannelInfo::is_sampler_channel);

  py::class_<TokenMetadata>(m, "TokenMetadata")
      .def(py::init<>())
      .def_readwrite("req_id", &TokenMetadata::req_id)
      .def_readwrite("exp_id", &TokenMetadata::exp_id)
      .def_readwrite("attn_dp_rank", &TokenMetadata::attn_dp_rank)
      .def_readwrite("init_prefill_len", &TokenMetadata::init_prefill_len)
      .def_readwrite("topk_weight", &TokenMetadata::topk_weight)
      .def_readwrite("position", &TokenMetadata::position)
      .def_readwrite("topk_slot", &TokenMetadata::topk_slot);

  py::class_<ParallelConfig>(m, "ParallelConfig")
      .def(py::init<>())
      .def_readwrite("tp", &ParallelConfig::tp)
      .def_readwrite("ep", &ParallelConfig::ep)
      .def_readwrite("dp", &ParallelConfig::dp)
      .def_readwrite("n_exp_per_rank", &ParallelConfig::n_exp_per_rank)
      .def_readwrite("expert_ranks", &ParallelConfig::expert_ranks)
      .def("rank_of", &ParallelConfig::rank_of);

  py::class_<SloStat>(m, "SloStat")
      .def(py::init<>())
      .def_readwrite("req_id", &SloStat::req_id)
      .def_readwrite("t_prefill", &SloStat::t_prefill)
      .def_readwrite("t_prefill_std", &SloStat::t_prefill_std)
      .def_readwrite("t_decode", &SloStat::t_decode)
      .def_readwrite("t_tokens", &SloStat::t_tokens);

  py::class_<SamplerStepInfo>(m, "SamplerStepInfo")
      .def(py::init<>())
      .def_readwrite("num_tokens", &SamplerStepInfo::num_tokens)
      .def_readwrite("time_stamp", &SamplerStepInfo::time_stamp);

  py::class_<TraceContext>(m, "TraceContext")
      .def_readonly("msg", &TraceContext::msg)
      .def_readonly("t_start", &TraceContext::t_start)
      .def_readonly("t_dur", &TraceContext::t_dur)
      .def_readonly("track_id", &TraceContext::track_id);

  py::class_<Metadata, std::shared_ptr<Metadata>>(m, "Metadata")
      .def(py::init<>())
      .def(py::init([](std::vector<int64_t> shape) {
        auto p = std::make_shared<Metadata>();
        p->shape = std::move(shape);
        return p;
      }))
      .def_readwrite("shape", &Metadata::shape)
      .def_readwrite("dtype", &Metadata::dtype)
      .def_readwrite("layer_id", &Metadata::layer_id)
      .def_property("req_ids", [](Metadata& s) { return s.tok.req_ids; }, [](Metadata& s, std::vector<int> v) { s.tok.req_ids = std::move(v); })
      .def_property("exp_ids", [](Metadata& s) { return s.tok.exp_ids; }, [](Metadata& s, std::vector<int> v) { s.tok.exp_ids = std::move(v); })
      .def_property("attn_dp_ranks", [](Metadata& s) { return s.tok.attn_dp_ranks; }, [](Metadata& s, std::vector<int> v) { s.tok.attn_dp_ranks = std::move(v); })
      .def_property("init_prefill_lens", [](Metadata& s) { return s.tok.init_prefill_lens; }, [](Metadata& s, std::vector<int> v) { s.tok.init_prefill_lens = std::move(v); })
      .def_property("positions", [](Metadata& s) { return s.tok.positions; }, [](Metadata& s, std::vector<int> v) { s.tok.positions = std::move(v); })
      .def_property("topk_slots", [](Metadata& s) { return s.tok.topk_slots; }, [](Metadata& s, std::vector<int> v) { s.tok.topk_slots = std::move(v); })
      .def_property("token_ids", [](Metadata& s) { return s.tok.token_ids; }, [](Metadata& s, std::vector<int> v) { s.tok.token_ids = std::move(v); })
      .def_property("topk_weights", [](Metadata& s) { return s.tok.topk_weights; }, [](Metadata& s, std::vector<float> v) { s.tok.topk_weights = std::move(v); })
      .def("num_tokens", &Metadata::num_tokens)
      .def("token_hidden_dim", &Metadata::token_hidden_dim)
      .def("num_element", &Metadata::num_element)
      .def("slice", [](Metadata& s, int l, int r) { return std::make_shared<Metadata>(s.slice(l, r)); })
      .def("at", [](Metadata& s, std::vector<int> ids) { return std::make_shared<Metadata>(s.at(ids)); })
      .def("info_at", &Metadata::info_at)
      .def("step_layer", &Metadata::step_layer)
      .def("get_expert_batch_sizes", &Metadata::get_expert_batch_sizes)
      .def("get_expert_offsets", &Metadata::get_expert_offsets)
      .def("update_exp_ids", &Metadata::update_exp_ids)
      .def("permute_token_infos", &Metadata::permute_token_infos)
      .def("duplicate_topk", &Metadata::duplicate_topk)
      .def("shrink_topk", &Metadata::shrink_topk)
      .def("sort_by_prefill_order", &Metadata::sort_by_prefill_order)
      .def("split", &Metadata::split)
      .def_static("merge_by_exp_ids", [](std::vector<metadata_t> metas) {
        std::vector<int> mapping;
        auto mm = Metadata::merge_by_exp_ids(metas, mapping);
        return std::make_pair(mm, mapping);
      })
      .def_static("concat", &Metadata::concat)
      .def("serialize", [](Metadata& s) { return py::bytes(to_bytes(s)); })
      .def_static("deserialize", [](const std::string& b) {
        auto p = std::make_shared<Metadata>();
        from_bytes(b, *p);
        return p;
      })
      .def("__repr__", &Metadata::str);

  py::class_<AttentionBatchMetadata, std::shared_ptr<AttentionBatchMetadata>>(m, "AttentionBatchMetadata")
      .def(py::init<>())
      .def_readwrite("layer_id", &AttentionBatchMetadata::layer_id)
      .def_readwrite("shape", &AttentionBatchMetadata::shape)
      .def_readwrite("dtype", &AttentionBatchMetadata::dtype)
      .def_readwrite("num_prefill_seqs", &AttentionBatchMetadata::num_prefill_seqs)
      .def_readwrite("num_prefill_tokens", &AttentionBatchMetadata::num_prefill_tokens)
      .def_readwrite("num_decode_tokens", &AttentionBatchMetadata::num_decode_tokens)
      .def_readwrite("seq_ids", &AttentionBatchMetadata::seq_ids)
      .def_readwrite("init_prefill_lens", &AttentionBatchMetadata::init_prefill_lens)
      .def_readwrite("positions", &AttentionBatchMetadata::positions)
      .def_readwrite("token_ids", &AttentionBatchMetadata::token_ids)
      .def_readwrite("expert_ids", &AttentionBatchMetadata::expert_ids)
      .def_readwrite("topk_weights", &AttentionBatchMetadata::topk_weights)
      .def_readwrite("attn_dp_ranks", &AttentionBatchMetadata::attn_dp_ranks)
      .def("num_tokens", &AttentionBatchMetadata::num_tokens)
      .def("to_metadata", &AttentionBatchMetadata::to_metadata)
      .def("recount", &AttentionBatchMetadata::recount)
      .def_static("from_metadata", &AttentionBatchMetadata::from_metadata)
      .def_static("merge", [](std::vector<attn_metadata_t> b) {
        std::vector<int> order;
        auto mm = AttentionBatchMetadata::merge(b, order);
        return std::make_pair(mm, order);
      })
      .def("serialize", [](AttentionBatchMetadata& s) { return py::bytes(to_bytes(s)); })
      .def_static("deserialize", [](const std::string& b) {
        auto p = std::make_shared<AttentionBatchMetadata>();
        from_bytes(b, *p);
        return p;
      });

  py::class_<TensorBatch>(m, "TensorBatch")
      .def(py::init<>())
      .def(py::init([](torch::Tensor data, metadata_t meta) { return TensorBatch{std::move(data), std::move(meta)}; }))
      .def_property("data", [](TensorBatch& b) -> py::object { return b.data.defined() ? py::cast(b.data) : py::none(); },
                    [](TensorBatch& b, torch::Tensor t) { b.data = std::move(t); })
      .def_readwrite("metadata", &TensorBatch::metadata)
      .def_static("merge", &TensorBatch::merge)
      .def_static("concat", &TensorBatch::concat);

  py::class_<AttentionBatch>(m, "AttentionBatch")
      .def(py::init<>())
      .def_property("data", [](AttentionBatch& b) -> py::object { return b.data.defined() ? py::cast(b.data) : py::none(); },
                    [](AttentionBatch& b, torch::Tensor t) { b.data = std::move(t); })
      .def_readwrite("metadata", &AttentionBatch::metadata)
      .def_readwrite("num_parts", &AttentionBatch::num_parts);

  // ---- block manager ---------------------------------------------------------------------------------
  py::class_<BlockManager, std::shared_ptr<BlockManager>>(m, "BlockManager")
      .def(py::init<int, int, int, int>(), py::arg("block_size"), py::arg("num_blocks"), py::arg("reserved_blocks"),
           py::arg("max_rows") = 0)
      .def("can_allocate", &BlockManager::can_allocate)
      .def("can_append", &BlockManager::can_append)
      .def("allocate", &BlockManager::allocate)
      .def("append_block", &BlockManager::append_block)
      .def("append_tokens", &BlockManager::append_tokens)
      .def("release", &BlockManager::release)
      .def("batch_release", &BlockManager::batch_release)
      .def("num_free_blocks", &BlockManager::num_free_blocks)
      .def("num_seqs", &BlockManager::num_seqs)
      .def("has_seq_block_list", &BlockManager::has_seq_block_list)
      .def("get_seq_block_list", &BlockManager::get_seq_block_list)
      .def("row_of", &BlockManager::row_of)
      .def("slot_of", &BlockManager::slot_of)
      .def("update_block_table", &BlockManager::update_block_table)
      .def("step_decode", &BlockManager::step_decode)
      .def("prepare_block_table", [](BlockManager& b, const AttentionBatchMetadata& meta, const std::vector<int>& lens) {
        int mb = 0;
        auto flat = b.prepare_block_table(meta, lens, &mb);
        auto t = torch::tensor(flat, torch::TensorOptions().dtype(torch::kInt32));
        return std::make_pair(t, mb);
      })
      .def("drain_updates", [](BlockManager& b) {
        std::vector<std::tuple<int, int, int>> out;
        for (auto& u : b.drain_updates()) out.emplace_back(u.row, u.col, u.block);
        return out;
      });
  // ---- serving scheduler of the fused data plane ------------------------------------------------------------------
  py::class_<FusedSeq, fused_seq_t>(m, "FusedSeq")
      .def(py::init([](int req_id, std::vector<int> prompt, int max_new_tokens, double t_arrival, int mb, int length,
                       int last_token, std::vector<int> outputs, std::vector<double> t_tokens) {
             auto s = std::make_shared<FusedSeq>();
             s->req_id = req_id; s->prompt = std::move(prompt); s->max_new_tokens = max_new_tokens;
             s->t_arrival = t_arrival; s->mb = mb; s->length = length; s->last_token = last_token;
             s->outputs = std::move(outputs); s->t_tokens = std::move(t_tokens);
             return s;
           }),
           py::arg("req_id"), py::arg("prompt"), py::arg("max_new_tokens"), py::arg("t_arrival") = 0.0, py::arg("mb") = -1,
           py::arg("length") = 0, py::arg("last_token") = 0, py::arg("outputs") = std::vector<int>{},
           py::arg("t_tokens") = std::vector<double>{})
      .def_readwrite("req_id", &FusedSeq::req_id)
      .def_readwrite("prompt", &FusedSeq::prompt)
      .def_readwrite("max_new_tokens", &FusedSeq::max_new_tokens)
      .def_readwrite("t_arrival", &FusedSeq::t_arrival)
      .def_readwrite("mb", &FusedSeq::mb)
      .def_readwrite("length", &FusedSeq::length)
      .def_readwrite("last_token", &FusedSeq::last_token)
      .def_readwrite("outputs", &FusedSeq::outputs)
      .def_readwrite("t_tokens", &FusedSeq::t_tokens);
  py::class_<FusedPlan>(m, "FusedPlan")
      .def(py::init<>())
      .def_readwrite("ids", &FusedPlan::ids)
      .def_readwrite("pos", &FusedPlan::pos)
      .def_readwrite("rows", &FusedPlan::rows)
      .def_readwrite("slots", &FusedPlan::slots)
      .def_readwrite("emit", &FusedPlan::emit)
      .def("__len__", &FusedPlan::size)
      .def("copy_to", [](const FusedPlan& p, torch::Tensor ids, torch::Tensor pos, torch::Tensor ctx, torch::Tensor rows,
                         torch::Tensor slots, int64_t offset) {
        const int64_t n = p.size();
        for (auto* t : {&ids, &pos, &ctx, &rows})
          DMOE_CHECK(t->scalar_type() == torch::kInt32 && t->is_contiguous() && !t->is_cuda() && t->numel() >= offset + n,
                     "copy_to: int32 contiguous host tensors with room for the plan are needed");
        DMOE_CHECK(slots.scalar_type() == torch::kInt64 && slots.is_contiguous() && !slots.is_cuda() &&
                       slots.numel() >= offset + n, "copy_to: slots must be an int64 contiguous host tensor");
        p.copy_to(ids.data_ptr<int32_t>() + offset, pos.data_ptr<int32_t>() + offset, ctx.data_ptr<int32_t>() + offset,
                  rows.data_ptr<int32_t>() + offset, slots.data_ptr<int64_t>() + offset);
      }, py::arg("ids"), py::arg("pos"), py::arg("ctx"), py::arg("rows"), py::arg("slots"), py::arg("offset") = 0);
  py::class_<FusedScheduler, std::shared_ptr<FusedScheduler>>(m, "FusedScheduler")
      .def(py::init<std::shared_ptr<BlockManager>, int, int, int, int, int, bool>(), py::arg("block_mgr"),
           py::arg("block_size"), py::arg("n_mb"), py::arg("max_seqs_per_mb"), py::arg("max_tokens_per_mb"),
           py::arg("max_prefill_tokens_per_mb") = 0, py::arg("ignore_eos") = true)
      .def("add_request", &FusedScheduler::add_request, py::arg("req_id"), py::arg("prompt"), py::arg("max_new_tokens"),
           py::arg("t_arrival"))
      .def("num_unfinished", &FusedScheduler::num_unfinished)
      .def("has_work", &FusedScheduler::has_work, py::arg("now"))
      .def("build", &FusedScheduler::build, py::arg("now"), py::call_guard<py::gil_scoped_release>())
      .def("commit", &FusedScheduler::commit, py::arg("plans"), py::arg("next_ids"), py::arg("now"))
      .def("restore_running", &FusedScheduler::restore_running, py::arg("mb"), py::arg("seq"))
      .def("restore_finished", &FusedScheduler::restore_finished, py::arg("seq"))
      .def_property_readonly("waiting", [](const FusedScheduler& s) { return s.waiting(); })
      .def_property_readonly("running", [](const FusedScheduler& s) {
        // per micro-batch: request id -> sequence, in admission order
        py::list out;
        for (auto& r : s.running()) {
          py::dict d;
          for (auto& q : r) d[py::int_(q->req_id)] = q;
          out.append(d);
        }
        return out;
      })
      .def_property_readonly("finished", [](const FusedScheduler& s) {
        py::dict d;
        for (auto& kv : s.finished()) d[py::int_(kv.first)] = kv.second;
        return d;
      })
      .def_property_readonly("pool_blocks", &FusedScheduler::pool_blocks)
      .def_property_readonly("max_tokens", &FusedScheduler::max_tokens)
      .def_property_readonly("max_seqs", &FusedScheduler::max_seqs)
      .def_property_readonly("max_prefill", &FusedScheduler::max_prefill)
      .def_readonly_static("MIN_CHUNK", &FusedScheduler::MIN_CHUNK);

  m.def("prepare_batch_infos", [](const AttentionBatchMetadata& meta, const std::vector<int>& lens) {
    return torch::tensor(prepare_batch_infos(meta, lens), torch::TensorOptions().dtype(torch::kInt32));
  });

  // ---- layer schedulers ------------------------------------------------------------------------------
  py::class_<LayerScheduler, std::shared_ptr<LayerScheduler>>(m, "LayerScheduler")
      .def(py::init([](int n, const std::string& policy) {
             return std::make_shared<LayerScheduler>(n, LayerScheduler::parse_policy(policy));
           }), py::arg("n_layers"), py::arg("policy") = "mbfs")
      .def("schedule", &LayerScheduler::schedule)
      .def("add_tokens_to_layer", py::overload_cast<int, int>(&LayerScheduler::add_tokens_to_layer))
      .def("remove_tokens_from_layer", &LayerScheduler::remove_tokens_from_layer)
      .def("set_schedule_type", &LayerScheduler::set_schedule_type)
      .def("set_block_size", &LayerScheduler::set_block_size)
      .def("get_tokens_per_layer", &LayerScheduler::get_tokens_per_layer);
  py::class_<AdvancedLayerScheduler, LayerScheduler, std::shared_ptr<AdvancedLayerScheduler>>(m, "AdvancedLayerScheduler")
      .def(py::init<int, int>(), py::arg("n_layers"), py::arg("hold_steps") = 2)
      .def("set_clock", &AdvancedLayerScheduler::set_clock);
  py::class_<GroupLayerScheduler, LayerScheduler, std::shared_ptr<GroupLayerScheduler>>(m, "GroupLayerScheduler")
      .def(py::init<int, int>())
      .def("add_tokens_to_group", py::overload_cast<int, int, int>(&GroupLayerScheduler::add_tokens_to_layer))
      .def("cell", &GroupLayerScheduler::cell);

  // ---- channels --------------------------------------------------------------------------------------
  py::class_<Channel, std::shared_ptr<Channel>>(m, "Channel")
      .def("instantiate", &Channel::instantiate, py::call_guard<py::gil_scoped_release>())
      .def("send", &Channel::send, py::call_guard<py::gil_scoped_release>())
      .def("recv", [](Channel& c, const Metadata& meta) {
        torch::Tensor t;
        {
          py::gil_scoped_release rel;
          c.recv(t, meta);
          c.sync();
        }
        return t;
      })
      .def("sync", &Channel::sync, py::call_guard<py::gil_scoped_release>());
  py::class_<NcclChannel, Channel, std::shared_ptr<NcclChannel>>(m, "NcclChannel");
  py::class_<LocalChannel, Channel, std::shared_ptr<LocalChannel>>(m, "TensorLocalChannel");
  py::class_<SocketChannel, Channel, std::shared_ptr<SocketChannel>>(m, "SocketChannel");
  py::class_<NcclGroupChannel, Channel, std::shared_ptr<NcclGroupChannel>>(m, "NcclGroupChannel")
      .def("all_reduce", &NcclGroupChannel::all_reduce, py::call_guard<py::gil_scoped_release>())
      .def("barrier", &NcclGroupChannel::barrier, py::call_guard<py::gil_scoped_release>())
      .def("bcast_obj", [](NcclGroupChannel& c, std::string b) {
        {
          py::gil_scoped_release rel;
          c.bcast_obj(b);
        }
        return py::bytes(b);
      })
      .def("send_metadata", &NcclGroupChannel::send_metadata, py::call_guard<py::gil_scoped_release>())
      .def("recv_metadata", [](NcclGroupChannel& c) {
        auto mm = std::make_shared<Metadata>();
        py::gil_scoped_release rel;
        c.recv_metadata(*mm);
        return mm;
      });
  m.def("create_channel", [](int local, int other, py::bytes uid) { return create_channel(local, other, std::string(uid)); });
  m.def("create_local_channel", &create_local_channel);
  m.def("create_socket_channel", &create_socket_channel, py::arg("local"), py::arg("other"), py::arg("is_sender"),
        py::arg("rank_offset") = 1);
  m.def("create_nccl_group_channel", [](int rank, int world, py::bytes uid) {
    return create_nccl_group_channel(rank, world, std::string(uid));
  });
  // Name-compatible factories of the reference module (csrc/bindings.cpp:190-196): one group channel per local rank
  // of an in-process party; a p2p channel whose id is picked from a {peer: id} map or given directly.
  m.def("create_nccl_group_channels", [](int root, const std::vector<int>& party_all, py::bytes uid) {
    DMOE_CHECK(root == 0, "the group root is rank 0");
    std::vector<std::shared_ptr<NcclGroupChannel>> out;
    const std::string id(uid);
    for (size_t i = 0; i < party_all.size(); ++i)
      out.push_back(create_nccl_group_channel(static_cast<int>(i), static_cast<int>(party_all.size()), id));
    return out;
  });
  m.def("create_channel_py_map", [](int local, int peer, const std::map<int, py::bytes>& uids) {
    auto it = uids.find(peer);
    DMOE_CHECK(it != uids.end(), "no channel id for peer " << peer);
    return create_channel(local, peer, std::string(it->second));
  });
  m.def("create_channel_py_single", [](int local, int peer, py::bytes uid) {
    return create_channel(local, peer, std::string(uid));
  });
  // Row scatter out[mappings[i]] = tokens[i / k], k = len(mappings) / len(tokens) (reference: csrc/permute.cu:53-112,
  // bound under the same name). This entry runs on any device through tensor ops; the sm_100a kernel of the same
  // operation is dmoe_permute_rows in the kernel library (disagmoe_b200.ops.memory.permute_tokens_cuda).
  m.def("permute_tokens_cuda", [](const torch::Tensor& tokens, const torch::Tensor& mappings, uintptr_t /*stream*/) {
    const int64_t n_out = mappings.numel();
    const int64_t k = std::max<int64_t>(1, n_out / std::max<int64_t>(1, tokens.size(0)));
    auto src = k > 1 ? tokens.repeat_interleave(k, 0) : tokens;
    auto out = torch::empty({n_out, tokens.size(1)}, tokens.options());
    out.index_copy_(0, mappings.to(torch::kLong).to(tokens.device()), src.slice(0, 0, n_out));
    return out;
  }, py::arg("tokens"), py::arg("mappings"), py::arg("stream") = 0);
  m.def("instantiate_channels", &instantiate_channels, py::call_guard<py::gil_scoped_release>());
  m.def("get_nccl_unique_id", [] { return py::bytes(get_nccl_unique_id()); });
  m.def("set_gpu_library_paths", &GpuApi::set_library_paths);
  m.def("gpu_transport_available", [] { return GpuApi::get().available(); });

  // ---- addressing ------------------------------------------------------------------------------------
  m.def("set_hosts", &set_hosts);
  m.def("get_zmq_addr", &get_zmq_addr, py::arg("device_id"), py::arg("is_gpu") = true, py::arg("offset") = 0,
        py::arg("group_hash") = 0);
  m.def("set_inproc_transport", &set_inproc_transport);
  m.def("set_send_fault", &set_send_fault, py::arg("kind"), py::arg("nth"), py::arg("delay_ms") = 0);
  m.def("send_faults_fired", &send_faults_fired);
  m.attr("SEND_FAULT_DROP") = static_cast<int>(SEND_FAULT_DROP);
  m.attr("SEND_FAULT_DUPLICATE") = static_cast<int>(SEND_FAULT_DUPLICATE);
  m.attr("SEND_FAULT_DELAY") = static_cast<int>(SEND_FAULT_DELAY);
  m.def("set_port_base", &set_port_base);
  m.def("is_embedding_node", &is_embedding_node);

  // ---- helpers ---------------------------------------------------------------------------------------
  py::class_<MuHelper, std::shared_ptr<MuHelper>>(m, "MuHelper")
      .def("start", &MuHelper::start)
      .def("terminate", &MuHelper::terminate, py::call_guard<py::gil_scoped_release>());
  py::class_<MuDispatcher, MuHelper, std::shared_ptr<MuDispatcher>>(m, "MuDispatcher")
      .def("put", &MuDispatcher::put, py::arg("batch"), py::arg("kind") = 0)
      .def("pending", &MuDispatcher::pending);
  py::class_<MuAttnDispatcher, MuDispatcher, std::shared_ptr<MuAttnDispatcher>>(m, "MuAttnDispatcher");
  py::class_<MuExpertDispatcher, MuDispatcher, std::shared_ptr<MuExpertDispatcher>>(m, "MuExpertDispatcher");
  py::class_<MuPool, MuHelper, std::shared_ptr<MuPool>>(m, "MuPool")
      .def("process_batch", [](MuPool& p, py::object t, metadata_t meta, int kind) {
        p.process_batch(t.is_none() ? torch::Tensor() : t.cast<torch::Tensor>(), meta, kind);
      }, py::arg("tensor"), py::arg("meta"), py::arg("kind") = 0)
      .def("get_pool_snapshot", &MuPool::get_pool_snapshot)
      .def("tokens_in_layer", &MuPool::tokens_in_layer);
  py::class_<MuAttentionPool, MuPool, std::shared_ptr<MuAttentionPool>>(m, "MuAttentionPool")
      .def("num_pending_tokens", &MuAttentionPool::num_pending_tokens)
      .def("release_seqs", &MuAttentionPool::release_seqs)
      .def("set_unordered_layer", &MuAttentionPool::set_unordered_layer)
      .def("fetch_attention_batch", &MuAttentionPool::fetch_attention_batch);

  py::class_<Scheduler, std::shared_ptr<Scheduler>>(m, "Scheduler")
      .def("schedule", &Scheduler::schedule)
      .def("wait_for_new_requests", &Scheduler::wait_for_new_requests, py::arg("timeout_ms") = 100,
           py::call_guard<py::gil_scoped_release>())
      .def("get_pool_snapshot", &Scheduler::get_pool_snapshot)
      .def("get_cur_queueing_delay", &Scheduler::get_cur_queueing_delay)
      .def("set_max_batch_size", &Scheduler::set_max_batch_size)
      .def("set_schedule_policy", &Scheduler::set_schedule_policy)
      .def("set_schedule_block", &Scheduler::set_schedule_block);
  py::class_<AttentionScheduler, std::shared_ptr<AttentionScheduler>>(m, "AttentionScheduler")
      .def("schedule", &AttentionScheduler::schedule)
      .def("wait_for_new_requests", &AttentionScheduler::wait_for_new_requests, py::arg("timeout_ms") = 100,
           py::call_guard<py::gil_scoped_release>())
      .def("get_pool_snapshot", &AttentionScheduler::get_pool_snapshot)
      .def("get_cur_queueing_delay", &AttentionScheduler::get_cur_queueing_delay)
      .def("set_max_batch_size", &AttentionScheduler::set_max_batch_size)
      .def("set_schedule_policy", &AttentionScheduler::set_schedule_policy)
      .def("set_schedule_block", &AttentionScheduler::set_schedule_block)
      .def("pool", &AttentionScheduler::pool);

  py::class_<Tokenizer, MuDispatcher, std::shared_ptr<Tokenizer>>(m, "Tokenizer")
      .def("put_request", &Tokenizer::put_request);
  py::class_<Sampler, MuDispatcher, std::shared_ptr<Sampler>>(m, "Sampler")
      .def("start_all", &Sampler::start_all)
      .def("stop_all", &Sampler::stop_all, py::call_guard<py::gil_scoped_release>())
      .def("set_request_output_len", &Sampler::set_request_output_len)
      .def("process_batch", &Sampler::process_batch)
      .def("fetch_finished_slo_stats", &Sampler::fetch_finished_slo_stats)
      .def("fetch_step_infos", &Sampler::fetch_step_infos)
      .def("wait_slo_stats", &Sampler::wait_slo_stats)
      .def("get_output_tokens", &Sampler::get_output_tokens)
      .def("num_finished", &Sampler::num_finished)
      .def("reset", &Sampler::reset);
  py::class_<TopKSampler, Sampler, std::shared_ptr<TopKSampler>>(m, "TopKSampler");

  // ---- engine factory --------------------------------------------------------------------------------
  py::class_<EngineArgs>(m, "EngineArgs")
      .def(py::init<>())
      .def_readwrite("local_id", &EngineArgs::local_id)
      .def_readwrite("top_k", &EngineArgs::top_k)
      .def_readwrite("has_attn", &EngineArgs::has_attn)
      .def_readwrite("has_expert", &EngineArgs::has_expert)
      .def_readwrite("cfg", &EngineArgs::cfg)
      .def_readwrite("attn_layer_ids", &EngineArgs::attn_layer_ids)
      .def_readwrite("expert_layer_ids", &EngineArgs::expert_layer_ids)
      .def_readwrite("in_device_ids", &EngineArgs::in_device_ids)
      .def_readwrite("out_device_ids", &EngineArgs::out_device_ids)
      .def_readwrite("out_channel_infos", &EngineArgs::out_channel_infos)
      .def_property("in_nccl_ids", [](EngineArgs& a) { std::map<int, py::bytes> o; for (auto& [k, v] : a.in_nccl_ids) o[k] = py::bytes(v); return o; },
                    [](EngineArgs& a, std::map<int, std::string> v) { a.in_nccl_ids = std::move(v); })
      .def_property("out_nccl_ids", [](EngineArgs& a) { std::map<int, py::bytes> o; for (auto& [k, v] : a.out_nccl_ids) o[k] = py::bytes(v); return o; },
                    [](EngineArgs& a, std::map<int, std::string> v) { a.out_nccl_ids = std::move(v); })
      .def_readwrite("attn_peer", &EngineArgs::attn_peer)
      .def_readwrite("parts_needed", &EngineArgs::parts_needed)
      .def_readwrite("sampler_id", &EngineArgs::sampler_id)
      .def_readwrite("num_dp_groups", &EngineArgs::num_dp_groups)
      .def_readwrite("device", &EngineArgs::device)
      .def_readwrite("attn_policy", &EngineArgs::attn_policy)
      .def_readwrite("expert_policy", &EngineArgs::expert_policy);
  py::class_<EngineHandles>(m, "EngineHandles")
      .def_readonly("scheduler", &EngineHandles::scheduler)
      .def_readonly("attn_scheduler", &EngineHandles::attn_scheduler)
      .def_readonly("attn_dispatcher", &EngineHandles::attn_dispatcher)
      .def_readonly("expert_dispatcher", &EngineHandles::expert_dispatcher)
      .def_readonly("expert_pool", &EngineHandles::expert_pool)
      .def_readonly("attn_pool", &EngineHandles::attn_pool);
  m.def("init_engine", &init_engine, py::call_guard<py::gil_scoped_release>());
  m.def("init_engine_colocate", &init_engine_colocate, py::call_guard<py::gil_scoped_release>());
  m.def("start_engine", &start_engine);
  m.def("helper_error", &helper_error);
  m.def("stop_engine", &stop_engine, py::call_guard<py::gil_scoped_release>());
  m.def("init_sampler", &init_sampler, py::arg("device_id"), py::arg("min_output_len"), py::arg("max_output_len"),
        py::arg("top_k"), py::arg("out_device_ids"), py::arg("attn_peer"), py::arg("ignore_eos") = true,
        py::arg("topk_partials") = false);
  m.def("init_tokenizer", &init_tokenizer);

  // ---- recorder --------------------------------------------------------------------------------------
  m.def("recorder_create", [](const std::string& name) { Recorder::instance().create(name); }, py::arg("name") = "");
  m.def("recorder_enable", [](bool on) { Recorder::instance().enable(on); });
  m.def("recorder_output", [] { return Recorder::instance().output(); });
  m.def("range_push", [](const std::string& msg) { Recorder::instance().push(msg); });
  m.def("range_pop", [] { Recorder::instance().pop(); });

  // ---- in-module tests -------------------------------------------------------------------------------
  m.def("test_socket_p2p", &test_socket_p2p, py::call_guard<py::gil_scoped_release>());
  m.def("test_parallel_attn_scheduler", &test_parallel_attn_scheduler, py::call_guard<py::gil_scoped_release>());
  m.def("test_recorder_threads", &test_recorder_threads, py::call_guard<py::gil_scoped_release>());
  m.def("test_nccl_p2p", &test_nccl_p2p, py::call_guard<py::gil_scoped_release>());
  m.def("test_nccl_group", &test_nccl_group, py::arg("devices"), py::call_guard<py::gil_scoped_release>());
  m.def("test_multi_launch", &test_multi_launch, py::arg("device") = 0, py::arg("launches") = 200, py::arg("n") = 4096,
        py::call_guard<py::gil_scoped_release>());
  m.def("test_op_overlap", &test_op_overlap, py::arg("dev_a") = 0, py::arg("dev_b") = 1, py::arg("mbytes") = 64,
        py::arg("launches") = 200, py::call_guard<py::gil_scoped_release>());
}
