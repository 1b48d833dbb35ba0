// Data-parallel gradient exchange over NCCL (see dp.h).  NCCL is loaded with dlopen on first use, so
// single-GPU users need no NCCL at all.
#include "host/dp.h"

#include <dlfcn.h>

#include <algorithm>
#include <chrono>
#include <cstring>
#include <future>
#include <thread>
#include <unordered_map>
#include <unordered_set>

#include "nrs_internal.h"

namespace nrs {

namespace {

[[noreturn]] void fail(int code, const std::string& m) { throw Error(code, m); }

// ------------------------------------------------------------------- NCCL
struct NcclId { char internal[128]; };
typedef void* ncclComm_p;
struct NcclApi {
  void* handle = nullptr;
  int (*GetUniqueId)(NcclId*) = nullptr;
  int (*CommInitRank)(ncclComm_p*, int, NcclId, int) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_p, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, ncclComm_p, cudaStream_t) = nullptr;
  int (*CommDestroy)(ncclComm_p) = nullptr;
  int (*CommAbort)(ncclComm_p) = nullptr;
  int (*CommGetAsyncError)(ncclComm_p, int*) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  std::string error;
};
constexpr int kNcclFloat32 = 7, kNcclUint64 = 5, kNcclSum = 0, kNcclSuccess = 0, kNcclInProgress = 7;

NcclApi* nccl_api() {
  static NcclApi api;
  static bool tried = false;
  if (tried) return api.handle ? &api : nullptr;
  tried = true;
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  for (const char* n : names) {
    api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (api.handle) break;
  }
  if (!api.handle) {
    const char* why = dlerror();
    api.error = std::string("cannot load libnccl.so.2: ") + (why ? why : "unknown");
    return nullptr;
  }
  auto sym = [&](const char* s) { return dlsym(api.handle, s); };
  api.GetUniqueId = (int (*)(NcclId*))sym("ncclGetUniqueId");
  api.CommInitRank = (int (*)(ncclComm_p*, int, NcclId, int))sym("ncclCommInitRank");
  api.AllReduce = (int (*)(const void*, void*, size_t, int, int, ncclComm_p, cudaStream_t))sym("ncclAllReduce");
  api.AllGather = (int (*)(const void*, void*, size_t, int, ncclComm_p, cudaStream_t))sym("ncclAllGather");
  api.CommDestroy = (int (*)(ncclComm_p))sym("ncclCommDestroy");
  api.CommAbort = (int (*)(ncclComm_p))sym("ncclCommAbort");
  api.CommGetAsyncError = (int (*)(ncclComm_p, int*))sym("ncclCommGetAsyncError");
  api.GetErrorString = (const char* (*)(int))sym("ncclGetErrorString");
  if (!api.GetUniqueId || !api.CommInitRank || !api.AllReduce || !api.AllGather || !api.CommDestroy || !api.CommAbort ||
      !api.CommGetAsyncError || !api.GetErrorString) {
    api.error = "libnccl.so.2 lacks a required symbol";
    dlclose(api.handle);
    api.handle = nullptr;
    return nullptr;
  }
  return &api;
}

NcclApi* require_nccl() {
  NcclApi* api = nccl_api();
  if (!api) fail(NRS_ERR_NCCL, "NCCL is not available");
  return api;
}

double now_ms() {
  using namespace std::chrono;
  return duration<double, std::milli>(steady_clock::now().time_since_epoch()).count();
}

}  // namespace

std::vector<DpBucket> dp_plan_buckets(const std::vector<size_t>& offsets, size_t total, size_t bucket_bytes) {
  std::vector<DpBucket> out;
  const int n = (int)offsets.size();
  if (n == 0) return out;
  const size_t want = std::max<size_t>(1, bucket_bytes / sizeof(float));
  size_t end = total;
  int last = n - 1;
  for (int i = n - 1; i >= 0; --i) {
    if (end - offsets[i] >= want || i == 0) {
      out.push_back({offsets[i], end, i, last});
      end = offsets[i];
      last = i - 1;
    }
  }
  return out;
}

uint64_t dp_fingerprint(const int64_t* param_lens, int n_params, size_t bucket_bytes, int global_batch, int world) {
  uint64_t h = 1469598103934665603ull;
  auto mix = [&](uint64_t v) {
    for (int i = 0; i < 8; ++i) {
      h ^= (v >> (8 * i)) & 0xffu;
      h *= 1099511628211ull;
    }
  };
  mix((uint64_t)n_params);
  for (int i = 0; i < n_params; ++i) mix((uint64_t)param_lens[i]);
  mix((uint64_t)bucket_bytes);
  mix((uint64_t)(int64_t)global_batch);
  mix((uint64_t)(int64_t)world);
  return h;
}

int dp_first_mismatch(const uint64_t* fingerprints, int world) {
  for (int r = 1; r < world; ++r)
    if (fingerprints[r] != fingerprints[0]) return r;
  return -1;
}

int dp_watchdog_wait(DpPollFn poll, void* user, double timeout_ms, double interval_us, double* waited_ms_out) {
  const double t0 = now_ms();
  int result = NRS_ERR_TIMEOUT;
  while (true) {
    const int st = poll(user);
    if (st > 0) { result = NRS_OK; break; }
    if (st < 0) { result = NRS_ERR_NCCL; break; }
    if (now_ms() - t0 >= timeout_ms) break;
    if (interval_us > 0) std::this_thread::sleep_for(std::chrono::duration<double, std::micro>(interval_us));
    else std::this_thread::yield();
  }
  if (waited_ms_out) *waited_ms_out = now_ms() - t0;
  return result;
}

void dp_unique_id(void* out_128_bytes) {
  NcclApi* api = require_nccl();
  NcclId id;
  const int rc = api->GetUniqueId(&id);
  if (rc != kNcclSuccess) fail(NRS_ERR_NCCL, std::string("ncclGetUniqueId: ") + api->GetErrorString(rc));
  std::memcpy(out_128_bytes, &id, sizeof(id));
}

DpGroup::DpGroup(nrs_ctx* ctx, int rank, int world, const void* unique_id, int global_batch, double timeout_ms)
    : ctx_(ctx), rank_(rank), world_(world), global_batch_(global_batch), timeout_ms_(timeout_ms) {
  if (!ctx) fail(NRS_ERR_ARG, "data parallel: null context");
  if (world < 1 || rank < 0 || rank >= world) fail(NRS_ERR_ARG, "data parallel: rank outside [0, world)");
  if (global_batch <= 0) fail(NRS_ERR_ARG, "data parallel: global batch must be positive");
  if (!(timeout_ms > 0)) fail(NRS_ERR_ARG, "data parallel: the deadline must be positive");
  if (world == 1) return;
  if (!unique_id) fail(NRS_ERR_ARG, "data parallel: null unique id");
  NcclApi* api = require_nccl();
  NcclId id;
  std::memcpy(&id, unique_id, sizeof(id));
  // ncclCommInitRank blocks until every rank has arrived; it runs on a helper thread so that a rank
  // that never comes turns into NRS_ERR_TIMEOUT here instead of a hang.  (The communicator stays an
  // ordinary blocking one: its collectives enqueue straight from the calling thread.)
  struct InitResult { ncclComm_p comm = nullptr; int rc = -1; };
  auto result = std::make_shared<std::promise<InitResult>>();
  std::future<InitResult> fut = result->get_future();
  const int device = ctx->device;
  std::thread([api, id, rank, world, device, result]() {
    InitResult r;
    cudaSetDevice(device);
    r.rc = api->CommInitRank(&r.comm, world, id, rank);
    result->set_value(r);
  }).detach();
  if (fut.wait_for(std::chrono::duration<double, std::milli>(timeout_ms)) != std::future_status::ready)
    fail(NRS_ERR_TIMEOUT, "data parallel: not every rank joined the communicator before the deadline");
  const InitResult r = fut.get();
  if (r.rc != kNcclSuccess) fail(NRS_ERR_NCCL, std::string("ncclCommInitRank: ") + api->GetErrorString(r.rc));
  comm_ = r.comm;
  auto cuda_ok = [&](cudaError_t e, const char* what) {
    if (e != cudaSuccess) fail(NRS_ERR_CUDA, std::string("data parallel: ") + what + ": " + cudaGetErrorString(e));
  };
  cuda_ok(cudaStreamCreateWithFlags(&comm_stream_, cudaStreamNonBlocking), "comm stream creation");
  cuda_ok(cudaEventCreateWithFlags(&ready_ev_, cudaEventDisableTiming), "event creation");
  cuda_ok(cudaEventCreateWithFlags(&done_ev_, cudaEventDisableTiming), "event creation");
  cuda_ok(cudaEventCreateWithFlags(&wait_ev_, cudaEventDisableTiming), "event creation");
}

DpGroup::~DpGroup() {
  if (comm_) {
    if (NcclApi* a = nccl_api()) {
      if (dead_) a->CommAbort(comm_); else a->CommDestroy(comm_);
    }
  }
  if (comm_stream_) cudaStreamDestroy(comm_stream_);
  for (cudaEvent_t e : {ready_ev_, done_ev_, wait_ev_})
    if (e) cudaEventDestroy(e);
}

void DpGroup::require_alive(const char* what) const {
  if (dead_) fail(NRS_ERR_NCCL, std::string(what) + ": the communicator was aborted (" + dead_reason_ + ")");
}

void DpGroup::abort_comm(const char* why) {
  dead_ = true;
  dead_reason_ = why;
  if (comm_) {
    if (NcclApi* a = nccl_api()) a->CommAbort(comm_);   // ends NCCL kernels still waiting for a peer
    comm_ = nullptr;
  }
}

int DpGroup::param_index(const Node* n) const {
  for (size_t i = 0; i < params_.size(); ++i)
    if (params_[i].get() == n) return (int)i;
  return -1;
}

void DpGroup::register_params(const std::vector<NodeP>& params, size_t bucket_bytes) {
  require_alive("bucket registration");
  if (params.empty()) fail(NRS_ERR_ARG, "data parallel: no parameters to register");
  if (in_step_) fail(NRS_ERR_ARG, "data parallel: registration inside a step");
  std::shared_ptr<FlatStore> fs = params[0]->flat;
  if (!fs || fs->offset.size() != params.size()) fs = nullptr;
  for (size_t i = 0; fs && i < params.size(); ++i)
    if (params[i]->flat != fs || params[i]->data != fs->data + fs->offset[i]) fs = nullptr;
  if (!fs) fs = cuda::flatten_params(params);   // values kept; gradients become ranges of one block
  flat_ = fs;
  params_ = params;
  const size_t bytes = bucket_bytes ? bucket_bytes : ((size_t)32 << 20);
  buckets_ = dp_plan_buckets(fs->offset, fs->total, bytes);
  ready_.assign(params.size(), 0);
  next_bucket_ = 0;
  if (world_ == 1) return;
  // Every rank must have planned the same exchange: compare fingerprints before any gradient moves.
  NcclApi* api = require_nccl();
  std::vector<int64_t> lens;
  for (const auto& p : params) lens.push_back((int64_t)p->len());
  const uint64_t mine = dp_fingerprint(lens.data(), (int)lens.size(), bytes, global_batch_, world_);
  void* dev = nullptr;
  check(ctx_, nrs_alloc(ctx_, sizeof(uint64_t) * (size_t)(world_ + 1), 0, &dev));
  uint64_t* all_dev = (uint64_t*)dev;
  std::vector<uint64_t> all((size_t)world_, 0);
  try {
    check(ctx_, nrs_h2d(ctx_, all_dev + world_, &mine, sizeof(mine)));
    const int rc = api->AllGather(all_dev + world_, all_dev, 1, kNcclUint64, comm_, ctx_->stream);
    if (rc != kNcclSuccess) fail(NRS_ERR_NCCL, std::string("ncclAllGather: ") + api->GetErrorString(rc));
    host_wait(ctx_->stream);
    check(ctx_, nrs_d2h(ctx_, all.data(), all_dev, sizeof(uint64_t) * (size_t)world_));
  } catch (...) {
    nrs_free(ctx_, dev);
    throw;
  }
  nrs_free(ctx_, dev);
  const int bad = dp_first_mismatch(all.data(), world_);
  if (bad >= 0)
    fail(NRS_ERR_SHAPE, "data parallel: rank " + std::to_string(bad) +
                            " registered different parameters, bucket size, global batch or world size than rank 0");
}

void DpGroup::begin_step() {
  require_alive("data-parallel step");
  std::fill(ready_.begin(), ready_.end(), 0);
  next_bucket_ = 0;
  in_step_ = true;
}

void DpGroup::launch_bucket(size_t index) {
  const DpBucket& b = buckets_[index];
  if (world_ > 1) {
    NcclApi* api = require_nccl();
    if (cudaEventRecord(ready_ev_, ctx_->stream) != cudaSuccess || cudaStreamWaitEvent(comm_stream_, ready_ev_, 0) != cudaSuccess)
      fail(NRS_ERR_CUDA, "data parallel: event hand-off to the comm stream failed");
    float* g = flat_->grad + b.begin;
    const int rc = api->AllReduce(g, g, b.end - b.begin, kNcclFloat32, kNcclSum, comm_, comm_stream_);
    if (rc != kNcclSuccess) fail(NRS_ERR_NCCL, std::string("ncclAllReduce: ") + api->GetErrorString(rc));
  }
  if (after_bucket) {
    cudaStream_t keep = ctx_->stream;
    if (world_ > 1) ctx_->stream = comm_stream_;
    try {
      after_bucket(b);
    } catch (...) {
      ctx_->stream = keep;
      throw;
    }
    ctx_->stream = keep;
  }
}

void DpGroup::grad_ready(int index) {
  require_alive("nrs_grad_ready");
  if (!in_step_) fail(NRS_ERR_ARG, "data parallel: gradient reported outside a step");
  if (index < 0 || index >= (int)params_.size()) fail(NRS_ERR_ARG, "data parallel: not a registered parameter");
  ready_[index] = 1;
  while (next_bucket_ < buckets_.size()) {
    const DpBucket& b = buckets_[next_bucket_];
    bool all = true;
    for (int p = b.first_param; p <= b.last_param; ++p) all = all && ready_[p];
    if (!all) break;
    // a parameter nothing wrote still goes out, as zeros
    for (int p = b.first_param; p <= b.last_param; ++p)
      if (!params_[p]->grad_valid) {
        check(ctx_, nrs_memset_zero(ctx_, params_[p]->grad, params_[p]->len() * sizeof(float)));
        params_[p]->grad_valid = true;
      }
    launch_bucket(next_bucket_);
    ++next_bucket_;
  }
}

void DpGroup::finish() {
  require_alive("nrs_allreduce_wait");
  if (!in_step_) fail(NRS_ERR_ARG, "data parallel: no step in progress");
  for (size_t p = 0; p < params_.size(); ++p)
    if (!ready_[p]) grad_ready((int)p);
  in_step_ = false;
  if (world_ > 1) {
    if (cudaEventRecord(done_ev_, comm_stream_) != cudaSuccess || cudaStreamWaitEvent(ctx_->stream, done_ev_, 0) != cudaSuccess)
      fail(NRS_ERR_CUDA, "data parallel: event hand-off from the comm stream failed");
  }
}

namespace {
struct WaitState {
  cudaEvent_t ev;
  NcclApi* api;
  void* comm;
  std::string error;
};
int poll_event_and_comm(void* user) {
  WaitState* w = (WaitState*)user;
  const cudaError_t e = cudaEventQuery(w->ev);
  if (e == cudaSuccess) return 1;
  if (e != cudaErrorNotReady) {
    w->error = std::string("CUDA error while waiting: ") + cudaGetErrorString(e);
    return -1;
  }
  if (w->comm) {
    int async = kNcclSuccess;
    const int rc = w->api->CommGetAsyncError(w->comm, &async);
    if (rc != kNcclSuccess || (async != kNcclSuccess && async != kNcclInProgress)) {
      w->error = std::string("NCCL reported an asynchronous error: ") + w->api->GetErrorString(rc != kNcclSuccess ? rc : async);
      return -1;
    }
  }
  return 0;
}
}  // namespace

void DpGroup::host_wait(cudaStream_t stream) {
  require_alive("data-parallel wait");
  if (world_ == 1) {
    if (cudaStreamSynchronize(stream) != cudaSuccess) fail(NRS_ERR_CUDA, "data parallel: stream synchronisation failed");
    return;
  }
  if (cudaEventRecord(wait_ev_, stream) != cudaSuccess) fail(NRS_ERR_CUDA, "data parallel: event record failed");
  host_wait_event(wait_ev_);
}

void DpGroup::host_wait_event(cudaEvent_t ev) {
  require_alive("data-parallel wait");
  if (world_ == 1) {
    if (cudaEventSynchronize(ev) != cudaSuccess) fail(NRS_ERR_CUDA, "data parallel: event synchronisation failed");
    return;
  }
  WaitState w{ev, require_nccl(), comm_, {}};
  double waited = 0.0;
  const int st = dp_watchdog_wait(poll_event_and_comm, &w, timeout_ms_, 20.0, &waited);
  if (st == NRS_OK) return;
  if (st == NRS_ERR_TIMEOUT) {
    abort_comm("a collective did not finish before the deadline");
    fail(NRS_ERR_TIMEOUT, "data parallel: the step did not finish within " + std::to_string((long)timeout_ms_) +
                              " ms (a rank is missing or stalled); the communicator was aborted");
  }
  abort_comm(w.error.c_str());
  fail(NRS_ERR_NCCL, "data parallel: " + w.error + "; the communicator was aborted");
}

void DpGroup::all_reduce_sum(float* dev, size_t count) {
  require_alive("all-reduce");
  if (world_ == 1 || count == 0) return;
  NcclApi* api = require_nccl();
  const int rc = api->AllReduce(dev, dev, count, kNcclFloat32, kNcclSum, comm_, ctx_->stream);
  if (rc != kNcclSuccess) fail(NRS_ERR_NCCL, std::string("ncclAllReduce: ") + api->GetErrorString(rc));
}

void backward_graph_dp(const NodeP& root, DpGroup* dp) {
  if (!root) fail(NRS_ERR_ARG, "backward_graph: null root");
  // post-order DFS, iterative (deep chains must not overflow the stack)
  std::vector<NodeP> topo;
  std::unordered_set<const Node*> seen;
  struct Frame { NodeP node; size_t next; };
  std::vector<Frame> stack;
  seen.insert(root.get());
  stack.push_back({root, 0});
  while (!stack.empty()) {
    Frame& f = stack.back();
    if (f.next < f.node->parents.size()) {
      NodeP p = f.node->parents[f.next++];
      if (seen.insert(p.get()).second) stack.push_back({p, 0});
    } else {
      topo.push_back(f.node);
      stack.pop_back();
    }
  }
  const bool track = dp && dp->registered();
  // reshape / flatten results alias their input's gradient: a reader of the view reads the parameter
  auto view_root = [](const NodeP& p) {
    const Node* r = p.get();
    while (r->view_of) r = r->view_of.get();
    return r;
  };
  // readers[i]: nodes with a backward closure that list parameter i among their parents
  std::unordered_map<const Node*, int> index_of;
  std::vector<int> readers;
  if (track) {
    for (const NodeP& n : topo) {
      const int pi = dp->param_index(n.get());
      if (pi >= 0) index_of[n.get()] = pi;
    }
    readers.assign(dp->param_count(), 0);
    for (const NodeP& n : topo)
      if (n->backward_fn)
        for (const NodeP& p : n->parents) {
          auto it = index_of.find(view_root(p));
          if (it != index_of.end()) ++readers[it->second];
        }
  }
  for (auto it = topo.rbegin(); it != topo.rend(); ++it) {
    const NodeP& n = *it;
    if (!n->backward_fn) continue;
    n->backward_fn();
    if (!track) continue;
    for (const NodeP& p : n->parents) {
      auto hit = index_of.find(view_root(p));
      if (hit != index_of.end() && --readers[hit->second] == 0) dp->grad_ready(hit->second);
    }
  }
}

}  // namespace nrs
