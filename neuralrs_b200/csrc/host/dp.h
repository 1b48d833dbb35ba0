// Data-parallel gradient exchange: flat buckets over a parameter block, all-reduced with NCCL on a
// second stream as soon as backward has produced them, with a host-side deadline on every wait.
//
// The reference is single-GPU (device 0 hard-coded, src/cuda/backend.rs:21; no distributed code), so
// nothing here has a counterpart in it.  The unit of work is the reference's own: a list of parameter
// nodes (what `parameters()` returns, src/nn/module.rs:21-27) whose gradients backward_graph fills.
#pragma once

#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "host/graph.h"

namespace nrs {

// A contiguous range [begin, end) of the flat gradient holding parameters first_param..last_param.
struct DpBucket {
  size_t begin, end;
  int first_param, last_param;
};

// Buckets over a flat gradient, walking parameters from the LAST to the first (the order backward
// finishes them); a bucket closes once it holds at least bucket_bytes.  `offsets` are the parameters'
// (padded) starts, `total` the end of the block.
std::vector<DpBucket> dp_plan_buckets(const std::vector<size_t>& offsets, size_t total, size_t bucket_bytes);

// What every rank must agree on before the first collective: parameter lengths (in order), bucket size,
// global batch and world size, folded into 64 bits (FNV-1a).  Ranks exchange the value on the host.
uint64_t dp_fingerprint(const int64_t* param_lens, int n_params, size_t bucket_bytes, int global_batch, int world);
// Index of the first rank whose fingerprint differs from rank 0's, or -1.
int dp_first_mismatch(const uint64_t* fingerprints, int world);

// Deadline loop over a poll function: 0 = still running, 1 = finished, negative = failed.  Returns
// NRS_OK, NRS_ERR_TIMEOUT (the deadline passed; `poll` was called at least once) or NRS_ERR_NCCL
// (poll reported a failure).  Sleeps interval_us between polls.
typedef int (*DpPollFn)(void* user);
int dp_watchdog_wait(DpPollFn poll, void* user, double timeout_ms, double interval_us, double* waited_ms_out);

class DpGroup {
 public:
  // Joins the communicator (blocking until every rank has arrived, or NRS_ERR_TIMEOUT after timeout_ms).
  DpGroup(nrs_ctx* ctx, int rank, int world, const void* unique_id_128_bytes, int global_batch, double timeout_ms);
  ~DpGroup();
  DpGroup(const DpGroup&) = delete;
  DpGroup& operator=(const DpGroup&) = delete;

  int rank() const { return rank_; }
  int world() const { return world_; }
  int global_batch() const { return global_batch_; }
  size_t bucket_count() const { return buckets_.size(); }
  const std::vector<DpBucket>& buckets() const { return buckets_; }
  void set_timeout_ms(double ms) { timeout_ms_ = ms; }

  // Takes the parameters of one FlatStore (in its order), plans the buckets and checks over the
  // communicator that every rank planned the same ones (NRS_ERR_SHAPE otherwise, before any gradient
  // is exchanged).
  void register_params(const std::vector<NodeP>& params, size_t bucket_bytes);
  bool registered() const { return !params_.empty(); }
  size_t param_count() const { return params_.size(); }
  int param_index(const Node* n) const;

  // One step: begin_step(); grad_ready(i) once parameter i's gradient is complete (any order; a
  // bucket is sent when it and every bucket before it are complete, so all ranks issue the same
  // sequence); finish() sends what is left (parameters that received no gradient go out as zeros) and
  // makes the compute stream wait for the exchange.
  void begin_step();
  void grad_ready(int param_index);
  void finish();
  // Runs on the COMM stream right after a bucket's all-reduce, with the context's stream switched to
  // it: the trainer updates the bucket's parameters there, overlapping the rest of backward.
  std::function<void(const DpBucket&)> after_bucket;

  // Waits on the host until everything enqueued on `stream` so far has finished, polling the
  // communicator for asynchronous errors; on an error or after the deadline the communicator is
  // aborted and every later call fails (NRS_ERR_NCCL / NRS_ERR_TIMEOUT).
  void host_wait(cudaStream_t stream);
  void host_wait_event(cudaEvent_t ev);   // the same for an event the caller recorded earlier
  // All-reduce (sum) of `count` floats at `dev` across the group on the compute stream (small values:
  // the loss share, statistics).
  void all_reduce_sum(float* dev, size_t count);
  nrs_ctx* context() const { return ctx_; }

 private:
  void launch_bucket(size_t index);
  void require_alive(const char* what) const;
  void abort_comm(const char* why);

  nrs_ctx* ctx_;
  int rank_, world_, global_batch_;
  double timeout_ms_;
  void* comm_ = nullptr;
  bool dead_ = false;
  std::string dead_reason_;
  cudaStream_t comm_stream_ = nullptr;
  cudaEvent_t ready_ev_ = nullptr, done_ev_ = nullptr, wait_ev_ = nullptr;
  std::shared_ptr<FlatStore> flat_;
  std::vector<NodeP> params_;
  std::vector<DpBucket> buckets_;
  std::vector<char> ready_;
  size_t next_bucket_ = 0;
  bool in_step_ = false;
};

// Topological backward pass (src/autograd/node.rs:113-151) that reports each registered parameter to
// the group as soon as the last node that reads it has run its backward closure.
void backward_graph_dp(const NodeP& root, DpGroup* dp);

// 128-byte rendezvous id made by rank 0 (ncclGetUniqueId).
void dp_unique_id(void* out_128_bytes);

}  // namespace nrs
