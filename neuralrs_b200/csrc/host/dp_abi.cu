// extern "C" face of the data-parallel gradient exchange (nrs_graph.h, "Data parallelism"): the
// operator-level entry points a define-by-run loop over nodes uses, and the host-only helpers.
#include <algorithm>
#include <cstring>

#include "host/dp.h"
#include "host/abi_types.h"
#include "nrs_graph.h"
#include "nrs_internal.h"

struct nrs_dp {
  nrs_ctx* ctx;
  std::unique_ptr<nrs::DpGroup> g;
};

namespace {

template <class F>
int guarded(nrs_ctx* ctx, F&& f) {
  try {
    f();
    return NRS_OK;
  } catch (const nrs::Error& e) {
    return nrs_fail(ctx, e.code, "%s", e.what());
  } catch (const std::bad_alloc&) {
    return nrs_fail(ctx, NRS_ERR_ALLOC, "host allocation failed");
  } catch (const std::exception& e) {
    return nrs_fail(ctx, NRS_ERR_ARG, "%s", e.what());
  }
}

}  // namespace

extern "C" {

int nrs_dp_unique_id(void* id_out) {
  if (!id_out) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_dp_unique_id: null output");
  return guarded(nullptr, [&] { nrs::dp_unique_id(id_out); });
}

int nrs_dp_create(nrs_ctx* ctx, int rank, int world, const void* unique_id, int global_batch, double timeout_ms, nrs_dp** out) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, out != nullptr, NRS_ERR_ARG, "nrs_dp_create: null out handle");
  *out = nullptr;
  return guarded(ctx, [&] {
    std::unique_ptr<nrs::DpGroup> g(new nrs::DpGroup(ctx, rank, world, unique_id, global_batch, timeout_ms > 0 ? timeout_ms : 300000.0));
    *out = new nrs_dp{ctx, std::move(g)};
  });
}

int nrs_dp_free(nrs_dp* dp) {
  if (dp && dp->ctx) cudaStreamSynchronize(dp->ctx->stream);
  delete dp;
  return NRS_OK;
}

int nrs_bucket_register(nrs_dp* dp, nrs_node* const* params, int count, size_t bucket_bytes) {
  if (!dp) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_bucket_register: null handle");
  NRS_REQUIRE(dp->ctx, params && count > 0, NRS_ERR_ARG, "nrs_bucket_register: no parameters");
  return guarded(dp->ctx, [&] {
    std::vector<nrs::NodeP> v;
    for (int i = 0; i < count; ++i) {
      if (!params[i] || !params[i]->p) throw nrs::Error(NRS_ERR_ARG, "nrs_bucket_register: null node in list");
      v.push_back(params[i]->p);
    }
    dp->g->register_params(v, bucket_bytes);
  });
}

int nrs_dp_bucket_count(const nrs_dp* dp) { return dp ? (int)dp->g->bucket_count() : -1; }

int nrs_dp_begin_step(nrs_dp* dp) {
  if (!dp) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_dp_begin_step: null handle");
  return guarded(dp->ctx, [&] { dp->g->begin_step(); });
}

int nrs_grad_ready(nrs_dp* dp, nrs_node* param) {
  if (!dp) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_grad_ready: null handle");
  NRS_REQUIRE(dp->ctx, param && param->p, NRS_ERR_ARG, "nrs_grad_ready: null node");
  return guarded(dp->ctx, [&] {
    const int i = dp->g->param_index(param->p.get());
    if (i < 0) throw nrs::Error(NRS_ERR_ARG, "nrs_grad_ready: the node was not registered with nrs_bucket_register");
    dp->g->grad_ready(i);
  });
}

int nrs_allreduce_wait(nrs_dp* dp) {
  if (!dp) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_allreduce_wait: null handle");
  return guarded(dp->ctx, [&] { dp->g->finish(); });
}

int nrs_backward_graph_dp(nrs_node* root, nrs_dp* dp) {
  if (!dp) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_backward_graph_dp: null handle");
  NRS_REQUIRE(dp->ctx, root && root->p, NRS_ERR_ARG, "nrs_backward_graph_dp: null root");
  return guarded(dp->ctx, [&] {
    dp->g->begin_step();
    nrs::backward_graph_dp(root->p, dp->g.get());
    dp->g->finish();
  });
}

int nrs_dp_host_wait(nrs_dp* dp) {
  if (!dp) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_dp_host_wait: null handle");
  return guarded(dp->ctx, [&] {
    dp->g->host_wait(dp->ctx->stream);
    nrs::check(dp->ctx, nrs_check_device_error(dp->ctx));
  });
}

int nrs_dp_set_timeout_ms(nrs_dp* dp, double timeout_ms) {
  if (!dp) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_dp_set_timeout_ms: null handle");
  NRS_REQUIRE(dp->ctx, timeout_ms > 0, NRS_ERR_ARG, "nrs_dp_set_timeout_ms: the deadline must be positive");
  dp->g->set_timeout_ms(timeout_ms);
  return NRS_OK;
}

int nrs_dp_all_reduce_sum(nrs_dp* dp, float* values_dev, size_t count) {
  if (!dp) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_dp_all_reduce_sum: null handle");
  NRS_REQUIRE(dp->ctx, values_dev || count == 0, NRS_ERR_ARG, "nrs_dp_all_reduce_sum: null pointer");
  return guarded(dp->ctx, [&] { dp->g->all_reduce_sum(values_dev, count); });
}

int nrs_dp_shard_range(int global_batch, int rank, int world, int* begin_out, int* end_out) {
  if (world < 1 || rank < 0 || rank >= world || global_batch < 0 || !begin_out || !end_out)
    return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_dp_shard_range: bad arguments");
  // Contiguous shards; the first (global_batch % world) ranks take one extra sample.
  const int base = global_batch / world, extra = global_batch % world;
  *begin_out = rank * base + std::min(rank, extra);
  *end_out = *begin_out + base + (rank < extra ? 1 : 0);
  return NRS_OK;
}

int nrs_dp_plan_buckets(const int64_t* param_lens, int n_params, size_t bucket_bytes, int64_t* starts_out,
                        int64_t* ends_out, int capacity) {
  if (n_params < 0 || (n_params > 0 && !param_lens)) return -1;
  std::vector<size_t> offsets;
  size_t total = 0;
  for (int i = 0; i < n_params; ++i) {
    if (param_lens[i] < 0) return -1;
    offsets.push_back(total);
    total += ((size_t)param_lens[i] + 3) / 4 * 4;
  }
  auto b = nrs::dp_plan_buckets(offsets, total, bucket_bytes ? bucket_bytes : ((size_t)32 << 20));
  if (starts_out && ends_out)
    for (int i = 0; i < (int)b.size() && i < capacity; ++i) {
      starts_out[i] = (int64_t)b[i].begin;
      ends_out[i] = (int64_t)b[i].end;
    }
  return (int)b.size();
}

uint64_t nrs_dp_fingerprint(const int64_t* param_lens, int n_params, size_t bucket_bytes, int global_batch, int world) {
  if (n_params < 0 || (n_params > 0 && !param_lens)) return 0;
  return nrs::dp_fingerprint(param_lens, n_params, bucket_bytes ? bucket_bytes : ((size_t)32 << 20), global_batch, world);
}

int nrs_dp_check_fingerprints(const uint64_t* fingerprints, int world) {
  if (!fingerprints || world < 1) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_dp_check_fingerprints: bad arguments");
  const int bad = nrs::dp_first_mismatch(fingerprints, world);
  if (bad >= 0)
    return nrs_fail(nullptr, NRS_ERR_SHAPE,
                    "data parallel: rank %d registered different parameters, bucket size, global batch or world size than rank 0", bad);
  return NRS_OK;
}

int nrs_watchdog_wait(nrs_poll_fn poll, void* user, double timeout_ms, double interval_us, double* waited_ms_out) {
  if (!poll || !(timeout_ms >= 0)) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_watchdog_wait: bad arguments");
  const int st = nrs::dp_watchdog_wait(poll, user, timeout_ms, interval_us, waited_ms_out);
  if (st == NRS_ERR_TIMEOUT) return nrs_fail(nullptr, st, "the wait did not finish within %.0f ms", timeout_ms);
  if (st != NRS_OK) return nrs_fail(nullptr, st, "the polled operation reported a failure");
  return NRS_OK;
}

}  // extern "C"
