// Context lifecycle, device memory pool and host<->device copies.
// Stands in for the reference's global backend and residency helpers
// (src/cuda/backend.rs:19-32, src/cuda/runtime.rs:39-124).
#include "nrs_internal.h"

static thread_local std::string g_no_ctx_error;

int nrs_fail(nrs_ctx* ctx, int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  if (ctx) ctx->err = buf; else g_no_ctx_error = buf;
  return code;
}

int nrs_workspace(nrs_ctx* ctx, size_t bytes, void** out) {
  if (bytes > ctx->workspace_bytes) {
    // The old block may still be read by kernels in flight on the stream.
    if (ctx->workspace) {
      NRS_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
      NRS_CUDA(ctx, cudaFree(ctx->workspace));
      ctx->workspace = nullptr;
      ctx->workspace_bytes = 0;
    }
    const size_t want = (bytes + ((size_t)1 << 20) - 1) >> 20 << 20;
    cudaError_t e = cudaMalloc(&ctx->workspace, want);
    if (e != cudaSuccess) {
      ctx->workspace = nullptr;
      (void)cudaGetLastError();
      return nrs_fail(ctx, NRS_ERR_ALLOC, "workspace: cudaMalloc(%zu) failed: %s", want,
                      cudaGetErrorString(e));
    }
    ctx->workspace_bytes = want;
  }
  *out = ctx->workspace;
  return NRS_OK;
}

int nrs_ws_slot(nrs_ctx* ctx, int slot, size_t bytes, void** out) {
  if (slot < 0 || slot >= NRS_WS_COUNT) return nrs_fail(ctx, NRS_ERR_ARG, "workspace: bad slot %d", slot);
  if (bytes > ctx->ws_slot_bytes[slot]) {
    if (ctx->ws_slot[slot]) {
      NRS_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // kernels in flight may still read the old block
      NRS_CUDA(ctx, cudaFree(ctx->ws_slot[slot]));
      ctx->ws_slot[slot] = nullptr;
      ctx->ws_slot_bytes[slot] = 0;
    }
    const size_t want = (bytes + ((size_t)1 << 20) - 1) >> 20 << 20;
    cudaError_t e = cudaMalloc(&ctx->ws_slot[slot], want);
    if (e != cudaSuccess) {
      ctx->ws_slot[slot] = nullptr;
      (void)cudaGetLastError();
      return nrs_fail(ctx, NRS_ERR_ALLOC, "workspace slot %d: cudaMalloc(%zu) failed: %s", slot, want, cudaGetErrorString(e));
    }
    ctx->ws_slot_bytes[slot] = want;
  }
  *out = ctx->ws_slot[slot];
  return NRS_OK;
}

int nrs_err_flag(nrs_ctx* ctx, int** out) {
  if (!ctx->err_flag) {
    NRS_CUDA(ctx, cudaMalloc(&ctx->err_flag, sizeof(int)));
    NRS_CUDA(ctx, cudaMemsetAsync(ctx->err_flag, 0, sizeof(int), ctx->stream));
  }
  *out = ctx->err_flag;
  return NRS_OK;
}

int nrs_fold_ticket(nrs_ctx* ctx, unsigned** out) {
  if (!ctx->fold_ticket) {
    NRS_CUDA(ctx, cudaMalloc(&ctx->fold_ticket, kNrsFoldTickets * sizeof(unsigned)));
    NRS_CUDA(ctx, cudaMemsetAsync(ctx->fold_ticket, 0, kNrsFoldTickets * sizeof(unsigned), ctx->stream));
  }
  *out = ctx->fold_ticket;
  return NRS_OK;
}

int nrs_check_device_error(nrs_ctx* ctx) {
  if (!ctx->err_flag) return NRS_OK;
  int code = 0;
  NRS_CUDA(ctx, cudaMemcpyAsync(&code, ctx->err_flag, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
  NRS_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (code == 0) return NRS_OK;
  NRS_CUDA(ctx, cudaMemsetAsync(ctx->err_flag, 0, sizeof(int), ctx->stream));
  if (code == 5)
    return nrs_fail(ctx, NRS_ERR_ARG, "an embedding lookup met a token index outside the vocabulary; that row was read as zeros");
  static const char* what[] = {"", "TMA producer waiting for a free ring slot", "UMMA issuer waiting for a filled ring slot",
                               "epilogue waiting for the accumulator", "draining outstanding TMA loads"};
  return nrs_fail(ctx, NRS_ERR_TIMEOUT, "a tensor-core kernel gave up a bounded wait (%s); its output is invalid",
                  code >= 1 && code <= 4 ? what[code] : "unknown stage");
}

static cudaEvent_t prof_event(nrs_ctx* ctx) {
  if (!ctx->prof_free_events.empty()) {
    cudaEvent_t e = ctx->prof_free_events.back();
    ctx->prof_free_events.pop_back();
    return e;
  }
  cudaEvent_t e = nullptr;
  if (cudaEventCreate(&e) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
  return e;
}

NrsProfScope::NrsProfScope(nrs_ctx* c, int kind, double work) : ctx(c) {
  if (!c || !c->profiling) return;
  rec.kind = kind;
  rec.work = work;
  rec.start = prof_event(c);
  rec.stop = prof_event(c);
  if (!rec.start || !rec.stop) return;
  active = cudaEventRecord(rec.start, c->stream) == cudaSuccess;
}

NrsProfScope::~NrsProfScope() {
  if (!active) return;
  if (cudaEventRecord(rec.stop, ctx->stream) == cudaSuccess) ctx->prof_records.push_back(rec);
}

extern "C" {

int nrs_selftest_smem_attr_bookkeeping(void) {
  NrsSmemAttr a;
  int bad = 0;
  bad += nrs_smem_attr_update(a, 0, 40 * 1024) ? 1 : 0;      // fits the default: never requested
  bad += nrs_smem_attr_update(a, 0, 100 * 1024) ? 0 : 1;     // first request on device 0
  bad += nrs_smem_attr_update(a, 0, 100 * 1024) ? 1 : 0;     // already set there
  bad += nrs_smem_attr_update(a, 0, 90 * 1024) ? 1 : 0;      // smaller than what is set
  bad += nrs_smem_attr_update(a, 1, 100 * 1024) ? 0 : 1;     // another device starts from nothing
  bad += nrs_smem_attr_update(a, 0, 200 * 1024) ? 0 : 1;     // growth
  bad += nrs_smem_attr_update(a, 1, 100 * 1024) ? 1 : 0;
  bad += nrs_smem_attr_update(a, kNrsMaxDevices, 100 * 1024) ? 0 : 1;   // untracked ordinals always request
  bad += nrs_smem_attr_update(a, kNrsMaxDevices, 100 * 1024) ? 0 : 1;
  return bad;
}

int nrs_profile_enable(nrs_ctx* ctx, int on) {
  NRS_REQUIRE_CTX(ctx);
  ctx->profiling = on != 0;
  return NRS_OK;
}

int nrs_profile_reset(nrs_ctx* ctx) {
  NRS_REQUIRE_CTX(ctx);
  NRS_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  for (auto& r : ctx->prof_records) {
    ctx->prof_free_events.push_back(r.start);
    ctx->prof_free_events.push_back(r.stop);
  }
  ctx->prof_records.clear();
  return NRS_OK;
}

int nrs_profile_get(nrs_ctx* ctx, int kind, double* ms_out, double* work_out, uint64_t* calls_out) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, kind >= 0 && kind < NRS_PROF_KINDS, NRS_ERR_ARG, "nrs_profile_get: unknown kind %d", kind);
  NRS_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  double ms = 0.0, work = 0.0;
  uint64_t calls = 0;
  for (auto& r : ctx->prof_records) {
    if (r.kind != kind) continue;
    float t = 0.0f;
    NRS_CUDA(ctx, cudaEventElapsedTime(&t, r.start, r.stop));
    ms += t;
    work += r.work;
    ++calls;
  }
  if (ms_out) *ms_out = ms;
  if (work_out) *work_out = work;
  if (calls_out) *calls_out = calls;
  return NRS_OK;
}

int nrs_init(int device, nrs_ctx** out) {
  if (!out) return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_init: null out pointer");
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) {
    (void)cudaGetLastError();
    return nrs_fail(nullptr, NRS_ERR_CUDA,
                    "nrs_init: no usable CUDA device (%s); this library has no CPU fallback",
                    e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0");
  }
  if (device < 0 || device >= count)
    return nrs_fail(nullptr, NRS_ERR_ARG, "nrs_init: device %d out of range [0,%d)", device, count);
  e = cudaSetDevice(device);
  if (e != cudaSuccess)
    return nrs_fail(nullptr, NRS_ERR_CUDA, "nrs_init: cudaSetDevice(%d): %s", device, cudaGetErrorString(e));
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess)
    return nrs_fail(nullptr, NRS_ERR_CUDA, "nrs_init: cudaGetDeviceProperties: %s", cudaGetErrorString(e));
  if (prop.major != 10)
    return nrs_fail(nullptr, NRS_ERR_CUDA,
                    "nrs_init: device %d is sm_%d%d; this library is built for sm_100a only",
                    device, prop.major, prop.minor);
  nrs_ctx* ctx = new nrs_ctx();
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  e = cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) {
    delete ctx;
    return nrs_fail(nullptr, NRS_ERR_CUDA, "nrs_init: cudaStreamCreate: %s", cudaGetErrorString(e));
  }
  ctx->stream = ctx->own_stream;
  *out = ctx;
  return NRS_OK;
}

int nrs_destroy(nrs_ctx* ctx) {
  if (!ctx) return NRS_OK;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  for (auto& kv : ctx->pool.free_blocks) cudaFree(kv.second);
  for (auto& kv : ctx->pool.live) cudaFree(kv.first);
  nrs_weight_set_clear(ctx);
  if (ctx->workspace) cudaFree(ctx->workspace);
  for (int i = 0; i < NRS_WS_COUNT; ++i) if (ctx->ws_slot[i]) cudaFree(ctx->ws_slot[i]);
  if (ctx->err_flag) cudaFree(ctx->err_flag);
  if (ctx->fold_ticket) cudaFree(ctx->fold_ticket);
  for (auto& r : ctx->prof_records) { cudaEventDestroy(r.start); cudaEventDestroy(r.stop); }
  for (auto& e : ctx->prof_free_events) cudaEventDestroy(e);
  if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
  delete ctx;
  return NRS_OK;
}

const char* nrs_last_error(const nrs_ctx* ctx) {
  return ctx ? ctx->err.c_str() : g_no_ctx_error.c_str();
}

int nrs_set_stream(nrs_ctx* ctx, void* cuda_stream) {
  NRS_REQUIRE_CTX(ctx);
  ctx->stream = cuda_stream ? (cudaStream_t)cuda_stream : ctx->own_stream;
  return NRS_OK;
}

void* nrs_get_stream(nrs_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

int nrs_set_math_mode(nrs_ctx* ctx, int mode) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, mode == NRS_MATH_3XTF32 || mode == NRS_MATH_TF32 || mode == NRS_MATH_FP32,
              NRS_ERR_ARG, "nrs_set_math_mode: unknown mode %d", mode);
  ctx->math_mode = mode;
  return NRS_OK;
}

int nrs_get_math_mode(const nrs_ctx* ctx) { return ctx ? ctx->math_mode : -1; }

uint64_t nrs_launch_count(const nrs_ctx* ctx) { return ctx ? ctx->launches : 0; }

int nrs_alloc(nrs_ctx* ctx, size_t bytes, int zero, void** dptr) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, dptr != nullptr, NRS_ERR_ARG, "nrs_alloc: null out pointer");
  *dptr = nullptr;
  const size_t want = NrsPool::round_up(bytes ? bytes : 1);
  void* p = nullptr;
  auto it = ctx->pool.free_blocks.find(want);
  if (it != ctx->pool.free_blocks.end()) {
    p = it->second;
    ctx->pool.free_blocks.erase(it);
  } else {
    cudaError_t e = cudaMalloc(&p, want);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      // Give cached blocks back to the driver and retry once.
      for (auto& kv : ctx->pool.free_blocks) { cudaFree(kv.second); ctx->pool.bytes_reserved -= kv.first; }
      ctx->pool.free_blocks.clear();
      e = cudaMalloc(&p, want);
      if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return nrs_fail(ctx, NRS_ERR_ALLOC, "nrs_alloc: cudaMalloc(%zu) failed: %s", want,
                        cudaGetErrorString(e));
      }
    }
    ctx->pool.bytes_reserved += want;
  }
  ctx->pool.live[p] = want;
  if (zero) NRS_CUDA(ctx, cudaMemsetAsync(p, 0, bytes, ctx->stream));
  *dptr = p;
  return NRS_OK;
}

int nrs_free(nrs_ctx* ctx, void* dptr) {
  NRS_REQUIRE_CTX(ctx);
  if (!dptr) return NRS_OK;
  auto it = ctx->pool.live.find(dptr);
  NRS_REQUIRE(ctx, it != ctx->pool.live.end(), NRS_ERR_ARG, "nrs_free: %p was not allocated by nrs_alloc", dptr);
  ctx->pool.free_blocks.emplace(it->second, dptr);
  ctx->pool.live.erase(it);
  return NRS_OK;
}

int nrs_memset_zero(nrs_ctx* ctx, void* dptr, size_t bytes) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, dptr || bytes == 0, NRS_ERR_ARG, "nrs_memset_zero: null pointer");
  if (bytes) NRS_CUDA(ctx, cudaMemsetAsync(dptr, 0, bytes, ctx->stream));
  return NRS_OK;
}

int nrs_h2d(nrs_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, (dst_dev && src_host) || bytes == 0, NRS_ERR_ARG, "nrs_h2d: null pointer");
  if (bytes) NRS_CUDA(ctx, cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
  return NRS_OK;
}

int nrs_d2h(nrs_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, (dst_host && src_dev) || bytes == 0, NRS_ERR_ARG, "nrs_d2h: null pointer");
  if (bytes) NRS_CUDA(ctx, cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  NRS_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return nrs_check_device_error(ctx);
}

int nrs_d2d(nrs_ctx* ctx, void* dst_dev, const void* src_dev, size_t bytes) {
  NRS_REQUIRE_CTX(ctx);
  NRS_REQUIRE(ctx, (dst_dev && src_dev) || bytes == 0, NRS_ERR_ARG, "nrs_d2d: null pointer");
  if (bytes) NRS_CUDA(ctx, cudaMemcpyAsync(dst_dev, src_dev, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
  return NRS_OK;
}

int nrs_sync(nrs_ctx* ctx) {
  NRS_REQUIRE_CTX(ctx);
  NRS_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return nrs_check_device_error(ctx);
}

}  // extern "C"
