// Data-parallel gradient exchange behind the C ABI: he_comm_* / he_allreduce_grads.
//
// The hot path shards by batch / tokens and its only cross-GPU step is the sum (or mean) of weight and
// bias gradients after the backward GEMMs.  The reference has no multi-GPU code (its optimiser consumes
// whatever gradient tensor it is handed, helium/src/optimizer/sgd.rs:35-62), so this is the piece a
// data-parallel helium host would call between `backward()` and `Optimizer::step`.
//
// NCCL is loaded at run time with dlopen (the library has no link-time dependency on it, so it still
// loads on a machine without NCCL); a process that already carries an NCCL (for instance PyTorch's) gets
// that copy.  Failure handling is host-side only: the communicator is created non-blocking, every
// call that may wait is polled with ncclCommGetAsyncError against a deadline, and a deadline that
// passes ends in ncclCommAbort and an error status -- no call in this file can block for ever.
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <memory>
#include <mutex>
#include <thread>

#include "he_internal.h"

namespace he {
namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetVersion)(int*) = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  std::string error;
};

// HE_NCCL_LIBRARY names the library to load (tests point it at a stand-in whose calls never complete);
// otherwise the NCCL already in the process, or the system's libnccl.so.2.
NcclApi* nccl_api() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* forced = getenv("HE_NCCL_LIBRARY");
    const char* names[] = {forced, "libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
      if (!n || !n[0]) continue;
      api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (api.handle) break;
      if (n == forced) break;   // an explicit choice that fails is an error, not a reason to fall through
    }
    if (!api.handle) {
      const char* why = dlerror();   // a second call would return NULL: the message is consumed by the first
      api.error = std::string("could not load NCCL: ") + (why ? why : "libnccl.so.2 not found");
      return;
    }
    auto sym = [&](const char* name) -> void* {
      void* p = dlsym(api.handle, name);
      if (!p && api.error.empty()) api.error = std::string("NCCL library lacks ") + name;
      return p;
    };
    api.GetVersion = reinterpret_cast<decltype(api.GetVersion)>(sym("ncclGetVersion"));
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRankConfig = reinterpret_cast<decltype(api.CommInitRankConfig)>(sym("ncclCommInitRankConfig"));
    api.CommGetAsyncError = reinterpret_cast<decltype(api.CommGetAsyncError)>(sym("ncclCommGetAsyncError"));
    api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(sym("ncclCommAbort"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
    api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
    api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
  });
  return &api;
}

int64_t now_ms() {
  return std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

}  // namespace
}  // namespace he

struct he_comm {
  he_ctx* ctx = nullptr;
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1;
  int max_ctas = 0;
  bool aborted = false;
  int32_t default_timeout_ms = 30000;
  // layouts (n, dtype, counts) that every rank has already been seen to agree on
  std::vector<uint64_t> agreed;
  uint64_t* d_check = nullptr;   // two u64 words for the layout check
};

using namespace he;

namespace {

// Polls the communicator until its pending operation has finished, `timeout_ms` passed (the
// communicator is then aborted) or NCCL reports an error (aborted as well).
int32_t wait_ready(he_comm* c, int32_t timeout_ms, const char* what) {
  NcclApi* n = nccl_api();
  const int64_t deadline = now_ms() + (timeout_ms > 0 ? timeout_ms : c->default_timeout_ms);
  for (;;) {
    ncclResult_t state = ncclSuccess;
    ncclResult_t r = n->CommGetAsyncError(c->comm, &state);
    if (r != ncclSuccess) state = r;
    if (state == ncclSuccess) return HE_OK;
    if (state != ncclInProgress) {
      n->CommAbort(c->comm);
      c->aborted = true;
      HE_FAIL(HE_ERR_COMM, "%s: NCCL reported '%s' on rank %d; the communicator was aborted", what, n->GetErrorString(state), c->rank);
    }
    if (now_ms() > deadline) {
      n->CommAbort(c->comm);
      c->aborted = true;
      HE_FAIL(HE_ERR_COMM_TIMEOUT, "%s: not complete after %d ms on rank %d of %d (a peer never joined?); the communicator was aborted",
              what, timeout_ms > 0 ? timeout_ms : c->default_timeout_ms, c->rank, c->world);
    }
    std::this_thread::sleep_for(std::chrono::microseconds(200));
  }
}

uint64_t layout_hash(const size_t* counts, int32_t n, int32_t dtype, int32_t mean) {
  uint64_t h = 1469598103934665603ull;   // FNV-1a
  auto mix = [&](uint64_t v) {
    for (int i = 0; i < 8; ++i) {
      h ^= (v >> (8 * i)) & 0xffu;
      h *= 1099511628211ull;
    }
  };
  mix((uint64_t)n); mix((uint64_t)dtype); mix((uint64_t)mean);
  for (int i = 0; i < n; ++i) mix((uint64_t)counts[i]);
  return h & 0x7fffffffffffffffull;
}

}  // namespace

extern "C" {

int32_t he_comm_unique_id(void* id_out) {
  if (!id_out) HE_FAIL(HE_ERR_INVALID, "he_comm_unique_id: null argument");
  NcclApi* n = nccl_api();
  if (!n->error.empty()) HE_FAIL(HE_ERR_COMM, "%s", n->error.c_str());
  static_assert(sizeof(ncclUniqueId) == HE_COMM_UNIQUE_ID_BYTES, "unique id size");
  ncclUniqueId id;
  ncclResult_t r = n->GetUniqueId(&id);
  if (r != ncclSuccess) HE_FAIL(HE_ERR_COMM, "ncclGetUniqueId failed: %s", n->GetErrorString(r));
  memcpy(id_out, &id, sizeof id);
  return HE_OK;
}

int32_t he_comm_create(he_ctx* ctx, int32_t rank, int32_t world, const void* unique_id, int32_t max_ctas, int32_t timeout_ms,
                       he_comm** out) {
  if (!out) HE_FAIL(HE_ERR_INVALID, "he_comm_create: null argument");
  *out = nullptr;
  if (!unique_id) HE_FAIL(HE_ERR_INVALID, "he_comm_create: null argument");
  if (world < 1 || rank < 0 || rank >= world) HE_FAIL(HE_ERR_INVALID, "he_comm_create: rank %d is not in [0, %d)", rank, world);
  NcclApi* n = nccl_api();
  if (!n->error.empty()) HE_FAIL(HE_ERR_COMM, "%s", n->error.c_str());
  // with a context the communicator lives on the context's device, without one on the calling thread's
  // current device (NCCL's own rule)
  std::unique_ptr<DeviceGuard> guard;
  if (ctx) {
    guard.reset(new DeviceGuard(ctx->device));
    HE_TRY(guard->status());
  }
  std::unique_ptr<he_comm> c(new he_comm());
  c->ctx = ctx;
  c->rank = rank;
  c->world = world;
  c->max_ctas = max_ctas > 0 ? max_ctas : 0;
  if (timeout_ms > 0) c->default_timeout_ms = timeout_ms;
  ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
  cfg.blocking = 0;                        // every call returns at once; completion is polled with a deadline
  if (max_ctas > 0) cfg.maxCTAs = max_ctas;   // SMs the collectives may occupy next to a persistent GEMM
  ncclUniqueId id;
  memcpy(&id, unique_id, sizeof id);
  ncclResult_t r = n->CommInitRankConfig(&c->comm, world, id, rank, &cfg);
  if (r != ncclSuccess && r != ncclInProgress) HE_FAIL(HE_ERR_COMM, "ncclCommInitRankConfig failed on rank %d: %s", rank, n->GetErrorString(r));
  HE_TRY(wait_ready(c.get(), timeout_ms, "he_comm_create"));
  *out = c.release();
  return HE_OK;
}

int32_t he_comm_info(const he_comm* comm, int32_t* rank, int32_t* world, int32_t* max_ctas) {
  if (!comm) HE_FAIL(HE_ERR_INVALID, "he_comm_info: null argument");
  if (rank) *rank = comm->rank;
  if (world) *world = comm->world;
  if (max_ctas) *max_ctas = comm->max_ctas;
  return HE_OK;
}

int32_t he_allreduce_grads(he_comm* comm, void* const* bufs, const size_t* counts, int32_t n, int32_t dtype, int32_t mean,
                           void* cu_stream) {
  if (!comm) HE_FAIL(HE_ERR_INVALID, "he_allreduce_grads: communicator is null");
  TraceRange range("he_allreduce_grads");
  if (comm->aborted) HE_FAIL(HE_ERR_COMM, "he_allreduce_grads: the communicator was aborted; create a new one");
  if (n < 0 || (n > 0 && (!bufs || !counts))) HE_FAIL(HE_ERR_INVALID, "he_allreduce_grads: null argument");
  ncclDataType_t dt;
  switch (dtype) {
    case HE_F16: dt = ncclFloat16; break;
    case HE_BF16: dt = ncclBfloat16; break;
    case HE_F32: dt = ncclFloat32; break;
    default: HE_FAIL(HE_ERR_INVALID, "he_allreduce_grads: gradients must be f16, bf16 or f32 (got dtype %d)", dtype);
  }
  for (int i = 0; i < n; ++i) {
    if (!bufs[i]) HE_FAIL(HE_ERR_INVALID, "he_allreduce_grads: buffer %d is null", i);
    if (counts[i] == 0 || counts[i] > (size_t)1 << 40) HE_FAIL(HE_ERR_INVALID, "he_allreduce_grads: buffer %d has %zu elements", i, counts[i]);
  }
  if (n == 0) return HE_OK;
  NcclApi* api = nccl_api();
  cudaStream_t stream = (cudaStream_t)cu_stream;
  std::unique_ptr<DeviceGuard> guard;
  if (comm->ctx) {
    guard.reset(new DeviceGuard(comm->ctx->device));
    HE_TRY(guard->status());
  }

  // A rank whose bucket layout differs from its peers' would deadlock or corrupt the sum.  The first time
  // a layout is used, all ranks compare a hash of (n, dtype, counts): max and min of it over the ranks,
  // in one 16-byte collective whose result is read back before anything else is enqueued.  Agreed layouts
  // are remembered, so steady-state calls pay nothing.
  const uint64_t h = layout_hash(counts, n, dtype, mean);
  bool known = false;
  for (uint64_t a : comm->agreed) known = known || a == h;
  if (!known && comm->world > 1) {
    uint64_t host[2] = {h, h};
    if (!comm->d_check) HE_CUDA(cudaMalloc(&comm->d_check, 16));   // once per communicator, outside any steady-state step
    HE_CUDA(cudaMemcpyAsync(comm->d_check, host, 16, cudaMemcpyHostToDevice, stream));
    ncclResult_t r = api->GroupStart();
    if (r == ncclSuccess || r == ncclInProgress) r = api->AllReduce(comm->d_check, comm->d_check, 1, ncclUint64, ncclMax, comm->comm, stream);
    if (r == ncclSuccess || r == ncclInProgress) r = api->AllReduce(comm->d_check + 1, comm->d_check + 1, 1, ncclUint64, ncclMin, comm->comm, stream);
    ncclResult_t e = api->GroupEnd();
    if (r == ncclSuccess || r == ncclInProgress) r = e;
    if (r != ncclSuccess && r != ncclInProgress) HE_FAIL(HE_ERR_COMM, "he_allreduce_grads: layout check failed to start: %s", api->GetErrorString(r));
    HE_TRY(wait_ready(comm, 0, "he_allreduce_grads (layout check)"));
    HE_CUDA(cudaMemcpyAsync(host, comm->d_check, 16, cudaMemcpyDeviceToHost, stream));
    // bounded wait for the two words
    const int64_t deadline = now_ms() + comm->default_timeout_ms;
    for (;;) {
      cudaError_t q = cudaStreamQuery(stream);
      if (q == cudaSuccess) break;
      if (q != cudaErrorNotReady) HE_FAIL(HE_ERR_CUDA, "he_allreduce_grads: %s while waiting for the layout check", cudaGetErrorString(q));
      if (now_ms() > deadline) {
        api->CommAbort(comm->comm);
        comm->aborted = true;
        HE_FAIL(HE_ERR_COMM_TIMEOUT, "he_allreduce_grads: the layout check did not complete within %d ms on rank %d; the communicator was aborted",
                comm->default_timeout_ms, comm->rank);
      }
      std::this_thread::sleep_for(std::chrono::microseconds(100));
    }
    if (host[0] != h || host[1] != h)
      HE_FAIL(HE_ERR_INVALID, "he_allreduce_grads: rank %d was called with a different bucket layout (count, sizes, dtype or mean flag) "
                              "than another rank; nothing was reduced", comm->rank);
    comm->agreed.push_back(h);
  }

  const ncclRedOp_t op = mean ? ncclAvg : ncclSum;
  ncclResult_t r = api->GroupStart();
  for (int i = 0; i < n && (r == ncclSuccess || r == ncclInProgress); ++i)
    r = api->AllReduce(bufs[i], bufs[i], counts[i], dt, op, comm->comm, stream);
  ncclResult_t e = api->GroupEnd();
  if (r == ncclSuccess || r == ncclInProgress) r = e;
  if (r != ncclSuccess && r != ncclInProgress) HE_FAIL(HE_ERR_COMM, "he_allreduce_grads: NCCL refused the collective: %s", api->GetErrorString(r));
  // non-blocking communicator: the enqueue itself may still be in progress; it is bounded like everything else
  return wait_ready(comm, 0, "he_allreduce_grads");
}

int32_t he_comm_poll(he_comm* comm) {
  if (!comm) HE_FAIL(HE_ERR_INVALID, "he_comm_poll: communicator is null");
  if (comm->aborted) HE_FAIL(HE_ERR_COMM, "the communicator was aborted");
  NcclApi* n = nccl_api();
  ncclResult_t state = ncclSuccess;
  ncclResult_t r = n->CommGetAsyncError(comm->comm, &state);
  if (r != ncclSuccess) state = r;
  if (state == ncclSuccess || state == ncclInProgress) return HE_OK;
  HE_FAIL(HE_ERR_COMM, "NCCL asynchronous error on rank %d: %s", comm->rank, n->GetErrorString(state));
}

int32_t he_comm_abort(he_comm* comm) {
  if (!comm) HE_FAIL(HE_ERR_INVALID, "he_comm_abort: communicator is null");
  if (!comm->aborted && comm->comm) {
    nccl_api()->CommAbort(comm->comm);
    comm->aborted = true;
  }
  return HE_OK;
}

void he_comm_destroy(he_comm* comm) {
  if (!comm) return;
  NcclApi* n = nccl_api();
  if (comm->comm && !comm->aborted) {
    // in-flight collectives belong to the caller's streams; by the time a communicator is destroyed the
    // caller has joined them, so a plain destroy does not wait on the device
    n->CommDestroy(comm->comm);
  }
  if (comm->d_check) cudaFree(comm->d_check);
  delete comm;
}

}  // extern "C"
