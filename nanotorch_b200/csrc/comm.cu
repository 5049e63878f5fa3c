// Data-parallel gradient exchange: one NCCL communicator per process (one process per GPU), fp32
// sum all-reduce on a dedicated communication stream, ordered against the compute stream with
// events so that the collective of one layer overlaps the backward kernels of the next.
//
// The reference has no multi-device code at all (its Device enum is {Cpu, Cuda} without an index,
// src/cpp/allocator.h:10); these entry points are additions behind the same C ABI.
//
// NCCL is bound at run time with dlopen so that the library also loads where NCCL is absent; the
// handful of signatures declared here are NCCL's stable public C API (nccl.h).
#include <dlfcn.h>

#include <chrono>
#include <condition_variable>
#include <cstdlib>
#include <memory>
#include <mutex>
#include <thread>

#include "nt_core.cuh"

namespace ntb {

typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
enum { ncclSuccess = 0, ncclInProgress = 7 };
enum { ncclFloat32 = 7 };
enum { ncclSum = 0 };
// Leading fields of NCCL's public ncclConfig_t (nccl.h, stable since 2.17); a library that knows more
// fields fills them with defaults from `size` and `version`.
struct NcclConfig {
  size_t size;
  unsigned int magic;
  unsigned int version;
  int blocking;
  int cgaClusterSize;
  int minCTAs;
  int maxCTAs;
  const char *netName;
  int splitShare;
};
constexpr int NCCL_UNDEF_INT = INT32_MIN;

struct Nccl {
  void *handle = nullptr;
  int (*GetUniqueId)(ncclUniqueId *) = nullptr;
  int (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  int (*CommInitRankConfig)(ncclComm_t *, int, ncclUniqueId, int, NcclConfig *) = nullptr; // may be absent
  int (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  int (*CommDestroy)(ncclComm_t) = nullptr;
  int (*CommAbort)(ncclComm_t) = nullptr;
  int (*CommGetAsyncError)(ncclComm_t, int *) = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1;
  bool in_group = false;
  bool side_work = false; // something was enqueued on the communication stream since the last join
  cudaEvent_t ready = nullptr, done = nullptr, exchanged = nullptr, updated = nullptr;
  bool update_work = false; // something was enqueued on the update stream since the last join
};
static Nccl &nccl() {
  static Nccl n;
  return n;
}

static void load_nccl() {
  Nccl &n = nccl();
  if (n.handle) return;
  const char *names[] = {"libnccl.so.2", "libnccl.so"};
  for (const char *nm : names) {
    n.handle = dlopen(nm, RTLD_NOW | RTLD_GLOBAL);
    if (n.handle) break;
  }
  if (!n.handle) fail_runtime(std::string("NCCL not found: ") + dlerror());
#define NT_SYM(field, name)                                                                        \
  n.field = reinterpret_cast<decltype(n.field)>(dlsym(n.handle, name));                            \
  if (!n.field) fail_runtime(std::string("NCCL symbol missing: ") + name);
  NT_SYM(GetUniqueId, "ncclGetUniqueId")
  NT_SYM(CommInitRank, "ncclCommInitRank")
  NT_SYM(AllReduce, "ncclAllReduce")
  NT_SYM(GroupStart, "ncclGroupStart")
  NT_SYM(GroupEnd, "ncclGroupEnd")
  NT_SYM(CommDestroy, "ncclCommDestroy")
  NT_SYM(CommAbort, "ncclCommAbort")
  NT_SYM(CommGetAsyncError, "ncclCommGetAsyncError")
  NT_SYM(GetErrorString, "ncclGetErrorString")
#undef NT_SYM
  n.CommInitRankConfig = reinterpret_cast<decltype(n.CommInitRankConfig)>(dlsym(n.handle, "ncclCommInitRankConfig"));
}

static void nccl_check(int rc, const char *what) {
  if (rc != ncclSuccess) fail_runtime(std::string(what) + " failed: " + nccl().GetErrorString(rc));
}

static void ensure_events() {
  Nccl &n = nccl();
  if (!n.ready) {
    NT_CUDA_CHECK(cudaEventCreateWithFlags(&n.ready, cudaEventDisableTiming));
    NT_CUDA_CHECK(cudaEventCreateWithFlags(&n.done, cudaEventDisableTiming));
    NT_CUDA_CHECK(cudaEventCreateWithFlags(&n.exchanged, cudaEventDisableTiming));
    NT_CUDA_CHECK(cudaEventCreateWithFlags(&n.updated, cudaEventDisableTiming));
  }
}

// Everything enqueued on the compute stream so far happens before what the communication stream is
// given next.
static void comm_after_compute() {
  Nccl &n = nccl();
  ensure_events();
  NT_CUDA_CHECK(cudaEventRecord(n.ready, compute_stream()));
  NT_CUDA_CHECK(cudaStreamWaitEvent(comm_stream(), n.ready, 0));
  n.side_work = true;
}

static void poll_async_error() {
  Nccl &n = nccl();
  int async_err = ncclSuccess;
  nccl_check(n.CommGetAsyncError(n.comm, &async_err), "ncclCommGetAsyncError");
  if (async_err != ncclSuccess && async_err != ncclInProgress) {
    n.CommAbort(n.comm);
    n.comm = nullptr;
    fail_runtime(std::string("NCCL asynchronous error: ") + n.GetErrorString(async_err));
  }
}

} // namespace ntb

using namespace ntb;

extern "C" {

int nt_comm_unique_id(uint8_t id[NT_COMM_ID_BYTES]) {
  NT_API_BEGIN
  load_nccl();
  static_assert(sizeof(ncclUniqueId) == NT_COMM_ID_BYTES, "unique id size");
  ncclUniqueId uid;
  nccl_check(nccl().GetUniqueId(&uid), "ncclGetUniqueId");
  std::memcpy(id, &uid, sizeof(uid));
  NT_API_END
}

int nt_comm_init_timeout(int rank, int world, const uint8_t id[NT_COMM_ID_BYTES], int64_t timeout_ms) {
  NT_API_BEGIN
  if (world < 1 || rank < 0 || rank >= world) fail_invalid("nt_comm_init: bad rank/world.");
  load_nccl();
  Nccl &n = nccl();
  if (n.comm) fail_runtime("nt_comm_init: communicator already initialised.");
  stream(); // selects the device and creates the streams
  int device = 0;
  NT_CUDA_CHECK(cudaGetDevice(&device));
  ncclUniqueId uid;
  std::memcpy(&uid, id, sizeof(uid));
  // NCCL's CTAs take whole SMs from the backward GEMMs they overlap (a GEMM CTA fills an SM): 16 was the
  // best trade at 8 ranks on NVSwitch -- 8 exposes the exchange, NCCL's own choice slows the GEMMs more than
  // it gains.  NT_NCCL_MAX_CTAS overrides it; 0 leaves the choice to NCCL.
  int max_ctas = 16;
  if (const char *e = std::getenv("NT_NCCL_MAX_CTAS")) max_ctas = std::atoi(e);
  // The rendezvous blocks until every rank has joined.  It runs on a helper thread so that a rank
  // that never arrives turns into an error here after `timeout_ms` instead of a hang; the helper
  // stays blocked in that case (there is no communicator yet that could be aborted) and the caller
  // is expected to exit.
  struct Shared {
    std::mutex mu;
    std::condition_variable cv;
    bool finished = false;
    int rc = ncclSuccess;
    ncclComm_t comm = nullptr;
  };
  auto sh = std::make_shared<Shared>();
  auto init_fn = n.CommInitRank;
  auto init_cfg_fn = n.CommInitRankConfig;
  std::thread([sh, init_fn, init_cfg_fn, uid, rank, world, device, max_ctas]() {
    cudaSetDevice(device);
    ncclComm_t c = nullptr;
    int rc;
    if (max_ctas > 0 && init_cfg_fn) {
      NcclConfig cfg{sizeof(NcclConfig), 0xcafebeefu, 21700u, NCCL_UNDEF_INT, NCCL_UNDEF_INT, NCCL_UNDEF_INT,
                     max_ctas, nullptr, NCCL_UNDEF_INT};
      rc = init_cfg_fn(&c, world, uid, rank, &cfg);
    } else {
      rc = init_fn(&c, world, uid, rank);
    }
    std::lock_guard<std::mutex> lk(sh->mu);
    sh->rc = rc;
    sh->comm = c;
    sh->finished = true;
    sh->cv.notify_all();
  }).detach();
  {
    std::unique_lock<std::mutex> lk(sh->mu);
    if (!sh->cv.wait_for(lk, std::chrono::milliseconds(timeout_ms > 0 ? timeout_ms : 1), [&] { return sh->finished; }))
      fail_runtime("nt_comm_init: the other ranks did not join within " + std::to_string(timeout_ms) + " ms.");
  }
  nccl_check(sh->rc, "ncclCommInitRank");
  n.comm = sh->comm;
  n.rank = rank;
  n.world = world;
  ensure_events();
  NT_API_END
}

int nt_comm_init(int rank, int world, const uint8_t id[NT_COMM_ID_BYTES]) {
  int64_t timeout_ms = 300000;
  if (const char *e = std::getenv("NT_COMM_TIMEOUT_MS")) timeout_ms = std::atoll(e);
  return nt_comm_init_timeout(rank, world, id, timeout_ms);
}

int nt_comm_group_begin(void) {
  NT_API_BEGIN
  Nccl &n = nccl();
  if (n.in_group) fail_runtime("nt_comm_group_begin: a group is already open.");
  comm_after_compute();
  if (n.comm) {
    poll_async_error();
    nccl_check(n.GroupStart(), "ncclGroupStart");
  }
  n.in_group = true;
  NT_API_END
}

int nt_comm_group_end(void) {
  NT_API_BEGIN
  Nccl &n = nccl();
  if (!n.in_group) fail_runtime("nt_comm_group_end: no group is open.");
  n.in_group = false;
  if (n.comm) nccl_check(n.GroupEnd(), "ncclGroupEnd");
  NT_API_END
}

int nt_comm_allreduce_sum(nt_storage *s) {
  NT_API_BEGIN
  Nccl &n = nccl();
  if (!n.comm) fail_runtime("nt_comm_allreduce_sum: communicator not initialised.");
  if (s->device != NT_CUDA || s->dtype != NT_FLOAT32) fail_invalid("nt_comm_allreduce_sum: Float32 Cuda storage only.");
  if (!n.in_group) {
    poll_async_error();
    comm_after_compute(); // the collective may start once everything enqueued on the compute stream so far has run
  }
  nccl_check(n.AllReduce(s->data, s->data, size_t(s->n), ncclFloat32, ncclSum, n.comm, comm_stream()), "ncclAllReduce");
  storage_touch(s);
  count_launch();
  NT_API_END
}

int nt_comm_sgd_update(const nt_view *param, const nt_view *grad, float lr, float grad_scale) {
  // same kernel and checks as nt_sgd_update, enqueued on the update stream: behind the collectives issued so
  // far on the communication stream (which itself is behind the kernels that produced the gradient)
  Nccl &n = nccl();
  try {
    comm_after_compute();
    NT_CUDA_CHECK(cudaEventRecord(n.exchanged, comm_stream()));
    NT_CUDA_CHECK(cudaStreamWaitEvent(update_stream(), n.exchanged, 0));
    n.update_work = true;
  } catch (const Error &e) {
    set_last_error(e.msg);
    return e.code;
  }
  StreamRedirect redirect(update_stream());
  return nt_sgd_update(param, grad, lr, grad_scale);
}

int nt_comm_wait(void) {
  NT_API_BEGIN
  Nccl &n = nccl();
  if (n.side_work) {
    NT_CUDA_CHECK(cudaEventRecord(n.done, comm_stream()));
    NT_CUDA_CHECK(cudaStreamWaitEvent(compute_stream(), n.done, 0));
    n.side_work = false;
  }
  if (n.update_work) {
    NT_CUDA_CHECK(cudaEventRecord(n.updated, update_stream()));
    NT_CUDA_CHECK(cudaStreamWaitEvent(compute_stream(), n.updated, 0));
    n.update_work = false;
  }
  NT_API_END
}

int nt_comm_sync(int64_t timeout_ms) {
  NT_API_BEGIN
  Nccl &n = nccl();
  if (!cuda_ok()) return NT_OK;
  ensure_events();
  cudaEvent_t ev = nullptr;
  NT_CUDA_CHECK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  NT_CUDA_CHECK(cudaEventRecord(ev, comm_stream()));
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (;;) {
    cudaError_t q = cudaEventQuery(ev);
    if (q == cudaSuccess) break;
    if (q != cudaErrorNotReady) {
      cudaEventDestroy(ev);
      fail_runtime(std::string("nt_comm_sync: ") + cudaGetErrorString(q));
    }
    if (n.comm) poll_async_error();
    if (std::chrono::steady_clock::now() > deadline) {
      cudaEventDestroy(ev);
      if (n.comm) { // a peer is gone or stuck: take the collective kernels down so the stream drains
        n.CommAbort(n.comm);
        n.comm = nullptr;
      }
      fail_runtime("nt_comm_sync: collectives still outstanding after " + std::to_string(timeout_ms) +
                   " ms; the communicator was aborted.");
    }
    std::this_thread::sleep_for(std::chrono::microseconds(200));
  }
  cudaEventDestroy(ev);
  NT_API_END
}

int nt_comm_abort(void) {
  NT_API_BEGIN
  Nccl &n = nccl();
  if (n.comm) {
    n.CommAbort(n.comm);
    n.comm = nullptr;
  }
  n.in_group = false;
  NT_API_END
}

int nt_comm_destroy(void) {
  NT_API_BEGIN
  Nccl &n = nccl();
  if (n.comm) {
    // a captured graph that contains a collective keeps the communicator busy: NCCL's destroy waits
    // for such graphs to be released, so release them first
    destroy_all_graphs();
    cudaStreamSynchronize(compute_stream());
    cudaStreamSynchronize(comm_stream());
    cudaStreamSynchronize(update_stream());
    n.CommDestroy(n.comm);
    n.comm = nullptr;
  }
  NT_API_END
}

} // extern "C"
