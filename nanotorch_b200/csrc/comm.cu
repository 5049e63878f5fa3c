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

#include "nt_core.cuh"

namespace ntb {

typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
enum { ncclSuccess = 0, ncclInProgress = 7 };
enum { ncclFloat32 = 7 };
enum { ncclSum = 0 };

struct Nccl {
  void *handle = nullptr;
  int (*GetUniqueId)(ncclUniqueId *) = nullptr;
  int (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  int (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*CommDestroy)(ncclComm_t) = nullptr;
  int (*CommAbort)(ncclComm_t) = nullptr;
  int (*CommGetAsyncError)(ncclComm_t, int *) = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1;
  cudaEvent_t ready = nullptr, done = nullptr;
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
  NT_SYM(CommDestroy, "ncclCommDestroy")
  NT_SYM(CommAbort, "ncclCommAbort")
  NT_SYM(CommGetAsyncError, "ncclCommGetAsyncError")
  NT_SYM(GetErrorString, "ncclGetErrorString")
#undef NT_SYM
}

static void nccl_check(int rc, const char *what) {
  if (rc != ncclSuccess) fail_runtime(std::string(what) + " failed: " + nccl().GetErrorString(rc));
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

int nt_comm_init(int rank, int world, const uint8_t id[NT_COMM_ID_BYTES]) {
  NT_API_BEGIN
  if (world < 1 || rank < 0 || rank >= world) fail_invalid("nt_comm_init: bad rank/world.");
  load_nccl();
  Nccl &n = nccl();
  if (n.comm) fail_runtime("nt_comm_init: communicator already initialised.");
  stream(); // selects the device and creates the streams
  ncclUniqueId uid;
  std::memcpy(&uid, id, sizeof(uid));
  nccl_check(n.CommInitRank(&n.comm, world, uid, rank), "ncclCommInitRank");
  n.rank = rank;
  n.world = world;
  NT_CUDA_CHECK(cudaEventCreateWithFlags(&n.ready, cudaEventDisableTiming));
  NT_CUDA_CHECK(cudaEventCreateWithFlags(&n.done, cudaEventDisableTiming));
  NT_API_END
}

int nt_comm_allreduce_sum(nt_storage *s) {
  NT_API_BEGIN
  Nccl &n = nccl();
  if (!n.comm) fail_runtime("nt_comm_allreduce_sum: communicator not initialised.");
  if (s->device != NT_CUDA || s->dtype != NT_FLOAT32) fail_invalid("nt_comm_allreduce_sum: Float32 Cuda storage only.");
  int async_err = ncclSuccess;
  nccl_check(n.CommGetAsyncError(n.comm, &async_err), "ncclCommGetAsyncError");
  if (async_err != ncclSuccess && async_err != ncclInProgress) {
    n.CommAbort(n.comm);
    n.comm = nullptr;
    fail_runtime(std::string("NCCL asynchronous error: ") + n.GetErrorString(async_err));
  }
  // the collective may start once everything enqueued on the compute stream so far has run
  NT_CUDA_CHECK(cudaEventRecord(n.ready, stream()));
  NT_CUDA_CHECK(cudaStreamWaitEvent(comm_stream(), n.ready, 0));
  nccl_check(n.AllReduce(s->data, s->data, size_t(s->n), ncclFloat32, ncclSum, n.comm, comm_stream()), "ncclAllReduce");
  count_launch();
  NT_API_END
}

int nt_comm_wait(void) {
  NT_API_BEGIN
  Nccl &n = nccl();
  if (!n.comm) return NT_OK;
  NT_CUDA_CHECK(cudaEventRecord(n.done, comm_stream()));
  NT_CUDA_CHECK(cudaStreamWaitEvent(stream(), n.done, 0));
  NT_API_END
}

int nt_comm_destroy(void) {
  NT_API_BEGIN
  Nccl &n = nccl();
  if (n.comm) {
    // a captured graph that contains a collective keeps the communicator busy: NCCL's destroy waits
    // for such graphs to be released, so release them first
    destroy_all_graphs();
    cudaStreamSynchronize(stream());
    cudaStreamSynchronize(comm_stream());
    n.CommDestroy(n.comm);
    n.comm = nullptr;
  }
  NT_API_END
}

} // extern "C"
