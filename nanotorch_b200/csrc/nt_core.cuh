// Shared runtime declarations for the sm_100a op-kernel library: status/error plumbing, the
// reference-counted storage object, the caching device arena, view normalisation (collapse of
// adjacent dimensions) and launch helpers.  Mirrors the roles of the reference's
// src/cpp/{storage.h,allocator.h,tensor_view.cuh,cuda.cuh}.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/nt_b200.h"

namespace ntb {

// ------------------------------------------------------------------------------------------
// Errors.  The three classes are the exception classes pybind11 raises for the reference
// (std::runtime_error / std::invalid_argument / py::type_error).
struct Error : std::exception {
  int code;
  std::string msg;
  Error(int c, std::string m) : code(c), msg(std::move(m)) {}
  const char *what() const noexcept override { return msg.c_str(); }
};
[[noreturn]] inline void fail_runtime(const std::string &m) { throw Error(NT_ERR_RUNTIME, m); }
[[noreturn]] inline void fail_invalid(const std::string &m) { throw Error(NT_ERR_INVALID, m); }
[[noreturn]] inline void fail_type(const std::string &m) { throw Error(NT_ERR_TYPE, m); }

void set_last_error(const std::string &m);

#define NT_CUDA_CHECK(expr)                                                                       \
  do {                                                                                            \
    cudaError_t _e = (expr);                                                                      \
    if (_e != cudaSuccess)                                                                        \
      ::ntb::fail_runtime(std::string(#expr " failed: ") + cudaGetErrorString(_e));               \
  } while (0)

#define NT_API_BEGIN try {
#define NT_API_END                                                                                \
  return NT_OK;                                                                                   \
  }                                                                                               \
  catch (const ::ntb::Error &e) {                                                                 \
    ::ntb::set_last_error(e.msg);                                                                 \
    return e.code;                                                                                \
  }                                                                                               \
  catch (const std::exception &e) {                                                               \
    ::ntb::set_last_error(e.what());                                                              \
    return NT_ERR_RUNTIME;                                                                        \
  }

// ------------------------------------------------------------------------------------------
// dtypes
inline int64_t dtype_itemsize(int dt) {
  switch (dt) {
  case NT_BOOL: return 1;
  case NT_INT32: return 4;
  case NT_INT64: return 8;
  case NT_FLOAT32: return 4;
  case NT_FLOAT64: return 8;
  default: fail_invalid("Unknown dtype.");
  }
}

// dtype -> template instantiation, the three dispatch families of src/cpp/dtype.h:23-79.
template <class F> auto dispatch_all(int dt, F &&f) {
  switch (dt) {
  case NT_BOOL: return f.template operator()<bool>();
  case NT_INT32: return f.template operator()<int32_t>();
  case NT_INT64: return f.template operator()<int64_t>();
  case NT_FLOAT32: return f.template operator()<float>();
  case NT_FLOAT64: return f.template operator()<double>();
  default: fail_invalid("Unknown dtype.");
  }
}
template <class F> auto dispatch_arith(int dt, F &&f) {
  switch (dt) {
  case NT_INT32: return f.template operator()<int32_t>();
  case NT_INT64: return f.template operator()<int64_t>();
  case NT_FLOAT32: return f.template operator()<float>();
  case NT_FLOAT64: return f.template operator()<double>();
  default: fail_invalid("Invalid dtype.");
  }
}
template <class F> auto dispatch_float(int dt, F &&f) {
  switch (dt) {
  case NT_FLOAT32: return f.template operator()<float>();
  case NT_FLOAT64: return f.template operator()<double>();
  default: fail_invalid("Invalid dtype.");
  }
}

// ------------------------------------------------------------------------------------------
// Runtime singletons
cudaStream_t stream();       // the one compute stream (non-blocking)
cudaStream_t comm_stream();  // collectives
cudaStream_t update_stream(); // the parameter updates that follow the collectives (lowest priority)
cudaStream_t compute_stream(); // the compute stream itself, whatever redirection is active
// While one of these lives, stream() returns `to`: kernels launched by the ordinary entry points go to
// that stream instead (used to run a parameter update on the communication stream, right behind the
// collective that produced its gradient).  Single-threaded use, like the rest of the library.
struct StreamRedirect {
  cudaStream_t prev;
  explicit StreamRedirect(cudaStream_t to);
  ~StreamRedirect();
  StreamRedirect(const StreamRedirect &) = delete;
  StreamRedirect &operator=(const StreamRedirect &) = delete;
};
void count_launch(uint64_t n = 1);
// matmul kernels call these around their launches (no-ops unless profiling is enabled)
void matmul_profile_begin();
bool matmul_profile_active();
void matmul_profile_extend(); // the launch just made belongs to the interval opened last
void matmul_profile_end();
bool cuda_ok();              // a device is present and usable
int gemm_tc_take_error();    // device-side error flag of the tensor-core GEMM (0 = none); call after a sync
void check_device_errors();  // after a stream synchronisation: raises if a bounded device-side wait ran out
long long wait_limit_clocks(); // limit of every bounded spin in device code, in SM clocks
bool is_capturing();         // a CUDA-graph capture is in progress on the compute stream
int capture_id();            // id of the graph being captured, 0 when none
uint64_t launches_so_far();  // kernels counted by check_launch since load
// Persistent device state that kernels expect to find zeroed (ticket counters of the reductions, the
// error flag of the tensor-core GEMM) and one-off function attributes: created eagerly, never inside
// a stream capture, where the zeroing would be recorded instead of executed.
void reduce_prepare();
void gemm_tc_prepare();
void gemm_tc_wait_probe();    // launches the bounded-wait probe kernel
int sm_count();
void destroy_all_graphs();   // captured graphs hold NCCL work: they must go before the communicator does

// Device arena: 256-byte granules up to 1 MiB, 1 MiB granules above; freed blocks are cached per
// rounded size and reused.  Reuse is safe without events because every consumer is on stream().
void *device_alloc(size_t nbytes, size_t *rounded);
void device_free(void *p, size_t rounded);
void *host_alloc(size_t nbytes, bool *pinned);
void host_free(void *p, bool pinned, size_t nbytes);

} // namespace ntb

// The storage object behind the opaque handle.
struct nt_storage {
  std::atomic<int64_t> refs{1};
  void *data = nullptr;
  size_t rounded = 0; // arena block size (device) or byte size (host)
  int64_t n = 0;
  int dtype = NT_FLOAT32;
  int device = NT_CPU;
  bool pinned = false;
  uint64_t version = 0;  // the reference's counter: bumped by the in-place ops only
  uint64_t mutation = 0; // bumped by EVERY entry point that writes into an existing storage (in-place ops,
                         // uploads, copy_view, scatter, all-reduce): what cached derived data is checked against
};

namespace ntb {

nt_storage *storage_new(int64_t n, int dtype, int device);
inline void storage_retain(nt_storage *s) { s->refs.fetch_add(1, std::memory_order_relaxed); }
void storage_release(nt_storage *s);
inline void storage_touch(nt_storage *s) { s->mutation += 1; }
// Cached operand planes of the tensor-core GEMM (gemm_tc.cu) die with the storage they were split from.
void gemm_tc_forget(nt_storage *s);
// Re-split, on the current stream(), every cached plane set of `s` (called right after a parameter
// update, so that the next forward pass finds its operand ready).
void gemm_tc_refresh(nt_storage *s);
float *gemm_tc_refresh_target(nt_storage *s, int64_t R, int64_t C); // see gemm_tc.cu
void gemm_tc_mark_refreshed(nt_storage *s);
// Cached planes written by work that was only captured, or overwritten by a graph replay behind the
// host's back, must not be trusted by later eager calls: a new epoch invalidates all of them.
void gemm_tc_new_epoch();
float *gemm_tc_adopt_planes(nt_storage *s, int64_t R, int64_t C); // see gemm_tc.cu

// RAII holder used while an entry point builds its result.
struct StorageRef {
  nt_storage *s = nullptr;
  StorageRef() = default;
  explicit StorageRef(nt_storage *p) : s(p) {}
  StorageRef(const StorageRef &) = delete;
  StorageRef &operator=(const StorageRef &) = delete;
  StorageRef(StorageRef &&o) noexcept : s(o.s) { o.s = nullptr; }
  ~StorageRef() {
    if (s) storage_release(s);
  }
  nt_storage *release() {
    nt_storage *p = s;
    s = nullptr;
    return p;
  }
  nt_storage *operator->() const { return s; }
};

// ------------------------------------------------------------------------------------------
// Views
inline int64_t view_numel(const nt_view &v) {
  int64_t n = 1;
  for (int i = 0; i < v.ndim; ++i) n *= v.shape[i];
  return n;
}

void check_view(const nt_view *v, const char *fname); // ndim range, non-null storage, bounds vs storage size
void require_cuda(const nt_view *v, const char *fname);
void require_same_shape(const nt_view *a, const nt_view *b, const char *fname);
void require_same_dtype(const nt_view *a, const nt_view *b, const char *fname);
void require_same_device(const nt_view *a, const nt_view *b, const char *fname);

// Device-side description of up to three operands over one shared iteration space.
// After collapse: size-1 dims dropped, adjacent dims merged when every operand allows it
// (stride[i] == stride[i+1]*shape[i+1]).  Strides are in elements; dim 0 is outermost.
template <int NOPS> struct IterSpace {
  int ndim;
  int64_t numel;
  int64_t shape[NT_MAX_DIMS];
  int64_t strides[NOPS][NT_MAX_DIMS];
  int64_t offset[NOPS];
};

template <int NOPS> IterSpace<NOPS> collapse(const nt_view *const (&views)[NOPS]) {
  IterSpace<NOPS> it{};
  const nt_view &v0 = *views[0];
  it.numel = view_numel(v0);
  for (int o = 0; o < NOPS; ++o) it.offset[o] = views[o]->offset;
  int nd = 0;
  for (int d = 0; d < v0.ndim; ++d) {
    if (v0.shape[d] == 1) continue;
    bool merged = false;
    if (nd > 0) {
      bool ok = true;
      for (int o = 0; o < NOPS; ++o)
        if (it.strides[o][nd - 1] != views[o]->strides[d] * v0.shape[d]) ok = false;
      if (ok) {
        it.shape[nd - 1] *= v0.shape[d];
        for (int o = 0; o < NOPS; ++o) it.strides[o][nd - 1] = views[o]->strides[d];
        merged = true;
      }
    }
    if (!merged) {
      it.shape[nd] = v0.shape[d];
      for (int o = 0; o < NOPS; ++o) it.strides[o][nd] = views[o]->strides[d];
      ++nd;
    }
  }
  it.ndim = nd;
  return it;
}

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

inline void check_launch(const char *what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) fail_runtime(std::string(what) + " launch failed: " + cudaGetErrorString(e));
  count_launch();
}

} // namespace ntb
