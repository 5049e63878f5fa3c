// Runtime half of the C ABI: error string, stream, caching arena, storage lifecycle, host<->device
// moves, on-device dtype cast, factories and the host RNG stream.
// Replaces src/cpp/{storage.cpp,allocator.cpp,factory.cu,random.h,cuda.cpp} of the reference.
#include <cstdlib>
#include <map>
#include <mutex>
#include <random>
#include <set>
#include <unordered_map>

#include "nt_core.cuh"

namespace ntb {

static thread_local std::string g_last_error;
void set_last_error(const std::string &m) { g_last_error = m; }

// ------------------------------------------------------------------------------------------
struct Runtime {
  std::mutex mu;
  bool probed = false;
  bool have_cuda = false;
  int device = 0;
  int sms = 148;
  cudaStream_t compute = nullptr;
  cudaStream_t comm = nullptr;
  cudaStream_t update = nullptr;
  cudaStream_t copy = nullptr;
  cudaStream_t redirect = nullptr;                     // when set, stream() hands this one out (StreamRedirect)
  cudaEvent_t copy_gate = nullptr, copy_done = nullptr;
  bool mm_profile = false;
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> mm_events;
  std::vector<int> mm_counts; // launches between each pair of events (2 for an overlapped pair of products)
  std::vector<cudaEvent_t> event_pool;
  std::map<size_t, std::vector<void *>> dev_cache;
  std::map<size_t, std::vector<void *>> pin_cache;
  // CUDA-graph capture: blocks handed out while a graph is being captured belong to that graph and
  // are recycled only inside it, so that eager work can never be given memory a replay will write.
  int capturing = 0;                                   // id of the graph being captured, 0 = none
  int next_graph_id = 1;
  std::unordered_map<void *, int> graph_owned;         // block -> graph id
  std::map<int, std::map<size_t, std::vector<void *>>> graph_cache;
  std::set<int> live_graphs;
  std::map<int, cudaGraphExec_t> graph_exec;
  uint64_t bytes_reserved = 0, bytes_in_use = 0, n_malloc = 0;
  uint64_t n_requests = 0;                             // device_alloc calls, served from the cache or not
  std::atomic<long long> wait_limit{1LL << 31};        // SM clocks a bounded device-side spin may take
  size_t pin_cached_bytes = 0;
  std::atomic<uint64_t> launches{0};
  std::mt19937_64 rng{std::random_device{}()};
  // device generator (rng_mode 1): Philox4x32-10 keyed by the seed; `philox_offset` counts the 128-bit
  // blocks handed out so far, so successive calls continue one stream
  int rng_mode = 0;
  uint64_t philox_seed = std::random_device{}();
  uint64_t philox_offset = 0;
};
static Runtime &rt() {
  static Runtime r;
  return r;
}

static void probe_locked(Runtime &r) {
  if (r.probed) return;
  r.probed = true;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count <= 0) {
    cudaGetLastError();
    r.have_cuda = false;
    return;
  }
  r.have_cuda = true;
}

static void ensure_streams_locked(Runtime &r) {
  probe_locked(r);
  if (!r.have_cuda) fail_runtime("CUDA device required: no usable GPU found (this library has no CPU compute path).");
  if (r.compute) return;
  NT_CUDA_CHECK(cudaSetDevice(r.device));
  // Three streams.  The compute stream and the communication stream (NCCL) run at the highest priority;
  // the update stream -- parameter updates and the re-split of their operand planes, issued behind each
  // bucket's exchange -- at the lowest, so that its CTAs fill SMs the backward GEMMs leave idle instead
  // of delaying their tiles.  NT_STREAM_PRIORITY=0 creates all three alike.
  int least = 0, greatest = 0;
  const char *prio = std::getenv("NT_STREAM_PRIORITY");
  const bool flat = prio && prio[0] == '0';
  if (!flat && cudaDeviceGetStreamPriorityRange(&least, &greatest) == cudaSuccess && least != greatest) {
    NT_CUDA_CHECK(cudaStreamCreateWithPriority(&r.compute, cudaStreamNonBlocking, greatest));
    NT_CUDA_CHECK(cudaStreamCreateWithPriority(&r.comm, cudaStreamNonBlocking, greatest));
    NT_CUDA_CHECK(cudaStreamCreateWithPriority(&r.update, cudaStreamNonBlocking, least));
  } else {
    cudaGetLastError();
    NT_CUDA_CHECK(cudaStreamCreateWithFlags(&r.compute, cudaStreamNonBlocking));
    NT_CUDA_CHECK(cudaStreamCreateWithFlags(&r.comm, cudaStreamNonBlocking));
    NT_CUDA_CHECK(cudaStreamCreateWithFlags(&r.update, cudaStreamNonBlocking));
  }
  NT_CUDA_CHECK(cudaStreamCreateWithFlags(&r.copy, cudaStreamNonBlocking));
  NT_CUDA_CHECK(cudaEventCreateWithFlags(&r.copy_gate, cudaEventDisableTiming));
  NT_CUDA_CHECK(cudaEventCreateWithFlags(&r.copy_done, cudaEventDisableTiming));
  cudaDeviceProp prop;
  NT_CUDA_CHECK(cudaGetDeviceProperties(&prop, r.device));
  r.sms = prop.multiProcessorCount;
}

bool cuda_ok() {
  Runtime &r = rt();
  std::lock_guard<std::mutex> lk(r.mu);
  probe_locked(r);
  return r.have_cuda;
}
cudaStream_t stream() {
  Runtime &r = rt();
  std::lock_guard<std::mutex> lk(r.mu);
  ensure_streams_locked(r);
  return r.redirect ? r.redirect : r.compute;
}
cudaStream_t compute_stream() {
  Runtime &r = rt();
  std::lock_guard<std::mutex> lk(r.mu);
  ensure_streams_locked(r);
  return r.compute;
}
StreamRedirect::StreamRedirect(cudaStream_t to) {
  Runtime &r = rt();
  std::lock_guard<std::mutex> lk(r.mu);
  prev = r.redirect;
  r.redirect = to;
}
StreamRedirect::~StreamRedirect() {
  Runtime &r = rt();
  std::lock_guard<std::mutex> lk(r.mu);
  r.redirect = prev;
}
cudaStream_t comm_stream() {
  Runtime &r = rt();
  std::lock_guard<std::mutex> lk(r.mu);
  ensure_streams_locked(r);
  return r.comm;
}
cudaStream_t update_stream() {
  Runtime &r = rt();
  std::lock_guard<std::mutex> lk(r.mu);
  ensure_streams_locked(r);
  return r.update;
}
uint64_t launches_so_far() { return rt().launches.load(); }
int capture_id() {
  Runtime &r = rt();
  std::lock_guard<std::mutex> lk(r.mu);
  return r.capturing;
}
bool is_capturing() {
  Runtime &r = rt();
  std::lock_guard<std::mutex> lk(r.mu);
  return r.capturing != 0;
}
long long wait_limit_clocks() { return rt().wait_limit.load(std::memory_order_relaxed); }
void check_device_errors() {
  const int tc_err = gemm_tc_take_error();
  if (tc_err != 0)
    fail_runtime("a bounded device-side wait ran out (code " + std::to_string(tc_err) +
                 "; gemm_3xtf32: 1 = producer waiting for a free stage, 2 = MMA waiting for data, 3 = epilogue "
                 "waiting for the accumulator, 4 = MMA waiting for a drained accumulator; 5 = the wait probe; "
                 "6 = the elementwise tile pipeline waiting for a tile); results of the launches since the last "
                 "synchronisation are invalid.");
}
int sm_count() {
  Runtime &r = rt();
  std::lock_guard<std::mutex> lk(r.mu);
  ensure_streams_locked(r);
  return r.sms;
}
static void graph_destroy_locked(Runtime &r, int graph_id) {
  auto it = r.graph_exec.find(graph_id);
  if (it != r.graph_exec.end()) {
    if (r.compute) cudaStreamSynchronize(r.compute);
    cudaGraphExecDestroy(it->second);
    r.graph_exec.erase(it);
  }
  r.live_graphs.erase(graph_id);
  auto gc = r.graph_cache.find(graph_id);
  if (gc != r.graph_cache.end()) { // its recycled blocks go back to the general cache
    for (auto &kv : gc->second)
      for (void *p : kv.second) {
        r.graph_owned.erase(p);
        r.dev_cache[kv.first].push_back(p);
      }
    r.graph_cache.erase(gc);
  }
}

void destroy_all_graphs() {
  Runtime &r = rt();
  std::lock_guard<std::mutex> lk(r.mu);
  std::vector<int> ids;
  for (auto &kv : r.graph_exec) ids.push_back(kv.first);
  for (int id : ids) graph_destroy_locked(r, id);
}
void count_launch(uint64_t n) { rt().launches.fetch_add(n, std::memory_order_relaxed); }

static cudaEvent_t pooled_event(Runtime &r) {
  if (!r.event_pool.empty()) {
    cudaEvent_t e = r.event_pool.back();
    r.event_pool.pop_back();
    return e;
  }
  cudaEvent_t e;
  NT_CUDA_CHECK(cudaEventCreate(&e));
  return e;
}
void matmul_profile_begin() {
  Runtime &r = rt();
  if (!r.mm_profile) return;
  cudaEvent_t a = pooled_event(r), b = pooled_event(r);
  NT_CUDA_CHECK(cudaEventRecord(a, r.compute));
  r.mm_events.emplace_back(a, b);
  r.mm_counts.push_back(1);
}
bool matmul_profile_active() { return rt().mm_profile; }
// One more launch belongs to the interval that was opened last (the second product of an overlapped pair).
void matmul_profile_extend() {
  Runtime &r = rt();
  if (!r.mm_profile || r.mm_counts.empty()) return;
  r.mm_counts.back() += 1;
}
void matmul_profile_end() {
  Runtime &r = rt();
  if (!r.mm_profile || r.mm_events.empty()) return;
  NT_CUDA_CHECK(cudaEventRecord(r.mm_events.back().second, r.compute));
}

static size_t round_block(size_t nbytes) {
  if (nbytes == 0) nbytes = 1;
  const size_t small = 256, big = size_t(1) << 20;
  if (nbytes <= big) return (nbytes + small - 1) / small * small;
  return (nbytes + big - 1) / big * big;
}

static void trim_locked(Runtime &r) {
  for (auto &kv : r.dev_cache) {
    for (void *p : kv.second) {
      cudaFree(p);
      r.bytes_reserved -= kv.first;
    }
    kv.second.clear();
  }
}

void *device_alloc(size_t nbytes, size_t *rounded) {
  Runtime &r = rt();
  std::lock_guard<std::mutex> lk(r.mu);
  ensure_streams_locked(r);
  size_t sz = round_block(nbytes);
  *rounded = sz;
  r.n_requests += 1;
  if (r.capturing) {
    auto &gc = r.graph_cache[r.capturing];
    auto git = gc.find(sz);
    if (git != gc.end() && !git->second.empty()) {
      void *p = git->second.back();
      git->second.pop_back();
      r.bytes_in_use += sz;
      return p;
    }
  }
  auto it = r.dev_cache.find(sz);
  if (it != r.dev_cache.end() && !it->second.empty()) {
    void *p = it->second.back();
    it->second.pop_back();
    r.bytes_in_use += sz;
    if (r.capturing) r.graph_owned[p] = r.capturing;
    return p;
  }
  void *p = nullptr;
  cudaError_t e = cudaMalloc(&p, sz);
  if (e == cudaErrorMemoryAllocation && !r.capturing) {
    cudaGetLastError();
    // Everything cached was freed behind work on the compute stream: drain it, give the cache
    // back to the driver, try once more.
    cudaStreamSynchronize(r.compute);
    trim_locked(r);
    e = cudaMalloc(&p, sz);
  }
  if (e != cudaSuccess) fail_runtime(std::string("cudaMalloc failed: ") + cudaGetErrorString(e));
  r.n_malloc += 1;
  r.bytes_reserved += sz;
  r.bytes_in_use += sz;
  if (r.capturing) r.graph_owned[p] = r.capturing;
  return p;
}
void device_free(void *p, size_t rounded) {
  if (!p) return;
  Runtime &r = rt();
  std::lock_guard<std::mutex> lk(r.mu);
  r.bytes_in_use -= rounded;
  auto own = r.graph_owned.find(p);
  if (own != r.graph_owned.end()) {
    if (r.live_graphs.count(own->second)) {
      r.graph_cache[own->second][rounded].push_back(p); // stays with its graph
      return;
    }
    r.graph_owned.erase(own); // the graph is gone: an ordinary block again
  }
  r.dev_cache[rounded].push_back(p);
}

void *host_alloc(size_t nbytes, bool *pinned) {
  Runtime &r = rt();
  size_t sz = round_block(nbytes);
  {
    std::lock_guard<std::mutex> lk(r.mu);
    probe_locked(r);
    if (r.have_cuda && nbytes >= (size_t(1) << 16)) {
      auto it = r.pin_cache.find(sz);
      if (it != r.pin_cache.end() && !it->second.empty()) {
        void *p = it->second.back();
        it->second.pop_back();
        r.pin_cached_bytes -= sz;
        *pinned = true;
        return p;
      }
      void *p = nullptr;
      if (cudaHostAlloc(&p, sz, cudaHostAllocDefault) == cudaSuccess) {
        *pinned = true;
        return p;
      }
      cudaGetLastError();
    }
  }
  *pinned = false;
  void *p = ::malloc(sz);
  if (!p) fail_runtime("host allocation failed");
  return p;
}
void host_free(void *p, bool pinned, size_t nbytes) {
  if (!p) return;
  if (!pinned) {
    ::free(p);
    return;
  }
  // pinned blocks are cached by size like device blocks (cudaFreeHost is slow and synchronising),
  // up to a bound so that a long session does not pin the whole host.
  Runtime &r = rt();
  size_t sz = round_block(nbytes);
  {
    std::lock_guard<std::mutex> lk(r.mu);
    if (r.pin_cached_bytes + sz <= (size_t(8) << 30)) {
      r.pin_cache[sz].push_back(p);
      r.pin_cached_bytes += sz;
      return;
    }
  }
  cudaFreeHost(p);
}

// ------------------------------------------------------------------------------------------
nt_storage *storage_new(int64_t n, int dtype, int device) {
  if (n < 0) fail_invalid("Storage size must be non-negative.");
  if (device != NT_CPU && device != NT_CUDA) fail_invalid("Unknown device.");
  size_t nbytes = size_t(n) * size_t(dtype_itemsize(dtype));
  nt_storage *s = new nt_storage();
  s->n = n;
  s->dtype = dtype;
  s->device = device;
  try {
    if (device == NT_CUDA) {
      s->data = device_alloc(nbytes, &s->rounded);
    } else {
      s->data = host_alloc(nbytes, &s->pinned);
      s->rounded = nbytes;
    }
  } catch (...) {
    delete s;
    throw;
  }
  return s;
}
void storage_release(nt_storage *s) {
  if (!s) return;
  if (s->refs.fetch_sub(1, std::memory_order_acq_rel) == 1) {
    if (s->device == NT_CUDA) gemm_tc_forget(s);
    if (s->device == NT_CUDA)
      device_free(s->data, s->rounded);
    else
      host_free(s->data, s->pinned, s->rounded);
    delete s;
  }
}

void check_view(const nt_view *v, const char *fname) {
  if (!v || !v->storage) fail_runtime(std::string(fname) + ": null view or storage.");
  if (v->ndim < 0 || v->ndim > NT_MAX_DIMS)
    fail_runtime(std::string(fname) + ": views of more than 8 dimensions are not supported on device.");
  int64_t lo = v->offset, hi = v->offset, n = 1;
  for (int i = 0; i < v->ndim; ++i) {
    if (v->shape[i] < 0) fail_runtime(std::string(fname) + ": negative extent.");
    n *= v->shape[i];
  }
  if (n == 0) return;
  for (int i = 0; i < v->ndim; ++i) {
    int64_t span = (v->shape[i] - 1) * v->strides[i];
    if (span < 0) lo += span; else hi += span;
  }
  if (lo < 0 || hi >= v->storage->n)
    fail_runtime(std::string(fname) + ": view exceeds its storage (index range [" + std::to_string(lo) + ", " +
                 std::to_string(hi) + "], capacity " + std::to_string(v->storage->n) + ").");
}
void require_cuda(const nt_view *v, const char *fname) {
  if (v->storage->device != NT_CUDA)
    fail_runtime(std::string(fname) + ": requires Cuda (this library has no CPU compute path).");
}
void require_same_shape(const nt_view *a, const nt_view *b, const char *fname) {
  bool same = a->ndim == b->ndim;
  for (int i = 0; same && i < a->ndim; ++i) same = a->shape[i] == b->shape[i];
  if (!same) fail_runtime(std::string(fname) + ": Expected two views of the same shape.");
}
void require_same_dtype(const nt_view *a, const nt_view *b, const char *fname) {
  if (a->storage->dtype != b->storage->dtype)
    fail_runtime(std::string(fname) + ": Expected two storages on the same dtype.");
}
void require_same_device(const nt_view *a, const nt_view *b, const char *fname) {
  if (a->storage->device != b->storage->device)
    fail_runtime(std::string(fname) + ": Expected two storages on the same device.");
}

// ------------------------------------------------------------------------------------------
// kernels of this file
template <class T> __global__ void fill_kernel(T *out, int64_t n, T value) {
  int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  int64_t step = int64_t(gridDim.x) * blockDim.x;
  for (; i < n; i += step) out[i] = value;
}

// Storage::cast semantics (src/cpp/storage.cpp:54-62): to Bool is `s != 0`, everything else static_cast
// -- which the reference always evaluates on the host, also for Cuda storages (it round-trips them).
// A floating-point value outside the integer type's range, or NaN, is undefined in C++; on the x86-64
// hosts the reference runs on the conversion instruction returns the "integer indefinite" value, the
// most negative integer, and that is what its tensors then hold.  The device's own conversion would
// saturate (and turn NaN into 0), so the range test is explicit here.
template <class S, class D> __device__ __forceinline__ D cast_value(S x) {
  if constexpr (std::is_same_v<D, bool>) {
    return x ? true : false;
  } else if constexpr (std::is_floating_point_v<S> && std::is_same_v<D, int32_t>) {
    return (x > S(-2147483649.0) && x < S(2147483648.0)) ? static_cast<int32_t>(x) : INT32_MIN;
  } else if constexpr (std::is_floating_point_v<S> && std::is_same_v<D, int64_t>) {
    return (x >= S(-9223372036854775808.0) && x < S(9223372036854775808.0)) ? static_cast<int64_t>(x) : INT64_MIN;
  } else {
    return static_cast<D>(x);
  }
}
template <class S, class D> __global__ void cast_kernel(const S *in, D *out, int64_t n) {
  int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  int64_t step = int64_t(gridDim.x) * blockDim.x;
  for (; i < n; i += step) out[i] = cast_value<S, D>(in[i]);
}

// eye(n): ones where row == column, i.e. at every (n + 1)-th element (src/cpp/factory.cu:51-59)
template <class T> __global__ void eye_kernel(T *out, int64_t n) {
  int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  int64_t step = int64_t(gridDim.x) * blockDim.x;
  for (; i < n * n; i += step) out[i] = static_cast<T>(i % (n + 1) == 0 ? 1 : 0);
}

// arange: static_cast<T>(start + i * step) in int64, as the reference's host loop (src/cpp/factory.cu:62-71)
template <class T> __global__ void arange_kernel(T *out, int64_t n, int64_t start, int64_t inc) {
  int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  int64_t step = int64_t(gridDim.x) * blockDim.x;
  for (; i < n; i += step) out[i] = static_cast<T>(start + i * inc);
}

// Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11):
// a counter-based generator -- block b of the stream is a pure function of (key, b), so every thread
// computes its own four words with no state shared between threads or launches.
__host__ __device__ inline void philox4x32_10(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  for (int round = 0; round < 10; ++round) {
    const uint64_t p0 = uint64_t(0xD2511F53u) * c[0];
    const uint64_t p1 = uint64_t(0xCD9E8D57u) * c[2];
    const uint32_t n0 = uint32_t(p1 >> 32) ^ c[1] ^ k0;
    const uint32_t n2 = uint32_t(p0 >> 32) ^ c[3] ^ k1;
    c[1] = uint32_t(p1);
    c[3] = uint32_t(p0);
    c[0] = n0;
    c[2] = n2;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

// U[0,1): float = top 24 bits * 2^-24 (4 per block); double = top 53 bits of two words * 2^-53 (2 per block)
template <class T> __global__ void philox_uniform_kernel(T *out, int64_t n, uint64_t seed, uint64_t offset) {
  constexpr int PER = std::is_same_v<T, float> ? 4 : 2;
  const int64_t blocks = (n + PER - 1) / PER;
  int64_t b = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t step = int64_t(gridDim.x) * blockDim.x;
  for (; b < blocks; b += step) {
    const uint64_t ctr = offset + uint64_t(b);
    uint32_t c[4] = {uint32_t(ctr), uint32_t(ctr >> 32), 0u, 0u};
    philox4x32_10(c, uint32_t(seed), uint32_t(seed >> 32));
    T v[PER];
    if constexpr (std::is_same_v<T, float>) {
      for (int j = 0; j < 4; ++j) v[j] = float(c[j] >> 8) * 5.9604644775390625e-08f;
    } else {
      for (int j = 0; j < 2; ++j)
        v[j] = double(((uint64_t(c[2 * j + 1]) << 32) | c[2 * j]) >> 11) * 1.1102230246251565e-16;
    }
    const int64_t at = b * PER;
    if (at + PER <= n) {
      if constexpr (std::is_same_v<T, float>)
        *reinterpret_cast<float4 *>(out + at) = make_float4(v[0], v[1], v[2], v[3]);
      else
        *reinterpret_cast<double2 *>(out + at) = make_double2(v[0], v[1]);
    } else {
      for (int j = 0; at + j < n; ++j) out[at + j] = v[j];
    }
  }
}

static int grid_for(int64_t n, int block) {
  int64_t g = ceil_div(n, block);
  int64_t cap = int64_t(sm_count()) * 16;
  return int(g < 1 ? 1 : (g > cap ? cap : g));
}

template <class T> static void fill_device(nt_storage *s, T value) {
  if (s->n == 0) return;
  fill_kernel<T><<<grid_for(s->n, 256), 256, 0, stream()>>>(static_cast<T *>(s->data), s->n, value);
  check_launch("fill");
}

template <class T> static T scalar_as(const nt_scalar *v) {
  switch (v->kind) {
  case 0: return static_cast<T>(v->i != 0);
  case 1: return static_cast<T>(v->i);
  case 2: return static_cast<T>(v->d);
  default: fail_type("Unknown scalar type.");
  }
}

static nt_storage *full_impl(int64_t n, const nt_scalar *value, int dtype, int device) {
  StorageRef out(storage_new(n, dtype, device));
  dispatch_all(dtype, [&]<class T>() {
    T v = scalar_as<T>(value);
    if (device == NT_CUDA) {
      fill_device<T>(out.s, v);
    } else {
      T *p = static_cast<T *>(out->data);
      for (int64_t i = 0; i < n; ++i) p[i] = v;
    }
  });
  return out.release();
}

static nt_storage *to_device_impl(nt_storage *s, int device) {
  if (s->device == device) {
    storage_retain(s);
    return s;
  }
  StorageRef out(storage_new(s->n, s->dtype, device));
  size_t nbytes = size_t(s->n) * dtype_itemsize(s->dtype);
  if (nbytes) {
    cudaStream_t st = stream();
    cudaMemcpyKind kind = (s->device == NT_CPU) ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost;
    NT_CUDA_CHECK(cudaMemcpyAsync(out->data, s->data, nbytes, kind, st));
    // The host side of either direction may be reused or read right after the call returns.
    NT_CUDA_CHECK(cudaStreamSynchronize(st));
    if (kind == cudaMemcpyDeviceToHost && !is_capturing()) check_device_errors(); // values are about to be read
  }
  return out.release();
}

} // namespace ntb

using namespace ntb;

extern "C" {

const char *nt_last_error(void) { return g_last_error.c_str(); }

int nt_is_cuda_available(void) {
  try {
    return cuda_ok() ? 1 : 0;
  } catch (...) {
    return 0;
  }
}

int nt_cuda_sync(void) {
  NT_API_BEGIN
  if (cuda_ok()) {
    NT_CUDA_CHECK(cudaStreamSynchronize(stream()));
    NT_CUDA_CHECK(cudaStreamSynchronize(comm_stream()));
    NT_CUDA_CHECK(cudaStreamSynchronize(update_stream()));
    NT_CUDA_CHECK(cudaStreamSynchronize(rt().copy));
    check_device_errors();
  }
  NT_API_END
}

int nt_set_device(int ordinal) {
  NT_API_BEGIN
  Runtime &r = rt();
  std::lock_guard<std::mutex> lk(r.mu);
  if (r.compute && r.device != ordinal) fail_runtime("nt_set_device: the device is already initialised.");
  probe_locked(r);
  if (!r.have_cuda) fail_runtime("nt_set_device: no CUDA device.");
  int count = 0;
  NT_CUDA_CHECK(cudaGetDeviceCount(&count));
  if (ordinal < 0 || ordinal >= count) fail_invalid("nt_set_device: ordinal out of range.");
  r.device = ordinal;
  NT_CUDA_CHECK(cudaSetDevice(ordinal));
  NT_API_END
}

int nt_device_count(int *out) {
  NT_API_BEGIN
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) {
    cudaGetLastError();
    count = 0;
  }
  *out = count;
  NT_API_END
}

void *nt_stream(void) {
  try {
    return (void *)stream();
  } catch (...) {
    return nullptr;
  }
}

int nt_launch_count(uint64_t *out) {
  NT_API_BEGIN
  *out = rt().launches.load();
  NT_API_END
}

int nt_allocator_stats(uint64_t *bytes_reserved, uint64_t *bytes_in_use, uint64_t *n_cuda_malloc) {
  NT_API_BEGIN
  Runtime &r = rt();
  std::lock_guard<std::mutex> lk(r.mu);
  if (bytes_reserved) *bytes_reserved = r.bytes_reserved;
  if (bytes_in_use) *bytes_in_use = r.bytes_in_use;
  if (n_cuda_malloc) *n_cuda_malloc = r.n_malloc;
  NT_API_END
}

int nt_allocator_requests(uint64_t *out) {
  NT_API_BEGIN
  Runtime &r = rt();
  std::lock_guard<std::mutex> lk(r.mu);
  *out = r.n_requests;
  NT_API_END
}

int nt_set_wait_limit_clocks(int64_t clocks) {
  NT_API_BEGIN
  if (clocks < 1000) fail_invalid("nt_set_wait_limit_clocks: at least 1000 clocks.");
  rt().wait_limit.store(clocks, std::memory_order_relaxed);
  NT_API_END
}
int64_t nt_get_wait_limit_clocks(void) { return rt().wait_limit.load(std::memory_order_relaxed); }

int nt_allocator_trim(void) {
  NT_API_BEGIN
  Runtime &r = rt();
  std::lock_guard<std::mutex> lk(r.mu);
  if (r.compute) NT_CUDA_CHECK(cudaStreamSynchronize(r.compute));
  trim_locked(r);
  NT_API_END
}

// ---------------------------------------------------------------- events, profiling
int nt_event_create(void **event) {
  NT_API_BEGIN
  stream();
  cudaEvent_t e;
  NT_CUDA_CHECK(cudaEventCreate(&e));
  *event = e;
  NT_API_END
}
int nt_event_record(void *event) {
  NT_API_BEGIN
  NT_CUDA_CHECK(cudaEventRecord(static_cast<cudaEvent_t>(event), stream()));
  NT_API_END
}
int nt_event_elapsed_ms(void *start, void *stop, float *ms) {
  NT_API_BEGIN
  NT_CUDA_CHECK(cudaEventSynchronize(static_cast<cudaEvent_t>(stop)));
  NT_CUDA_CHECK(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop)));
  NT_API_END
}
int nt_event_destroy(void *event) {
  NT_API_BEGIN
  if (event) NT_CUDA_CHECK(cudaEventDestroy(static_cast<cudaEvent_t>(event)));
  NT_API_END
}
int nt_matmul_profile_enable(int on) {
  NT_API_BEGIN
  stream();
  rt().mm_profile = on != 0;
  NT_API_END
}
int nt_matmul_profile_read(double *total_ms, int64_t *launches) {
  NT_API_BEGIN
  Runtime &r = rt();
  double total = 0.0;
  int64_t n = 0;
  for (auto &pr : r.mm_events) {
    float ms = 0.f;
    NT_CUDA_CHECK(cudaEventSynchronize(pr.second));
    NT_CUDA_CHECK(cudaEventElapsedTime(&ms, pr.first, pr.second));
    total += ms;
    r.event_pool.push_back(pr.first);
    r.event_pool.push_back(pr.second);
  }
  for (int c : r.mm_counts) n += c;
  r.mm_events.clear();
  r.mm_counts.clear();
  *total_ms = total;
  *launches = n;
  NT_API_END
}

// ---------------------------------------------------------------- CUDA graphs
int nt_graph_begin_capture(int *graph_id) {
  NT_API_BEGIN
  cudaStream_t st = stream();
  // state that kernels expect to find zeroed must exist before the capture starts: created inside
  // it, its zeroing would only be recorded, and eager launches issued before the first replay
  // would find it uninitialised
  reduce_prepare();
  gemm_tc_prepare();
  Runtime &r = rt();
  std::lock_guard<std::mutex> lk(r.mu);
  if (r.capturing) fail_runtime("nt_graph_begin_capture: a capture is already in progress.");
  if (r.mm_profile) fail_runtime("nt_graph_begin_capture: switch the matmul profile off first.");
  NT_CUDA_CHECK(cudaStreamBeginCapture(st, cudaStreamCaptureModeRelaxed));
  r.capturing = r.next_graph_id++;
  r.live_graphs.insert(r.capturing);
  *graph_id = r.capturing;
  NT_API_END
}
int nt_graph_end_capture(int graph_id) {
  NT_API_BEGIN
  Runtime &r = rt();
  std::lock_guard<std::mutex> lk(r.mu);
  if (r.capturing != graph_id || graph_id == 0) fail_runtime("nt_graph_end_capture: not the graph being captured.");
  r.capturing = 0;
  gemm_tc_new_epoch(); // what the captured calls "computed" does not exist on the device yet
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(r.compute, &graph);
  if (e != cudaSuccess || !graph) {
    r.live_graphs.erase(graph_id);
    fail_runtime(std::string("cudaStreamEndCapture failed: ") + cudaGetErrorString(e));
  }
  cudaGraphExec_t exec = nullptr;
  e = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) {
    r.live_graphs.erase(graph_id);
    fail_runtime(std::string("cudaGraphInstantiate failed: ") + cudaGetErrorString(e));
  }
  r.graph_exec[graph_id] = exec;
  NT_API_END
}
int nt_graph_launch(int graph_id) {
  NT_API_BEGIN
  cudaStream_t st = stream();
  Runtime &r = rt();
  auto it = r.graph_exec.find(graph_id);
  if (it == r.graph_exec.end()) fail_invalid("nt_graph_launch: unknown graph.");
  NT_CUDA_CHECK(cudaGraphLaunch(it->second, st));
  gemm_tc_new_epoch(); // the replay rewrites storages behind the host's counters
  count_launch();
  NT_API_END
}
int nt_graph_destroy(int graph_id) {
  NT_API_BEGIN
  Runtime &r = rt();
  std::lock_guard<std::mutex> lk(r.mu);
  graph_destroy_locked(r, graph_id);
  NT_API_END
}

int nt_storage_upload_async(nt_storage *dst, const void *host_src, int64_t nbytes) {
  NT_API_BEGIN
  if (dst->device != NT_CUDA) fail_runtime("nt_storage_upload_async: destination must be a Cuda storage.");
  if (nbytes < 0 || size_t(nbytes) > size_t(dst->n) * dtype_itemsize(dst->dtype))
    fail_runtime("nt_storage_upload_async: byte count exceeds the storage.");
  cudaStream_t st = stream();
  Runtime &r = rt();
  NT_CUDA_CHECK(cudaEventRecord(r.copy_gate, st));
  NT_CUDA_CHECK(cudaStreamWaitEvent(r.copy, r.copy_gate, 0));
  if (nbytes) NT_CUDA_CHECK(cudaMemcpyAsync(dst->data, host_src, size_t(nbytes), cudaMemcpyHostToDevice, r.copy));
  storage_touch(dst);
  NT_API_END
}
int nt_upload_fence(void) {
  NT_API_BEGIN
  cudaStream_t st = stream();
  Runtime &r = rt();
  NT_CUDA_CHECK(cudaEventRecord(r.copy_done, r.copy));
  NT_CUDA_CHECK(cudaStreamWaitEvent(st, r.copy_done, 0));
  NT_API_END
}
int nt_host_register(void *ptr, int64_t nbytes) {
  NT_API_BEGIN
  stream();
  NT_CUDA_CHECK(cudaHostRegister(ptr, size_t(nbytes), cudaHostRegisterDefault));
  NT_API_END
}
int nt_host_unregister(void *ptr) {
  NT_API_BEGIN
  NT_CUDA_CHECK(cudaHostUnregister(ptr));
  NT_API_END
}

// ---------------------------------------------------------------- storage
int nt_storage_allocate(int64_t n, int dtype, int device, nt_storage **out) {
  NT_API_BEGIN
  *out = storage_new(n, dtype, device);
  NT_API_END
}
int nt_storage_retain(nt_storage *s) {
  NT_API_BEGIN
  if (!s) fail_runtime("null storage");
  storage_retain(s);
  NT_API_END
}
int nt_storage_release(nt_storage *s) {
  NT_API_BEGIN
  storage_release(s);
  NT_API_END
}
int64_t nt_storage_size(const nt_storage *s) { return s->n; }
int64_t nt_storage_itemsize(const nt_storage *s) {
  try {
    return dtype_itemsize(s->dtype);
  } catch (...) {
    return 0;
  }
}
int nt_storage_dtype(const nt_storage *s) { return s->dtype; }
int nt_storage_device(const nt_storage *s) { return s->device; }
uint64_t nt_storage_version(const nt_storage *s) { return s->version; }
void *nt_storage_data(nt_storage *s) { return s->data; }

int nt_storage_clone(const nt_storage *s, nt_storage **out) {
  NT_API_BEGIN
  StorageRef o(storage_new(s->n, s->dtype, s->device));
  size_t nbytes = size_t(s->n) * dtype_itemsize(s->dtype);
  if (nbytes) {
    if (s->device == NT_CPU)
      std::memcpy(o->data, s->data, nbytes);
    else
      NT_CUDA_CHECK(cudaMemcpyAsync(o->data, s->data, nbytes, cudaMemcpyDeviceToDevice, stream()));
  }
  *out = o.release();
  NT_API_END
}

int nt_storage_to(nt_storage *s, int device, nt_storage **out) {
  NT_API_BEGIN
  if (device != NT_CPU && device != NT_CUDA) fail_invalid("Unknown device.");
  *out = to_device_impl(s, device);
  NT_API_END
}

int nt_storage_cast(nt_storage *s, int dtype, nt_storage **out) {
  NT_API_BEGIN
  dtype_itemsize(dtype);
  if (dtype == s->dtype) { // no copy on same dtype (src/cpp/storage.cpp:48-49)
    storage_retain(s);
    *out = s;
    return NT_OK;
  }
  StorageRef o(storage_new(s->n, dtype, s->device));
  if (s->n) {
    dispatch_all(s->dtype, [&]<class S>() {
      dispatch_all(dtype, [&]<class D>() {
        const S *in = static_cast<const S *>(s->data);
        D *dst = static_cast<D *>(o->data);
        if (s->device == NT_CUDA) {
          cast_kernel<S, D><<<grid_for(s->n, 256), 256, 0, stream()>>>(in, dst, s->n);
          check_launch("cast");
        } else {
          // host staging buffers only: the cast of a CPU storage is bookkeeping for tensor
          // construction (python scalars, index arrays), not a compute path.
          for (int64_t i = 0; i < s->n; ++i) {
            if constexpr (std::is_same_v<D, bool>)
              dst[i] = in[i] ? true : false;
            else
              dst[i] = static_cast<D>(in[i]);
          }
        }
      });
    });
  }
  *out = o.release();
  NT_API_END
}

int nt_storage_upload(nt_storage *dst, const void *host_src, int64_t nbytes) {
  NT_API_BEGIN
  if (nbytes < 0 || size_t(nbytes) > size_t(dst->n) * dtype_itemsize(dst->dtype))
    fail_runtime("nt_storage_upload: byte count exceeds the storage.");
  if (nbytes == 0) return NT_OK;
  if (dst->device == NT_CPU) {
    std::memcpy(dst->data, host_src, size_t(nbytes));
  } else {
    cudaStream_t st = stream();
    NT_CUDA_CHECK(cudaMemcpyAsync(dst->data, host_src, size_t(nbytes), cudaMemcpyHostToDevice, st));
    NT_CUDA_CHECK(cudaStreamSynchronize(st));
  }
  storage_touch(dst);
  NT_API_END
}

int nt_storage_download(const nt_storage *src, void *host_dst, int64_t nbytes) {
  NT_API_BEGIN
  if (nbytes < 0 || size_t(nbytes) > size_t(src->n) * dtype_itemsize(src->dtype))
    fail_runtime("nt_storage_download: byte count exceeds the storage.");
  if (nbytes == 0) return NT_OK;
  if (src->device == NT_CPU) {
    std::memcpy(host_dst, src->data, size_t(nbytes));
  } else {
    cudaStream_t st = stream();
    NT_CUDA_CHECK(cudaMemcpyAsync(host_dst, src->data, size_t(nbytes), cudaMemcpyDeviceToHost, st));
    NT_CUDA_CHECK(cudaStreamSynchronize(st));
    check_device_errors(); // the caller is about to read these values
  }
  NT_API_END
}

// ---------------------------------------------------------------- factories
int nt_zeros(int64_t n, int dtype, int device, nt_storage **out) {
  NT_API_BEGIN
  nt_scalar z{1, 0, 0.0};
  *out = full_impl(n, &z, dtype, device);
  NT_API_END
}
int nt_ones(int64_t n, int dtype, int device, nt_storage **out) {
  NT_API_BEGIN
  nt_scalar o{1, 1, 1.0};
  *out = full_impl(n, &o, dtype, device);
  NT_API_END
}
int nt_full(int64_t n, const nt_scalar *value, int dtype, int device, nt_storage **out) {
  NT_API_BEGIN
  *out = full_impl(n, value, dtype, device);
  NT_API_END
}

int nt_eye(int64_t n, int dtype, int device, nt_storage **out) {
  NT_API_BEGIN
  if (n < 0) fail_invalid("eye: negative size.");
  StorageRef o(storage_new(n * n, dtype, device));
  dispatch_all(dtype, [&]<class T>() {
    T *p = static_cast<T *>(o->data);
    if (device == NT_CUDA) {
      if (n > 0) {
        eye_kernel<T><<<grid_for(n * n, 256), 256, 0, stream()>>>(p, n);
        check_launch("eye");
      }
    } else {
      for (int64_t i = 0; i < n * n; ++i) p[i] = static_cast<T>(0);
      for (int64_t i = 0; i < n; ++i) p[i * n + i] = static_cast<T>(1);
    }
  });
  *out = o.release();
  NT_API_END
}

int nt_arange(int64_t n, int64_t start, int64_t step, int dtype, int device, nt_storage **out) {
  NT_API_BEGIN
  if (n < 0) fail_invalid("arange: negative size.");
  StorageRef o(storage_new(n, dtype, device));
  dispatch_all(dtype, [&]<class T>() {
    T *p = static_cast<T *>(o->data);
    if (device == NT_CUDA) {
      if (n > 0) {
        arange_kernel<T><<<grid_for(n, 256), 256, 0, stream()>>>(p, n, start, step);
        check_launch("arange");
      }
    } else {
      for (int64_t i = 0; i < n; ++i) p[i] = static_cast<T>(start + i * step);
    }
  });
  *out = o.release();
  NT_API_END
}

int nt_manual_seed(uint64_t seed) {
  NT_API_BEGIN
  rt().rng.seed(seed);
  rt().philox_seed = seed;
  rt().philox_offset = 0;
  NT_API_END
}

int nt_set_rng_mode(int mode) {
  NT_API_BEGIN
  if (mode != 0 && mode != 1) fail_invalid("nt_set_rng_mode: mode must be 0 (host mt19937_64) or 1 (device Philox4x32-10).");
  rt().rng_mode = mode;
  NT_API_END
}
int nt_get_rng_mode(void) { return rt().rng_mode; }

// Mode 0: the same host generator and distribution as the reference (src/cpp/random.h:6-9,
// factory.cu:73-83), so a seed reproduces the reference's parameter initialisation value for value.
// Mode 1 (Cuda storages): generated on the device, no host loop and no host-to-device copy.
int nt_uniform(int64_t n, int dtype, int device, nt_storage **out) {
  NT_API_BEGIN
  if (n < 0) fail_invalid("uniform: negative size.");
  if (rt().rng_mode == 1 && device == NT_CUDA) {
    StorageRef o(storage_new(n, dtype, NT_CUDA));
    dispatch_float(dtype, [&]<class T>() {
      constexpr int per = std::is_same_v<T, float> ? 4 : 2;
      const int64_t blocks = ceil_div(n, per);
      if (n > 0) {
        philox_uniform_kernel<T><<<grid_for(blocks, 256), 256, 0, stream()>>>(static_cast<T *>(o->data), n,
                                                                              rt().philox_seed, rt().philox_offset);
        check_launch("philox_uniform");
      }
      rt().philox_offset += uint64_t(blocks);
    });
    *out = o.release();
    return NT_OK;
  }
  StorageRef host(storage_new(n, dtype, NT_CPU));
  dispatch_float(dtype, [&]<class T>() {
    T *p = static_cast<T *>(host->data);
    std::uniform_real_distribution<T> dist(0.0, 1.0);
    auto &rng = rt().rng;
    for (int64_t i = 0; i < n; ++i) p[i] = static_cast<T>(dist(rng));
  });
  *out = to_device_impl(host.s, device);
  NT_API_END
}

} // extern "C"
