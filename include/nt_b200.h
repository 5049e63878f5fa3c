/*
 * nt_b200.h -- C ABI of the B200 (sm_100a) op-kernel library behind nanotorch's `_C` module.
 *
 * Every entry point mirrors one function or method of the reference's native module
 * (`PYBIND11_MODULE(_C, m)`, src/cpp/_C.cpp:12-24, typed in src/nanotorch/_C.pyi:1-136).  The
 * reference passes `TensorView` (storage + shape + strides + offset, strides in elements, 0 and
 * negative allowed; src/cpp/tensor_view.cuh:10-15) and returns a fresh `Storage`; this ABI passes
 * `const nt_view*` and returns `nt_storage*` through an out-parameter with an `int` status.
 *
 * Conventions
 *   - return value: NT_OK or an nt_status error class; the message is in nt_last_error()
 *     (thread-local).  The classes map one-to-one to the Python exception the reference raises:
 *     NT_ERR_RUNTIME -> RuntimeError (std::runtime_error, CUDA failures),
 *     NT_ERR_INVALID -> ValueError   (std::invalid_argument),
 *     NT_ERR_TYPE    -> TypeError    (py::type_error).
 *   - compute entry points accept CUDA storages only.  There is no CPU compute path in this
 *     library: a CPU storage handed to an op is NT_ERR_RUNTIME ("requires Cuda").  CPU storages
 *     exist as host staging buffers (construction, tolist/item, H2D/D2H).
 *   - all work is enqueued on one non-blocking stream owned by the library; calls return without
 *     synchronising unless stated; the sync entry point below waits for it.
 *   - storages are reference counted; every `nt_storage**` result carries one reference owned by
 *     the caller (release with nt_storage_release).
 *   - nothing here names a torch type.
 */
#ifndef NT_B200_H
#define NT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NT_MAX_DIMS 8 /* src/cpp/tensor_view.cuh:8 */

/* src/cpp/dtype.h:21 -- enum order is the promotion order. */
typedef enum { NT_BOOL = 0, NT_INT32 = 1, NT_INT64 = 2, NT_FLOAT32 = 3, NT_FLOAT64 = 4 } nt_dtype;
/* src/cpp/allocator.h:10 */
typedef enum { NT_CPU = 0, NT_CUDA = 1 } nt_device;

typedef enum {
  NT_OK = 0,
  NT_ERR_RUNTIME = 1, /* RuntimeError */
  NT_ERR_INVALID = 2, /* ValueError   */
  NT_ERR_TYPE = 3,    /* TypeError    */
  NT_ERR_INDEX = 4    /* IndexError (index-array entry points only) */
} nt_status;

/* Opaque, reference-counted flat typed buffer (src/cpp/storage.h:34-66). */
typedef struct nt_storage nt_storage;

/* Strided view (src/cpp/tensor_view.cuh:10-21). */
typedef struct {
  nt_storage *storage;
  int32_t ndim; /* 0..NT_MAX_DIMS */
  int64_t shape[NT_MAX_DIMS];
  int64_t strides[NT_MAX_DIMS]; /* in elements */
  int64_t offset;               /* in elements */
} nt_view;

/* Scalar argument of pow/full (src/cpp/storage.h:68-101): the Python bool/int/float variant. */
typedef struct {
  int32_t kind; /* 0 = bool, 1 = int64, 2 = double */
  int64_t i;
  double d;
} nt_scalar;

/* ------------------------------------------------------------------ errors, device, stream */
const char *nt_last_error(void);
int nt_is_cuda_available(void);       /* src/cpp/cuda.h:20-24 */
int nt_cuda_sync(void);               /* src/cpp/cuda.h:26 (cudaDeviceSynchronize there; the library stream here) */
int nt_set_device(int ordinal);       /* no counterpart: the reference never calls cudaSetDevice */
int nt_device_count(int *out);
void *nt_stream(void);                /* the cudaStream_t every kernel is launched on */
int nt_launch_count(uint64_t *out);   /* kernels launched by this library since load (bench evidence) */
int nt_allocator_stats(uint64_t *bytes_reserved, uint64_t *bytes_in_use, uint64_t *n_cuda_malloc);
int nt_allocator_trim(void);          /* return cached blocks to the driver */
int nt_allocator_requests(uint64_t *out); /* requests made to the device arena since load, cache hits included */

/* Every spin in device code (the mbarrier waits of the tensor-core GEMM pipeline) is bounded: past the
 * limit the kernel records which role gave up, stops issuing, and returns; the next synchronising call
 * (nt_cuda_sync, a download, to(Cpu)) reports it as NT_ERR_RUNTIME and clears it, and the context stays
 * usable.  No counterpart in the reference, whose kernels never wait on one another.  The limit is in SM
 * clocks, default 2^31 (about a second).  nt_wait_probe launches a one-thread kernel that waits, with
 * that same helper and limit, on a barrier nothing arrives on: the way to exercise the time-out path
 * without faulting or hanging anything. */
int nt_set_wait_limit_clocks(int64_t clocks);
int64_t nt_get_wait_limit_clocks(void);
int nt_wait_probe(void);

/* Timing on the library stream (no counterpart in the reference, which times with perf_counter
 * around a device sync, scripts/profile_ops.py:61-89). */
int nt_event_create(void **event);
int nt_event_record(void *event);                               /* on the compute stream */
int nt_event_elapsed_ms(void *start, void *stop, float *ms);    /* waits for `stop` */
int nt_event_destroy(void *event);
/* Per-launch timing of the matmul kernels: when enabled every matmul launch is bracketed by two
 * events; nt_matmul_profile_read waits for them and returns (and clears) their sum and count. */
int nt_matmul_profile_enable(int on);
int nt_matmul_profile_read(double *total_ms, int64_t *launches);

/* CUDA-graph capture of everything enqueued between begin and end (no counterpart in the reference,
 * whose ~40 launches per training step are issued one by one from Python).  Device blocks handed out
 * during the capture belong to the graph and are recycled only inside it, so replays never write
 * memory that eager work owns; they return to the general cache at nt_graph_destroy.  Do not call a
 * synchronising entry point (download, to(Cpu), equals, sync) or the matmul profile inside a capture.
 * Warm the step up once before capturing it: first-use set-up (streams, shared-memory opt-in, the
 * scratch counters) must not land inside the capture. */
int nt_graph_begin_capture(int *graph_id);
int nt_graph_end_capture(int graph_id);
int nt_graph_launch(int graph_id);      /* replay on the compute stream */
int nt_graph_destroy(int graph_id);

/* ------------------------------------------------------------------ storage (src/cpp/storage.cpp:4-70) */
int nt_storage_allocate(int64_t n, int dtype, int device, nt_storage **out); /* Storage::allocate */
int nt_storage_retain(nt_storage *s);
int nt_storage_release(nt_storage *s);
int64_t nt_storage_size(const nt_storage *s);
int64_t nt_storage_itemsize(const nt_storage *s);
int nt_storage_dtype(const nt_storage *s);
int nt_storage_device(const nt_storage *s);
uint64_t nt_storage_version(const nt_storage *s);
void *nt_storage_data(nt_storage *s);                 /* host or device pointer */
int nt_storage_clone(const nt_storage *s, nt_storage **out);            /* Storage::clone */
int nt_storage_to(nt_storage *s, int device, nt_storage **out);         /* Storage::to; same device -> same storage, retained */
int nt_storage_cast(nt_storage *s, int dtype, nt_storage **out);        /* Storage::cast; on device, no host round trip */
int nt_storage_upload(nt_storage *dst, const void *host_src, int64_t nbytes);   /* H2D (or memcpy for CPU storages) */
int nt_storage_download(const nt_storage *src, void *host_dst, int64_t nbytes); /* D2H, synchronises */
/* Overlapped input feed (no counterpart: the reference's Storage::to is a blocking cudaMemcpy).
 * The copy runs on a dedicated stream, ordered after everything enqueued on the compute stream so
 * far (so a buffer that an earlier step still reads is not overwritten early); `host_src` must be
 * pinned and stay valid until the fence.  nt_upload_fence makes the compute stream wait for every
 * copy issued so far. */
int nt_storage_upload_async(nt_storage *dst, const void *host_src, int64_t nbytes);
int nt_upload_fence(void);
int nt_host_register(void *ptr, int64_t nbytes);   /* pin caller-owned host memory (cudaHostRegister) */
int nt_host_unregister(void *ptr);

/* ------------------------------------------------------------------ factories (src/cpp/factory.cu:35-83) */
int nt_zeros(int64_t n, int dtype, int device, nt_storage **out);
int nt_ones(int64_t n, int dtype, int device, nt_storage **out);
int nt_full(int64_t n, const nt_scalar *value, int dtype, int device, nt_storage **out);
/* eye / arange are written by a kernel when device is Cuda (host loop + copy in the reference). */
int nt_eye(int64_t n, int dtype, int device, nt_storage **out);
int nt_arange(int64_t n, int64_t start, int64_t step, int dtype, int device, nt_storage **out);
int nt_manual_seed(uint64_t seed);                                       /* src/cpp/random.h:12; seeds both generators below */
/* U[0,1).  Generator mode 0 (default): the reference's host stream -- std::mt19937_64 through
 * std::uniform_real_distribution, then a host-to-device copy (src/cpp/factory.cu:73-83) -- so that a
 * seed reproduces the reference's values, parameter initialisation included.  Mode 1 (no counterpart
 * in the reference): Philox4x32-10 keyed by the seed, generated by a kernel straight into the Cuda
 * storage; consecutive calls continue one counter stream (4 floats or 2 doubles per 128-bit block,
 * a call starts on a fresh block); float = (word >> 8) * 2^-24, double = 53 bits of two words. */
int nt_uniform(int64_t n, int dtype, int device, nt_storage **out);
int nt_set_rng_mode(int mode);
int nt_get_rng_mode(void);

/* ------------------------------------------------------------------ pointwise binary (src/cpp/ops/binary_ops.cu:97-113) */
int nt_add(const nt_view *x1, const nt_view *x2, nt_storage **out);
int nt_subtract(const nt_view *x1, const nt_view *x2, nt_storage **out);
int nt_multiply(const nt_view *x1, const nt_view *x2, nt_storage **out);
int nt_divide(const nt_view *x1, const nt_view *x2, nt_storage **out);
int nt_pw_equal(const nt_view *x1, const nt_view *x2, nt_storage **out);      /* Bool output */
int nt_pw_greater(const nt_view *x1, const nt_view *x2, nt_storage **out);    /* Bool output */
int nt_pw_greater_eq(const nt_view *x1, const nt_view *x2, nt_storage **out); /* Bool output */
int nt_equals(const nt_view *x1, const nt_view *x2, int *out);                /* src/cpp/ops/binary_ops.cu:160-176; synchronises */

/* ------------------------------------------------------------------ pointwise unary (src/cpp/ops/unary_ops.cu:58-107) */
int nt_exp(const nt_view *x, nt_storage **out);
int nt_log(const nt_view *x, nt_storage **out);
int nt_sqrt(const nt_view *x, nt_storage **out);
int nt_tanh(const nt_view *x, nt_storage **out);
/* fp32 tanh mode.  0 (default): the correctly rounded value, by one double-precision evaluation --
 * within 2 ulp of the host libm's tanhf that the reference's CPU path calls (src/cpp/ops/unary_ops.cu:106).
 * 1: that libm's algorithm restated operation for operation -- bit-for-bit equal to the reference's CPU
 * result, at ~2.6x the instruction count. */
int nt_set_tanh_mode(int mode);
int nt_get_tanh_mode(void);
int nt_sigmoid(const nt_view *x, nt_storage **out);
int nt_neg(const nt_view *x, nt_storage **out);
int nt_relu(const nt_view *x, nt_storage **out);
int nt_pow(const nt_view *x, const nt_scalar *exponent, nt_storage **out);

/* ------------------------------------------------------------------ reductions (src/cpp/ops/reduction_ops.cu:225-259) */
int nt_sum(const nt_view *x, const int64_t *axes, int32_t n_axes, int dtype, nt_storage **out);
/* MeanOp's two kernels (sum, then a true division by the element count; autograd/ops_reduction.py:112-127)
 * in one launch for Float32 views: the rounded fp32 sum is divided by `count` where the reduction finishes,
 * same bits as nt_sum followed by nt_divide.  *out stays NULL when the view takes none of the single-launch
 * fp32 reduction kernels; the caller then composes the two steps. */
int nt_mean_f32(const nt_view *x, const int64_t *axes, int32_t n_axes, float count, nt_storage **out);
int nt_max(const nt_view *x, const int64_t *axes, int32_t n_axes, nt_storage **out);
int nt_min(const nt_view *x, const int64_t *axes, int32_t n_axes, nt_storage **out);
int nt_argmax(const nt_view *x, const int64_t *axes, int32_t n_axes, nt_storage **out); /* Int64 output */
int nt_argmin(const nt_view *x, const int64_t *axes, int32_t n_axes, nt_storage **out); /* Int64 output */

/* Row sums of a dense fp32 matrix, out[r] = sum_c in[r * row_len + c], that allocate nothing.
 * No counterpart in the reference.  For callers that must not let the library touch the device
 * allocator: a host runtime that handed all device memory to its own arena at start-up, or a
 * latency-critical loop in which cudaMalloc's device-wide synchronisation would stall every stream.
 * `in` and `out` are device pointers owned by the caller (n_rows * row_len and n_rows floats).  The
 * cross-CTA scratch of the reduction sits in a fixed 9 KB device array inside the library (held by
 * every GPU that loads it, until exit) instead of coming from the arena.  Rows are split over several
 * CTAs when there are too few of them to fill the GPU (fewer than 8 per SM) and they are longer than
 * 8192 elements; such a call may have at most 256 rows and 2048 partial sums, beyond that it is refused
 * with NT_ERR_INVALID -- use nt_sum for those.  Shapes that need no split have no limit.  The first call on a device looks up the array's device
 * address; make that first call before any stream capture.  All calls share the one array and each
 * leaves its partial sums behind: two calls that overlap on the GPU (different streams or
 * processes' threads) race; calls issued through this library's single stream do not.  The looked-up
 * address is cached per device without a lock: like the rest of the library (the allocator aside) the
 * entry point is for one calling thread at a time.  Runs on the library stream, asynchronously. */
int nt_sum_rows_noalloc(const float *in, int64_t n_rows, int64_t row_len, float *out);

/* ------------------------------------------------------------------ matmul (src/cpp/ops/matmul.cu:236-273) */
int nt_matmul(const nt_view *x1, const nt_view *x2, nt_storage **out);
/* x @ w + bias in one call (no single counterpart: nn.Linear.forward composes matmul and a broadcast add,
 * src/nanotorch/nn/module.py:64-76).  bias is 1-D with one fp32 value per output column.  Two rounded
 * steps, exactly as the composed form: the product rounded to fp32, then the sum with the bias rounded
 * again -- bit-identical to nt_matmul followed by nt_add.  In matmul mode 1 the second step runs in the
 * GEMM kernel's epilogue (no extra launch, no second pass over the output). */
int nt_linear(const nt_view *x, const nt_view *w, const nt_view *bias, nt_storage **out);
/* fp32 product mode.
 *   0  exact FP32 on the CUDA cores (FMA, sequential in k: the rounding of the reference's CUDA kernels);
 *   1  (default) 3xTF32 on the tcgen05 tensor cores with promoted accumulation: chains of 256 values of k
 *      accumulate in tensor memory, their sums are added round-to-nearest in registers -- the error of an
 *      ordinary fp32 summation (2e-6 of max|C| at K = 4096 and at K = 16384);
 *   2  FP32 on the CUDA cores with separate multiply and add, sequential in k: bit-for-bit the reference's
 *      CPU loop (src/cpp/ops/matmul.cu:31-45);
 *   3  3xTF32 with a single accumulation chain per output: ~1 % faster than mode 1; the tensor core's
 *      round-toward-zero accumulate then shows as a bias of 1e-5 of max|C| at K = 4096, 4e-5 at 16384. */
int nt_set_matmul_mode(int mode);
int nt_get_matmul_mode(void);
/* In modes 1 and 3 a product of at most this many multiply-adds (batch*M*N*K, default 2^21) takes the
 * exact FP32 kernel of mode 0 instead: that small, the tensor-core path's operand-split launches cost more
 * than they save, and tiny products keep the accuracy of the reference's CUDA kernels.  0 sends every fp32
 * product to the tensor cores. */
/* Mode 1 splits each fp32 operand into two TF32 planes (hi, lo) before the product.  natural != 0 (default):
 * the planes keep the operand's own row-major order whichever of its two matrix dims has unit stride -- the
 * kernel reads them K-major or MN-major -- so no operand is transposed on the way.  cached != 0 (default): the
 * planes are remembered per storage and view and reused until that storage is written again through any
 * entry point of this library (in-place ops, sgd_update, uploads, copy_view, scatter, all-reduce): an
 * activation is split once for the forward product and the weight-gradient product, a gradient once for
 * its two products; nt_sgd_update / nt_comm_sgd_update write the new planes of a weight that has been an operand
 * in the same pass (a dense 2-D parameter with whole 128-byte rows) or re-split it right behind the update.
 * Inside a graph capture cached planes are trusted only when they were split inside that capture or belong
 * to a parameter whose update keeps them current; everything else
 * (an input batch that an eager warm-up step had split) is split again inside the graph, so a replay reads
 * what the input buffers hold at that moment.  Do not write to a parameter from outside the graph between
 * replays other than through nt_sgd_update.  Each storage keeps at most 32 cached views.  Writes through
 * nt_storage_data() pointers are not seen.  nt_matmul_split_stats: operand-split launches and cache hits since load. */
int nt_set_matmul_operand_planes(int natural, int cached);
/* on != 0 (default): nt_tanh and nt_tanh_backward, when their result is a dense 2-D Float32 matrix of at
 * least 2^20 elements whose rows are whole 128-byte lines, also write the result's TF32 planes and register
 * them in the cache above -- an activation or its gradient is then never read back by an operand split.
 * Costs 8 extra bytes written per element if no product ever uses the result. */
int nt_set_producer_planes(int on);
/* on != 0 (default): an elementwise op on Float32 operands of at least 2^20 elements, one of which is
 * transposed over the last two dims (unit stride on the second-to-last), runs as a persistent kernel fed
 * by TMA loads and drained by TMA stores when every operand fits a tensor map (16-byte aligned base and
 * strides, no broadcast operand, at most one leading dim); 0: always the register-staged tile kernel.
 * Same result bits either way.  Replaces the strided path of src/cpp/ops/elementwise.cu for such views. */
int nt_set_transposed_tile_pipeline(int on);
int nt_matmul_split_stats(uint64_t *split_launches, uint64_t *cache_hits);
/* Scheduling of the mode-1 tensor-core kernel.  max_splits (1..8, default 8; NT_GEMM_SPLITK): a product with
 * so few output tiles that most SMs would idle (tiles x splits still within one wave of CTAs) is cut along k
 * into up to that many parts per tile, each at least 512 long; the parts' fp32 sums are added in part order
 * by the CTA that finishes last, so the result does not depend on timing.  1 = never.  panel (default 8;
 * NT_GEMM_PANEL): width in n-tiles of the panels the CTAs walk the output in, 0 = row by row. */
int nt_set_matmul_schedule(int max_splits, int panel);
/* Two independent products in one call, *out1 = a1 @ b1 and *out2 = a2 @ b2 -- what MatmulOp.backward computes
 * (autograd/ops_binary.py:253-267: g @ x2^T and x1^T @ g).  Same bits as two nt_matmul calls.  In mode 1, when the
 * second product's operand planes are already cached, its kernel can be launched as the programmatic dependent of
 * the first: its CTAs start on the SMs that the first product's last, partly filled wave leaves idle (256 tiles on
 * 148 SMs at a 2048-row batch) and wait for the first grid before they exit, so later work in the stream
 * still sees both complete.  The overlap is off by default (measured gain on the training step: 0.3-0.6 % at
 * 2048-4096 rows per GPU, none at 16384); nt_set_matmul_pair_overlap(1) or NT_GEMM_PAIR_OVERLAP=1 switches it on. */
int nt_matmul_pair(const nt_view *a1, const nt_view *b1, const nt_view *a2, const nt_view *b2, nt_storage **out1,
                   nt_storage **out2);
int nt_set_matmul_pair_overlap(int on);
int nt_set_matmul_tc_min_macs(int64_t macs);
int64_t nt_get_matmul_tc_min_macs(void);

/* ------------------------------------------------------------------ in-place (src/cpp/ops/inplace_ops.cu:75-79); bump the version */
int nt_add_inplace(const nt_view *out, const nt_view *other);
int nt_sub_inplace(const nt_view *out, const nt_view *other);
int nt_mul_inplace(const nt_view *out, const nt_view *other);
int nt_div_inplace(const nt_view *out, const nt_view *other);
int nt_copy_inplace(const nt_view *out, const nt_view *other);

/* ------------------------------------------------------------------ copies (src/cpp/ops/copy_ops.cu:172-217) */
int nt_copy_view(const nt_view *src, const nt_view *out);                    /* copy_view: strided -> strided; version untouched, as in the reference */
int nt_clone_contiguous_view_from(const nt_view *src, nt_storage **out);     /* also the materialising broadcast */

/* ------------------------------------------------------------------ index-array ("fancy") gather / scatter
 * src/cpp/ops/copy_ops.cu:85-160 (gather_from_axes) and :7-83 (scatter_to_axes), which the reference
 * implements for CPU storages only; argument meaning is the reference's:
 *   fancy_dims_in_src[p]   dim of the indexed tensor that index array p addresses;
 *   fancy_dims_data[p]     Int64 Cuda views, all of one (already broadcast) shape;
 *   out_axis_is_fancy[i], out_axis_target[i]   for axis i of the iteration space (the result shape
 *       for gather, the shape of `src` for scatter): an axis of the index arrays, or a basic dim of
 *       the indexed tensor.
 * Negative indices wrap.  Unless NT_INDEX_CHECKED is set, a pass over the index arrays first rejects
 * values outside [-extent, extent) with NT_ERR_INDEX before anything is written (the check the
 * reference's Python layer does on the host, src/nanotorch/core.py:712-718); that pass synchronises.
 * Scatter: where several source positions address one destination, the destination ends with the
 * value of the last of them in row-major order of `src`, as the reference's sequential loop leaves
 * it; NT_INDEX_UNIQUE (the caller vouches that destinations are distinct) skips the ordering pass
 * and its scratch (8 bytes per 16-byte destination item, 16 beyond 2^31 items).  Storage::version is not bumped, as in the
 * reference. */
#define NT_INDEX_CHECKED 1u
#define NT_INDEX_UNIQUE 2u
int nt_gather_from_axes(const nt_view *x, const int64_t *new_shape, int32_t new_ndim, const int64_t *fancy_dims_in_src,
                        int32_t n_fancy, const nt_view *fancy_dims_data, const uint8_t *out_axis_is_fancy,
                        const int64_t *out_axis_target, uint32_t flags, nt_storage **out);
int nt_scatter_to_axes(const nt_view *src, const nt_view *out, const int64_t *fancy_dims_in_src, int32_t n_fancy,
                       const nt_view *fancy_dims_data, const uint8_t *out_axis_is_fancy, const int64_t *out_axis_target,
                       uint32_t flags);

/* ------------------------------------------------------------------ fused backward kernels
 * No single counterpart in the reference: each replaces the chain of primitive kernels that the
 * reference's Python `backward` composes, and reproduces that chain's per-step fp32 rounding.
 * `g` is the upstream gradient view; results are fresh contiguous fp32 storages. */
int nt_relu_backward(const nt_view *g, const nt_view *y, nt_storage **out);    /* g * float(y > 0)             autograd/ops_unary.py:287-289 */
int nt_tanh_backward(const nt_view *g, const nt_view *t, nt_storage **out);    /* g * (1 - powf(t,2))          autograd/ops_unary.py:180-182 */
int nt_sigmoid_backward(const nt_view *g, const nt_view *s, nt_storage **out); /* (g*s) * (1 - s)              autograd/ops_unary.py:218-220 */
int nt_exp_backward(const nt_view *g, const nt_view *e, nt_storage **out);     /* g * e                        autograd/ops_unary.py:69-70   */
int nt_log_backward(const nt_view *g, const nt_view *x, nt_storage **out);     /* g * powf(x,-1)               autograd/ops_unary.py:105-106 */
int nt_sqrt_backward(const nt_view *g, const nt_view *r, nt_storage **out);    /* (g*0.5) * powf(r,-1)         autograd/ops_unary.py:142-144 */
int nt_pow_backward(const nt_view *g, const nt_view *x, float exponent, nt_storage **out); /* (g*e) * powf(x,e-1)  autograd/ops_unary.py:264-266 */
int nt_div_backward_x2(const nt_view *g, const nt_view *x1, const nt_view *x2, nt_storage **out); /* ((-x1)/powf(x2,2))*g  autograd/ops_binary.py:197-202 */
/* Both gradients of x1 * x2 (x2*g, x1*g; autograd/ops_binary.py:150-156) or of x1 / x2 (g/x2, ((-x1)/powf(x2,2))*g;
 * autograd/ops_binary.py:192-202) in one pass over g, x1, x2 -- 20 bytes per element instead of the 24 of two
 * launches.  For three equally shaped dense views; otherwise both results stay NULL and the caller composes
 * the single-gradient kernels. */
int nt_mul_backward(const nt_view *g, const nt_view *x1, const nt_view *x2, nt_storage **dx1, nt_storage **dx2);
int nt_div_backward(const nt_view *g, const nt_view *x1, const nt_view *x2, nt_storage **dx1, nt_storage **dx2);
/* Max/Min backward: g_expanded * mask where mask = (x == m_expanded) and zero on every tied slice
 * (integer-division quirk of the reference, autograd/ops_reduction.py:201-212, 275-286). */
int nt_extremum_backward(const nt_view *g_expanded, const nt_view *x, const nt_view *m_expanded,
                         const int64_t *axes, int32_t n_axes, nt_storage **out);
/* SGD update p <- p - (g*lr), the two rounded steps of `p -= p.grad * lr` (nn/optimizers.py:45-51); bumps the version.
 * `grad_scale` multiplies g first when != 1 (data-parallel mean over ranks). */
int nt_sgd_update(const nt_view *param, const nt_view *grad, float lr, float grad_scale);

/* ------------------------------------------------------------------ data-parallel exchange (NCCL; no counterpart in the reference) */
#define NT_COMM_ID_BYTES 128
int nt_comm_unique_id(uint8_t id[NT_COMM_ID_BYTES]);
/* The rendezvous waits for every rank; it is bounded: NT_ERR_RUNTIME after NT_COMM_TIMEOUT_MS (default
 * 300 000) or the explicit limit, instead of hanging on a rank that never joins.  NCCL is capped at 16 CTAs
 * per collective (they take whole SMs from the backward GEMMs they overlap); NT_NCCL_MAX_CTAS in the
 * environment overrides that, 0 leaves the choice to NCCL. */
int nt_comm_init(int rank, int world, const uint8_t id[NT_COMM_ID_BYTES]);
int nt_comm_init_timeout(int rank, int world, const uint8_t id[NT_COMM_ID_BYTES], int64_t timeout_ms);
/* A bucket: nt_comm_group_begin orders the communication stream after everything enqueued on the compute
 * stream so far; the all-reduces issued until nt_comm_group_end leave as one NCCL launch.  Works without
 * a communicator too (one rank): it then only orders the side stream. */
int nt_comm_group_begin(void);
int nt_comm_group_end(void);
int nt_comm_allreduce_sum(nt_storage *s);       /* in place, fp32, on the communication stream; ordered after prior work */
/* nt_sgd_update enqueued on the update stream (a third stream, of the lowest priority, so that its CTAs fill
 * idle SMs instead of delaying the GEMM tiles of the compute stream), behind the collectives issued so far
 * on the communication stream: the update of one layer overlaps the backward kernels of the layers below it.  The caller vouches that no kernel still
 * to be enqueued on the compute stream before the next nt_comm_wait reads the parameter. */
int nt_comm_sgd_update(const nt_view *param, const nt_view *grad, float lr, float grad_scale);
int nt_comm_wait(void);                         /* make the compute stream wait for the communication and update streams (device-side join) */
/* Host-side wait for the communication stream with a time limit.  Past it the communicator is aborted
 * (ncclCommAbort takes the stuck collective kernels down, so the stream drains) and NT_ERR_RUNTIME is
 * returned: a peer that died between steps shows up here instead of as a hang. */
int nt_comm_sync(int64_t timeout_ms);
int nt_comm_abort(void);
int nt_comm_destroy(void);

#ifdef __cplusplus
}
#endif
#endif /* NT_B200_H */
