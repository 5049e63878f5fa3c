// Pointwise entry points of the C ABI: binary, comparison, unary, pow, in-place, strided copies,
// the fused backward kernels and the SGD update.  All arithmetic is compiled with FMA contraction
// off, so every functor rounds exactly where the reference's separate kernels round.
#include "elementwise.cuh"
#include "tanh_exact.h"
#include "cr_math.h"
#include "sigmoid_f32.h"

namespace ntb {

// =============================================================================================
// Functors.  `in_t`/`out_t` drive the launcher; bool arithmetic follows C++ integer promotion then
// conversion back to bool, as `static_cast<O>(func(T, T))` does in src/cpp/ops/binary_ops.cu:16.
#define NT_BINARY_FUNCTOR(name, expr)                                                              \
  template <class T> struct name {                                                                 \
    using in_t = T;                                                                                \
    using out_t = T;                                                                               \
    __device__ __forceinline__ T operator()(T a, T b) const { return static_cast<T>(expr); }      \
  };
NT_BINARY_FUNCTOR(AddF, a + b)
NT_BINARY_FUNCTOR(SubF, a - b)
NT_BINARY_FUNCTOR(MulF, a *b)
NT_BINARY_FUNCTOR(DivF, a / b)
NT_BINARY_FUNCTOR(SecondF, b) // copy_inplace: out <- other

#define NT_COMPARE_FUNCTOR(name, expr)                                                             \
  template <class T> struct name {                                                                 \
    using in_t = T;                                                                                \
    using out_t = bool;                                                                            \
    __device__ __forceinline__ bool operator()(T a, T b) const { return expr; }                    \
  };
NT_COMPARE_FUNCTOR(EqF, a == b)
NT_COMPARE_FUNCTOR(GtF, a > b)
NT_COMPARE_FUNCTOR(GeF, a >= b)

template <class T> struct IdentityF {
  using in_t = T;
  using out_t = T;
  __device__ __forceinline__ T operator()(T a) const { return a; }
};
template <class T> struct NegF {
  using in_t = T;
  using out_t = T;
  __device__ __forceinline__ T operator()(T a) const { return -a; }
};
// (a >= 0) ? a : 0  -- relu(-0.0) = -0.0, relu(NaN) = 0   (src/cpp/ops/unary_ops.cu:104)
template <class T> struct ReluF {
  using in_t = T;
  using out_t = T;
  __device__ __forceinline__ T operator()(T a) const { return (a >= T(0)) ? a : T(0); }
};
template <class T> struct SqrtF {
  using in_t = T;
  using out_t = T;
  __device__ __forceinline__ T operator()(T a) const {
    if constexpr (std::is_same_v<T, float>) return __fsqrt_rn(a);
    else return __dsqrt_rn(a);
  }
};

template <class T> struct ExpF {
  using in_t = T;
  using out_t = T;
  __device__ __forceinline__ T operator()(T a) const {
    // fp32: the CUDA library's expf (documented error <= 2 ulp; measured against the host libm on 2^24
    // N(0,1) and 2^24 U(-87,88) arguments: never more than 2 ulp apart), ~4x fewer issue slots than
    // the double-precision evaluation above
    if constexpr (std::is_same_v<T, float>) return expf(a);
    else return exp(a);
  }
};
template <class T> struct LogF {
  using in_t = T;
  using out_t = T;
  __device__ __forceinline__ T operator()(T a) const {
    if constexpr (std::is_same_v<T, float>) return logf(a);
    else return log(a);
  }
};
// T(1) / (T(1) + exp(-a)): three rounded steps (src/cpp/ops/unary_ops.cu:107)
template <class T> struct SigmoidF {
  using in_t = T;
  using out_t = T;
  __device__ __forceinline__ T operator()(T a) const {
    if constexpr (std::is_same_v<T, float>) return nt_sigmoid_f32(a); // the same three steps in fp32, see sigmoid_f32.h
    else return 1.0 / (1.0 + exp(-a));
  }
};

// ---- tanh, fp32, two modes (nt_set_tanh_mode):
//   0 (default)  correctly rounded through one double-precision evaluation (cr_math.h): within 2 ulp of
//                the host libm, ~100 thread instructions per element as measured;
//   1            bit for bit the host libm's algorithm (tanh_exact.h), ~130 instructions per element.
template <class T> struct TanhF {
  using in_t = T;
  using out_t = T;
  __device__ __forceinline__ T operator()(T a) const {
    if constexpr (std::is_same_v<T, float>) return nt_tanh_fast_f32(a);
    else return tanh(a);
  }
};
template <class T> struct TanhExactF {
  using in_t = T;
  using out_t = T;
  __device__ __forceinline__ T operator()(T a) const {
    if constexpr (std::is_same_v<T, float>) return nt_tanh_f32(a);
    else return tanh(a);
  }
};
static std::atomic<int> g_tanh_mode{0};

// ---- pow.  fp32: the small integer exponents that training uses are exact products / reciprocals
// (<= 1 ulp from a correctly rounded powf); any other exponent goes through double precision.
__device__ __forceinline__ float pow_f32(float a, float e, int special) {
  switch (special) {
  case 1: return 1.0f;
  case 2: return a;
  case 3: return a * a;
  case 4: return (a * a) * a;
  case 5: return 1.0f / a;
  case 6: {
    // a*a is a denormal (fewer than 24 significant bits) below |a| ~ 1.1e-19 while 1/a^2 is still
    // finite down to |a| ~ 5.4e-20, and a*a overflows above |a| ~ 1.8e19 while 1/a^2 is still a non-zero
    // denormal: both slivers take the double-precision quotient
    if (fabsf(a) < 1.1e-19f || fabsf(a) > 1.8e19f) return (float)(1.0 / ((double)a * (double)a));
    return 1.0f / (a * a);
  }
  default: return (float)pow((double)a, (double)e);
  }
}
inline int pow_special(float e) {
  if (e == 0.0f) return 1;
  if (e == 1.0f) return 2;
  if (e == 2.0f) return 3;
  if (e == 3.0f) return 4;
  if (e == -1.0f) return 5;
  if (e == -2.0f) return 6;
  return 0;
}
struct SquareF { // pow(x, 2.0f): the exponent training uses (the MSE loss), without the general path's registers
  using in_t = float;
  using out_t = float;
  __device__ __forceinline__ float operator()(float a) const { return a * a; }
};
template <class T> struct PowF {
  using in_t = T;
  using out_t = T;
  T value;
  int special;
  __device__ __forceinline__ T operator()(T a) const {
    if constexpr (std::is_integral_v<T>) { // square-and-multiply, src/cpp/ops/unary_ops.cu:40-49
      T r = 1, n = value;
      while (n > 0) {
        if (n & 1) r *= a;
        a *= a;
        n >>= 1;
      }
      return r;
    } else if constexpr (std::is_same_v<T, float>) {
      return pow_f32(a, value, special);
    } else {
      return pow(a, value);
    }
  }
};

// ---- fused backward functors (fp32).  Each line is one rounded kernel of the reference's chain.
struct ReluBwdF { // g * float(y > 0)
  using in_t = float;
  using out_t = float;
  __device__ __forceinline__ float operator()(float g, float y) const { return g * ((y > 0.0f) ? 1.0f : 0.0f); }
};
struct TanhBwdF { // g * (1 - t**2)
  using in_t = float;
  using out_t = float;
  __device__ __forceinline__ float operator()(float g, float t) const {
    float p = t * t;
    float q = 1.0f - p;
    return g * q;
  }
};
struct SigmoidBwdF { // (g * s) * (1 - s)
  using in_t = float;
  using out_t = float;
  __device__ __forceinline__ float operator()(float g, float s) const {
    float gs = g * s;
    float q = 1.0f - s;
    return gs * q;
  }
};
struct LogBwdF { // g * x**-1
  using in_t = float;
  using out_t = float;
  __device__ __forceinline__ float operator()(float g, float x) const { return g * (1.0f / x); }
};
struct SqrtBwdF { // (g * 0.5) * r**-1
  using in_t = float;
  using out_t = float;
  __device__ __forceinline__ float operator()(float g, float r) const { return (g * 0.5f) * (1.0f / r); }
};
struct PowBwdF { // (g * e) * x**(e-1)
  using in_t = float;
  using out_t = float;
  float e, em1;
  int special;
  __device__ __forceinline__ float operator()(float g, float x) const { return (g * e) * pow_f32(x, em1, special); }
};
struct DivBwdX2F { // ((-x1) / x2**2) * g
  using in_t = float;
  using out_t = float;
  __device__ __forceinline__ float operator()(float g, float x1, float x2) const {
    float d = x2 * x2;
    return ((-x1) / d) * g;
  }
};
// both gradients of a product / a quotient, each the reference's own expression (one rounding per step)
struct MulBwdBothF { // x2 * g, x1 * g                          autograd/ops_binary.py:150-156
  __device__ __forceinline__ void operator()(float g, float x1, float x2, float *d1, float *d2) const {
    *d1 = x2 * g;
    *d2 = x1 * g;
  }
};
struct DivBwdBothF { // g / x2, ((-x1) / x2**2) * g             autograd/ops_binary.py:192-202
  __device__ __forceinline__ void operator()(float g, float x1, float x2, float *d1, float *d2) const {
    *d1 = g / x2;
    float d = x2 * x2;
    *d2 = ((-x1) / d) * g;
  }
};
struct SgdF { // p - (g * lr)  [optionally (g * scale) first]
  using in_t = float;
  using out_t = float;
  float lr, scale;
  bool scaled;
  __device__ __forceinline__ float operator()(float p, float g) const {
    if (scaled) g = g * scale;
    return p - g * lr;
  }
};

// =============================================================================================
// Shared entry-point bodies
static void binary_checks(const nt_view *x1, const nt_view *x2, const char *fname) {
  check_view(x1, fname);
  check_view(x2, fname);
  require_same_shape(x1, x2, fname);
  require_same_device(x1, x2, fname);
  require_same_dtype(x1, x2, fname);
  require_cuda(x1, fname);
}

template <template <class> class F, bool ARITH_ONLY>
static nt_storage *binary_same_dtype(const nt_view *x1, const nt_view *x2) {
  binary_checks(x1, x2, "_dispatch_binary");
  const int dt = x1->storage->dtype;
  StorageRef out(storage_new(view_numel(*x1), dt, NT_CUDA));
  nt_view ov = fresh_view(out.s, *x1);
  auto run = [&]<class T>() {
    const nt_view *views[3] = {&ov, x1, x2};
    ew_launch<F<T>, 2>(F<T>{}, views);
  };
  if constexpr (ARITH_ONLY) dispatch_arith(dt, run);
  else dispatch_all(dt, run);
  return out.release();
}

template <template <class> class F> static nt_storage *compare_impl(const nt_view *x1, const nt_view *x2) {
  binary_checks(x1, x2, "_dispatch_binary");
  StorageRef out(storage_new(view_numel(*x1), NT_BOOL, NT_CUDA));
  nt_view ov = fresh_view(out.s, *x1);
  dispatch_all(x1->storage->dtype, [&]<class T>() {
    const nt_view *views[3] = {&ov, x1, x2};
    ew_launch<F<T>, 2>(F<T>{}, views);
  });
  return out.release();
}

template <template <class> class F, int FAMILY /*0 float, 1 arith*/> static nt_storage *unary_impl(const nt_view *x, const char *fname) {
  check_view(x, fname);
  require_cuda(x, fname);
  const int dt = x->storage->dtype;
  if (FAMILY == 0 && dt != NT_FLOAT32 && dt != NT_FLOAT64) fail_invalid("Invalid dtype.");
  if (FAMILY == 1 && dt == NT_BOOL) fail_invalid("Invalid dtype.");
  StorageRef out(storage_new(view_numel(*x), dt, NT_CUDA));
  nt_view ov = fresh_view(out.s, *x);
  auto run = [&]<class T>() {
    const nt_view *views[2] = {&ov, x};
    ew_launch<F<T>, 1>(F<T>{}, views);
  };
  if constexpr (FAMILY == 0) dispatch_float(dt, run);
  else dispatch_arith(dt, run);
  return out.release();
}

template <template <class> class F, bool ARITH_ONLY> static void inplace_impl(const nt_view *out, const nt_view *other) {
  const char *fname = "_dispatch_inplace_apply";
  check_view(out, fname);
  check_view(other, fname);
  require_same_device(out, other, fname);
  require_same_dtype(out, other, fname);
  require_same_shape(out, other, fname);
  require_cuda(out, fname);
  auto run = [&]<class T>() {
    const nt_view *views[3] = {out, out, other};
    ew_launch<F<T>, 2>(F<T>{}, views);
  };
  if constexpr (ARITH_ONLY) dispatch_arith(out->storage->dtype, run);
  else dispatch_all(out->storage->dtype, run);
  out->storage->version += 1;
  storage_touch(out->storage);
}

// fp32-only fused entry: every view must be Float32 on Cuda with the shape of `shape_of`.
static void fused_checks(const nt_view *const *views, int n, const char *fname) {
  for (int i = 0; i < n; ++i) {
    check_view(views[i], fname);
    require_cuda(views[i], fname);
    if (views[i]->storage->dtype != NT_FLOAT32) fail_invalid(std::string(fname) + ": Float32 only.");
    if (i) require_same_shape(views[0], views[i], fname);
  }
}
template <class F> static nt_storage *fused2(F f, const nt_view *a, const nt_view *b, const char *fname) {
  const nt_view *chk[2] = {a, b};
  fused_checks(chk, 2, fname);
  StorageRef out(storage_new(view_numel(*a), NT_FLOAT32, NT_CUDA));
  nt_view ov = fresh_view(out.s, *a);
  const nt_view *views[3] = {&ov, a, b};
  ew_launch<F, 2>(f, views);
  return out.release();
}

// A producer of GEMM operands (an activation, its gradient): a dense 2-D fp32 result, large enough for the
// tensor-core path, with rows that are whole 128-byte lines -- it writes its own TF32 planes (ew_contig_planes)
// and registers them in the operand-plane cache, so the products that follow find them ready.
std::atomic<int> g_tile_pipeline{1};
static std::atomic<int> g_producer_planes{1};
static bool dense_2d(const nt_view *v) {
  return v->ndim == 2 && v->strides[1] == 1 && v->strides[0] == v->shape[1] && v->storage->dtype == NT_FLOAT32 &&
         v->storage->device == NT_CUDA;
}
template <class F, int NIN> static nt_storage *produce_with_planes(F f, const nt_view *a, const nt_view *b) {
  if (!g_producer_planes.load() || nt_get_matmul_mode() != 1 || !dense_2d(a)) return nullptr;
  const int64_t R = a->shape[0], C = a->shape[1];
  if (C % 32 != 0 || R * C < (int64_t(1) << 20)) return nullptr;
  const float *pa = static_cast<const float *>(a->storage->data) + a->offset, *pb = nullptr;
  if (!aligned16(pa)) return nullptr;
  if constexpr (NIN == 2) {
    if (!dense_2d(b) || b->shape[0] != R || b->shape[1] != C) return nullptr;
    pb = static_cast<const float *>(b->storage->data) + b->offset;
    if (!aligned16(pb)) return nullptr;
  }
  StorageRef out(storage_new(R * C, NT_FLOAT32, NT_CUDA));
  float *hi = gemm_tc_adopt_planes(out.s, R, C);
  if (!hi) return nullptr;
  const int64_t n = R * C;
  ew_contig_planes<F, NIN><<<unsigned(ceil_div(n >> 2, 256 * 4)), 256, 0, stream()>>>(f, static_cast<float *>(out->data), pa, pb, n,
                                                                                      hi, hi + n);
  check_launch("ew_contig_planes");
  return out.release();
}

// equality flag for nt_equals
template <class T> struct NeqFlagF {
  using in_t = T;
  using out_t = T;
  int *flag;
  __device__ __forceinline__ T operator()(T a, T b) const {
    if (a != b) *flag = 1;
    return a;
  }
};

// Both gradients in one launch; *out1 stays NULL when the three views are not equally shaped dense fp32
// runs (the caller then composes the single-gradient kernels).
template <class F> static void binary_backward_both(F f, const nt_view *g, const nt_view *x1, const nt_view *x2,
                                                    nt_storage **out1, nt_storage **out2, const char *fname) {
  *out1 = *out2 = nullptr;
  const nt_view *chk[3] = {g, x1, x2};
  fused_checks(chk, 3, fname);
  const int64_t n = view_numel(*g);
  const float *p[3];
  for (int i = 0; i < 3; ++i) {
    int64_t acc = 1; // dense row-major?
    for (int d = chk[i]->ndim - 1; d >= 0; --d) {
      if (chk[i]->shape[d] != 1 && chk[i]->strides[d] != acc) return;
      acc *= chk[i]->shape[d];
    }
    p[i] = static_cast<const float *>(chk[i]->storage->data) + chk[i]->offset;
    if (!aligned16(p[i])) return;
  }
  if (n < 4) return;
  StorageRef o1(storage_new(n, NT_FLOAT32, NT_CUDA)), o2(storage_new(n, NT_FLOAT32, NT_CUDA));
  ew_contig_two<F><<<unsigned(ceil_div(n >> 2, 256 * 2)), 256, 0, stream()>>>(f, static_cast<float *>(o1->data),
                                                                            static_cast<float *>(o2->data), p[0], p[1], p[2], n);
  check_launch("ew_contig_two");
  *out1 = o1.release();
  *out2 = o2.release();
}

} // namespace ntb

using namespace ntb;

extern "C" {

int nt_add(const nt_view *x1, const nt_view *x2, nt_storage **out) {
  NT_API_BEGIN
  *out = binary_same_dtype<AddF, false>(x1, x2);
  NT_API_END
}
int nt_subtract(const nt_view *x1, const nt_view *x2, nt_storage **out) {
  NT_API_BEGIN
  *out = binary_same_dtype<SubF, false>(x1, x2);
  NT_API_END
}
int nt_multiply(const nt_view *x1, const nt_view *x2, nt_storage **out) {
  NT_API_BEGIN
  *out = binary_same_dtype<MulF, false>(x1, x2);
  NT_API_END
}
int nt_divide(const nt_view *x1, const nt_view *x2, nt_storage **out) {
  NT_API_BEGIN
  *out = binary_same_dtype<DivF, true>(x1, x2);
  NT_API_END
}
int nt_pw_equal(const nt_view *x1, const nt_view *x2, nt_storage **out) {
  NT_API_BEGIN
  *out = compare_impl<EqF>(x1, x2);
  NT_API_END
}
int nt_pw_greater(const nt_view *x1, const nt_view *x2, nt_storage **out) {
  NT_API_BEGIN
  *out = compare_impl<GtF>(x1, x2);
  NT_API_END
}
int nt_pw_greater_eq(const nt_view *x1, const nt_view *x2, nt_storage **out) {
  NT_API_BEGIN
  *out = compare_impl<GeF>(x1, x2);
  NT_API_END
}

int nt_equals(const nt_view *x1, const nt_view *x2, int *result) {
  NT_API_BEGIN
  check_view(x1, "equals");
  check_view(x2, "equals");
  require_same_shape(x1, x2, "equals");
  require_same_dtype(x1, x2, "equals");
  require_same_device(x1, x2, "equals");
  require_cuda(x1, "equals");
  // one int of device scratch from the arena; the compare kernel writes its first input back
  // into a throw-away buffer only to reuse the launcher (n is small wherever this is used).
  StorageRef flag(storage_new(1, NT_INT32, NT_CUDA));
  NT_CUDA_CHECK(cudaMemsetAsync(flag->data, 0, sizeof(int), stream()));
  StorageRef sink(storage_new(view_numel(*x1), x1->storage->dtype, NT_CUDA));
  nt_view sv = fresh_view(sink.s, *x1);
  dispatch_all(x1->storage->dtype, [&]<class T>() {
    const nt_view *views[3] = {&sv, x1, x2};
    ew_launch<NeqFlagF<T>, 2>(NeqFlagF<T>{static_cast<int *>(flag->data)}, views);
  });
  int host = 0;
  NT_CUDA_CHECK(cudaMemcpyAsync(&host, flag->data, sizeof(int), cudaMemcpyDeviceToHost, stream()));
  NT_CUDA_CHECK(cudaStreamSynchronize(stream()));
  *result = (host == 0) ? 1 : 0;
  NT_API_END
}

int nt_exp(const nt_view *x, nt_storage **out) {
  NT_API_BEGIN
  *out = unary_impl<ExpF, 0>(x, "exp");
  NT_API_END
}
int nt_log(const nt_view *x, nt_storage **out) {
  NT_API_BEGIN
  *out = unary_impl<LogF, 0>(x, "log");
  NT_API_END
}
int nt_sqrt(const nt_view *x, nt_storage **out) {
  NT_API_BEGIN
  *out = unary_impl<SqrtF, 0>(x, "sqrt");
  NT_API_END
}
int nt_tanh(const nt_view *x, nt_storage **out) {
  NT_API_BEGIN
  check_view(x, "tanh");
  if (g_tanh_mode.load() == 0 && (*out = produce_with_planes<TanhF<float>, 1>(TanhF<float>{}, x, nullptr))) return NT_OK;
  *out = (g_tanh_mode.load() == 1) ? unary_impl<TanhExactF, 0>(x, "tanh") : unary_impl<TanhF, 0>(x, "tanh");
  NT_API_END
}
int nt_set_transposed_tile_pipeline(int on) {
  NT_API_BEGIN
  g_tile_pipeline.store(on ? 1 : 0);
  NT_API_END
}
int nt_set_producer_planes(int on) {
  NT_API_BEGIN
  g_producer_planes.store(on ? 1 : 0);
  NT_API_END
}
int nt_set_tanh_mode(int mode) {
  NT_API_BEGIN
  if (mode != 0 && mode != 1) fail_invalid("tanh mode must be 0 (correctly rounded) or 1 (bit-exact host libm).");
  g_tanh_mode.store(mode);
  NT_API_END
}
int nt_get_tanh_mode(void) { return g_tanh_mode.load(); }
int nt_sigmoid(const nt_view *x, nt_storage **out) {
  NT_API_BEGIN
  *out = unary_impl<SigmoidF, 0>(x, "sigmoid");
  NT_API_END
}
int nt_neg(const nt_view *x, nt_storage **out) {
  NT_API_BEGIN
  *out = unary_impl<NegF, 1>(x, "neg");
  NT_API_END
}
int nt_relu(const nt_view *x, nt_storage **out) {
  NT_API_BEGIN
  *out = unary_impl<ReluF, 1>(x, "relu");
  NT_API_END
}

int nt_pow(const nt_view *x, const nt_scalar *exponent, nt_storage **out) {
  NT_API_BEGIN
  check_view(x, "pow");
  require_cuda(x, "pow");
  if (!exponent || exponent->kind < 0 || exponent->kind > 2) fail_type("Unknown scalar type.");
  const int dt = x->storage->dtype;
  if (dt == NT_BOOL) fail_invalid("Invalid dtype.");
  StorageRef o(storage_new(view_numel(*x), dt, NT_CUDA));
  nt_view ov = fresh_view(o.s, *x);
  dispatch_arith(dt, [&]<class T>() {
    T v = (exponent->kind == 2) ? static_cast<T>(exponent->d) : static_cast<T>(exponent->i);
    PowF<T> f{v, 0};
    const nt_view *views[2] = {&ov, x};
    if constexpr (std::is_same_v<T, float>) {
      f.special = pow_special(v);
      if (f.special == 3) {
        ew_launch<SquareF, 1>(SquareF{}, views);
        return;
      }
    }
    ew_launch<PowF<T>, 1>(f, views);
  });
  *out = o.release();
  NT_API_END
}

int nt_add_inplace(const nt_view *out, const nt_view *other) {
  NT_API_BEGIN
  inplace_impl<AddF, false>(out, other);
  NT_API_END
}
int nt_sub_inplace(const nt_view *out, const nt_view *other) {
  NT_API_BEGIN
  inplace_impl<SubF, false>(out, other);
  NT_API_END
}
int nt_mul_inplace(const nt_view *out, const nt_view *other) {
  NT_API_BEGIN
  inplace_impl<MulF, false>(out, other);
  NT_API_END
}
int nt_div_inplace(const nt_view *out, const nt_view *other) {
  NT_API_BEGIN
  inplace_impl<DivF, true>(out, other);
  NT_API_END
}
int nt_copy_inplace(const nt_view *out, const nt_view *other) {
  NT_API_BEGIN
  inplace_impl<SecondF, false>(out, other);
  NT_API_END
}

int nt_copy_view(const nt_view *src, const nt_view *out) {
  NT_API_BEGIN
  const char *fname = "copy_view";
  check_view(src, fname);
  check_view(out, fname);
  require_same_shape(src, out, fname);
  require_same_dtype(src, out, fname);
  require_same_device(src, out, fname);
  require_cuda(src, fname);
  dispatch_all(src->storage->dtype, [&]<class T>() {
    const nt_view *views[2] = {out, src};
    ew_launch<IdentityF<T>, 1>(IdentityF<T>{}, views);
  });
  storage_touch(out->storage);
  // no version bump: the reference's copy_view leaves Storage::version alone (only the *_inplace
  // family bumps it, src/cpp/ops/inplace_ops.cu:60)
  NT_API_END
}

int nt_clone_contiguous_view_from(const nt_view *src, nt_storage **out) {
  NT_API_BEGIN
  const char *fname = "clone_contiguous_view_from";
  check_view(src, fname);
  require_cuda(src, fname);
  StorageRef o(storage_new(view_numel(*src), src->storage->dtype, NT_CUDA));
  nt_view ov = fresh_view(o.s, *src);
  dispatch_all(src->storage->dtype, [&]<class T>() {
    const nt_view *views[2] = {&ov, src};
    ew_launch<IdentityF<T>, 1>(IdentityF<T>{}, views);
  });
  *out = o.release();
  NT_API_END
}

// ---------------------------------------------------------------- fused backward
int nt_relu_backward(const nt_view *g, const nt_view *y, nt_storage **out) {
  NT_API_BEGIN
  *out = fused2(ReluBwdF{}, g, y, "relu_backward");
  NT_API_END
}
int nt_tanh_backward(const nt_view *g, const nt_view *t, nt_storage **out) {
  NT_API_BEGIN
  {
    const nt_view *chk[2] = {g, t};
    fused_checks(chk, 2, "tanh_backward");
  }
  if ((*out = produce_with_planes<TanhBwdF, 2>(TanhBwdF{}, g, t))) return NT_OK;
  *out = fused2(TanhBwdF{}, g, t, "tanh_backward");
  NT_API_END
}
int nt_sigmoid_backward(const nt_view *g, const nt_view *s, nt_storage **out) {
  NT_API_BEGIN
  *out = fused2(SigmoidBwdF{}, g, s, "sigmoid_backward");
  NT_API_END
}
int nt_exp_backward(const nt_view *g, const nt_view *e, nt_storage **out) {
  NT_API_BEGIN
  *out = fused2(MulF<float>{}, g, e, "exp_backward");
  NT_API_END
}
int nt_log_backward(const nt_view *g, const nt_view *x, nt_storage **out) {
  NT_API_BEGIN
  *out = fused2(LogBwdF{}, g, x, "log_backward");
  NT_API_END
}
int nt_sqrt_backward(const nt_view *g, const nt_view *r, nt_storage **out) {
  NT_API_BEGIN
  *out = fused2(SqrtBwdF{}, g, r, "sqrt_backward");
  NT_API_END
}
int nt_pow_backward(const nt_view *g, const nt_view *x, float exponent, nt_storage **out) {
  NT_API_BEGIN
  // exponent - 1 is computed in fp32 as the reference does on its 0-d tensors
  float em1 = exponent - 1.0f;
  *out = fused2(PowBwdF{exponent, em1, pow_special(em1)}, g, x, "pow_backward");
  NT_API_END
}
int nt_div_backward_x2(const nt_view *g, const nt_view *x1, const nt_view *x2, nt_storage **out) {
  NT_API_BEGIN
  const nt_view *chk[3] = {g, x1, x2};
  fused_checks(chk, 3, "div_backward_x2");
  StorageRef o(storage_new(view_numel(*g), NT_FLOAT32, NT_CUDA));
  nt_view ov = fresh_view(o.s, *g);
  const nt_view *views[4] = {&ov, g, x1, x2};
  ew_launch<DivBwdX2F, 3>(DivBwdX2F{}, views);
  *out = o.release();
  NT_API_END
}

int nt_mul_backward(const nt_view *g, const nt_view *x1, const nt_view *x2, nt_storage **dx1, nt_storage **dx2) {
  NT_API_BEGIN
  binary_backward_both(MulBwdBothF{}, g, x1, x2, dx1, dx2, "mul_backward");
  NT_API_END
}
int nt_div_backward(const nt_view *g, const nt_view *x1, const nt_view *x2, nt_storage **dx1, nt_storage **dx2) {
  NT_API_BEGIN
  binary_backward_both(DivBwdBothF{}, g, x1, x2, dx1, dx2, "div_backward");
  NT_API_END
}

int nt_sgd_update(const nt_view *param, const nt_view *grad, float lr, float grad_scale) {
  NT_API_BEGIN
  const nt_view *chk[2] = {param, grad};
  fused_checks(chk, 2, "sgd_update");
  const SgdF f{lr, grad_scale, grad_scale != 1.0f};
  // A weight that has been a matmul operand: its TF32 planes follow the update.  When the parameter is the whole
  // of a dense 2-D storage the update writes them itself (20 bytes per element in one launch instead of 12 + 12
  // in two); otherwise the cached views are split again behind the update.
  if (g_producer_planes.load() && nt_get_matmul_mode() == 1 && dense_2d(param) && dense_2d(grad) && param->offset == 0 &&
      param->shape[0] * param->shape[1] == param->storage->n) {
    const int64_t R = param->shape[0], C = param->shape[1], n = R * C;
    float *pp = static_cast<float *>(param->storage->data);
    const float *pg = static_cast<const float *>(grad->storage->data) + grad->offset;
    float *hi = (n >= 4 && aligned16(pp) && aligned16(pg)) ? gemm_tc_refresh_target(param->storage, R, C) : nullptr;
    if (hi) {
      ew_contig_planes<SgdF, 2><<<unsigned(ceil_div(n >> 2, 256 * 4)), 256, 0, stream()>>>(f, pp, pp, pg, n, hi, hi + n);
      check_launch("ew_contig_planes");
      param->storage->version += 1;
      storage_touch(param->storage);
      gemm_tc_mark_refreshed(param->storage);
      return NT_OK;
    }
  }
  const nt_view *views[3] = {param, param, grad};
  ew_launch<SgdF, 2>(f, views);
  param->storage->version += 1;
  storage_touch(param->storage);
  gemm_tc_refresh(param->storage);
  NT_API_END
}

} // extern "C"
