/*
 * nt_oracle.c -- CPU restatement of the reference's op kernels.  TEST INFRASTRUCTURE ONLY.
 *
 * Nothing shipped may link, import or call this file: it is the checker that the CUDA library is
 * compared against (tests/, the smoke check, and the cpu_baseline leg of the benchmark).
 *
 * Each function restates, in plain C, the single-threaded CPU loop the reference runs for the same
 * call, and cites it.  Pinned against the reference itself: tests/golden/*.npz holds outputs of the
 * reference's own Python package + native module on seeded inputs (tests/golden/make_golden.py),
 * and tests/test_oracle.py requires this file to reproduce them bit for bit; where the reference's
 * native module is present (oracle/_ref, built by oracle/Makefile) the two are also compared
 * directly on random views.
 *
 * Build: gcc -O2 -std=c11 -fPIC -shared -ffp-contract=off nt_oracle.c -lm   (see Makefile).
 * -ffp-contract=off and no -ffast-math: the reference is built without FMA contraction on x86-64
 * (no -march flags in its CMakeLists), so multiply and add round separately.
 * Transcendentals resolve to the host libm exactly as the reference's std::exp/log/pow/tanh do
 * (src/cpp/ops/unary_ops.cu:56,101-107).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#define NTO_MAX_DIMS 8

typedef struct {
  int32_t ndim;
  int64_t shape[NTO_MAX_DIMS];
  int64_t strides[NTO_MAX_DIMS]; /* elements */
  int64_t offset;                /* elements */
} nto_view;

/* src/cpp/tensor_view.cuh:43-52 -- linear index -> storage index, innermost dim fastest */
static int64_t unravel(int64_t i, const nto_view *v) {
  int64_t idx = v->offset;
  for (int j = v->ndim - 1; j >= 0; --j) {
    int64_t coord = i % v->shape[j];
    i /= v->shape[j];
    idx += coord * v->strides[j];
  }
  return idx;
}
static int64_t numel(const nto_view *v) {
  int64_t n = 1;
  for (int j = 0; j < v->ndim; ++j) n *= v->shape[j];
  return n;
}

/* ---------------------------------------------------------------- binary
 * src/cpp/ops/binary_ops.cu:6-20 (_cpu_binary_op_generic) with the functors of :107-113 */
enum { NTO_ADD = 0, NTO_SUB = 1, NTO_MUL = 2, NTO_DIV = 3, NTO_EQ = 4, NTO_GT = 5, NTO_GE = 6 };

int nto_binary_f32(int op, const float *a, const nto_view *va, const float *b, const nto_view *vb, float *out) {
  int64_t n = numel(va);
  for (int64_t i = 0; i < n; ++i) {
    float x = a[unravel(i, va)], y = b[unravel(i, vb)];
    switch (op) {
    case NTO_ADD: out[i] = x + y; break;
    case NTO_SUB: out[i] = x - y; break;
    case NTO_MUL: out[i] = x * y; break;
    case NTO_DIV: out[i] = x / y; break;
    default: return 1;
    }
  }
  return 0;
}
int nto_compare_f32(int op, const float *a, const nto_view *va, const float *b, const nto_view *vb, uint8_t *out) {
  int64_t n = numel(va);
  for (int64_t i = 0; i < n; ++i) {
    float x = a[unravel(i, va)], y = b[unravel(i, vb)];
    switch (op) {
    case NTO_EQ: out[i] = (x == y); break;
    case NTO_GT: out[i] = (x > y); break;
    case NTO_GE: out[i] = (x >= y); break;
    default: return 1;
    }
  }
  return 0;
}

/* ---------------------------------------------------------------- in-place
 * src/cpp/ops/inplace_ops.cu:6-16 (_cpu_inplace_apply), functors :75-79; NTO_COPY = `b` */
enum { NTO_COPY = 7 };
int nto_inplace_f32(int op, float *out, const nto_view *vo, const float *other, const nto_view *vx) {
  int64_t n = numel(vo);
  for (int64_t i = 0; i < n; ++i) {
    int64_t io = unravel(i, vo);
    float a = out[io], b = other[unravel(i, vx)];
    switch (op) {
    case NTO_ADD: out[io] = a + b; break;
    case NTO_SUB: out[io] = a - b; break;
    case NTO_MUL: out[io] = a * b; break;
    case NTO_DIV: out[io] = a / b; break;
    case NTO_COPY: out[io] = b; break;
    default: return 1;
    }
  }
  return 0;
}

/* ---------------------------------------------------------------- unary
 * src/cpp/ops/unary_ops.cu:6-17 (_cpu_unary_op_generic), functors :101-107, PowOp :50-57 */
enum { NTO_EXP = 0, NTO_LOG = 1, NTO_NEG = 2, NTO_RELU = 3, NTO_SQRT = 4, NTO_TANH = 5, NTO_SIGMOID = 6, NTO_POW = 7 };

int nto_unary_f32(int op, const float *x, const nto_view *vx, float *out, double pow_value) {
  int64_t n = numel(vx);
  const float e = (float)pow_value; /* Scalar::item<float>() */
  for (int64_t i = 0; i < n; ++i) {
    float a = x[unravel(i, vx)];
    switch (op) {
    case NTO_EXP: out[i] = expf(a); break;
    case NTO_LOG: out[i] = logf(a); break;
    case NTO_NEG: out[i] = -a; break;
    case NTO_RELU: out[i] = (a >= 0) ? a : 0; break;
    case NTO_SQRT: out[i] = sqrtf(a); break;
    case NTO_TANH: out[i] = tanhf(a); break;
    case NTO_SIGMOID: out[i] = 1.0f / (1.0f + expf(-a)); break;
    case NTO_POW: out[i] = powf(a, e); break;
    default: return 1;
    }
  }
  return 0;
}

/* ---------------------------------------------------------------- reductions
 * src/cpp/ops/reduction_ops.cu:52-83 (_generic_reduction_cpu) + the view split of :174-220.
 * The accumulator is an (index, value) item; neutral values and the combiner are those of
 * :13-50 (max: lowest(), min: max(), ties keep the lower index; sum: 0). */
enum { NTO_SUM = 0, NTO_MAX = 1, NTO_MIN = 2, NTO_ARGMAX = 3, NTO_ARGMIN = 4 };

static void split_views(const nto_view *x, const int64_t *axes, int n_axes, nto_view *keep, nto_view *drop) {
  keep->ndim = 0;
  keep->offset = x->offset;
  drop->ndim = 0;
  drop->offset = 0;
  for (int p = 0; p < x->ndim; ++p) {
    int dropped = 0;
    for (int a = 0; a < n_axes; ++a) dropped |= (axes[a] == p);
    if (!dropped) {
      keep->shape[keep->ndim] = x->shape[p];
      keep->strides[keep->ndim] = x->strides[p];
      keep->ndim++;
    }
  }
  /* dropped dims are visited in the order the caller listed them (src/cpp/ops/reduction_ops.cu:213-217) */
  for (int a = 0; a < n_axes; ++a) {
    drop->shape[drop->ndim] = x->shape[axes[a]];
    drop->strides[drop->ndim] = x->strides[axes[a]];
    drop->ndim++;
  }
}

int nto_reduce_f32(int op, const float *x, const nto_view *vx, const int64_t *axes, int n_axes, float *out_value,
                   int64_t *out_index) {
  nto_view keep, drop;
  split_views(vx, axes, n_axes, &keep, &drop);
  int64_t n_keep = numel(&keep), n_drop = numel(&drop);
  for (int64_t i = 0; i < n_keep; ++i) {
    int64_t base = unravel(i, &keep);
    int64_t acc_idx;
    float acc;
    switch (op) {
    case NTO_SUM: acc_idx = -1; acc = 0.0f; break;
    case NTO_MAX: case NTO_ARGMAX: acc_idx = INT64_MAX; acc = -3.402823466e+38f; break;
    case NTO_MIN: case NTO_ARGMIN: acc_idx = INT64_MAX; acc = 3.402823466e+38f; break;
    default: return 1;
    }
    for (int64_t j = 0; j < n_drop; ++j) {
      float v = x[base + unravel(j, &drop)];
      if (op == NTO_SUM) {
        acc = acc + v;
      } else if (op == NTO_MAX || op == NTO_ARGMAX) {
        if (!(acc > v || (acc == v && acc_idx < j))) { acc = v; acc_idx = j; }
      } else {
        if (!(acc < v || (acc == v && acc_idx < j))) { acc = v; acc_idx = j; }
      }
    }
    if (out_value) out_value[i] = acc;
    if (out_index) out_index[i] = acc_idx;
  }
  return 0;
}

/* ---------------------------------------------------------------- matmul
 * src/cpp/ops/matmul.cu:21-57 (_cpu_matmul): per output element, acc += A*B for c = 0..K-1,
 * separate multiply and add, batch dims share coordinates between the operands. */
int nto_matmul_f32(const float *A, const nto_view *va, const float *B, const nto_view *vb, float *C) {
  int nd = va->ndim;
  if (nd != vb->ndim || nd < 2) return 1;
  int64_t M = va->shape[nd - 2], K = va->shape[nd - 1], N = vb->shape[nd - 1];
  if (vb->shape[nd - 2] != K) return 1;
  int64_t batch = 1;
  for (int d = 0; d < nd - 2; ++d) batch *= va->shape[d];
  int64_t loc[NTO_MAX_DIMS] = {0};
  int64_t total = batch * M * N;
  for (int64_t ci = 0; ci < total; ++ci) {
    float acc = 0.0f;
    int64_t base1 = va->offset + loc[nd - 2] * va->strides[nd - 2];
    int64_t base2 = vb->offset + loc[nd - 1] * vb->strides[nd - 1];
    for (int d = 0; d < nd - 2; ++d) {
      base1 += va->strides[d] * loc[d];
      base2 += vb->strides[d] * loc[d];
    }
    for (int64_t c = 0; c < K; ++c) acc += A[base1 + c * va->strides[nd - 1]] * B[base2 + c * vb->strides[nd - 2]];
    C[ci] = acc;
    /* odometer over the output shape (batch..., M, N) */
    for (int j = nd - 1; j >= 0; --j) {
      int64_t extent = (j == nd - 1) ? N : (j == nd - 2) ? M : va->shape[j];
      if (++loc[j] < extent) break;
      loc[j] = 0;
    }
  }
  return 0;
}

/* ---------------------------------------------------------------- strided copy
 * src/cpp/ops/copy_ops.cu (clone_contiguous_view_from): out[i] = src[unravel(i)] */
int nto_clone_f32(const float *x, const nto_view *vx, float *out) {
  int64_t n = numel(vx);
  for (int64_t i = 0; i < n; ++i) out[i] = x[unravel(i, vx)];
  return 0;
}

/* ---------------------------------------------------------------- RNG
 * src/cpp/random.h:6-12 + src/cpp/factory.cu:73-83: std::mt19937_64 seeded by manual_seed,
 * std::uniform_real_distribution<float>(0,1).  mt19937_64 is the published 64-bit Mersenne Twister
 * (Matsumoto & Nishimura; parameters fixed by the C++ standard, [rand.predef]).  libstdc++'s
 * generate_canonical<float,24> draws ONE 64-bit word per float: float(word) / 2^64, and returns
 * nextafter(1,0) when that rounds to 1. */
#define MT_N 312
#define MT_M 156
typedef struct {
  uint64_t mt[MT_N];
  int idx;
} nto_rng;

void nto_rng_seed(nto_rng *r, uint64_t seed) {
  r->mt[0] = seed;
  for (int i = 1; i < MT_N; ++i) r->mt[i] = 6364136223846793005ULL * (r->mt[i - 1] ^ (r->mt[i - 1] >> 62)) + (uint64_t)i;
  r->idx = MT_N;
}
static uint64_t rng_next(nto_rng *r) {
  if (r->idx >= MT_N) {
    const uint64_t upper = 0xFFFFFFFF80000000ULL, lower = 0x7FFFFFFFULL, a = 0xB5026F5AA96619E9ULL;
    for (int i = 0; i < MT_N; ++i) {
      uint64_t x = (r->mt[i] & upper) | (r->mt[(i + 1) % MT_N] & lower);
      r->mt[i] = r->mt[(i + MT_M) % MT_N] ^ (x >> 1) ^ ((x & 1) ? a : 0);
    }
    r->idx = 0;
  }
  uint64_t x = r->mt[r->idx++];
  x ^= (x >> 29) & 0x5555555555555555ULL;
  x ^= (x << 17) & 0x71D67FFFEDA60000ULL;
  x ^= (x << 37) & 0xFFF7EEE000000000ULL;
  x ^= (x >> 43);
  return x;
}
void nto_uniform_f32(nto_rng *r, float *out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    float u = (float)rng_next(r) / 18446744073709551616.0f;
    if (u >= 1.0f) u = nextafterf(1.0f, 0.0f);
    out[i] = u;
  }
}
int64_t nto_rng_sizeof(void) { return (int64_t)sizeof(nto_rng); }

/* ---------------------------------------------------------------- index-array gather / scatter
 * src/cpp/ops/copy_ops.cu:85-160 (gather_from_axes) and :7-83 (scatter_to_axes): an odometer walks
 * the iteration space (the result shape for gather, the source shape for scatter) in row-major
 * order; each iteration axis either drives one axis of the (equally shaped) index arrays or one
 * basic dim of the indexed operand; the coordinate of an indexed dim is read from its index array.
 * Indices arrive already wrapped and range-checked (the reference's Python layer does that,
 * src/nanotorch/core.py:712-718).  Elements are copied as `itemsize` raw bytes (DispatchAll there).
 * Scatter visits the source in row-major order, so of several writers to one destination the last
 * one wins. */
typedef struct {
  const int64_t *data; /* Int64 index array storage */
  nto_view view;
} nto_index_array;

static void index_walk(int scatter, int itemsize, const char *lin_data, const nto_view *lin, char *ix_data_w,
                       const char *ix_data_r, const nto_view *ix, const int64_t *fancy_dims, int n_fancy,
                       const nto_index_array *ind, const uint8_t *axis_is_fancy, const int64_t *axis_target,
                       char *lin_data_w) {
  int64_t pos[NTO_MAX_DIMS] = {0};         /* odometer over the iteration space */
  int64_t ix_basic[NTO_MAX_DIMS] = {0};    /* coordinates of the indexed operand's basic dims */
  int64_t ind_coord[NTO_MAX_DIMS] = {0};   /* coordinates into the index arrays */
  int fancy_slot[NTO_MAX_DIMS];
  for (int d = 0; d < NTO_MAX_DIMS; ++d) fancy_slot[d] = -1;
  for (int q = 0; q < n_fancy; ++q) fancy_slot[fancy_dims[q]] = q;
  const int64_t n = numel(lin);
  for (int64_t it = 0; it < n; ++it) {
    for (int a = 0; a < lin->ndim; ++a) {
      if (axis_is_fancy[a]) ind_coord[axis_target[a]] = pos[a];
      else ix_basic[axis_target[a]] = pos[a];
    }
    int64_t at_lin = lin->offset;
    for (int a = 0; a < lin->ndim; ++a) at_lin += lin->strides[a] * pos[a];
    int64_t at_ix = ix->offset;
    for (int d = 0; d < ix->ndim; ++d) {
      int64_t coord = ix_basic[d];
      const int q = fancy_slot[d];
      if (q >= 0) {
        int64_t flat = ind[q].view.offset;
        for (int k = 0; k < ind[q].view.ndim; ++k) flat += ind[q].view.strides[k] * ind_coord[k];
        coord = ind[q].data[flat];
      }
      at_ix += ix->strides[d] * coord;
    }
    if (scatter) memcpy(ix_data_w + at_ix * itemsize, lin_data + at_lin * itemsize, (size_t)itemsize);
    else memcpy(lin_data_w + at_lin * itemsize, ix_data_r + at_ix * itemsize, (size_t)itemsize);
    for (int a = lin->ndim - 1; a >= 0; --a) {
      if (++pos[a] < lin->shape[a]) break;
      pos[a] = 0;
    }
  }
}

/* out: contiguous buffer of prod(out_view->shape) elements; out_view carries the result shape with
 * contiguous strides and offset 0. */
int nto_gather_from_axes(int itemsize, const void *x, const nto_view *vx, void *out, const nto_view *out_view,
                         const int64_t *fancy_dims, int n_fancy, const nto_index_array *ind,
                         const uint8_t *axis_is_fancy, const int64_t *axis_target) {
  index_walk(0, itemsize, NULL, out_view, NULL, (const char *)x, vx, fancy_dims, n_fancy, ind, axis_is_fancy,
             axis_target, (char *)out);
  return 0;
}

int nto_scatter_to_axes(int itemsize, const void *src, const nto_view *vsrc, void *out, const nto_view *vout,
                        const int64_t *fancy_dims, int n_fancy, const nto_index_array *ind,
                        const uint8_t *axis_is_fancy, const int64_t *axis_target) {
  index_walk(1, itemsize, (const char *)src, vsrc, (char *)out, NULL, vout, fancy_dims, n_fancy, ind, axis_is_fancy,
             axis_target, NULL);
  return 0;
}

/* ---------------------------------------------------------------- Philox4x32-10
 * No counterpart in the reference (whose only generator is the host mt19937_64 above): the checker
 * of the library's optional device generator.  Published algorithm: Salmon, Moraes, Dror, Shaw,
 * "Parallel random numbers: as easy as 1, 2, 3" (SC'11), 10 rounds, multipliers 0xD2511F53 /
 * 0xCD9E8D57, Weyl key increments 0x9E3779B9 / 0xBB67AE85; pinned by the known-answer vectors
 * distributed with the authors' Random123 library (tests/test_rng_philox.py). */
void nto_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]) {
  uint32_t c0 = ctr[0], c1 = ctr[1], c2 = ctr[2], c3 = ctr[3], k0 = key[0], k1 = key[1];
  for (int r = 0; r < 10; ++r) {
    uint64_t a = (uint64_t)0xD2511F53u * c0, b = (uint64_t)0xCD9E8D57u * c2;
    uint32_t n0 = (uint32_t)(b >> 32) ^ c1 ^ k0, n2 = (uint32_t)(a >> 32) ^ c3 ^ k1;
    c1 = (uint32_t)b;
    c3 = (uint32_t)a;
    c0 = n0;
    c2 = n2;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

/* The library's stream layout: block b = philox(ctr = {lo(offset+b), hi(offset+b), 0, 0}, key = seed);
 * four floats per block, (word >> 8) * 2^-24. */
void nto_philox_uniform_f32(uint64_t seed, uint64_t offset, float *out, int64_t n) {
  for (int64_t b = 0; b * 4 < n; ++b) {
    uint64_t at = offset + (uint64_t)b;
    uint32_t ctr[4] = {(uint32_t)at, (uint32_t)(at >> 32), 0u, 0u}, key[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)}, w[4];
    nto_philox4x32_10(ctr, key, w);
    for (int j = 0; j < 4 && b * 4 + j < n; ++j) out[b * 4 + j] = (float)(w[j] >> 8) * 5.9604644775390625e-08f;
  }
}
void nto_philox_uniform_f64(uint64_t seed, uint64_t offset, double *out, int64_t n) {
  for (int64_t b = 0; b * 2 < n; ++b) {
    uint64_t at = offset + (uint64_t)b;
    uint32_t ctr[4] = {(uint32_t)at, (uint32_t)(at >> 32), 0u, 0u}, key[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)}, w[4];
    nto_philox4x32_10(ctr, key, w);
    for (int j = 0; j < 2 && b * 2 + j < n; ++j)
      out[b * 2 + j] = (double)((((uint64_t)w[2 * j + 1] << 32) | w[2 * j]) >> 11) * 1.1102230246251565e-16;
  }
}
