// Reductions of the C ABI: sum / max / min / argmax / argmin over any set of axes of a strided view.
//
// fp32 sum/max/min take one of two single-launch kernels, both HBM-bound at 4 bytes per input
// element (the reference's accounting, autograd/ops_reduction.py:80-82):
//   reduce_rows  the dropped dims collapse to one unit-stride run (last-dim and full reductions):
//                128-bit loads, four accumulators per thread, warp shuffles, then shared memory
//                across the CTA's warps.  Long rows are split over several CTAs; each writes one
//                partial and the CTA that draws the last ticket folds the partials in index order
//                and writes the result -- one launch, deterministic, no (index,value) payload.
//   reduce_cols  the innermost kept dim has unit stride and one strided dim is dropped (dim-0
//                reductions, bias gradients): lanes run along the kept columns so every row read
//                is coalesced; row ranges are split over CTAs with the same ticket finish.
// Everything else (other dtypes, argmax/argmin, exotic views) takes reduce_generic, a direct
// restatement of the reference's combiner with its (index,value) items.
//
// Replaces _reduce_kernel/_extract_kernel and their multi-pass host loop
// (src/cpp/ops/reduction_ops.cu:86-171), which re-launches over 16-byte partial items, reads one
// element per thread for dim-1 and strides lanes by a whole row for dim-0.
#include <cuda/std/limits>

#include "elementwise.cuh"

namespace ntb {

// ---------------------------------------------------------------------------------------------
// fp32 combiners.  Neutral elements are the reference's: 0, lowest() and max() -- not infinities
// (src/cpp/ops/reduction_ops.cu:15-50), so max over an all -inf slice is -FLT_MAX there and here.
struct RSum {
  static __device__ __forceinline__ float neutral() { return 0.0f; }
  static __device__ __forceinline__ float combine(float a, float b) { return a + b; }
};
// NaN: the reference folds a slice sequentially and a NaN replaces the running extremum, only to be
// replaced itself by the next element, so its answer depends on where in the slice the NaN sits.  A
// parallel reduction cannot follow an order-dependent rule; fmaxf / fminf return the other operand when
// one is NaN, so the extremum of the non-NaN elements comes out whatever the order, and a slice of
// nothing but NaN gives the neutral element every accumulator starts from.  Of +0 and -0 the maximum is
// +0 and the minimum -0 (the reference keeps whichever comes first).
struct RMax {
  static __device__ __forceinline__ float neutral() { return -3.402823466e+38f; }
  static __device__ __forceinline__ float combine(float a, float b) { return fmaxf(a, b); }
};
struct RMin {
  static __device__ __forceinline__ float neutral() { return 3.402823466e+38f; }
  static __device__ __forceinline__ float combine(float a, float b) { return fminf(a, b); }
};

template <class Op> __device__ __forceinline__ float warp_reduce(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v = Op::combine(v, __shfl_xor_sync(0xffffffffu, v, s));
  return v;
}

struct KeepIndex { // kept dims of the input view, outermost first
  int ndim;
  int64_t shape[NT_MAX_DIMS];
  int64_t strides[NT_MAX_DIMS];
};
__device__ __forceinline__ int64_t keep_offset(const KeepIndex &k, int64_t lin) {
  int64_t off = 0;
  for (int d = k.ndim - 1; d >= 0; --d) {
    int64_t q = lin / k.shape[d];
    off += (lin - q * k.shape[d]) * k.strides[d];
    lin = q;
  }
  return off;
}

// ---------------------------------------------------------------------------------------------
// Row reduction.  Block b handles split (b % S) of row (b / S); elements [lo, hi) of the row.
template <class Op>
__global__ void __launch_bounds__(256) reduce_rows(const float *__restrict__ in, float *__restrict__ out,
                                                   float *__restrict__ partials, unsigned *__restrict__ tickets,
                                                   KeepIndex keep, int64_t L, int S, int64_t chunk, float divisor) {
  // divisor != 0: the finished value is divided by it (one IEEE division of the rounded fp32 result:
  // the bits of a sum kernel followed by a divide kernel -- MeanOp's two steps in one launch)
  __shared__ float warp_part[8];
  __shared__ bool is_last;
  const int64_t row = blockIdx.x / S;
  const int split = int(blockIdx.x - row * S);
  const float *p = in + keep_offset(keep, row);
  const int64_t lo = int64_t(split) * chunk;
  int64_t hi = lo + chunk;
  if (hi > L) hi = L;

  float a0 = Op::neutral(), a1 = Op::neutral(), a2 = Op::neutral(), a3 = Op::neutral();
  const bool aligned = ((reinterpret_cast<uintptr_t>(p) & 15) == 0); // lo is a multiple of 4
  if (aligned) {
    const int64_t nvec = (hi - lo) >> 2;
    const float4 *pv = reinterpret_cast<const float4 *>(p + lo);
    int64_t i = threadIdx.x;
    // four vectors in flight per thread
    for (; i + 3 * 256 < nvec; i += 4 * 256) {
      float4 v0 = __ldcs(pv + i), v1 = __ldcs(pv + i + 256), v2 = __ldcs(pv + i + 512), v3 = __ldcs(pv + i + 768);
      a0 = Op::combine(a0, Op::combine(Op::combine(v0.x, v0.y), Op::combine(v0.z, v0.w)));
      a1 = Op::combine(a1, Op::combine(Op::combine(v1.x, v1.y), Op::combine(v1.z, v1.w)));
      a2 = Op::combine(a2, Op::combine(Op::combine(v2.x, v2.y), Op::combine(v2.z, v2.w)));
      a3 = Op::combine(a3, Op::combine(Op::combine(v3.x, v3.y), Op::combine(v3.z, v3.w)));
    }
    for (; i < nvec; i += 256) {
      float4 v = __ldcs(pv + i);
      a0 = Op::combine(a0, Op::combine(Op::combine(v.x, v.y), Op::combine(v.z, v.w)));
    }
    for (int64_t j = lo + (nvec << 2) + threadIdx.x; j < hi; j += 256) a1 = Op::combine(a1, p[j]);
  } else {
    int64_t j = lo + threadIdx.x;
    for (; j + 3 * 256 < hi; j += 4 * 256) {
      float v0 = p[j], v1 = p[j + 256], v2 = p[j + 512], v3 = p[j + 768];
      a0 = Op::combine(a0, v0);
      a1 = Op::combine(a1, v1);
      a2 = Op::combine(a2, v2);
      a3 = Op::combine(a3, v3);
    }
    for (; j < hi; j += 256) a0 = Op::combine(a0, p[j]);
  }
  float v = Op::combine(Op::combine(a0, a1), Op::combine(a2, a3));
  v = warp_reduce<Op>(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) warp_part[warp] = v;
  __syncthreads();
  if (warp == 0) {
    v = (lane < 8) ? warp_part[lane] : Op::neutral();
    v = warp_reduce<Op>(v);
  }
  if (S == 1) {
    if (threadIdx.x == 0) out[row] = (divisor != 0.0f) ? v / divisor : v;
    return;
  }
  // single-pass grid finish
  if (threadIdx.x == 0) {
    partials[row * S + split] = v;
    __threadfence();
    unsigned t = atomicAdd(&tickets[row], 1u);
    is_last = (t == unsigned(S - 1));
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // fold the S partials in index order: fixed thread->index map, fixed tree => deterministic
  float acc = Op::neutral();
  for (int i = threadIdx.x; i < S; i += 256) acc = Op::combine(acc, __ldcg(partials + row * S + i));
  acc = warp_reduce<Op>(acc);
  if (lane == 0) warp_part[warp] = acc;
  __syncthreads();
  if (warp == 0) {
    acc = (lane < 8) ? warp_part[lane] : Op::neutral();
    acc = warp_reduce<Op>(acc);
    if (lane == 0) {
      out[row] = (divisor != 0.0f) ? acc / divisor : acc;
      tickets[row] = 0; // leave the counter ready for the next launch
    }
  }
}

// Short rows: a warp takes four rows at a time (their loads are issued together, so that a lane has four
// 128-bit loads in flight instead of one), 32 rows per CTA.
template <class Op>
__global__ void __launch_bounds__(256) reduce_rows_warp(const float *__restrict__ in, float *__restrict__ out,
                                                        KeepIndex keep, int64_t n_rows, int64_t L, float divisor) {
  const int64_t row0 = (int64_t(blockIdx.x) * 8 + (threadIdx.x >> 5)) * 4;
  if (row0 >= n_rows) return;
  const int lane = threadIdx.x & 31;
  const float *p[4];
  bool vec = true;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int64_t row = (row0 + r < n_rows) ? row0 + r : n_rows - 1; // a row past the end re-reads the last one, unused
    p[r] = in + keep_offset(keep, row);
    vec = vec && ((reinterpret_cast<uintptr_t>(p[r]) & 15) == 0);
  }
  float a[4] = {Op::neutral(), Op::neutral(), Op::neutral(), Op::neutral()};
  if (vec) {
    const int64_t nvec = L >> 2;
    for (int64_t i = lane; i < nvec; i += 32) {
      float4 v[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) v[r] = __ldcs(reinterpret_cast<const float4 *>(p[r]) + i);
#pragma unroll
      for (int r = 0; r < 4; ++r) a[r] = Op::combine(a[r], Op::combine(Op::combine(v[r].x, v[r].y), Op::combine(v[r].z, v[r].w)));
    }
    for (int64_t j = (nvec << 2) + lane; j < L; j += 32) {
#pragma unroll
      for (int r = 0; r < 4; ++r) a[r] = Op::combine(a[r], p[r][j]);
    }
  } else {
    for (int64_t j = lane; j < L; j += 32) {
#pragma unroll
      for (int r = 0; r < 4; ++r) a[r] = Op::combine(a[r], p[r][j]);
    }
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    a[r] = warp_reduce<Op>(a[r]);
    if (lane == 0 && row0 + r < n_rows) out[row0 + r] = (divisor != 0.0f) ? a[r] / divisor : a[r];
  }
}

// ---------------------------------------------------------------------------------------------
// Column reduction over a [Z][R][C] view with strides (keep-outer, sR, 1).
// grid.x = column tile, grid.y = row split, grid.z = outer kept index.  VEC = 4: a warp spans 128
// columns; VEC = 1: 32 columns.  The 8 warps of the CTA interleave over the rows of the split.
template <class Op, int VEC>
__global__ void __launch_bounds__(256) reduce_cols(const float *__restrict__ in, float *__restrict__ out,
                                                   float *__restrict__ partials, unsigned *__restrict__ tickets,
                                                   KeepIndex keep_outer, int64_t R, int64_t C, int64_t sR,
                                                   int64_t rows_per_split, float divisor) {
  constexpr int TW = 32 * VEC; // tile width in columns
  __shared__ float part[8][TW];
  __shared__ bool is_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t c0 = int64_t(blockIdx.x) * TW + lane * VEC;
  const int S = gridDim.y, split = blockIdx.y;
  const int64_t z = blockIdx.z;
  const float *base = in + keep_offset(keep_outer, z);
  int64_t r_lo = int64_t(split) * rows_per_split, r_hi = r_lo + rows_per_split;
  if (r_hi > R) r_hi = R;

  float acc[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) acc[e] = Op::neutral();
  if (c0 < C) {
    if constexpr (VEC == 4) {
      float4 b0, b1, b2, b3;
      int64_t r = r_lo + warp;
      for (; r + 24 < r_hi; r += 32) { // four rows in flight per thread
        b0 = __ldcs(reinterpret_cast<const float4 *>(base + r * sR + c0));
        b1 = __ldcs(reinterpret_cast<const float4 *>(base + (r + 8) * sR + c0));
        b2 = __ldcs(reinterpret_cast<const float4 *>(base + (r + 16) * sR + c0));
        b3 = __ldcs(reinterpret_cast<const float4 *>(base + (r + 24) * sR + c0));
        acc[0] = Op::combine(acc[0], Op::combine(Op::combine(b0.x, b1.x), Op::combine(b2.x, b3.x)));
        acc[1] = Op::combine(acc[1], Op::combine(Op::combine(b0.y, b1.y), Op::combine(b2.y, b3.y)));
        acc[2] = Op::combine(acc[2], Op::combine(Op::combine(b0.z, b1.z), Op::combine(b2.z, b3.z)));
        acc[3] = Op::combine(acc[3], Op::combine(Op::combine(b0.w, b1.w), Op::combine(b2.w, b3.w)));
      }
      for (; r < r_hi; r += 8) {
        b0 = __ldcs(reinterpret_cast<const float4 *>(base + r * sR + c0));
        acc[0] = Op::combine(acc[0], b0.x);
        acc[1] = Op::combine(acc[1], b0.y);
        acc[2] = Op::combine(acc[2], b0.z);
        acc[3] = Op::combine(acc[3], b0.w);
      }
    } else {
      int64_t r = r_lo + warp;
      for (; r + 24 < r_hi; r += 32) {
        float b0 = base[r * sR + c0], b1 = base[(r + 8) * sR + c0], b2 = base[(r + 16) * sR + c0],
              b3 = base[(r + 24) * sR + c0];
        acc[0] = Op::combine(acc[0], Op::combine(Op::combine(b0, b1), Op::combine(b2, b3)));
      }
      for (; r < r_hi; r += 8) acc[0] = Op::combine(acc[0], base[r * sR + c0]);
    }
  }
#pragma unroll
  for (int e = 0; e < VEC; ++e) part[warp][lane * VEC + e] = acc[e];
  __syncthreads();
  // 8 warps -> 1, in warp order; thread t owns column t of the tile
  float v = Op::neutral();
  const int64_t c = int64_t(blockIdx.x) * TW + threadIdx.x;
  const bool owner = (threadIdx.x < TW) && (c < C);
  if (threadIdx.x < TW) {
#pragma unroll
    for (int w = 0; w < 8; ++w) v = Op::combine(v, part[w][threadIdx.x]);
  }
  const int64_t out_base = z * C;
  if (S == 1) {
    if (owner) out[out_base + c] = (divisor != 0.0f) ? v / divisor : v;
    return;
  }
  if (owner) partials[(z * S + split) * C + c] = v;
  __threadfence();
  __syncthreads();
  const int64_t tile_id = z * gridDim.x + blockIdx.x;
  if (threadIdx.x == 0) {
    unsigned t = atomicAdd(&tickets[tile_id], 1u);
    is_last = (t == unsigned(S - 1));
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  if (owner) {
    float a = Op::neutral();
    for (int s = 0; s < S; ++s) a = Op::combine(a, __ldcg(partials + (z * S + s) * C + c));
    out[out_base + c] = (divisor != 0.0f) ? a / divisor : a;
  }
  if (threadIdx.x == 0) tickets[tile_id] = 0;
}

// Column reduction for wide matrices (C >= 1024, 128-bit alignment): a CTA streams whole 4 KB row segments --
// its 8 warps sit side by side, each thread owns 4 columns of every row of the CTA's row range, 8 rows in
// flight per thread -- so DRAM sees long sequential bursts instead of the 512-byte strips of reduce_cols, and
// no cross-warp step is needed.  grid.x = 1024-column tile, grid.y = row split, grid.z = outer kept index.
template <class Op>
__global__ void __launch_bounds__(256) reduce_cols_wide(const float *__restrict__ in, float *__restrict__ out,
                                                        float *__restrict__ partials, unsigned *__restrict__ tickets,
                                                        KeepIndex keep_outer, int64_t R, int64_t C, int64_t sR,
                                                        int64_t rows_per_split, float divisor) {
  __shared__ bool is_last;
  const int64_t c0 = int64_t(blockIdx.x) * 1024 + threadIdx.x * 4;
  const int S = gridDim.y, split = blockIdx.y;
  const int64_t z = blockIdx.z;
  const float *base = in + keep_offset(keep_outer, z) + c0;
  int64_t r_lo = int64_t(split) * rows_per_split, r_hi = r_lo + rows_per_split;
  if (r_hi > R) r_hi = R;
  const bool live = c0 < C; // C is a multiple of 4: a live thread owns 4 valid columns
  float4 acc = make_float4(Op::neutral(), Op::neutral(), Op::neutral(), Op::neutral());
  if (live) {
    int64_t r = r_lo;
    for (; r + 7 < r_hi; r += 8) {
      float4 b[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) b[u] = __ldcs(reinterpret_cast<const float4 *>(base + (r + u) * sR));
      // fixed tree over the 8 rows, then into the running value: the order never depends on the grid
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        b[u].x = Op::combine(b[u].x, b[u + 4].x);
        b[u].y = Op::combine(b[u].y, b[u + 4].y);
        b[u].z = Op::combine(b[u].z, b[u + 4].z);
        b[u].w = Op::combine(b[u].w, b[u + 4].w);
      }
      acc.x = Op::combine(acc.x, Op::combine(Op::combine(b[0].x, b[1].x), Op::combine(b[2].x, b[3].x)));
      acc.y = Op::combine(acc.y, Op::combine(Op::combine(b[0].y, b[1].y), Op::combine(b[2].y, b[3].y)));
      acc.z = Op::combine(acc.z, Op::combine(Op::combine(b[0].z, b[1].z), Op::combine(b[2].z, b[3].z)));
      acc.w = Op::combine(acc.w, Op::combine(Op::combine(b[0].w, b[1].w), Op::combine(b[2].w, b[3].w)));
    }
    for (; r < r_hi; ++r) {
      float4 b = __ldcs(reinterpret_cast<const float4 *>(base + r * sR));
      acc.x = Op::combine(acc.x, b.x);
      acc.y = Op::combine(acc.y, b.y);
      acc.z = Op::combine(acc.z, b.z);
      acc.w = Op::combine(acc.w, b.w);
    }
  }
  float *o = out + z * C + c0;
  if (S == 1) {
    if (live) {
      if (divisor != 0.0f) acc = make_float4(acc.x / divisor, acc.y / divisor, acc.z / divisor, acc.w / divisor);
      *reinterpret_cast<float4 *>(o) = acc;
    }
    return;
  }
  if (live) *reinterpret_cast<float4 *>(partials + (z * S + split) * C + c0) = acc;
  __threadfence();
  __syncthreads();
  const int64_t tile_id = z * gridDim.x + blockIdx.x;
  if (threadIdx.x == 0) {
    unsigned t = atomicAdd(&tickets[tile_id], 1u);
    is_last = (t == unsigned(S - 1));
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  if (live) {
    float4 a = make_float4(Op::neutral(), Op::neutral(), Op::neutral(), Op::neutral());
    const float *pp = partials + z * S * C + c0;
    int s = 0;
    for (; s + 3 < S; s += 4) { // partial sums in split order, four loads in flight
      float4 p0 = __ldcg(reinterpret_cast<const float4 *>(pp + int64_t(s) * C));
      float4 p1 = __ldcg(reinterpret_cast<const float4 *>(pp + int64_t(s + 1) * C));
      float4 p2 = __ldcg(reinterpret_cast<const float4 *>(pp + int64_t(s + 2) * C));
      float4 p3 = __ldcg(reinterpret_cast<const float4 *>(pp + int64_t(s + 3) * C));
      a.x = Op::combine(Op::combine(Op::combine(Op::combine(a.x, p0.x), p1.x), p2.x), p3.x);
      a.y = Op::combine(Op::combine(Op::combine(Op::combine(a.y, p0.y), p1.y), p2.y), p3.y);
      a.z = Op::combine(Op::combine(Op::combine(Op::combine(a.z, p0.z), p1.z), p2.z), p3.z);
      a.w = Op::combine(Op::combine(Op::combine(Op::combine(a.w, p0.w), p1.w), p2.w), p3.w);
    }
    for (; s < S; ++s) {
      float4 p0 = __ldcg(reinterpret_cast<const float4 *>(pp + int64_t(s) * C));
      a.x = Op::combine(a.x, p0.x);
      a.y = Op::combine(a.y, p0.y);
      a.z = Op::combine(a.z, p0.z);
      a.w = Op::combine(a.w, p0.w);
    }
    if (divisor != 0.0f) a = make_float4(a.x / divisor, a.y / divisor, a.z / divisor, a.w / divisor);
    *reinterpret_cast<float4 *>(o) = a;
  }
  if (threadIdx.x == 0) tickets[tile_id] = 0;
}

// ---------------------------------------------------------------------------------------------
// Generic path: the reference's (index, value) combiner, any dtype pair.
template <class O> struct Item {
  int64_t idx;
  O value;
};
struct GSum {
  static constexpr bool returns_idx = false;
  template <class O> static __device__ Item<O> neutral() { return Item<O>{-1, O(0)}; }
  template <class O> static __device__ Item<O> combine(Item<O> a, Item<O> b) { return Item<O>{-1, O(a.value + b.value)}; }
};
struct GArgMin {
  static constexpr bool returns_idx = true;
  template <class O> static __device__ Item<O> neutral() {
    return Item<O>{cuda::std::numeric_limits<int64_t>::max(), cuda::std::numeric_limits<O>::max()};
  }
  template <class O> static __device__ Item<O> combine(Item<O> a, Item<O> b) {
    return (a.value < b.value || (a.value == b.value && a.idx < b.idx)) ? a : b;
  }
};
struct GArgMax {
  static constexpr bool returns_idx = true;
  template <class O> static __device__ Item<O> neutral() {
    return Item<O>{cuda::std::numeric_limits<int64_t>::max(), cuda::std::numeric_limits<O>::lowest()};
  }
  template <class O> static __device__ Item<O> combine(Item<O> a, Item<O> b) {
    return (a.value > b.value || (a.value == b.value && a.idx < b.idx)) ? a : b;
  }
};
struct GMin : GArgMin {
  static constexpr bool returns_idx = false;
};
struct GMax : GArgMax {
  static constexpr bool returns_idx = false;
};

// One CTA of 256 threads per kept element (GROUP = 256) or one warp (GROUP = 32).
template <class T, class O, class Op, int GROUP>
__global__ void __launch_bounds__(256) reduce_generic(const T *__restrict__ in, void *__restrict__ out_raw,
                                                      KeepIndex keep, KeepIndex drop, int64_t n_keep,
                                                      int64_t n_drop) {
  constexpr int PER_CTA = 256 / GROUP;
  __shared__ Item<O> buf[256];
  const int sub = threadIdx.x / GROUP, t = threadIdx.x % GROUP;
  const int64_t k = int64_t(blockIdx.x) * PER_CTA + sub;
  Item<O> acc = Op::template neutral<O>();
  if (k < n_keep) {
    const T *p = in + keep_offset(keep, k);
    for (int64_t j = t; j < n_drop; j += GROUP)
      acc = Op::template combine<O>(acc, Item<O>{j, static_cast<O>(p[keep_offset(drop, j)])});
  }
  buf[threadIdx.x] = acc;
  __syncthreads();
  for (int s = GROUP / 2; s > 0; s >>= 1) {
    if (t < s) buf[threadIdx.x] = Op::template combine<O>(buf[threadIdx.x], buf[threadIdx.x + s]);
    __syncthreads();
  }
  if (t == 0 && k < n_keep) {
    if constexpr (Op::returns_idx)
      static_cast<int64_t *>(out_raw)[k] = buf[threadIdx.x].idx;
    else
      static_cast<O *>(out_raw)[k] = buf[threadIdx.x].value;
  }
}

// ---------------------------------------------------------------------------------------------
// Host side
struct Ticket {
  unsigned *ptr = nullptr;
  int64_t capacity = 0;
};
// Zero-initialised once; every kernel leaves the counters it used at zero.
static unsigned *tickets(int64_t need) {
  static Ticket t;
  if (need > t.capacity) {
    if (is_capturing())
      fail_runtime("reduction: the ticket counters must grow, which cannot happen inside a graph capture; run the "
                   "step once eagerly before capturing it.");
    int64_t cap = need < 65536 ? 65536 : need;
    size_t rounded;
    void *p = device_alloc(size_t(cap) * sizeof(unsigned), &rounded);
    NT_CUDA_CHECK(cudaMemsetAsync(p, 0, size_t(cap) * sizeof(unsigned), stream()));
    // the previous block (if any) stays allocated: kernels in flight may still hold it
    t.ptr = static_cast<unsigned *>(p);
    t.capacity = cap;
  }
  return t.ptr;
}

void reduce_prepare() { tickets(1); }

struct Plan {
  KeepIndex keep{}, drop{};
  int64_t n_keep = 1, n_drop = 1;
};

static void collapse_group(KeepIndex &g) {
  KeepIndex r{};
  for (int d = 0; d < g.ndim; ++d) {
    if (g.shape[d] == 1) continue;
    if (r.ndim > 0 && r.strides[r.ndim - 1] == g.strides[d] * g.shape[d]) {
      r.shape[r.ndim - 1] *= g.shape[d];
      r.strides[r.ndim - 1] = g.strides[d];
    } else {
      r.shape[r.ndim] = g.shape[d];
      r.strides[r.ndim] = g.strides[d];
      ++r.ndim;
    }
  }
  g = r;
}

static Plan make_plan(const nt_view *x, const int64_t *axes, int32_t n_axes) {
  Plan pl;
  bool dropped[NT_MAX_DIMS] = {};
  for (int i = 0; i < n_axes; ++i) {
    if (axes[i] < 0 || axes[i] >= x->ndim) fail_runtime("reduction: axis out of range.");
    if (dropped[axes[i]]) fail_runtime("reduction: repeated axis.");
    dropped[axes[i]] = true;
  }
  for (int d = 0; d < x->ndim; ++d) {
    KeepIndex &g = dropped[d] ? pl.drop : pl.keep;
    g.shape[g.ndim] = x->shape[d];
    g.strides[g.ndim] = x->strides[d];
    ++g.ndim;
    (dropped[d] ? pl.n_drop : pl.n_keep) *= x->shape[d];
  }
  collapse_group(pl.keep);
  collapse_group(pl.drop);
  return pl;
}

template <class Op> static bool try_fast_f32(const nt_view *x, const Plan &pl, float *out, float divisor = 0.0f) {
  const float *in = static_cast<const float *>(x->storage->data) + x->offset;
  cudaStream_t st = stream();
  const int sms = sm_count();
  const int64_t target_ctas = int64_t(sms) * 8;

  // rows: dropped dims are one unit-stride run
  if (pl.drop.ndim == 1 && pl.drop.strides[0] == 1) {
    const int64_t L = pl.n_drop, n_rows = pl.n_keep;
    if (L < 1024 && n_rows >= 64) {
      int64_t blocks = ceil_div(n_rows, 32);
      if (blocks > 0x7fffffffLL) return false;
      reduce_rows_warp<Op><<<unsigned(blocks), 256, 0, st>>>(in, out, pl.keep, n_rows, L, divisor);
      check_launch("reduce_rows_warp");
      return true;
    }
    int64_t S = ceil_div(target_ctas, n_rows);
    int64_t max_s = ceil_div(L, 8192);
    if (S > max_s) S = max_s;
    if (S > 1024) S = 1024;
    if (S < 1) S = 1;
    int64_t chunk = ceil_div(ceil_div(L, S), 1024) * 1024;
    S = ceil_div(L, chunk);
    if (n_rows * S > 0x7fffffffLL) return false;
    float *partials = nullptr;
    unsigned *tk = nullptr;
    size_t rounded = 0;
    if (S > 1) {
      partials = static_cast<float *>(device_alloc(size_t(n_rows * S) * sizeof(float), &rounded));
      tk = tickets(n_rows);
    }
    reduce_rows<Op><<<unsigned(n_rows * S), 256, 0, st>>>(in, out, partials, tk, pl.keep, L, int(S), chunk, divisor);
    if (partials) device_free(partials, rounded); // stream-ordered reuse: later work queues behind this launch
    check_launch("reduce_rows");
    return true;
  }

  // columns: innermost kept dim has unit stride, exactly one strided dim is dropped
  if (pl.drop.ndim == 1 && pl.keep.ndim >= 1 && pl.keep.strides[pl.keep.ndim - 1] == 1) {
    const int64_t R = pl.n_drop, sR = pl.drop.strides[0];
    const int64_t C = pl.keep.shape[pl.keep.ndim - 1];
    KeepIndex outer = pl.keep;
    outer.ndim -= 1;
    int64_t Z = 1;
    for (int d = 0; d < outer.ndim; ++d) Z *= outer.shape[d];
    if (Z > 65535) return false;
    bool vec = (C % 4 == 0) && (sR % 4 == 0) && aligned16(in);
    for (int d = 0; d < outer.ndim; ++d) vec = vec && (outer.strides[d] % 4 == 0);
    if (vec && C >= 1024 && aligned16(out)) {
      const int64_t tiles = ceil_div(C, 1024);
      // row splits: 4 CTAs per SM for large inputs; for inputs of up to 128 MB the finish -- one CTA per tile
      // reading S partial rows -- weighs as much as the main pass, so half as many, longer splits
      const int64_t per_sm = (R * C * Z * 4 <= (int64_t(128) << 20)) ? 2 : 4;
      int64_t S = ceil_div(int64_t(sms) * per_sm, tiles * Z);
      int64_t max_s = ceil_div(R, 32);
      if (S > max_s) S = max_s;
      if (S > 65535) S = 65535;
      if (S < 1) S = 1;
      int64_t rows_per_split = ceil_div(ceil_div(R, S), 8) * 8;
      S = ceil_div(R, rows_per_split);
      float *partials = nullptr;
      unsigned *tk = nullptr;
      size_t rounded = 0;
      if (S > 1) {
        partials = static_cast<float *>(device_alloc(size_t(Z * S * C) * sizeof(float), &rounded));
        tk = tickets(Z * tiles);
      }
      dim3 grid{unsigned(tiles), unsigned(S), unsigned(Z)};
      reduce_cols_wide<Op><<<grid, 256, 0, st>>>(in, out, partials, tk, outer, R, C, sR, rows_per_split, divisor);
      if (partials) device_free(partials, rounded);
      check_launch("reduce_cols_wide");
      return true;
    }
    const int TW = vec ? 128 : 32;
    const int64_t tiles = ceil_div(C, TW);
    if (tiles > 0x7fffffffLL) return false;
    int64_t S = ceil_div(target_ctas, tiles * Z);
    int64_t max_s = ceil_div(R, 64);
    if (S > max_s) S = max_s;
    if (S > 65535) S = 65535;
    if (S < 1) S = 1;
    int64_t rows_per_split = ceil_div(R, S);
    S = ceil_div(R, rows_per_split);
    float *partials = nullptr;
    unsigned *tk = nullptr;
    size_t rounded = 0;
    if (S > 1) {
      partials = static_cast<float *>(device_alloc(size_t(Z * S * C) * sizeof(float), &rounded));
      tk = tickets(Z * tiles);
    }
    dim3 grid{unsigned(tiles), unsigned(S), unsigned(Z)};
    if (vec)
      reduce_cols<Op, 4><<<grid, 256, 0, st>>>(in, out, partials, tk, outer, R, C, sR, rows_per_split, divisor);
    else
      reduce_cols<Op, 1><<<grid, 256, 0, st>>>(in, out, partials, tk, outer, R, C, sR, rows_per_split, divisor);
    if (partials) device_free(partials, rounded);
    check_launch("reduce_cols");
    return true;
  }
  return false;
}

template <class T, class O, class Op> static void launch_generic(const nt_view *x, const Plan &pl, void *out) {
  const T *in = static_cast<const T *>(x->storage->data) + x->offset;
  cudaStream_t st = stream();
  if (pl.n_drop > 256) {
    if (pl.n_keep > 0x7fffffffLL) fail_runtime("reduction: too many kept elements.");
    reduce_generic<T, O, Op, 256><<<unsigned(pl.n_keep), 256, 0, st>>>(in, out, pl.keep, pl.drop, pl.n_keep, pl.n_drop);
  } else {
    int64_t blocks = ceil_div(pl.n_keep, 8);
    if (blocks > 0x7fffffffLL) fail_runtime("reduction: too many kept elements.");
    reduce_generic<T, O, Op, 32><<<unsigned(blocks), 256, 0, st>>>(in, out, pl.keep, pl.drop, pl.n_keep, pl.n_drop);
  }
  check_launch("reduce_generic");
}

template <class GOp, class FastOp>
static nt_storage *reduce_impl(const nt_view *x, const int64_t *axes, int32_t n_axes, int out_dtype, const char *fname) {
  check_view(x, fname);
  require_cuda(x, fname);
  if (n_axes < 0 || n_axes > x->ndim) fail_runtime(std::string(fname) + ": bad axis list.");
  Plan pl = make_plan(x, axes, n_axes);
  const int in_dtype = x->storage->dtype;
  if (out_dtype == NT_BOOL) fail_invalid("Invalid dtype.");
  dtype_itemsize(out_dtype);
  const int storage_dtype = GOp::returns_idx ? NT_INT64 : out_dtype;
  StorageRef out(storage_new(pl.n_keep, storage_dtype, NT_CUDA));
  if (pl.n_keep == 0) return out.release();

  if constexpr (!std::is_same_v<FastOp, void>) {
    if (in_dtype == NT_FLOAT32 && out_dtype == NT_FLOAT32 && pl.n_drop > 0) {
      if (try_fast_f32<FastOp>(x, pl, static_cast<float *>(out->data))) return out.release();
    }
  }
  dispatch_all(in_dtype, [&]<class T>() {
    dispatch_arith(out_dtype, [&]<class O>() { launch_generic<T, O, GOp>(x, pl, out->data); });
  });
  return out.release();
}

// mask helpers of the extremum backward
struct EqMaskF { // float(x == m)
  using in_t = float;
  using out_t = float;
  __device__ __forceinline__ float operator()(float x, float m) const { return (x == m) ? 1.0f : 0.0f; }
};
struct UniqueMaskMulF { // g * float(mask && count == 1)
  using in_t = float;
  using out_t = float;
  __device__ __forceinline__ float operator()(float g, float mask, float count) const {
    return g * ((mask != 0.0f && count == 1.0f) ? 1.0f : 0.0f);
  }
};


// ---------------------------------------------------------------------------------------------
// Max/Min backward without materialising the mask: two launches over x.
//   extremum_count_*  counts, per reduced slice, the positions equal to the slice's extremum
//                     (integer atomics: exact, order-free);
//   extremum_apply    out = g_slice * float(x == m_slice && count_slice == 1).
// x is seen as [n_keep slices] x [n_drop] with the dropped dims either the trailing run (ROWS:
// x[row_base + j]) or the leading dim of a dense matrix (COLS: x[i * sR + c]).  g and m are read once
// per slice through their own kept-dim strides (they are stride-0 along the dropped dims).
// Algorithmic bytes: x twice + out once = 12 per element (the composed chain moves 20).
struct SliceScalars {
  KeepIndex x_keep, g_keep, m_keep; // same shapes, each operand's strides over the kept dims
};
// offset of slice `lin`: a single kept dim needs no division at all
__device__ __forceinline__ int64_t slice_offset(const KeepIndex &k, int64_t lin) {
  if (k.ndim == 0) return 0;
  if (k.ndim == 1) return lin * k.strides[0];
  return keep_offset(k, lin);
}

__global__ void __launch_bounds__(256) extremum_count_rows(const float *__restrict__ x, const float *__restrict__ m,
                                                           int *__restrict__ count, SliceScalars sc, int64_t L,
                                                           int chunks_per_row, int64_t chunk) {
  __shared__ int warp_cnt[8];
  const int64_t row = blockIdx.x / chunks_per_row;
  const int c = int(blockIdx.x - row * chunks_per_row);
  const float *p = x + slice_offset(sc.x_keep, row);
  const float mv = m[slice_offset(sc.m_keep, row)];
  const int64_t lo = int64_t(c) * chunk;
  int64_t hi = lo + chunk;
  if (hi > L) hi = L;
  int n = 0;
  if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
    const int64_t nvec = (hi - lo) >> 2;
    const float4 *pv = reinterpret_cast<const float4 *>(p + lo);
    for (int64_t i = threadIdx.x; i < nvec; i += 256) {
      float4 v = __ldcs(pv + i);
      n += (v.x == mv) + (v.y == mv) + (v.z == mv) + (v.w == mv);
    }
    for (int64_t j = lo + (nvec << 2) + threadIdx.x; j < hi; j += 256) n += (p[j] == mv);
  } else {
    for (int64_t j = lo + threadIdx.x; j < hi; j += 256) n += (p[j] == mv);
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) n += __shfl_xor_sync(0xffffffffu, n, s);
  if ((threadIdx.x & 31) == 0) warp_cnt[threadIdx.x >> 5] = n;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += warp_cnt[w];
    if (t) atomicAdd(count + row, t);
  }
}

// COLS: block = 128 columns (32 lanes x 4) x rows_per_block rows, 8 warps interleaved over the rows.
__global__ void __launch_bounds__(256) extremum_count_cols(const float *__restrict__ x, const float *__restrict__ m,
                                                           int *__restrict__ count, SliceScalars sc, int64_t R, int64_t C,
                                                           int64_t sR, int64_t rows_per_block, int vec) {
  __shared__ int part[8][128];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t c0 = int64_t(blockIdx.x) * 128 + lane * 4;
  int64_t r_lo = int64_t(blockIdx.y) * rows_per_block, r_hi = r_lo + rows_per_block;
  if (r_hi > R) r_hi = R;
  int n[4] = {0, 0, 0, 0};
  float mv[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) mv[e] = (c0 + e < C) ? m[slice_offset(sc.m_keep, c0 + e)] : 0.0f;
  if (c0 < C) {
    for (int64_t r = r_lo + warp; r < r_hi; r += 8) {
      const float *q = x + r * sR + c0;
      if (vec) {
        float4 v = __ldcs(reinterpret_cast<const float4 *>(q));
        n[0] += (v.x == mv[0]); n[1] += (v.y == mv[1]); n[2] += (v.z == mv[2]); n[3] += (v.w == mv[3]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (c0 + e < C) n[e] += (q[e] == mv[e]);
      }
    }
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) part[warp][lane * 4 + e] = n[e];
  __syncthreads();
  if (threadIdx.x < 128) {
    int t = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += part[w][threadIdx.x];
    const int64_t c = int64_t(blockIdx.x) * 128 + threadIdx.x;
    if (t && c < C) atomicAdd(count + c, t);
  }
}

// One thread per 4 consecutive output elements.  ROWS: slice = idx / L (L % 4 == 0 when vec);
// COLS: slice = idx % C.
template <bool ROWS>
__global__ void __launch_bounds__(256) extremum_apply(const float *__restrict__ x, const float *__restrict__ g,
                                                      const float *__restrict__ m, const int *__restrict__ count,
                                                      float *__restrict__ out, SliceScalars sc, int64_t n_outer, int64_t L,
                                                      int64_t sR, int vec) {
  // ROWS: n_outer slices of L elements; COLS: n_outer rows of L columns (slice = column).
  // total < 2^40 is guaranteed by the host; the common case fits 32-bit division.
  const int64_t total = n_outer * L;
  const int64_t t = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (t >= total) return;
  int64_t outer, inner;
  if (total < (int64_t(1) << 32)) {
    const uint32_t o32 = uint32_t(t) / uint32_t(L);
    outer = o32;
    inner = uint32_t(t) - o32 * uint32_t(L);
  } else {
    outer = t / L;
    inner = t - outer * L;
  }
  float res[4];
  if (vec) { // the four elements share `outer` (L % 4 == 0) and are contiguous in x
    const float *px = ROWS ? x + slice_offset(sc.x_keep, outer) + inner : x + outer * sR + inner;
    const float4 v = __ldcs(reinterpret_cast<const float4 *>(px));
    const float xv[4] = {v.x, v.y, v.z, v.w};
    if (ROWS) {
      const float gv = g[slice_offset(sc.g_keep, outer)], mv = m[slice_offset(sc.m_keep, outer)];
      const bool unique = count[outer] == 1;
#pragma unroll
      for (int e = 0; e < 4; ++e) res[e] = gv * ((xv[e] == mv && unique) ? 1.0f : 0.0f);
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int64_t c = inner + e;
        const float gv = g[slice_offset(sc.g_keep, c)], mv = m[slice_offset(sc.m_keep, c)];
        res[e] = gv * ((xv[e] == mv && count[c] == 1) ? 1.0f : 0.0f);
      }
    }
    __stcs(reinterpret_cast<float4 *>(out + t), make_float4(res[0], res[1], res[2], res[3]));
    return;
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int64_t idx = t + e;
    if (idx >= total) break;
    const int64_t o = idx / L, i = idx - o * L;
    const int64_t slice = ROWS ? o : i;
    const float xv = ROWS ? x[slice_offset(sc.x_keep, o) + i] : x[o * sR + i];
    const float gv = g[slice_offset(sc.g_keep, slice)], mv = m[slice_offset(sc.m_keep, slice)];
    out[idx] = gv * ((xv == mv && count[slice] == 1) ? 1.0f : 0.0f);
  }
}

// Vector form of extremum_apply: a CTA owns 1024 consecutive elements of ONE outer index (a slice for
// ROWS, a matrix row for COLS), so the outer index and -- for ROWS -- the slice's g, m and count are
// block-uniform and no thread divides anything.
template <bool ROWS>
__global__ void __launch_bounds__(256) extremum_apply_vec(const float *__restrict__ x, const float *__restrict__ g,
                                                          const float *__restrict__ m, const int *__restrict__ count,
                                                          float *__restrict__ out, SliceScalars sc, int64_t L, int64_t sR,
                                                          int chunks) {
  const int64_t outer = blockIdx.x / chunks;
  const int64_t inner = int64_t(blockIdx.x - outer * chunks) * 1024 + threadIdx.x * 4;
  if (inner >= L) return;
  const float *px = ROWS ? x + slice_offset(sc.x_keep, outer) + inner : x + outer * sR + inner;
  const float4 v = __ldcs(reinterpret_cast<const float4 *>(px));
  const float xv[4] = {v.x, v.y, v.z, v.w};
  float res[4];
  if (ROWS) {
    const float gv = g[slice_offset(sc.g_keep, outer)], mv = m[slice_offset(sc.m_keep, outer)];
    const bool unique = count[outer] == 1;
#pragma unroll
    for (int e = 0; e < 4; ++e) res[e] = gv * ((xv[e] == mv && unique) ? 1.0f : 0.0f);
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int64_t c = inner + e;
      const float gv = g[slice_offset(sc.g_keep, c)], mv = m[slice_offset(sc.m_keep, c)];
      res[e] = gv * ((xv[e] == mv && count[c] == 1) ? 1.0f : 0.0f);
    }
  }
  __stcs(reinterpret_cast<float4 *>(out + outer * L + inner), make_float4(res[0], res[1], res[2], res[3]));
}

// Optimistic single pass for the long-slice and leading-dim cases: ties are rare, so write g * float(x == m)
// straight away (x read once, 8 bytes per element) and count the matches per slice on the side -- one atomic per
// match, i.e. one per slice unless it is tied.  extremum_fix_ties then revisits only the slices whose count is
// above 1 and turns their matches into g * 0, which is what the reference's integer 1 // count leaves there.
template <bool ROWS>
__global__ void __launch_bounds__(256) extremum_apply_count_vec(const float *__restrict__ x, const float *__restrict__ g,
                                                                const float *__restrict__ m, int *__restrict__ count,
                                                                float *__restrict__ out, SliceScalars sc, int64_t L,
                                                                int64_t sR, int chunks, int gm_vec) {
  // a CTA owns 4096 consecutive elements of ONE outer index (a slice for ROWS, a matrix row for COLS); a thread
  // owns four 128-bit vectors 1024 elements apart, all loaded before the first use
  const int64_t outer = blockIdx.x / chunks;
  const int64_t base = int64_t(blockIdx.x - outer * chunks) * 4096 + threadIdx.x * 4;
  const float *px = ROWS ? x + slice_offset(sc.x_keep, outer) : x + outer * sR;
  float4 v[4];
#pragma unroll
  for (int u = 0; u < 4; ++u)
    if (base + u * 1024 < L) v[u] = __ldcs(reinterpret_cast<const float4 *>(px + base + u * 1024));
  float gs = 0.0f, ms = 0.0f;
  if (ROWS) {
    gs = g[slice_offset(sc.g_keep, outer)];
    ms = m[slice_offset(sc.m_keep, outer)];
  }
  int hits = 0;
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int64_t inner = base + u * 1024;
    if (inner >= L) break;
    const float xv[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
    float gv[4], mv[4];
    if (ROWS) {
#pragma unroll
      for (int e = 0; e < 4; ++e) gv[e] = gs, mv[e] = ms;
    } else if (gm_vec) { // g and m are dense vectors over the columns: one 128-bit load each
      const float4 g4 = __ldg(reinterpret_cast<const float4 *>(g + inner)), m4 = __ldg(reinterpret_cast<const float4 *>(m + inner));
      gv[0] = g4.x, gv[1] = g4.y, gv[2] = g4.z, gv[3] = g4.w;
      mv[0] = m4.x, mv[1] = m4.y, mv[2] = m4.z, mv[3] = m4.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        gv[e] = g[slice_offset(sc.g_keep, inner + e)];
        mv[e] = m[slice_offset(sc.m_keep, inner + e)];
      }
    }
    float res[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const bool eq = xv[e] == mv[e];
      if (ROWS) hits += eq ? 1 : 0;
      else if (eq) atomicAdd(count + inner + e, 1);
      res[e] = gv[e] * (eq ? 1.0f : 0.0f);
    }
    __stcs(reinterpret_cast<float4 *>(out + outer * L + inner), make_float4(res[0], res[1], res[2], res[3]));
  }
  if (ROWS && hits) atomicAdd(count + outer, hits);
}

// ROWS: one CTA per slice (n_slices CTAs), COLS: one thread per column.  Slices with a unique extremum -- all of
// them, normally -- cost one read of their counter.
template <bool ROWS>
__global__ void __launch_bounds__(256) extremum_fix_ties(const float *__restrict__ x, const float *__restrict__ g,
                                                         const float *__restrict__ m, const int *__restrict__ count,
                                                         float *__restrict__ out, SliceScalars sc, int64_t n_slices,
                                                         int64_t n_drop, int64_t sR) {
  if (ROWS) {
    const int64_t slice = blockIdx.x;
    if (count[slice] <= 1) return;
    const float *px = x + slice_offset(sc.x_keep, slice);
    const float gv = g[slice_offset(sc.g_keep, slice)], mv = m[slice_offset(sc.m_keep, slice)];
    for (int64_t j = threadIdx.x; j < n_drop; j += 256)
      if (px[j] == mv) out[slice * n_drop + j] = gv * 0.0f;
  } else {
    const int64_t c = int64_t(blockIdx.x) * 256 + threadIdx.x;
    if (c >= n_slices || count[c] <= 1) return;
    const float gv = g[slice_offset(sc.g_keep, c)], mv = m[slice_offset(sc.m_keep, c)];
    for (int64_t r = 0; r < n_drop; ++r)
      if (x[r * sR + c] == mv) out[r * n_slices + c] = gv * 0.0f;
  }
}

// One pass for ROWS slices of at most 16384 elements: a CTA keeps its whole slice in registers (VPT
// 128-bit vectors per thread), counts the positions equal to the extremum, and writes the gradient from
// the registers -- x is read once: 8 bytes per element instead of 12, no counter array, one launch.
template <int VPT>
__global__ void __launch_bounds__(256) extremum_rows_onepass(const float *__restrict__ x, const float *__restrict__ g,
                                                             const float *__restrict__ m, float *__restrict__ out,
                                                             SliceScalars sc, int64_t L) {
  __shared__ int warp_cnt[8];
  const int64_t row = blockIdx.x;
  const float4 *pv = reinterpret_cast<const float4 *>(x + slice_offset(sc.x_keep, row));
  const float mv = m[slice_offset(sc.m_keep, row)];
  const float gv = g[slice_offset(sc.g_keep, row)];
  const int nvec = int(L >> 2);
  float4 v[VPT];
  int n = 0;
#pragma unroll
  for (int u = 0; u < VPT; ++u) {
    const int i = threadIdx.x + u * 256;
    if (i < nvec) {
      v[u] = __ldcs(pv + i);
      n += (v[u].x == mv) + (v[u].y == mv) + (v[u].z == mv) + (v[u].w == mv);
    }
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) n += __shfl_xor_sync(0xffffffffu, n, s);
  if ((threadIdx.x & 31) == 0) warp_cnt[threadIdx.x >> 5] = n;
  __syncthreads();
  int total = 0;
#pragma unroll
  for (int w = 0; w < 8; ++w) total += warp_cnt[w];
  const bool unique = total == 1;
  float4 *po = reinterpret_cast<float4 *>(out + row * L);
#pragma unroll
  for (int u = 0; u < VPT; ++u) {
    const int i = threadIdx.x + u * 256;
    if (i < nvec) {
      float4 r;
      r.x = gv * ((v[u].x == mv && unique) ? 1.0f : 0.0f);
      r.y = gv * ((v[u].y == mv && unique) ? 1.0f : 0.0f);
      r.z = gv * ((v[u].z == mv && unique) ? 1.0f : 0.0f);
      r.w = gv * ((v[u].w == mv && unique) ? 1.0f : 0.0f);
      __stcs(po + i, r);
    }
  }
}

// Returns false when the views do not have one of the two shapes above (the caller then composes).
static bool extremum_backward_fused(const nt_view *g, const nt_view *x, const nt_view *m, const int64_t *axes,
                                    int32_t n_axes, float *out) {
  const int nd = x->ndim;
  if (n_axes < 1 || n_axes > nd) return false;
  bool dropped[NT_MAX_DIMS] = {};
  for (int i = 0; i < n_axes; ++i) {
    if (axes[i] < 0 || axes[i] >= nd || dropped[axes[i]]) return false;
    dropped[axes[i]] = true;
  }
  bool trailing = true, leading = true;
  for (int d = 0; d < nd; ++d) {
    if (dropped[d] != (d >= nd - n_axes)) trailing = false;
    if (dropped[d] != (d < n_axes)) leading = false;
  }
  if (!trailing && !leading) return false;
  // g and m must not vary along the dropped dims
  for (int d = 0; d < nd; ++d)
    if (dropped[d] && x->shape[d] > 1 && (g->strides[d] != 0 || m->strides[d] != 0)) return false;
  Plan pl = make_plan(x, axes, n_axes);
  if (pl.n_keep == 0 || pl.n_drop == 0) return false;
  SliceScalars sc{};
  for (int d = 0; d < nd; ++d) {
    if (dropped[d] || x->shape[d] == 1) continue;
    const int k = sc.x_keep.ndim;
    sc.x_keep.shape[k] = sc.g_keep.shape[k] = sc.m_keep.shape[k] = x->shape[d];
    sc.x_keep.strides[k] = x->strides[d];
    sc.g_keep.strides[k] = g->strides[d];
    sc.m_keep.strides[k] = m->strides[d];
    sc.x_keep.ndim = sc.g_keep.ndim = sc.m_keep.ndim = k + 1;
  }
  const float *xp = static_cast<const float *>(x->storage->data) + x->offset;
  const float *gp = static_cast<const float *>(g->storage->data) + g->offset;
  const float *mp = static_cast<const float *>(m->storage->data) + m->offset;
  cudaStream_t st = stream();
  const bool rows = trailing && pl.drop.ndim == 1 && pl.drop.strides[0] == 1;
  const bool cols = !rows && leading && pl.drop.ndim == 1 && pl.keep.ndim == 1 && pl.keep.strides[0] == 1;
  if (!rows && !cols) return false;
  if (pl.n_keep * pl.n_drop >= (int64_t(1) << 40)) return false;
  if (rows) {
    const int64_t L = pl.n_drop;
    bool vec = (L % 4 == 0) && aligned16(xp) && aligned16(out);
    for (int k = 0; k < sc.x_keep.ndim; ++k) vec = vec && (sc.x_keep.strides[k] % 4 == 0);
    if (vec && L <= 16384 && pl.n_keep >= sm_count() && pl.n_keep <= 0x7fffffffLL) {
      const unsigned grid = unsigned(pl.n_keep);
      const int64_t per_thread = ceil_div(L / 4, 256);
      if (per_thread <= 1) extremum_rows_onepass<1><<<grid, 256, 0, st>>>(xp, gp, mp, out, sc, L);
      else if (per_thread <= 2) extremum_rows_onepass<2><<<grid, 256, 0, st>>>(xp, gp, mp, out, sc, L);
      else if (per_thread <= 4) extremum_rows_onepass<4><<<grid, 256, 0, st>>>(xp, gp, mp, out, sc, L);
      else if (per_thread <= 8) extremum_rows_onepass<8><<<grid, 256, 0, st>>>(xp, gp, mp, out, sc, L);
      else extremum_rows_onepass<16><<<grid, 256, 0, st>>>(xp, gp, mp, out, sc, L);
      check_launch("extremum_rows_onepass");
      return true;
    }
  }
  size_t rounded = 0;
  int *count = static_cast<int *>(device_alloc(size_t(pl.n_keep) * sizeof(int), &rounded));
  NT_CUDA_CHECK(cudaMemsetAsync(count, 0, size_t(pl.n_keep) * sizeof(int), st));
  const int64_t total = pl.n_keep * pl.n_drop;
  const int64_t apply_blocks = ceil_div(ceil_div(total, 4), 256);
  if (rows) {
    const int64_t L = pl.n_drop;
    const int64_t chunk = 16384; // elements per counting CTA (a multiple of 4)
    const int64_t chunks = ceil_div(L, chunk);
    if (pl.n_keep * chunks > 0x7fffffffLL || apply_blocks > 0x7fffffffLL) {
      device_free(count, rounded);
      return false;
    }
    bool vec = (L % 4 == 0) && aligned16(xp) && aligned16(out);
    for (int k = 0; k < sc.x_keep.ndim; ++k) vec = vec && (sc.x_keep.strides[k] % 4 == 0);
    const int64_t vchunks = ceil_div(L, 4096);
    if (vec && pl.n_keep * vchunks <= 0x7fffffffLL) {
      extremum_apply_count_vec<true><<<unsigned(pl.n_keep * vchunks), 256, 0, st>>>(xp, gp, mp, count, out, sc, L, 0, int(vchunks), 0);
      check_launch("extremum_apply_count_vec");
      extremum_fix_ties<true><<<unsigned(pl.n_keep), 256, 0, st>>>(xp, gp, mp, count, out, sc, pl.n_keep, L, 0);
      check_launch("extremum_fix_ties");
    } else {
      extremum_count_rows<<<unsigned(pl.n_keep * chunks), 256, 0, st>>>(xp, mp, count, sc, L, int(chunks), chunk);
      check_launch("extremum_count_rows");
      extremum_apply<true><<<unsigned(apply_blocks), 256, 0, st>>>(xp, gp, mp, count, out, sc, pl.n_keep, L, 0, vec ? 1 : 0);
      check_launch("extremum_apply");
    }
  } else {
    const int64_t R = pl.n_drop, C = pl.n_keep, sR = pl.drop.strides[0];
    const bool vec = (C % 4 == 0) && (sR % 4 == 0) && aligned16(xp) && aligned16(out);
    const int64_t tiles = ceil_div(C, 128);
    int64_t row_blocks = ceil_div(int64_t(sm_count()) * 8, tiles);
    if (row_blocks > ceil_div(R, 32)) row_blocks = ceil_div(R, 32);
    if (row_blocks < 1) row_blocks = 1;
    if (row_blocks > 65535) row_blocks = 65535;
    const int64_t rows_per_block = ceil_div(R, row_blocks);
    row_blocks = ceil_div(R, rows_per_block);
    if (tiles > 0x7fffffffLL || apply_blocks > 0x7fffffffLL) {
      device_free(count, rounded);
      return false;
    }
    dim3 grid{unsigned(tiles), unsigned(row_blocks), 1};
    const int64_t vchunks = ceil_div(C, 4096);
    if (vec && R * vchunks <= 0x7fffffffLL) {
      const int gm_vec = (sc.g_keep.ndim == 1 && sc.g_keep.strides[0] == 1 && sc.m_keep.ndim == 1 && sc.m_keep.strides[0] == 1 &&
                          aligned16(gp) && aligned16(mp)) ? 1 : 0;
      extremum_apply_count_vec<false><<<unsigned(R * vchunks), 256, 0, st>>>(xp, gp, mp, count, out, sc, C, sR, int(vchunks), gm_vec);
      check_launch("extremum_apply_count_vec");
      extremum_fix_ties<false><<<unsigned(ceil_div(C, 256)), 256, 0, st>>>(xp, gp, mp, count, out, sc, C, R, sR);
      check_launch("extremum_fix_ties");
    } else {
      extremum_count_cols<<<grid, 256, 0, st>>>(xp, mp, count, sc, R, C, sR, rows_per_block, vec ? 1 : 0);
      check_launch("extremum_count_cols");
      extremum_apply<false><<<unsigned(apply_blocks), 256, 0, st>>>(xp, gp, mp, count, out, sc, R, C, sR, vec ? 1 : 0);
      check_launch("extremum_apply");
    }
  }
  device_free(count, rounded);
  return true;
}

// ---------------------------------------------------------------------------------------------
// Row sums without any allocation: the cross-CTA scratch of reduce_rows (one partial per CTA, one
// ticket per row) lives in this fixed device array instead of coming from the arena.
constexpr int64_t NOALLOC_MAX_PARTIALS = 2048; // floats
constexpr int64_t NOALLOC_MAX_ROWS = 256;      // tickets: rows that are long enough to be split over CTAs
struct NoAllocScratch {
  float partials[NOALLOC_MAX_PARTIALS];
  unsigned tickets[NOALLOC_MAX_ROWS];
};
static __device__ __align__(256) NoAllocScratch g_noalloc_scratch; // 9 KB on every GPU that loads the library

// `g_noalloc_scratch` named in host code is only a host-side handle; the kernel needs the device
// address, looked up once per device with that device current.
static NoAllocScratch *noalloc_scratch_device_ptr() {
  static NoAllocScratch *per_device[64] = {};
  int dev = 0;
  NT_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) fail_runtime("nt_sum_rows_noalloc: device ordinal out of range.");
  if (!per_device[dev]) {
    void *p = nullptr;
    NT_CUDA_CHECK(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    per_device[dev] = static_cast<NoAllocScratch *>(p);
  }
  return per_device[dev];
}

} // namespace ntb

using namespace ntb;

extern "C" {

int nt_sum_rows_noalloc(const float *in, int64_t n_rows, int64_t row_len, float *out) {
  NT_API_BEGIN
  if (!in || !out) fail_invalid("nt_sum_rows_noalloc: null pointer.");
  if (n_rows < 0 || row_len < 1) fail_invalid("nt_sum_rows_noalloc: n_rows must be >= 0 and row_len >= 1.");
  if (n_rows == 0) return NT_OK;
  cudaStream_t st = stream();
  NoAllocScratch *scratch = noalloc_scratch_device_ptr();
  // same split rule as the allocating path (try_fast_f32), so both entry points add in the same order
  const int64_t target_ctas = int64_t(sm_count()) * 8;
  KeepIndex keep{};
  keep.ndim = 1;
  keep.shape[0] = n_rows;
  keep.strides[0] = row_len;
  if (row_len < 1024 && n_rows >= 64) {
    int64_t blocks = ceil_div(n_rows, 32);
    if (blocks > 0x7fffffffLL) fail_invalid("nt_sum_rows_noalloc: too many rows for one launch.");
    reduce_rows_warp<RSum><<<unsigned(blocks), 256, 0, st>>>(in, out, keep, n_rows, row_len, 0.0f);
    check_launch("reduce_rows_warp");
    return NT_OK;
  }
  int64_t S = ceil_div(target_ctas, n_rows);
  int64_t max_s = ceil_div(row_len, 8192);
  if (S > max_s) S = max_s;
  if (S > 1024) S = 1024;
  if (S < 1) S = 1;
  int64_t chunk = ceil_div(ceil_div(row_len, S), 1024) * 1024;
  S = ceil_div(row_len, chunk);
  if (n_rows * S > 0x7fffffffLL) fail_invalid("nt_sum_rows_noalloc: too many rows for one launch.");
  if (S > 1 && (n_rows * S > NOALLOC_MAX_PARTIALS || n_rows > NOALLOC_MAX_ROWS))
    fail_invalid("nt_sum_rows_noalloc: this shape needs " + std::to_string(n_rows * S) + " partial sums over " +
                 std::to_string(n_rows) + " rows; the fixed scratch holds " + std::to_string(NOALLOC_MAX_PARTIALS) +
                 " partials and " + std::to_string(NOALLOC_MAX_ROWS) + " row tickets. Use nt_sum for larger inputs.");
  if (S > 1) // tickets must start at zero whatever the previous call left behind
    NT_CUDA_CHECK(cudaMemsetAsync(scratch->tickets, 0, size_t(n_rows) * sizeof(unsigned), st));
  reduce_rows<RSum><<<unsigned(n_rows * S), 256, 0, st>>>(in, out, scratch->partials, scratch->tickets, keep, row_len,
                                                        int(S), chunk, 0.0f);
  check_launch("reduce_rows");
  NT_API_END
}

int nt_sum(const nt_view *x, const int64_t *axes, int32_t n_axes, int dtype, nt_storage **out) {
  NT_API_BEGIN
  *out = reduce_impl<GSum, RSum>(x, axes, n_axes, dtype, "sum");
  NT_API_END
}
int nt_mean_f32(const nt_view *x, const int64_t *axes, int32_t n_axes, float count, nt_storage **out) {
  NT_API_BEGIN
  *out = nullptr;
  check_view(x, "mean");
  require_cuda(x, "mean");
  if (n_axes < 0 || n_axes > x->ndim) fail_runtime("mean: bad axis list.");
  if (x->storage->dtype != NT_FLOAT32 || count == 0.0f) return NT_OK;
  Plan pl = make_plan(x, axes, n_axes);
  if (pl.n_keep == 0 || pl.n_drop == 0) return NT_OK;
  StorageRef o(storage_new(pl.n_keep, NT_FLOAT32, NT_CUDA));
  if (try_fast_f32<RSum>(x, pl, static_cast<float *>(o->data), count)) *out = o.release();
  NT_API_END
}
int nt_max(const nt_view *x, const int64_t *axes, int32_t n_axes, nt_storage **out) {
  NT_API_BEGIN
  check_view(x, "max");
  *out = reduce_impl<GMax, RMax>(x, axes, n_axes, x->storage->dtype, "max");
  NT_API_END
}
int nt_min(const nt_view *x, const int64_t *axes, int32_t n_axes, nt_storage **out) {
  NT_API_BEGIN
  check_view(x, "min");
  *out = reduce_impl<GMin, RMin>(x, axes, n_axes, x->storage->dtype, "min");
  NT_API_END
}
int nt_argmax(const nt_view *x, const int64_t *axes, int32_t n_axes, nt_storage **out) {
  NT_API_BEGIN
  check_view(x, "argmax");
  *out = reduce_impl<GArgMax, void>(x, axes, n_axes, x->storage->dtype, "argmax");
  NT_API_END
}
int nt_argmin(const nt_view *x, const int64_t *axes, int32_t n_axes, nt_storage **out) {
  NT_API_BEGIN
  check_view(x, "argmin");
  *out = reduce_impl<GArgMin, void>(x, axes, n_axes, x->storage->dtype, "argmin");
  NT_API_END
}

int nt_extremum_backward(const nt_view *g_expanded, const nt_view *x, const nt_view *m_expanded,
                         const int64_t *axes, int32_t n_axes, nt_storage **out) {
  NT_API_BEGIN
  const char *fname = "extremum_backward";
  const nt_view *chk[3] = {g_expanded, x, m_expanded};
  for (int i = 0; i < 3; ++i) {
    check_view(chk[i], fname);
    require_cuda(chk[i], fname);
    if (chk[i]->storage->dtype != NT_FLOAT32) fail_invalid(std::string(fname) + ": Float32 only.");
    require_same_shape(chk[0], chk[i], fname);
  }
  const int64_t n = view_numel(*x);
  if (n > 0) {
    StorageRef fused(storage_new(n, NT_FLOAT32, NT_CUDA));
    if (extremum_backward_fused(g_expanded, x, m_expanded, axes, n_axes, static_cast<float *>(fused->data))) {
      *out = fused.release();
      return NT_OK;
    }
  }
  // general views: compose mask, count and product
  // mask = float(x == m)
  StorageRef mask(storage_new(n, NT_FLOAT32, NT_CUDA));
  nt_view mv = fresh_view(mask.s, *x);
  {
    const nt_view *views[3] = {&mv, x, m_expanded};
    ew_launch<EqMaskF, 2>(EqMaskF{}, views);
  }
  // count of extremal positions per slice, kept dims set to 1 and expanded back with stride 0
  StorageRef count(reduce_impl<GSum, RSum>(&mv, axes, n_axes, NT_FLOAT32, fname));
  nt_view cv{};
  cv.storage = count.s;
  cv.ndim = x->ndim;
  cv.offset = 0;
  {
    bool dropped[NT_MAX_DIMS] = {};
    for (int i = 0; i < n_axes; ++i) dropped[axes[i]] = true;
    int64_t st = 1;
    for (int d = x->ndim - 1; d >= 0; --d) {
      cv.shape[d] = x->shape[d];
      if (dropped[d]) {
        cv.strides[d] = 0;
      } else {
        cv.strides[d] = st;
        st *= x->shape[d];
      }
    }
  }
  StorageRef o(storage_new(n, NT_FLOAT32, NT_CUDA));
  nt_view ov = fresh_view(o.s, *x);
  {
    const nt_view *views[4] = {&ov, g_expanded, &mv, &cv};
    ew_launch<UniqueMaskMulF, 3>(UniqueMaskMulF{}, views);
  }
  *out = o.release();
  NT_API_END
}

} // extern "C"
