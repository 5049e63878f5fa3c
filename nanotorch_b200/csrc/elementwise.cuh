// Elementwise kernel framework for sm_100a: one functor, three kernels.
//
//   ew_contig   every operand is one contiguous run: 128-bit loads/stores, four vectors in flight
//               per operand per thread, streaming cache hints.  HBM-bound: (NIN+1)*4 bytes/element.
//   ew_strided  any strides (0 = broadcast, negative, transposed) over up to 8 collapsed dims;
//               a thread owns 4 consecutive elements of the innermost dim when that dim allows
//               it, so unit-stride operands still move as 128-bit vectors and stride-0 operands
//               as one load.
//   ew_tile2d   fp32, the last two collapsed dims: operands whose unit stride is on the *outer*
//               of the two (transposed views) are staged through a 64x64 shared-memory tile so
//               that both global sides stay coalesced.
//
// Operand 0 is always the output (fresh contiguous storage, or the `out` view of an in-place op).
// Replaces _binary_kernel/_binary_kernel_contig_f4 (src/cpp/ops/binary_ops.cu:22-41),
// _unary_kernel (src/cpp/ops/unary_ops.cu:19-26) and _inplace_apply_kernel
// (src/cpp/ops/inplace_ops.cu:18-27) of the reference, whose strided path does a chain of int64
// divisions per element per operand (src/cpp/tensor_view.cuh:43-52) with 4-byte accesses.
#pragma once

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <type_traits>

#include "ew_tile_tma.cuh"
#include "nt_core.cuh"
#include "tf32_split.cuh"

namespace ntb {

constexpr int EW_MAX_IN = 3;

struct EwParams {
  int ndim;                               // collapsed dims, 0..8 (0 => single element)
  int64_t numel;
  int64_t shape[NT_MAX_DIMS];
  // 32-bit index path: n / shape[d] == __umulhi(n, div_mul[d]) >> div_shift[d] for every n < 2^31
  // (div_mul == 0 marks an extent of 1)
  uint32_t div_mul[NT_MAX_DIMS];
  uint32_t div_shift[NT_MAX_DIMS];
  int64_t strides[EW_MAX_IN + 1][NT_MAX_DIMS]; // [0] = output
  void *out;                              // already advanced by the view offset
  const void *in[EW_MAX_IN];              // already advanced by the view offsets
  // per operand: 0 = four scalar accesses, 1 = one 128-bit access, 2 = one scalar access (stride 0)
  int vec_mode[EW_MAX_IN + 1];
  // tile2d only: non-zero => the operand is unit-stride along dim ndim-2 and is staged through
  // shared-memory slot (value - 1)
  int col_major[EW_MAX_IN + 1];
};

__device__ __forceinline__ float4 ld_stream(const float4 *p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float4 *p, float4 v) { __stcs(p, v); }

// ---------------------------------------------------------------------------------------------
// Contiguous fp32-sized kernel.  TI/TO are 4-byte types.
template <class F, int NIN>
__global__ void __launch_bounds__(256) ew_contig(F f, typename F::out_t *out, const typename F::in_t *a,
                                                 const typename F::in_t *b, const typename F::in_t *c, int64_t n) {
  // no __restrict__: in-place ops pass the same pointer as `out` and `a`
  using TI = typename F::in_t;
  using TO = typename F::out_t;
  static_assert(sizeof(TI) == 4 && sizeof(TO) == 4, "vector path is for 4-byte types");
  constexpr int UNROLL = 4;
  const int64_t nvec = n >> 2;
  const int64_t base = (int64_t(blockIdx.x) * UNROLL) * blockDim.x + threadIdx.x;
  float4 va[UNROLL], vb[UNROLL], vc[UNROLL];
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    int64_t i = base + int64_t(u) * blockDim.x;
    if (i < nvec) {
      va[u] = ld_stream(reinterpret_cast<const float4 *>(a) + i);
      if constexpr (NIN >= 2) vb[u] = ld_stream(reinterpret_cast<const float4 *>(b) + i);
      if constexpr (NIN >= 3) vc[u] = ld_stream(reinterpret_cast<const float4 *>(c) + i);
    }
  }
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    int64_t i = base + int64_t(u) * blockDim.x;
    if (i < nvec) {
      const TI *pa = reinterpret_cast<const TI *>(&va[u]);
      const TI *pb = reinterpret_cast<const TI *>(&vb[u]);
      const TI *pc = reinterpret_cast<const TI *>(&vc[u]);
      float4 r;
      TO *pr = reinterpret_cast<TO *>(&r);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if constexpr (NIN == 1) pr[e] = f(pa[e]);
        if constexpr (NIN == 2) pr[e] = f(pa[e], pb[e]);
        if constexpr (NIN == 3) pr[e] = f(pa[e], pb[e], pc[e]);
      }
      st_stream(reinterpret_cast<float4 *>(out) + i, r);
    }
  }
  // ragged tail (n % 4 elements) by the first threads of block 0
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    int64_t i = (nvec << 2) + threadIdx.x;
    if constexpr (NIN == 1) out[i] = f(a[i]);
    if constexpr (NIN == 2) out[i] = f(a[i], b[i]);
    if constexpr (NIN == 3) out[i] = f(a[i], b[i], c[i]);
  }
}

// ew_contig for an fp32 result that the next kernel will multiply on the tensor cores: besides the result it
// writes the result's two TF32 planes (hi at `hi`, lo at `lo`, same indexing as `out`), so that the
// GEMM's operand split -- a read of the result and a write of both planes in a launch of its own --
// never runs.  n is a multiple of 4.
template <class F, int NIN>
__global__ void __launch_bounds__(256) ew_contig_planes(F f, float *out, const float *a, const float *b, int64_t n,
                                                        float *hi, float *lo) {
  constexpr int UNROLL = 4;
  const int64_t nvec = n >> 2;
  const int64_t base = (int64_t(blockIdx.x) * UNROLL) * blockDim.x + threadIdx.x;
  float4 va[UNROLL], vb[UNROLL];
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    int64_t i = base + int64_t(u) * blockDim.x;
    if (i < nvec) {
      va[u] = ld_stream(reinterpret_cast<const float4 *>(a) + i);
      if constexpr (NIN >= 2) vb[u] = ld_stream(reinterpret_cast<const float4 *>(b) + i);
    }
  }
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    int64_t i = base + int64_t(u) * blockDim.x;
    if (i < nvec) {
      float4 r;
      if constexpr (NIN == 1) r = make_float4(f(va[u].x), f(va[u].y), f(va[u].z), f(va[u].w));
      else r = make_float4(f(va[u].x, vb[u].x), f(va[u].y, vb[u].y), f(va[u].z, vb[u].z), f(va[u].w, vb[u].w));
      reinterpret_cast<float4 *>(out)[i] = r; // read again soon (backward, the next product): no streaming hint
      const float h0 = split_hi(r.x), h1 = split_hi(r.y), h2 = split_hi(r.z), h3 = split_hi(r.w);
      reinterpret_cast<float4 *>(hi)[i] = make_float4(h0, h1, h2, h3);
      reinterpret_cast<float4 *>(lo)[i] = make_float4(split_lo(r.x, h0), split_lo(r.y, h1), split_lo(r.z, h2), split_lo(r.w, h3));
    }
  }
}

// [R, C] op [C]: one operand is a single row broadcast over the rows of the other (a bias, a per-column scale).
// The contiguous kernel with the row operand indexed modulo the row length -- it stays in the L1 -- instead of the
// general strided kernel's per-dim index arithmetic.  C % 4 == 0, fewer than 2^31 vectors.  ROW_FIRST: the row is
// the first argument of f.
template <class F, bool ROW_FIRST>
__global__ void __launch_bounds__(256) ew_contig_rowbcast(F f, float *out, const float *a, const float *row, int64_t nvec,
                                                          uint32_t cvec, uint32_t div_mul, uint32_t div_shift) {
  constexpr int UNROLL = 4;
  const int64_t base = (int64_t(blockIdx.x) * UNROLL) * blockDim.x + threadIdx.x;
  float4 va[UNROLL], vr[UNROLL];
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    const int64_t i = base + int64_t(u) * blockDim.x;
    if (i < nvec) {
      va[u] = ld_stream(reinterpret_cast<const float4 *>(a) + i);
      const uint32_t lin = uint32_t(i);
      const uint32_t quo = div_mul ? (__umulhi(lin, div_mul) >> div_shift) : lin;
      vr[u] = __ldg(reinterpret_cast<const float4 *>(row) + (lin - quo * cvec));
    }
  }
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    const int64_t i = base + int64_t(u) * blockDim.x;
    if (i < nvec) {
      const float4 x = va[u], r = vr[u];
      float4 y;
      if constexpr (ROW_FIRST) y = make_float4(f(r.x, x.x), f(r.y, x.y), f(r.z, x.z), f(r.w, x.w));
      else y = make_float4(f(x.x, r.x), f(x.y, r.y), f(x.z, r.z), f(x.w, r.w));
      st_stream(reinterpret_cast<float4 *>(out) + i, y);
    }
  }
}

// A unary op on one broadcast row: out[r][c] = f(row[c]) for every r (write-only apart from the row).
template <class F>
__global__ void __launch_bounds__(256) ew_contig_rowbcast1(F f, float *out, const float *row, int64_t nvec, uint32_t cvec,
                                                           uint32_t div_mul, uint32_t div_shift) {
  constexpr int UNROLL = 4;
  const int64_t base = (int64_t(blockIdx.x) * UNROLL) * blockDim.x + threadIdx.x;
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    const int64_t i = base + int64_t(u) * blockDim.x;
    if (i < nvec) {
      const uint32_t lin = uint32_t(i);
      const uint32_t quo = div_mul ? (__umulhi(lin, div_mul) >> div_shift) : lin;
      const float4 r = __ldg(reinterpret_cast<const float4 *>(row) + (lin - quo * cvec));
      st_stream(reinterpret_cast<float4 *>(out) + i, make_float4(f(r.x), f(r.y), f(r.z), f(r.w)));
    }
  }
}

// Two results from three contiguous fp32 inputs in one pass (the two gradients of a binary op: g, x1, x2
// -> dx1, dx2; 20 bytes per element instead of the 24 of two launches).  f(g, x1, x2, &r1, &r2).
template <class F>
__global__ void __launch_bounds__(256) ew_contig_two(F f, float *out1, float *out2, const float *g, const float *x1,
                                                     const float *x2, int64_t n) {
  constexpr int UNROLL = 2;
  const int64_t nvec = n >> 2;
  const int64_t base = (int64_t(blockIdx.x) * UNROLL) * blockDim.x + threadIdx.x;
  float4 vg[UNROLL], v1[UNROLL], v2[UNROLL];
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    int64_t i = base + int64_t(u) * blockDim.x;
    if (i < nvec) {
      vg[u] = ld_stream(reinterpret_cast<const float4 *>(g) + i);
      v1[u] = ld_stream(reinterpret_cast<const float4 *>(x1) + i);
      v2[u] = ld_stream(reinterpret_cast<const float4 *>(x2) + i);
    }
  }
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) {
    int64_t i = base + int64_t(u) * blockDim.x;
    if (i < nvec) {
      float4 r1, r2;
      f(vg[u].x, v1[u].x, v2[u].x, &r1.x, &r2.x);
      f(vg[u].y, v1[u].y, v2[u].y, &r1.y, &r2.y);
      f(vg[u].z, v1[u].z, v2[u].z, &r1.z, &r2.z);
      f(vg[u].w, v1[u].w, v2[u].w, &r1.w, &r2.w);
      st_stream(reinterpret_cast<float4 *>(out1) + i, r1);
      st_stream(reinterpret_cast<float4 *>(out2) + i, r2);
    }
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    int64_t i = (nvec << 2) + threadIdx.x;
    f(g[i], x1[i], x2[i], out1 + i, out2 + i);
  }
}

// ---------------------------------------------------------------------------------------------
// Strided kernel.  IDX is uint32_t when every extent and offset fits, else uint64_t.
// VEC == 4: a thread owns UNROLL groups of 4 consecutive elements of the innermost dim (groups of
// one block are interleaved so that a warp touches consecutive vectors); all loads are issued before
// the first use.  VEC == 1: one element per thread, any dtype.
// ND > 0: the number of collapsed dims is known at compile time (the loop unrolls and every extent,
// reciprocal and stride is read straight from the constant bank); ND == 0: any ndim.
template <class IDX, int NOPS, int ND = 0>
__device__ __forceinline__ void ew_offsets(const EwParams &p, IDX lin, int64_t (&off)[NOPS]) {
#pragma unroll
  for (int o = 0; o < NOPS; ++o) off[o] = 0;
  const int nd = (ND > 0) ? ND : p.ndim;
#pragma unroll
  for (int d = nd - 1; d >= 0; --d) {
    IDX ext = IDX(p.shape[d]);
    IDX q;
    if constexpr (sizeof(IDX) == 4) // multiply-high by a precomputed reciprocal instead of a division
      q = p.div_mul[d] ? (__umulhi(lin, p.div_mul[d]) >> p.div_shift[d]) : lin;
    else
      q = lin / ext;
    IDX r = lin - q * ext;
    lin = q;
#pragma unroll
    for (int o = 0; o < NOPS; ++o) off[o] += int64_t(r) * p.strides[o][d];
  }
}

// Reciprocal of a divisor d >= 1 for the 32-bit path above: with p = 31 + ceil(log2 d) and
// m = ceil(2^p / d) < 2^32, floor(n / d) == (n * m) >> p for all 0 <= n < 2^31.
inline void ew_fast_divisor(int64_t d, uint32_t *mul, uint32_t *shift) {
  if (d <= 1) {
    *mul = 0;
    *shift = 0;
    return;
  }
  int cl = 0;
  while ((int64_t(1) << cl) < d) ++cl;
  const int p = 31 + cl;
  const unsigned __int128 one = 1;
  const unsigned __int128 m = ((one << p) + (unsigned __int128)d - 1) / (unsigned __int128)d;
  *mul = uint32_t(m);
  *shift = uint32_t(p - 32);
}

template <class F, int NIN, int VEC, class IDX, int ND = 0>
__global__ void __launch_bounds__(256) ew_strided(F f, EwParams p) {
  using TI = typename F::in_t;
  using TO = typename F::out_t;
  if constexpr (VEC == 1) {
    int64_t t = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= p.numel) return;
    int64_t off[NIN + 1];
    ew_offsets<IDX, NIN + 1>(p, IDX(t), off);
    const TI *in[NIN];
#pragma unroll
    for (int o = 0; o < NIN; ++o) in[o] = static_cast<const TI *>(p.in[o]) + off[o + 1];
    TO *out = static_cast<TO *>(p.out) + off[0];
    if constexpr (NIN == 1) *out = f(*in[0]);
    if constexpr (NIN == 2) *out = f(*in[0], *in[1]);
    if constexpr (NIN == 3) *out = f(*in[0], *in[1], *in[2]);
  } else {
    static_assert(sizeof(TI) == 4 && sizeof(TO) == 4, "vector path is for 4-byte types");
    constexpr int UNROLL = 4;
    const int64_t nvec = p.numel / VEC;
    const int last = ((ND > 0) ? ND : p.ndim) - 1;
    const int64_t base = (int64_t(blockIdx.x) * UNROLL) * blockDim.x + threadIdx.x;
    TI v[UNROLL][NIN][4];
    int64_t out_off[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int64_t t = base + int64_t(u) * blockDim.x;
      if (t >= nvec) continue;
      int64_t off[NIN + 1];
      ew_offsets<IDX, NIN + 1, ND>(p, IDX(t) * VEC, off);
      out_off[u] = off[0];
#pragma unroll
      for (int o = 0; o < NIN; ++o) {
        const TI *src = static_cast<const TI *>(p.in[o]) + off[o + 1];
        const int mode = p.vec_mode[o + 1];
        if (mode == 1) {
          float4 x = *reinterpret_cast<const float4 *>(src);
          const TI *px = reinterpret_cast<const TI *>(&x);
#pragma unroll
          for (int e = 0; e < 4; ++e) v[u][o][e] = px[e];
        } else if (mode == 2) {
          TI x = *src;
#pragma unroll
          for (int e = 0; e < 4; ++e) v[u][o][e] = x;
        } else {
          const int64_t s = p.strides[o + 1][last];
#pragma unroll
          for (int e = 0; e < 4; ++e) v[u][o][e] = src[e * s];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int64_t t = base + int64_t(u) * blockDim.x;
      if (t >= nvec) continue;
      TO r[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if constexpr (NIN == 1) r[e] = f(v[u][0][e]);
        if constexpr (NIN == 2) r[e] = f(v[u][0][e], v[u][1][e]);
        if constexpr (NIN == 3) r[e] = f(v[u][0][e], v[u][1][e], v[u][2][e]);
      }
      TO *out = static_cast<TO *>(p.out) + out_off[u];
      if (p.vec_mode[0] == 1) {
        __stcs(reinterpret_cast<float4 *>(out), *reinterpret_cast<const float4 *>(r));
      } else {
        const int64_t s = p.strides[0][last];
#pragma unroll
        for (int e = 0; e < 4; ++e) out[e * s] = r[e];
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// 2-D tile kernel (fp32-sized types).  Grid: x = tiles along the last dim (J), y = tiles along the
// second-to-last (I), z = product of the leading dims.  256 threads own a 64x64 tile; in output
// order a thread holds rows ty+16r (r=0..3), columns 4*tx..4*tx+3.
constexpr int TILE = 64;
constexpr int TILE_PITCH = TILE + 1;
// Shared memory is dynamic: one TILE x (TILE+1) slot per staged (column-major) operand, so that a launch
// with a single transposed operand holds 8 CTAs per SM instead of 6.  The row-major operands' global
// loads are issued before the staging barrier: their latency overlaps the staging of the tile.
template <class F, int NIN>
__global__ void __launch_bounds__(256, 4) ew_tile2d(F f, EwParams p) {
  using TI = typename F::in_t;
  using TO = typename F::out_t;
  static_assert(sizeof(TI) == 4 && sizeof(TO) == 4, "tile path is for 4-byte types");
  extern __shared__ __align__(16) unsigned char tile_raw[];
  TI(*tile)[TILE][TILE_PITCH] = reinterpret_cast<TI(*)[TILE][TILE_PITCH]>(tile_raw);

  const int dI = p.ndim - 2, dJ = p.ndim - 1;
  const int64_t nI = p.shape[dI], nJ = p.shape[dJ];
  const int64_t i0 = int64_t(blockIdx.y) * TILE, j0 = int64_t(blockIdx.x) * TILE;

  // leading dims -> per-operand base offsets
  int64_t base[NIN + 1];
#pragma unroll
  for (int o = 0; o <= NIN; ++o) base[o] = 0;
  {
    int64_t lin = blockIdx.z;
    for (int d = p.ndim - 3; d >= 0; --d) {
      int64_t q = lin / p.shape[d];
      int64_t r = lin - q * p.shape[d];
      lin = q;
#pragma unroll
      for (int o = 0; o <= NIN; ++o) base[o] += r * p.strides[o][d];
    }
  }

  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;

  // (1) row-major operands: this thread's output-order values (rows ty+16r, columns 4tx..4tx+3), loaded now
  TI v[4][NIN][4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int64_t i = i0 + ty + 16 * r;
    const int64_t j = j0 + 4 * tx;
    const bool live = i < nI && j < nJ;
    const bool full = (j + 3 < nJ);
#pragma unroll
    for (int o = 0; o < NIN; ++o) {
      if (p.col_major[o + 1] || !live) continue;
      const TI *src = static_cast<const TI *>(p.in[o]) + base[o + 1] + i * p.strides[o + 1][dI];
      const int64_t sJ = p.strides[o + 1][dJ];
      if (sJ == 0) {
        TI x = *src;
#pragma unroll
        for (int e = 0; e < 4; ++e) v[r][o][e] = x;
      } else if (p.vec_mode[o + 1] == 1 && full) {
        float4 x = __ldcs(reinterpret_cast<const float4 *>(src + j));
        const TI *px = reinterpret_cast<const TI *>(&x);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[r][o][e] = px[e];
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) v[r][o][e] = (j + e < nJ) ? src[(j + e) * sJ] : TI(0);
      }
    }
  }

  // (2) stage the column-major operands: read along I (their unit-stride dim), 4 elements per thread
#pragma unroll
  for (int o = 0; o < NIN; ++o) {
    if (p.col_major[o + 1]) {
      const int slot = p.col_major[o + 1] - 1;
      const TI *src = static_cast<const TI *>(p.in[o]) + base[o + 1];
      const int64_t sJ = p.strides[o + 1][dJ]; // stride along J; stride along I is 1
      float4 x[4];
      bool vec[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int64_t j = j0 + ty + 16 * r;
        const int64_t i = i0 + 4 * tx;
        vec[r] = j < nJ && p.vec_mode[o + 1] == 1 && i + 3 < nI;
        if (vec[r]) x[r] = __ldcs(reinterpret_cast<const float4 *>(src + j * sJ + i));
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int64_t j = j0 + ty + 16 * r;
        const int64_t i = i0 + 4 * tx;
        if (j >= nJ) continue;
        if (vec[r]) {
          const TI *px = reinterpret_cast<const TI *>(&x[r]);
#pragma unroll
          for (int e = 0; e < 4; ++e) tile[slot][ty + 16 * r][4 * tx + e] = px[e];
        } else {
          const TI *q = src + j * sJ + i;
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (i + e < nI) tile[slot][ty + 16 * r][4 * tx + e] = q[e];
        }
      }
    }
  }
  __syncthreads();

  // (3) transposed reads from the tile, the functor, coalesced stores
  TO *dst = static_cast<TO *>(p.out) + base[0];
  const int64_t oI = p.strides[0][dI], oJ = p.strides[0][dJ];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int64_t i = i0 + ty + 16 * r;
    const int64_t j = j0 + 4 * tx;
    if (i >= nI || j >= nJ) continue;
    const bool full = (j + 3 < nJ);
#pragma unroll
    for (int o = 0; o < NIN; ++o) {
      if (p.col_major[o + 1]) {
        const int slot = p.col_major[o + 1] - 1;
#pragma unroll
        for (int e = 0; e < 4; ++e) v[r][o][e] = tile[slot][4 * tx + e][ty + 16 * r];
      }
    }
    TO res[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if constexpr (NIN == 1) res[e] = f(v[r][0][e]);
      if constexpr (NIN == 2) res[e] = f(v[r][0][e], v[r][1][e]);
      if constexpr (NIN == 3) res[e] = f(v[r][0][e], v[r][1][e], v[r][2][e]);
    }
    TO *q = dst + i * oI + j * oJ;
    if (p.vec_mode[0] == 1 && full) {
      __stcs(reinterpret_cast<float4 *>(q), *reinterpret_cast<const float4 *>(res));
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (j + e < nJ) q[e * oJ] = res[e];
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Host-side planner + launcher.
inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Large fp32 operands with a transposed one among them go through the copy-engine pipeline of
// ew_tile_tma.cuh when every operand can be described by a tensor map: unit stride along J (row-major) or
// along I (column-major), all other strides and the base 16-byte aligned, no broadcast operand, at most one
// leading dim.  Returns false when the case does not qualify (the register-staged tile kernel takes it).
extern std::atomic<int> g_tile_pipeline; // nt_set_transposed_tile_pipeline
template <class F, int NIN>
bool ew_launch_tile_pipeline(F f, const IterSpace<NIN + 1> &it, float *out, const float *const *in, const int *col_major) {
  if (!g_tile_pipeline.load(std::memory_order_relaxed)) return false;
  if (it.ndim != 2 && it.ndim != 3) return false;
  const int dI = it.ndim - 2, dJ = it.ndim - 1;
  const int64_t nI = it.shape[dI], nJ = it.shape[dJ], lead = it.ndim == 3 ? it.shape[0] : 1;
  if (nI < 64 || nJ < 64 || it.numel < (int64_t(1) << 20) || nI > 0x7fffffffLL || nJ > 0x7fffffffLL || lead > 0x7fffffffLL)
    return false;
  constexpr int64_t MAX_STRIDE = int64_t(1) << 37; // elements: 2^39 bytes, below the 2^40 of a tensor map
  for (int o = 0; o <= NIN; ++o) {
    const void *base = o == 0 ? static_cast<const void *>(out) : static_cast<const void *>(in[o - 1]);
    if (!aligned16(base)) return false;
    const bool col = o > 0 && col_major[o] != 0;
    const int64_t unit = it.strides[o][col ? dI : dJ], other = it.strides[o][col ? dJ : dI];
    if (unit != 1 || other <= 0 || (other & 3) != 0 || other >= MAX_STRIDE) return false;
    if (it.ndim == 3) {
      const int64_t ls = it.strides[o][0];
      if (ls <= 0 || (ls & 3) != 0 || ls >= MAX_STRIDE) return false;
    }
  }
  auto map_of = [&](int o, bool prefetch_box = false) {
    const void *base = o == 0 ? static_cast<const void *>(out) : static_cast<const void *>(in[o - 1]);
    const bool col = o > 0 && col_major[o] != 0;
    const int64_t other = it.strides[o][col ? dJ : dI];
    const int64_t inner = col ? nI : nJ, rows = col ? nJ : nI;
    const int64_t ls = it.ndim == 3 ? it.strides[o][0] : other * rows;
    return tile_tma::make_map(base, inner, rows, lead, other, ls, o == 0 ? 8u : 64u, prefetch_box);
  };
  tile_tma::Args a{};
  a.tiles_i = int32_t(ceil_div(nI, tile_tma::T));
  a.tiles_j = int32_t(ceil_div(nJ, tile_tma::T));
  static const int group_log2 = [] {
    const char *e = getenv("NT_TILE_GROUP_LOG2");
    const int v = (e && *e) ? atoi(e) : 2;
    return v < 0 ? 0 : (v > 6 ? 6 : v);
  }();
  const int G = 1 << group_log2;
  a.group_log2 = group_log2;
  a.groups_j = (a.tiles_j + G - 1) / G;
  a.slots_per_lead = int64_t(G) * G * ((a.tiles_i + G - 1) / G) * a.groups_j;
  a.total = a.slots_per_lead * lead;
  for (int o = 0; o < NIN; ++o) a.col[o] = col_major[o + 1] != 0;
  a.wait_limit = wait_limit_clocks();
  a.error_flag = pipeline_error_flag();
  // Measured on [4096, 4096]: with two operands the L2 prefetch two rounds ahead gains 3 % (0.83 -> 0.86 of
  // the copy rate); with one operand it loses 8 % (the prefetches queue in front of the tile loads of a ring
  // that has less time per tile), so it is off there.  NT_TILE_PREFETCH overrides both.
  static const int prefetch_rounds = [] {
    const char *e = getenv("NT_TILE_PREFETCH");
    const int v = (e && *e) ? atoi(e) : (NIN == 2 ? 2 : 0);
    return v < 0 ? 0 : (v > 8 ? 8 : v);
  }();
  a.prefetch_rounds = prefetch_rounds;
  const CUtensorMap m_out = map_of(0), m0 = map_of(1), m1 = map_of(NIN == 2 ? 2 : 1);
  const CUtensorMap pf0 = map_of(1, true), pf1 = map_of(NIN == 2 ? 2 : 1, true);
  const size_t smem = tile_tma::smem_bytes(NIN);
  static bool configured = false; // one per instantiation
  if (!configured) {
    NT_CUDA_CHECK(cudaFuncSetAttribute(tile_tma::ew_tile_tma<F, NIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    configured = true;
  }
  const int64_t tiles = int64_t(a.tiles_i) * a.tiles_j * lead;
  const unsigned grid = unsigned(std::min<int64_t>(tiles, sm_count()));
  tile_tma::ew_tile_tma<F, NIN><<<grid, tile_tma::THREADS, smem, stream()>>>(f, m_out, m0, m1, pf0, pf1, a);
  check_launch("ew_tile_tma");
  return true;
}

// views[0] is the output view (for fresh outputs: contiguous, offset 0).
template <class F, int NIN> void ew_launch(F f, const nt_view *const (&views)[NIN + 1]) {
  using TI = typename F::in_t;
  using TO = typename F::out_t;
  IterSpace<NIN + 1> it = collapse<NIN + 1>(views);
  if (it.numel == 0) return;
  cudaStream_t st = stream();

  TO *out = static_cast<TO *>(views[0]->storage->data) + it.offset[0];
  const TI *in[EW_MAX_IN] = {nullptr, nullptr, nullptr};
  for (int o = 0; o < NIN; ++o) in[o] = static_cast<const TI *>(views[o + 1]->storage->data) + it.offset[o + 1];

  constexpr bool VECTOR_TYPES = (sizeof(TI) == 4 && sizeof(TO) == 4);

  // (1) every operand one contiguous run
  bool all_contig = it.ndim <= 1;
  if (all_contig && it.ndim == 1)
    for (int o = 0; o <= NIN; ++o) all_contig = all_contig && it.strides[o][0] == 1;
  if constexpr (VECTOR_TYPES) {
    bool al = aligned16(out);
    for (int o = 0; o < NIN; ++o) al = al && aligned16(in[o]);
    if (all_contig && al && it.numel >= 4) {
      int64_t nvec = it.numel >> 2;
      int64_t blocks = ceil_div(nvec, 256 * 4);
      ew_contig<F, NIN><<<unsigned(blocks), 256, 0, st>>>(f, out, in[0], in[1], in[2], it.numel);
      check_launch("ew_contig");
      return;
    }
  }

  // (1b) a dense [R, C] operand against one broadcast row
  if constexpr (NIN == 2 && std::is_same<TI, float>::value && std::is_same<TO, float>::value) {
    if (it.ndim == 2 && (it.shape[1] & 3) == 0 && (it.numel >> 2) < (int64_t(1) << 31) && it.strides[0][0] == it.shape[1] &&
        it.strides[0][1] == 1 && aligned16(out) && aligned16(in[0]) && aligned16(in[1])) {
      const int64_t C = it.shape[1];
      auto dense = [&](int o) { return it.strides[o][0] == C && it.strides[o][1] == 1; };
      auto row = [&](int o) { return it.strides[o][0] == 0 && it.strides[o][1] == 1; };
      const int which = (row(1) && dense(2)) ? 1 : (dense(1) && row(2)) ? 2 : 0;
      if (which) {
        uint32_t mul, shift;
        ew_fast_divisor(C >> 2, &mul, &shift);
        const int64_t nvec = it.numel >> 2;
        const unsigned blocks = unsigned(ceil_div(nvec, 256 * 4));
        if (which == 1)
          ew_contig_rowbcast<F, true><<<blocks, 256, 0, st>>>(f, out, in[1], in[0], nvec, uint32_t(C >> 2), mul, shift);
        else
          ew_contig_rowbcast<F, false><<<blocks, 256, 0, st>>>(f, out, in[0], in[1], nvec, uint32_t(C >> 2), mul, shift);
        check_launch("ew_contig_rowbcast");
        return;
      }
    }
  }

  if constexpr (NIN == 1 && std::is_same<TI, float>::value && std::is_same<TO, float>::value) {
    if (it.ndim == 2 && (it.shape[1] & 3) == 0 && (it.numel >> 2) < (int64_t(1) << 31) && it.strides[0][0] == it.shape[1] &&
        it.strides[0][1] == 1 && it.strides[1][0] == 0 && it.strides[1][1] == 1 && aligned16(out) && aligned16(in[0])) {
      uint32_t mul, shift;
      ew_fast_divisor(it.shape[1] >> 2, &mul, &shift);
      const int64_t nvec = it.numel >> 2;
      ew_contig_rowbcast1<F><<<unsigned(ceil_div(nvec, 256 * 4)), 256, 0, st>>>(f, out, in[0], nvec, uint32_t(it.shape[1] >> 2), mul, shift);
      check_launch("ew_contig_rowbcast1");
      return;
    }
  }

  EwParams p{};
  p.ndim = it.ndim;
  p.numel = it.numel;
  for (int d = 0; d < it.ndim; ++d) {
    p.shape[d] = it.shape[d];
    ew_fast_divisor(it.shape[d], &p.div_mul[d], &p.div_shift[d]);
    for (int o = 0; o <= NIN; ++o) p.strides[o][d] = it.strides[o][d];
  }
  p.out = out;
  for (int o = 0; o < NIN; ++o) p.in[o] = in[o];

  // 128-bit access along the last dim is legal for an operand when that dim has unit stride, the
  // base is 16-byte aligned and every other stride keeps rows 16-byte aligned.
  auto vec_ok = [&](int o, int unit_dim) {
    const void *base = (o == 0) ? static_cast<const void *>(out) : static_cast<const void *>(in[o - 1]);
    if (!aligned16(base)) return false;
    if (it.strides[o][unit_dim] != 1) return false;
    for (int d = 0; d < it.ndim; ++d)
      if (d != unit_dim && (it.strides[o][d] & 3) != 0) return false;
    return true;
  };

  if constexpr (VECTOR_TYPES) {
    // (2) a transposed operand: unit stride on the second-to-last dim, not on the last
    if (it.ndim >= 2) {
      const int dI = it.ndim - 2, dJ = it.ndim - 1;
      bool any_col = false, ok = true;
      int n_col = 0;
      for (int o = 1; o <= NIN; ++o) {
        bool col = it.strides[o][dI] == 1 && it.strides[o][dJ] != 1 && it.strides[o][dJ] != 0;
        p.col_major[o] = col ? ++n_col : 0; // 1-based shared-memory slot
        any_col = any_col || col;
      }
      if (n_col > 2) ok = false;
      // the output must be written along J for the tile mapping to pay off
      if (it.strides[0][dJ] != 1) ok = false;
      int64_t lead = 1;
      for (int d = 0; d < it.ndim - 2; ++d) lead *= it.shape[d];
      if (lead > 65535 || ceil_div(it.shape[dI], TILE) > 65535) ok = false;
      if (any_col && ok && it.shape[dI] >= 16 && it.shape[dJ] >= 16) {
        for (int o = 0; o <= NIN; ++o) {
          if (o > 0 && p.col_major[o])
            p.vec_mode[o] = vec_ok(o, dI) ? 1 : 0;
          else
            p.vec_mode[o] = vec_ok(o, dJ) ? 1 : 0;
        }
        if constexpr (NIN <= 2 && std::is_same<TI, float>::value && std::is_same<TO, float>::value) {
          if (ew_launch_tile_pipeline<F, NIN>(f, it, out, in, p.col_major)) return;
        }
        dim3 grid(unsigned(ceil_div(it.shape[dJ], TILE)), unsigned(ceil_div(it.shape[dI], TILE)), unsigned(lead));
        const size_t smem = size_t(n_col) * TILE * TILE_PITCH * sizeof(TI); // at most 2 slots = 33 KB: below the 48 KB default limit
        ew_tile2d<F, NIN><<<grid, 256, smem, st>>>(f, p);
        check_launch("ew_tile2d");
        return;
      }
      for (int o = 0; o <= NIN; ++o) p.col_major[o] = 0;
    }
  }

  // (3) general strided
  bool idx32 = it.numel < (int64_t(1) << 31);
  bool vec4 = false;
  if constexpr (VECTOR_TYPES) {
    if (it.ndim >= 1 && (it.shape[it.ndim - 1] & 3) == 0) {
      vec4 = true;
      const int last = it.ndim - 1;
      for (int o = 0; o <= NIN; ++o) {
        if (o > 0 && it.strides[o][last] == 0)
          p.vec_mode[o] = 2;
        else
          p.vec_mode[o] = vec_ok(o, last) ? 1 : 0;
      }
      // an output that aliases itself along the vector (stride 0) cannot be written 4-wide
      if (it.strides[0][last] == 0) vec4 = false;
    }
  }
  if (it.ndim == 0) { // single element
    p.ndim = 1;
    p.shape[0] = 1;
    for (int o = 0; o <= NIN; ++o) p.strides[o][0] = 1;
  }
  if constexpr (VECTOR_TYPES) {
    if (vec4) {
      int64_t blocks = ceil_div(it.numel / 4, 256 * 4);
      if (idx32 && p.ndim == 2) // the common case ([R, C] with a broadcast or sliced operand): unrolled index math
        ew_strided<F, NIN, 4, uint32_t, 2><<<unsigned(blocks), 256, 0, st>>>(f, p);
      else if (idx32)
        ew_strided<F, NIN, 4, uint32_t><<<unsigned(blocks), 256, 0, st>>>(f, p);
      else
        ew_strided<F, NIN, 4, uint64_t><<<unsigned(blocks), 256, 0, st>>>(f, p);
      check_launch("ew_strided");
      return;
    }
  }
  int64_t blocks = ceil_div(it.numel, 256);
  if (blocks > 0x7fffffffLL) fail_runtime("elementwise: tensor too large for one launch.");
  if (idx32)
    ew_strided<F, NIN, 1, uint32_t><<<unsigned(blocks), 256, 0, st>>>(f, p);
  else
    ew_strided<F, NIN, 1, uint64_t><<<unsigned(blocks), 256, 0, st>>>(f, p);
  check_launch("ew_strided");
}

// Builds the contiguous view of a freshly allocated result with the shape of `like`.
inline nt_view fresh_view(nt_storage *s, const nt_view &like) {
  nt_view v{};
  v.storage = s;
  v.ndim = like.ndim;
  int64_t st = 1;
  for (int d = like.ndim - 1; d >= 0; --d) {
    v.shape[d] = like.shape[d];
    v.strides[d] = st;
    st *= like.shape[d];
  }
  v.offset = 0;
  return v;
}

} // namespace ntb
