// nt_matmul: batched C[..., M, N] = A[..., M, K] x B[..., K, N] over arbitrary strided views.
//
// fp32 has three modes (nt_set_matmul_mode):
//   1 (default) 3xTF32 on the tcgen05 tensor cores with promoted accumulation, see gemm_tc.cu;
//   3           3xTF32 with one accumulation chain per output (1 % faster, 5-20x the rounding bias);
//   0           exact FP32 on the CUDA cores: 128x128x16 shared-memory tiles, 8x8 register
//               micro-tiles, register-prefetch double buffering, one FMA per multiply-add,
//               accumulated in ascending k -- the rounding of the reference's CUDA kernels
//               (src/cpp/ops/matmul.cu:60-205);
//   2           same kernel with separate multiply and add roundings: bit for bit the reference's
//               CPU triple loop (src/cpp/ops/matmul.cu:21-57).
// Operand tiles are read straight from the strided views -- vectorised along whichever of the two
// matrix dims has unit stride -- so the transposed views of MatmulOp.backward
// (autograd/ops_binary.py:265-266) and N % 4 != 0 never drop to a one-thread-per-output kernel as
// they do in the reference (src/cpp/ops/matmul.cu:218-233).
// Other dtypes (Int32/Int64/Float64) use a plain one-output-per-thread kernel.
#include "nt_core.cuh"

namespace ntb {

// implemented in gemm_tc.cu; returns false when the shape/layout is outside what it supports
bool gemm_3xtf32(const float *A, const float *B, float *C, int64_t batch, int64_t M, int64_t N, int64_t K,
                 int64_t a_sb, int64_t a_sm, int64_t a_sk, int64_t b_sb, int64_t b_sk, int64_t b_sn,
                 const float *bias, int64_t bias_stride, bool *bias_done);
void gemm_tc_set_promoted(bool on);
// mode 1 over natural-layout, cached operand planes; false when an operand has no unit-stride matrix dim
bool gemm_3xtf32_natural(nt_storage *sa, int64_t a_off, nt_storage *sb, int64_t b_off, float *C, int64_t batch, int64_t M,
                         int64_t N, int64_t K, int64_t a_sb, int64_t a_sm, int64_t a_sk, int64_t b_sb, int64_t b_sk,
                         int64_t b_sn, const float *bias, int64_t bias_stride, bool *bias_done);
void gemm_tc_set_operand_cache(bool on);
void gemm_tc_set_schedule(int max_splits, int panel);
void gemm_tc_pair_role(int role);
void gemm_tc_set_pair_overlap(bool on);
void gemm_tc_split_stats(uint64_t *launches, uint64_t *hits);
static std::atomic<int> g_natural_planes{1};

static std::atomic<int> g_matmul_mode{1};
static std::atomic<int64_t> g_tc_min_macs{int64_t(1) << 21}; // batch*M*N*K at or below this: exact FP32 kernel

constexpr int BM = 128, BN = 128, BK = 16;

struct BatchIndex {
  int ndim;
  int64_t shape[NT_MAX_DIMS];
  int64_t a_strides[NT_MAX_DIMS];
  int64_t b_strides[NT_MAX_DIMS];
};

enum LoadMode { LOAD_SCALAR = 0, LOAD_VEC_K = 1, LOAD_VEC_MN = 2 };

struct GemmArgs {
  const float *A, *B;
  float *C;
  int64_t M, N, K;
  int64_t a_sm, a_sk, b_sk, b_sn;
  BatchIndex batch;
  int c_vec; // C rows may be written 128 bits at a time
};

template <int AMODE, int BMODE, bool FUSED_MAD>
__global__ void __launch_bounds__(256) sgemm_tiled(GemmArgs g) {
  __shared__ __align__(16) float As[2][BK][BM];
  __shared__ __align__(16) float Bs[2][BK][BN];

  const int tid = threadIdx.x;
  const int64_t m0 = int64_t(blockIdx.y) * BM, n0 = int64_t(blockIdx.x) * BN;

  const float *A = g.A, *B = g.B;
  {
    int64_t lin = blockIdx.z;
    for (int d = g.batch.ndim - 1; d >= 0; --d) {
      int64_t q = lin / g.batch.shape[d];
      int64_t r = lin - q * g.batch.shape[d];
      lin = q;
      A += r * g.batch.a_strides[d];
      B += r * g.batch.b_strides[d];
    }
  }
  float *C = g.C + int64_t(blockIdx.z) * g.M * g.N;

  float ra[8], rb[8]; // staged global loads of the next k-tile

  auto load_a = [&](int64_t k0) {
    if constexpr (AMODE == LOAD_VEC_K) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int64_t m = m0 + (tid >> 2) + 64 * i, k = k0 + (tid & 3) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (m < g.M && k < g.K) v = *reinterpret_cast<const float4 *>(A + m * g.a_sm + k);
        ra[4 * i + 0] = v.x; ra[4 * i + 1] = v.y; ra[4 * i + 2] = v.z; ra[4 * i + 3] = v.w;
      }
    } else if constexpr (AMODE == LOAD_VEC_MN) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int64_t k = k0 + (tid >> 5) + 8 * i, m = m0 + (tid & 31) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (m < g.M && k < g.K) v = *reinterpret_cast<const float4 *>(A + k * g.a_sk + m);
        ra[4 * i + 0] = v.x; ra[4 * i + 1] = v.y; ra[4 * i + 2] = v.z; ra[4 * i + 3] = v.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int idx = tid + 256 * i;
        const int64_t m = m0 + (idx & (BM - 1)), k = k0 + (idx >> 7);
        ra[i] = (m < g.M && k < g.K) ? A[m * g.a_sm + k * g.a_sk] : 0.f;
      }
    }
  };
  auto load_b = [&](int64_t k0) {
    if constexpr (BMODE == LOAD_VEC_K) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int64_t n = n0 + (tid >> 2) + 64 * i, k = k0 + (tid & 3) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (n < g.N && k < g.K) v = *reinterpret_cast<const float4 *>(B + n * g.b_sn + k);
        rb[4 * i + 0] = v.x; rb[4 * i + 1] = v.y; rb[4 * i + 2] = v.z; rb[4 * i + 3] = v.w;
      }
    } else if constexpr (BMODE == LOAD_VEC_MN) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int64_t k = k0 + (tid >> 5) + 8 * i, n = n0 + (tid & 31) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (n < g.N && k < g.K) v = *reinterpret_cast<const float4 *>(B + k * g.b_sk + n);
        rb[4 * i + 0] = v.x; rb[4 * i + 1] = v.y; rb[4 * i + 2] = v.z; rb[4 * i + 3] = v.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int idx = tid + 256 * i;
        const int64_t n = n0 + (idx & (BN - 1)), k = k0 + (idx >> 7);
        rb[i] = (n < g.N && k < g.K) ? B[k * g.b_sk + n * g.b_sn] : 0.f;
      }
    }
  };
  auto store_a = [&](int buf) {
    if constexpr (AMODE == LOAD_VEC_K) {
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) As[buf][(tid & 3) * 4 + e][(tid >> 2) + 64 * i] = ra[4 * i + e];
    } else if constexpr (AMODE == LOAD_VEC_MN) {
#pragma unroll
      for (int i = 0; i < 2; ++i)
        *reinterpret_cast<float4 *>(&As[buf][(tid >> 5) + 8 * i][(tid & 31) * 4]) =
            make_float4(ra[4 * i], ra[4 * i + 1], ra[4 * i + 2], ra[4 * i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int idx = tid + 256 * i;
        As[buf][idx >> 7][idx & (BM - 1)] = ra[i];
      }
    }
  };
  auto store_b = [&](int buf) {
    if constexpr (BMODE == LOAD_VEC_K) {
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) Bs[buf][(tid & 3) * 4 + e][(tid >> 2) + 64 * i] = rb[4 * i + e];
    } else if constexpr (BMODE == LOAD_VEC_MN) {
#pragma unroll
      for (int i = 0; i < 2; ++i)
        *reinterpret_cast<float4 *>(&Bs[buf][(tid >> 5) + 8 * i][(tid & 31) * 4]) =
            make_float4(rb[4 * i], rb[4 * i + 1], rb[4 * i + 2], rb[4 * i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int idx = tid + 256 * i;
        Bs[buf][idx >> 7][idx & (BN - 1)] = rb[i];
      }
    }
  };

  // thread (ty, tx) owns rows {4ty..4ty+3, 64+4ty..} and columns {4tx..4tx+3, 64+4tx..}
  const int ty = tid >> 4, tx = tid & 15;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  load_a(0);
  load_b(0);
  store_a(0);
  store_b(0);
  __syncthreads();

  int buf = 0;
  for (int64_t k0 = 0; k0 < g.K; k0 += BK) {
    const bool more = (k0 + BK < g.K);
    if (more) {
      load_a(k0 + BK);
      load_b(k0 + BK);
    }
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float4 a_lo = *reinterpret_cast<const float4 *>(&As[buf][k][4 * ty]);
      float4 a_hi = *reinterpret_cast<const float4 *>(&As[buf][k][64 + 4 * ty]);
      float4 b_lo = *reinterpret_cast<const float4 *>(&Bs[buf][k][4 * tx]);
      float4 b_hi = *reinterpret_cast<const float4 *>(&Bs[buf][k][64 + 4 * tx]);
      const float av[8] = {a_lo.x, a_lo.y, a_lo.z, a_lo.w, a_hi.x, a_hi.y, a_hi.z, a_hi.w};
      const float bv[8] = {b_lo.x, b_lo.y, b_lo.z, b_lo.w, b_hi.x, b_hi.y, b_hi.z, b_hi.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if constexpr (FUSED_MAD) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
          else acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(av[i], bv[j]));
        }
    }
    if (more) {
      store_a(buf ^ 1);
      store_b(buf ^ 1);
      __syncthreads();
      buf ^= 1;
    }
  }

#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int64_t m = m0 + ((i < 4) ? (4 * ty + i) : (64 + 4 * ty + i - 4));
    if (m >= g.M) continue;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int64_t n = n0 + 64 * h + 4 * tx;
      float *dst = C + m * g.N + n;
      if (g.c_vec && n + 3 < g.N) {
        *reinterpret_cast<float4 *>(dst) = make_float4(acc[i][4 * h], acc[i][4 * h + 1], acc[i][4 * h + 2], acc[i][4 * h + 3]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (n + e < g.N) dst[e] = acc[i][4 * h + e];
      }
    }
  }
}

// One output element per thread, any arithmetic dtype (the shape of the reference's fallback).
template <class T>
__global__ void matmul_naive(const T *A, const T *B, T *C, int64_t M, int64_t N, int64_t K, int64_t a_sm, int64_t a_sk,
                             int64_t b_sk, int64_t b_sn, BatchIndex batch, int64_t total) {
  int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  int64_t n = i % N, r = i / N;
  int64_t m = r % M;
  int64_t lin = r / M;
  for (int d = batch.ndim - 1; d >= 0; --d) {
    int64_t q = lin / batch.shape[d];
    int64_t c = lin - q * batch.shape[d];
    lin = q;
    A += c * batch.a_strides[d];
    B += c * batch.b_strides[d];
  }
  T acc = 0;
  for (int64_t k = 0; k < K; ++k) acc += A[m * a_sm + k * a_sk] * B[k * b_sk + n * b_sn];
  C[i] = acc;
}

static bool al16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <int AMODE, int BMODE> static void launch_simt(const GemmArgs &g, dim3 grid, bool fused) {
  if (fused)
    sgemm_tiled<AMODE, BMODE, true><<<grid, 256, 0, stream()>>>(g);
  else
    sgemm_tiled<AMODE, BMODE, false><<<grid, 256, 0, stream()>>>(g);
}

static void sgemm_simt(GemmArgs g, int64_t nbatch, bool fused) {
  bool batch_al = true;
  for (int d = 0; d < g.batch.ndim; ++d) batch_al = batch_al && (g.batch.a_strides[d] % 4 == 0);
  int amode = LOAD_SCALAR;
  if (al16(g.A) && batch_al) {
    if (g.a_sk == 1 && g.K % 4 == 0 && g.a_sm % 4 == 0) amode = LOAD_VEC_K;
    else if (g.a_sm == 1 && g.M % 4 == 0 && g.a_sk % 4 == 0) amode = LOAD_VEC_MN;
  }
  batch_al = true;
  for (int d = 0; d < g.batch.ndim; ++d) batch_al = batch_al && (g.batch.b_strides[d] % 4 == 0);
  int bmode = LOAD_SCALAR;
  if (al16(g.B) && batch_al) {
    if (g.b_sn == 1 && g.N % 4 == 0 && g.b_sk % 4 == 0) bmode = LOAD_VEC_MN;
    else if (g.b_sk == 1 && g.K % 4 == 0 && g.b_sn % 4 == 0) bmode = LOAD_VEC_K;
  }
  g.c_vec = (g.N % 4 == 0) ? 1 : 0;
  if (nbatch > 65535 || ceil_div(g.M, BM) > 65535) fail_runtime("matmul: too many tiles for one launch.");
  dim3 grid{unsigned(ceil_div(g.N, BN)), unsigned(ceil_div(g.M, BM)), unsigned(nbatch)};
#define NT_CASE(a, b)                                                                              \
  if (amode == a && bmode == b) {                                                                  \
    launch_simt<a, b>(g, grid, fused);                                                             \
  } else
  NT_CASE(LOAD_SCALAR, LOAD_SCALAR)
  NT_CASE(LOAD_SCALAR, LOAD_VEC_K)
  NT_CASE(LOAD_SCALAR, LOAD_VEC_MN)
  NT_CASE(LOAD_VEC_K, LOAD_SCALAR)
  NT_CASE(LOAD_VEC_K, LOAD_VEC_K)
  NT_CASE(LOAD_VEC_K, LOAD_VEC_MN)
  NT_CASE(LOAD_VEC_MN, LOAD_SCALAR)
  NT_CASE(LOAD_VEC_MN, LOAD_VEC_K)
  NT_CASE(LOAD_VEC_MN, LOAD_VEC_MN) {}
#undef NT_CASE
  check_launch("sgemm_tiled");
}

} // namespace ntb

using namespace ntb;

extern "C" {

int nt_set_matmul_mode(int mode) {
  NT_API_BEGIN
  if (mode < 0 || mode > 3)
    fail_invalid("matmul mode must be 0 (exact fp32), 1 (3xTF32), 2 (fp32, unfused multiply-add) or 3 (3xTF32, single accumulation chain).");
  g_matmul_mode.store(mode);
  gemm_tc_set_promoted(mode == 1);
  NT_API_END
}
int nt_get_matmul_mode(void) { return g_matmul_mode.load(); }
int nt_set_matmul_schedule(int max_splits, int panel) {
  NT_API_BEGIN
  if (max_splits < 1 || max_splits > 8) fail_invalid("nt_set_matmul_schedule: max_splits must be 1..8.");
  if (panel < 0) fail_invalid("nt_set_matmul_schedule: negative panel width.");
  gemm_tc_set_schedule(max_splits, panel);
  NT_API_END
}
int nt_set_matmul_tc_min_macs(int64_t macs) {
  NT_API_BEGIN
  if (macs < 0) fail_invalid("nt_set_matmul_tc_min_macs: negative.");
  g_tc_min_macs.store(macs);
  NT_API_END
}
int64_t nt_get_matmul_tc_min_macs(void) { return g_tc_min_macs.load(); }

int nt_set_matmul_operand_planes(int natural, int cached) {
  NT_API_BEGIN
  g_natural_planes.store(natural ? 1 : 0);
  gemm_tc_set_operand_cache(cached != 0);
  NT_API_END
}
int nt_matmul_split_stats(uint64_t *split_launches, uint64_t *cache_hits) {
  NT_API_BEGIN
  gemm_tc_split_stats(split_launches, cache_hits);
  NT_API_END
}
int nt_wait_probe(void) {
  NT_API_BEGIN
  gemm_tc_wait_probe();
  NT_API_END
}

// x1 @ x2, plus -- when `bias` is given (fp32, N values) -- the broadcast add of the bias as a second
// rounded step: in the tensor-core kernel's epilogue where that kernel runs, by an in-place add launch
// otherwise.  Either way the bits are those of matmul followed by add.
static nt_storage *matmul_impl(const nt_view *x1, const nt_view *x2, const nt_view *bias) {
  check_view(x1, "matmul");
  check_view(x2, "matmul");
  require_same_device(x1, x2, "matmul");
  require_same_dtype(x1, x2, "matmul");
  if (x1->ndim != x2->ndim) fail_invalid("matmul: x1 and x2 have different ndim.");
  if (x1->ndim < 2) fail_invalid("matmul: kernel should be called with >=2d tensors.");
  const int nd = x1->ndim;
  BatchIndex bi{};
  int64_t nbatch = 1;
  for (int d = 0; d < nd - 2; ++d) {
    if (x1->shape[d] != x2->shape[d]) fail_invalid("Invalid broacast shapes.");
    if (x1->shape[d] == 1) continue;
    bi.shape[bi.ndim] = x1->shape[d];
    bi.a_strides[bi.ndim] = x1->strides[d];
    bi.b_strides[bi.ndim] = x2->strides[d];
    ++bi.ndim;
    nbatch *= x1->shape[d];
  }
  const int64_t M = x1->shape[nd - 2], K = x1->shape[nd - 1], N = x2->shape[nd - 1];
  if (K != x2->shape[nd - 2]) fail_invalid("Invalid matmul shape.");
  require_cuda(x1, "matmul");
  const int dt = x1->storage->dtype;
  if (dt == NT_BOOL) fail_invalid("Invalid dtype.");

  const int64_t total = nbatch * M * N;
  StorageRef o(storage_new(total, dt, NT_CUDA));
  if (total == 0) return o.release();
  bool bias_done = false;
  const int64_t a_sm = x1->strides[nd - 2], a_sk = x1->strides[nd - 1];
  const int64_t b_sk = x2->strides[nd - 2], b_sn = x2->strides[nd - 1];

  if (dt == NT_FLOAT32) {
    GemmArgs g{};
    g.A = static_cast<const float *>(x1->storage->data) + x1->offset;
    g.B = static_cast<const float *>(x2->storage->data) + x2->offset;
    g.C = static_cast<float *>(o->data);
    g.M = M; g.N = N; g.K = K;
    g.a_sm = a_sm; g.a_sk = a_sk; g.b_sk = b_sk; g.b_sn = b_sn;
    g.batch = bi;
    const int mode = g_matmul_mode.load();
    bool done = false;
    // Tiny products (a single tile of the exact kernel) take the exact FP32 kernel: one launch instead of
    // up to three, and the full fp32 accuracy of the reference's own CUDA kernels on the small cases.
    const bool big_enough = double(nbatch) * double(M) * double(N) * double(K) > double(g_tc_min_macs.load());
    if ((mode == 1 || mode == 3) && K > 0 && big_enough) {
      // the tensor-core path takes a single (collapsed) batch stride per operand
      int64_t a_sb = 0, b_sb = 0;
      bool single = true;
      if (bi.ndim == 1) {
        a_sb = bi.a_strides[0];
        b_sb = bi.b_strides[0];
      } else if (bi.ndim > 1) {
        // mergeable batch dims: stride[d] == stride[d+1] * shape[d+1]
        for (int d = 0; d + 1 < bi.ndim; ++d)
          if (bi.a_strides[d] != bi.a_strides[d + 1] * bi.shape[d + 1] ||
              bi.b_strides[d] != bi.b_strides[d + 1] * bi.shape[d + 1])
            single = false;
        a_sb = bi.a_strides[bi.ndim - 1];
        b_sb = bi.b_strides[bi.ndim - 1];
      }
      const float *bp = bias ? static_cast<const float *>(bias->storage->data) + bias->offset : nullptr;
      if (single && mode == 1 && g_natural_planes.load())
        done = gemm_3xtf32_natural(x1->storage, x1->offset, x2->storage, x2->offset, g.C, nbatch, M, N, K, a_sb, a_sm,
                                   a_sk, b_sb, b_sk, b_sn, bp, bias ? bias->strides[0] : 0, &bias_done);
      if (single && !done)
        done = gemm_3xtf32(g.A, g.B, g.C, nbatch, M, N, K, a_sb, a_sm, a_sk, b_sb, b_sk, b_sn, bp,
                           bias ? bias->strides[0] : 0, &bias_done);
    }
    if (!done) {
      matmul_profile_begin();
      sgemm_simt(g, nbatch, /*fused=*/mode != 2);
      matmul_profile_end();
    }
  } else {
    dispatch_arith(dt, [&]<class T>() {
      if constexpr (!std::is_same_v<T, float>) {
        const T *A = static_cast<const T *>(x1->storage->data) + x1->offset;
        const T *B = static_cast<const T *>(x2->storage->data) + x2->offset;
        int64_t blocks = ceil_div(total, 256);
        if (blocks > 0x7fffffffLL) fail_runtime("matmul: output too large for one launch.");
        matmul_naive<T><<<unsigned(blocks), 256, 0, stream()>>>(A, B, static_cast<T *>(o->data), M, N, K, a_sm, a_sk,
                                                                b_sk, b_sn, bi, total);
        check_launch("matmul_naive");
      }
    });
  }
  if (bias && !bias_done) {
    // out += bias (broadcast over the rows) through the ordinary in-place add
    nt_view ov{}, bv{};
    ov.storage = o.s;
    ov.ndim = nd;
    bv.storage = bias->storage;
    bv.ndim = nd;
    bv.offset = bias->offset;
    int64_t acc = 1;
    for (int d = nd - 1; d >= 0; --d) {
      ov.shape[d] = bv.shape[d] = (d == nd - 1) ? N : (d == nd - 2 ? M : x1->shape[d]);
      ov.strides[d] = acc;
      acc *= ov.shape[d];
      bv.strides[d] = (d == nd - 1) ? bias->strides[0] : 0;
    }
    if (nt_add_inplace(&ov, &bv) != NT_OK) fail_runtime(std::string("linear: bias add failed: ") + nt_last_error());
    o->version = 0; // a fresh result, not a mutated tensor
  }
  return o.release();
}

int nt_matmul(const nt_view *x1, const nt_view *x2, nt_storage **out) {
  NT_API_BEGIN
  *out = matmul_impl(x1, x2, nullptr);
  NT_API_END
}

// Two independent products in one call (the two gradients of a product: g @ b^T and a^T @ g).  In mode 1 the second
// tensor-core launch is made the programmatic dependent of the first when nothing had to be launched in between,
// so its first CTAs run on the SMs that the first product's last wave leaves idle.  Results are those of two
// nt_matmul calls, bit for bit.
int nt_matmul_pair(const nt_view *a1, const nt_view *b1, const nt_view *a2, const nt_view *b2, nt_storage **out1,
                   nt_storage **out2) {
  NT_API_BEGIN
  *out1 = *out2 = nullptr;
  struct Leave {
    ~Leave() { gemm_tc_pair_role(0); }
  } leave;
  gemm_tc_pair_role(1);
  nt_storage *first = matmul_impl(a1, b1, nullptr);
  gemm_tc_pair_role(2);
  nt_storage *second = nullptr;
  try {
    second = matmul_impl(a2, b2, nullptr);
  } catch (...) {
    storage_release(first);
    throw;
  }
  *out1 = first;
  *out2 = second;
  NT_API_END
}
int nt_set_matmul_pair_overlap(int on) {
  NT_API_BEGIN
  gemm_tc_set_pair_overlap(on != 0);
  NT_API_END
}

int nt_linear(const nt_view *x, const nt_view *w, const nt_view *bias, nt_storage **out) {
  NT_API_BEGIN
  check_view(bias, "linear");
  check_view(w, "linear");
  if (bias->ndim != 1 || w->ndim < 2 || bias->shape[0] != w->shape[w->ndim - 1])
    fail_invalid("linear: bias must be 1-D with one value per output column.");
  if (bias->storage->dtype != NT_FLOAT32 || w->storage->dtype != NT_FLOAT32 || x->storage == nullptr ||
      x->storage->dtype != NT_FLOAT32)
    fail_invalid("linear: Float32 only.");
  require_cuda(bias, "linear");
  *out = matmul_impl(x, w, bias);
  NT_API_END
}

} // extern "C"
