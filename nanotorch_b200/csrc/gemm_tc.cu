// fp32 GEMM on the Blackwell tensor cores with 3xTF32 split precision.
//
//   C[b][m][n] = sum_k A[b][m][k] * B[b][k][n],  every operand fp32, result within fp32 rounding of
//   the exact product.
//
// Two kernels:
//
//  split_pack      reads one operand through its strided view (any strides; coalesced along
//                  whichever matrix dim has unit stride, through a shared-memory transpose when that
//                  is not k) and writes two K-major planes  hi = tf32(x),  lo = tf32(x - hi)
//                  [plane][batch][rows][Kp], Kp = K rounded up to the k-block, zero padded.
//                  x = hi + lo to 2^-22 relative, and both planes are exactly representable in TF32.
//
//  gemm_3xtf32_kernel   one CTA per 128 x 256 output tile.  Warp 0 streams 16-wide k-blocks of the
//                  four planes into a 4-stage shared-memory ring with TMA (cp.async.bulk.tensor,
//                  64-byte swizzle, mbarrier completion; no multicast).  Warp 1 issues, per 8-wide
//                  k-step, three tcgen05.mma kind::tf32 instructions  hi*hi + hi*lo + lo*hi  that
//                  accumulate in fp32 in tensor memory (two 256-column accumulators, summed by the
//                  epilogue), and releases each stage with
//                  tcgen05.commit.  Warps 2-5 drain the accumulator with tcgen05.ld and store C.
//                  The dropped lo*lo term is below 2^-22 relative.
//
// Every wait on an mbarrier is bounded: past the limit the kernel records a code in a device flag,
// stops issuing work, lets in-flight copies land, frees its tensor memory and returns; the host
// reports the flag at the next synchronisation.
//
// Replaces _matmul_contig_fp32 / _matmul_fallback (src/cpp/ops/matmul.cu:60-205), plain SIMT FFMA
// kernels, for fp32 operands.
#include <cuda.h>

#include <atomic>
#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "nt_core.cuh"
#include "tf32_split.cuh"
#include "tma.cuh"

namespace ntb {

constexpr int TC_BM = 128;   // UMMA M
constexpr int TC_BN = 256;   // UMMA N
constexpr int TC_BK = 16;    // k-block per stage: 16 fp32 = 64 bytes = one 64B-swizzle row
constexpr int TC_STAGES = 4;
constexpr int TC_UMMA_K = 8; // tf32: 32 bytes of k per instruction
constexpr int TC_TMEM_COLS = 512; // two fp32 accumulators of 256 columns: hi*hi, and hi*lo + lo*hi
constexpr uint32_t TC_A_PLANE_BYTES = TC_BM * TC_BK * 4;  // 8 KB
constexpr uint32_t TC_B_PLANE_BYTES = TC_BN * TC_BK * 4;  // 16 KB
constexpr uint32_t TC_STAGE_BYTES = 2 * TC_A_PLANE_BYTES + 2 * TC_B_PLANE_BYTES; // 48 KB
constexpr uint32_t TC_SMEM_BYTES = TC_STAGES * TC_STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;

// ---------------------------------------------------------------------------------------------
// split_pack
struct SplitArgs {
  const float *src;
  float *hi, *lo;       // [batch][R][Kp]
  int64_t R, K, Kp;
  int64_t s_r, s_k, s_b; // element strides of the source view
  int mode;              // 0 generic, 1 unit stride along k (128-bit), 2 unit stride along r (128-bit + transpose)
};

__device__ __forceinline__ void split_store4(const SplitArgs &a, int64_t idx, float x0, float x1, float x2, float x3) {
  const float h0 = split_hi(x0), h1 = split_hi(x1), h2 = split_hi(x2), h3 = split_hi(x3);
  __stcs(reinterpret_cast<float4 *>(a.hi + idx), make_float4(h0, h1, h2, h3));
  __stcs(reinterpret_cast<float4 *>(a.lo + idx),
         make_float4(split_lo(x0, h0), split_lo(x1, h1), split_lo(x2, h2), split_lo(x3, h3)));
}

// One CTA converts a 64 (r) x 64 (k) tile.  Kp is a multiple of 32, so every 4-group of k inside Kp is
// either fully stored or fully outside.
__global__ void __launch_bounds__(256) split_pack(SplitArgs a) {
  __shared__ float tile[64][65];
  const int64_t r0 = int64_t(blockIdx.y) * 64, k0 = int64_t(blockIdx.x) * 64;
  const int64_t b = blockIdx.z;
  const float *src = a.src + b * a.s_b;
  const int64_t plane_off = b * a.R * a.Kp;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4; // 16 x 16
  if (a.mode == 1) {
    // thread: rows ty + 16 i, k group 4 tx
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t r = r0 + ty + 16 * i, k = k0 + 4 * tx;
      if (r < a.R && k < a.Kp) {
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (k + 3 < a.K) {
          x = __ldcs(reinterpret_cast<const float4 *>(src + r * a.s_r + k));
        } else {
          if (k + 0 < a.K) x.x = src[r * a.s_r + k + 0];
          if (k + 1 < a.K) x.y = src[r * a.s_r + k + 1];
          if (k + 2 < a.K) x.z = src[r * a.s_r + k + 2];
        }
        split_store4(a, plane_off + r * a.Kp + k, x.x, x.y, x.z, x.w);
      }
    }
    return;
  }
  if (a.mode == 2) {
    // read along r (unit stride): rows of the tile in smem are k
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t k = k0 + ty + 16 * i, r = r0 + 4 * tx;
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      if (k < a.K && r < a.R) {
        if (r + 3 < a.R) {
          x = __ldcs(reinterpret_cast<const float4 *>(src + k * a.s_k + r));
        } else {
          if (r + 0 < a.R) x.x = src[k * a.s_k + r + 0];
          if (r + 1 < a.R) x.y = src[k * a.s_k + r + 1];
          if (r + 2 < a.R) x.z = src[k * a.s_k + r + 2];
        }
      }
      tile[ty + 16 * i][4 * tx + 0] = x.x;
      tile[ty + 16 * i][4 * tx + 1] = x.y;
      tile[ty + 16 * i][4 * tx + 2] = x.z;
      tile[ty + 16 * i][4 * tx + 3] = x.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int kk = (threadIdx.x & 63), rr = (threadIdx.x >> 6) + 4 * i;
      const int64_t k = k0 + kk, r = r0 + rr;
      tile[kk][rr] = (k < a.K && r < a.R) ? src[r * a.s_r + k * a.s_k] : 0.0f;
    }
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t r = r0 + ty + 16 * i, k = k0 + 4 * tx;
    if (r < a.R && k < a.Kp)
      split_store4(a, plane_off + r * a.Kp + k, tile[4 * tx + 0][ty + 16 * i], tile[4 * tx + 1][ty + 16 * i],
                   tile[4 * tx + 2][ty + 16 * i], tile[4 * tx + 3][ty + 16 * i]);
  }
}

// ---------------------------------------------------------------------------------------------
// PTX wrappers (the mbarrier and TMA ones are in tma.cuh)
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major operand tile in the 64-byte swizzle layout that TMA wrote: rows of 64 bytes, groups of 8
// rows (512 bytes) back to back.  Fields: start address >> 4 in bits [0,14); leading byte offset >> 4
// in [16,30) (unused for this layout, set to 1); stride byte offset >> 4 in [32,46) = 512 bytes between
// 8-row groups; descriptor version 1 in [46,48); layout type SWIZZLE_64B = 4 in [61,64).
__device__ __forceinline__ uint64_t umma_desc_sw64(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr & 0x3FFFF) >> 4);
  d |= uint64_t(1) << 16;
  d |= uint64_t(512 >> 4) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(4) << 61;
  return d;
}
// MN-major operand tile of 32-bit values.  The one shared-memory layout the tensor core accepts for it is
// the 128-byte swizzle with 32-byte atoms: a row of 128 bytes holds 32 consecutive values of the m (or n)
// index for one k, the 32-byte chunks of a row are permuted by the row number modulo 4, so 4 rows (512
// bytes) form one swizzle atom -- what the tensor map mode SWIZZLE_128B_ATOM_32B writes.  An instruction
// of kind::tf32 consumes 8 values of k = two atoms, `sbo` bytes apart; the atoms of the next 32 m (or n)
// values lie `lbo` bytes further.  Same field positions as above; layout type 1.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr & 0x3FFFF) >> 4);
  d |= uint64_t((lbo >> 4) & 0x3FFF) << 16;
  d |= uint64_t((sbo >> 4) & 0x3FFF) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(1) << 61;
  return d;
}
// Instruction descriptor, kind::tf32: D format F32 (1) in bits [4,6); A and B format TF32 (2) in [7,10) and
// [10,13); A and B K-major (0) in bits 15, 16; N >> 3 in [17,23); M >> 4 in [24,29).
constexpr uint32_t TC_IDESC = (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(TC_BN >> 3) << 17) | (uint32_t(TC_BM >> 4) << 24);

__device__ __forceinline__ void umma_tf32_idesc(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\t"
               "setp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
               : "memory");
}
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
  umma_tf32_idesc(tmem_d, adesc, bdesc, TC_IDESC, accumulate);
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

struct TcArgs {
  float *C;
  int64_t M, N;
  int32_t num_kb;   // k-blocks of TC_BK
  int32_t batch;    // number of batches (plane index of `lo` = batch + b)
  int32_t c_vec;    // rows of C may be written 128 bits at a time
  const float *bias;    // promoted kernel only: C[m][n] = fl(fl(sum) + bias[n * bias_stride]) when non-null
  int64_t bias_stride;
  int *error_flag;
  long long wait_limit; // SM clocks a pipeline wait may take before the kernel gives up
  uint32_t mn_lbo, mn_sbo; // byte offsets of the MN-major descriptors (see umma_desc_mn_sw128)
  int32_t panel;           // promoted kernel: tiles are walked in panels this many n-tiles wide (0 = row by row)
  // promoted kernel, split-K: `splits` CTAs share an output tile, each over kb_per_split k-blocks; they leave
  // their sums in `partials` ([tile][split][32 chunks][256 threads][4]) and the one that draws the last ticket
  // adds them up in split order.  splits == 1: one CTA per tile, no workspace.
  int32_t splits, kb_per_split;
  float *partials;
  unsigned int *tickets;
  // promoted kernel: launched as the programmatic dependent of the product before it (nt_matmul_pair): it did not
  // wait for that grid on entry, so every CTA waits for it before leaving -- this grid never completes first
  int32_t wait_for_primary_at_end;
};

// Output tile of this CTA.  CTAs are dispatched in the order of their linear index (x fastest); walking the
// n-tiles of a whole row before the next m-tile makes every wave of CTAs touch all of B, which at these
// sizes (two planes of B: 134 MB for 4096 x 4096) no longer fits the L2 and is fetched from DRAM once per
// wave.  With panels of `panel` n-tiles a wave covers more m-tiles and fewer n-tiles, and a panel's slice of
// B stays in the L2 while the CTAs walk down the m-tiles.
__device__ __forceinline__ void tile_of_cta(const TcArgs &g, int &tm, int &tn, int &split) {
  const int splits = g.splits > 1 ? g.splits : 1;
  tm = blockIdx.y;
  tn = blockIdx.x / splits; // the CTAs of one tile are neighbours in the dispatch order: their partial sums meet in the L2
  split = blockIdx.x - tn * splits;
  if (g.panel > 0) {
    const int tiles_n = gridDim.x / splits, tiles_m = gridDim.y;
    const int lin = tm * tiles_n + tn;
    const int per_panel = g.panel * tiles_m;
    const int p = lin / per_panel;
    const int within = lin - p * per_panel;
    const int pw = min(g.panel, tiles_n - p * g.panel);
    tm = within / pw;
    tn = p * g.panel + within % pw;
  }
}

__global__ void __launch_bounds__(192, 1)
gemm_3xtf32_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, TcArgs g) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + TC_STAGES * TC_STAGE_BYTES;
  // barriers: full[s] at bar_base + 8 s, empty[s] at + 32 + 8 s, accumulator-ready at + 64; tmem slot at + 72
  const uint32_t full0 = bar_base, empty0 = bar_base + 32, acc_bar = bar_base + 64;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem_raw + (bar_base - smem_u32(smem_raw)) + 72);
  volatile int *poison_slot = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * TC_BM, n0 = blockIdx.x * TC_BN, b = blockIdx.z;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(acc_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // a wait already ran out in this launch (or an earlier one since the last synchronisation): the
    // whole CTA agrees to do nothing instead of spending another wait limit per role
    *poison_slot = *reinterpret_cast<volatile int *>(g.error_flag);
  }
  if (warp == 1) { // one warp allocates the accumulator columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TC_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_acc = *tmem_slot;
  const bool poisoned = *poison_slot != 0;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && !poisoned) {
      uint32_t phase = 0;
      int s = 0;
      for (int kb = 0; kb < g.num_kb; ++kb) {
        if (!mbar_wait(empty0 + 8 * s, phase ^ 1, g.wait_limit)) {
          atomicExch(g.error_flag, 1);
          break;
        }
        const uint32_t st = smem_base + s * TC_STAGE_BYTES;
        mbar_expect_tx(full0 + 8 * s, TC_STAGE_BYTES);
        const int k = kb * TC_BK;
        tma_load_3d(st, &map_a, full0 + 8 * s, k, m0, b);                                           // A hi
        tma_load_3d(st + TC_A_PLANE_BYTES, &map_a, full0 + 8 * s, k, m0, g.batch + b);              // A lo
        tma_load_3d(st + 2 * TC_A_PLANE_BYTES, &map_b, full0 + 8 * s, k, n0, b);                    // B hi
        tma_load_3d(st + 2 * TC_A_PLANE_BYTES + TC_B_PLANE_BYTES, &map_b, full0 + 8 * s, k, n0, g.batch + b); // B lo
        if (++s == TC_STAGES) {
          s = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && !poisoned) {
      uint32_t phase = 0;
      int s = 0;
      bool ok = true;
      for (int kb = 0; kb < g.num_kb; ++kb) {
        if (!mbar_wait(full0 + 8 * s, phase, g.wait_limit)) {
          atomicExch(g.error_flag, 2);
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const uint32_t st = smem_base + s * TC_STAGE_BYTES;
#pragma unroll
        for (int ks = 0; ks < TC_BK / TC_UMMA_K; ++ks) {
          const uint32_t koff = ks * TC_UMMA_K * 4; // 32 bytes along the swizzled row
          const uint64_t a_hi = umma_desc_sw64(st + koff);
          const uint64_t a_lo = umma_desc_sw64(st + TC_A_PLANE_BYTES + koff);
          const uint64_t b_hi = umma_desc_sw64(st + 2 * TC_A_PLANE_BYTES + koff);
          const uint64_t b_lo = umma_desc_sw64(st + 2 * TC_A_PLANE_BYTES + TC_B_PLANE_BYTES + koff);
          // The tensor core's fp32 accumulation rounds toward zero, a bias that grows with the number
          // of accumulations into one accumulator.  The large term gets an accumulator of its own
          // (K/8 accumulations); the two cross terms, 2^-11 smaller, share the other one.
          umma_tf32(tmem_acc, a_hi, b_hi, (kb | ks) != 0);
          umma_tf32(tmem_acc + TC_BN, a_hi, b_lo, (kb | ks) != 0);
          umma_tf32(tmem_acc + TC_BN, a_lo, b_hi, 1);
        }
        umma_commit(empty0 + 8 * s); // the stage may be refilled once these MMAs have read it
        if (++s == TC_STAGES) {
          s = 0;
          phase ^= 1;
        }
      }
      if (ok) umma_commit(acc_bar);
      else asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_bar) : "memory"); // release the epilogue
    }
  } else {
    // ------------------------------------------------------------------ epilogue, warps 2..5
    const int quad = warp & 3; // the 32-lane group of tensor memory this warp may read
    bool ok = !poisoned && mbar_wait(acc_bar, 0, g.wait_limit);
    if (!ok && !poisoned) atomicExch(g.error_flag, 3);
    ok = ok && (*reinterpret_cast<volatile int *>(g.error_flag) == 0);
    tcgen05_fence_after();
    const int64_t m = int64_t(m0) + quad * 32 + lane;
    float *crow = g.C + (int64_t(b) * g.M + m) * g.N;
#pragma unroll 1
    for (int c = 0; c < (poisoned ? 0 : TC_BN); c += 32) {
      uint32_t v[32], w[32];
      const uint32_t taddr = tmem_acc + (uint32_t(quad * 32) << 16) + uint32_t(c);
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
          "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
          "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
          : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]),
            "=r"(w[8]), "=r"(w[9]), "=r"(w[10]), "=r"(w[11]), "=r"(w[12]), "=r"(w[13]), "=r"(w[14]), "=r"(w[15]),
            "=r"(w[16]), "=r"(w[17]), "=r"(w[18]), "=r"(w[19]), "=r"(w[20]), "=r"(w[21]), "=r"(w[22]), "=r"(w[23]),
            "=r"(w[24]), "=r"(w[25]), "=r"(w[26]), "=r"(w[27]), "=r"(w[28]), "=r"(w[29]), "=r"(w[30]), "=r"(w[31])
          : "r"(taddr + uint32_t(TC_BN))
          : "memory");
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
          "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
          "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
          : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
            "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
            "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
            "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
          : "r"(taddr)
          : "memory");
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) + __uint_as_float(w[e]));
      if (ok && m < g.M) {
        const int64_t n = int64_t(n0) + c;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const int64_t nn = n + 4 * q;
          if (g.c_vec && nn + 3 < g.N) {
            *reinterpret_cast<float4 *>(crow + nn) =
                make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]), __uint_as_float(v[4 * q + 2]),
                            __uint_as_float(v[4 * q + 3]));
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (nn + e < g.N) crow[nn + e] = __uint_as_float(v[4 * q + e]);
          }
        }
      }
    }
  }

  // If anything timed out, give copies that are still in flight time to land before the shared
  // memory of this CTA is handed to another one.
  if (!poisoned && *reinterpret_cast<volatile int *>(g.error_flag) != 0) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) {
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(TC_TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------
// Variant with promoted accumulation (matmul mode 1, the default; the kernel above is mode 3).
//
// The tensor core adds into its fp32 accumulator with round-toward-zero, so a long accumulation chain
// carries a bias that grows with its length.  Here a chain is only TC_PERIOD_KB k-blocks (256 values of
// k, 96 MMAs) long: the two 256-column halves of tensor memory alternate as the accumulator of
// successive periods; while the MMA warp fills one, eight epilogue warps drain the other with
// tcgen05.ld and add it -- round-to-nearest -- into running sums they keep in registers (128 per
// thread).  The result has the error of an ordinary fp32 summation (2e-6 of max|C| at K = 4096 and 16384;
// chains of 128 measured 1e-6 at 3 % more time, one chain per output 1e-5 .. 4e-5).
constexpr int TC_PERIOD_KB = 16; // k-blocks (of TC_BK = 16) per accumulation chain

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

// A_MN / B_MN: the operand's planes keep the source tensor's own row-major order and the contraction
// index k runs down the rows (A seen as its transpose, B as stored): the tile arrives through a 4-D
// tensor map {32 m|n, k, (m|n)/32, plane} into 128-byte-swizzle / 32-byte-atom rows and the instruction
// reads it MN-major.  Otherwise k runs along the rows (K-major): 3-D map, 64-byte swizzle.  Every combination is
// one instantiation, so forward (A K-major, B MN-major), input gradient (both K-major) and weight
// gradient (both MN-major) all read planes that were split once, without a transpose.
template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(320, 1)
gemm_3xtf32_promoted_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, TcArgs g) {
  constexpr uint32_t IDESC = TC_IDESC | (A_MN ? (1u << 15) : 0u) | (B_MN ? (1u << 16) : 0u);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + TC_STAGES * TC_STAGE_BYTES;
  // full[s] at +8 s, empty[s] at +32 + 8 s, acc_full[b] at +64 + 8 b, acc_empty[b] at +80 + 8 b, tmem slot at +96
  const uint32_t full0 = bar_base, empty0 = bar_base + 32, acc_full0 = bar_base + 64, acc_empty0 = bar_base + 80;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem_raw + (bar_base - smem_u32(smem_raw)) + 96);
  volatile int *poison_slot = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // A grid launched behind this one with the programmatic-serialization attribute may take the SMs this grid's
  // last wave leaves idle; it has nothing to wait for here.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  int tile_m, tile_n, split;
  tile_of_cta(g, tile_m, tile_n, split);
  const int m0 = tile_m * TC_BM, n0 = tile_n * TC_BN, b = blockIdx.z;
  // this CTA's share of the contraction: k-blocks [kb0, kb0 + nkb)
  const int kb0 = g.splits > 1 ? split * g.kb_per_split : 0;
  const int nkb = g.splits > 1 ? min(g.kb_per_split, g.num_kb - kb0) : g.num_kb;
  const int num_periods = (nkb + TC_PERIOD_KB - 1) / TC_PERIOD_KB;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(acc_full0 + 8 * i, 1);
      mbar_init(acc_empty0 + 8 * i, 8); // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    *poison_slot = *reinterpret_cast<volatile int *>(g.error_flag); // see gemm_3xtf32_kernel
    poison_slot[1] = 0; // split-K: an epilogue warp gave up
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_acc = *tmem_slot;
  const bool poisoned = *poison_slot != 0;

  if (warp == 0) {
    if (lane == 0 && !poisoned) {
      uint32_t phase = 0;
      int s = 0;
      for (int kb = 0; kb < nkb; ++kb) {
        if (!mbar_wait(empty0 + 8 * s, phase ^ 1, g.wait_limit)) {
          atomicExch(g.error_flag, 1);
          break;
        }
        const uint32_t st = smem_base + s * TC_STAGE_BYTES;
        mbar_expect_tx(full0 + 8 * s, TC_STAGE_BYTES);
        const int k = (kb0 + kb) * TC_BK;
        if constexpr (A_MN) {
          tma_load_4d(st, &map_a, full0 + 8 * s, 0, k, m0 >> 5, b);
          tma_load_4d(st + TC_A_PLANE_BYTES, &map_a, full0 + 8 * s, 0, k, m0 >> 5, g.batch + b);
        } else {
          tma_load_3d(st, &map_a, full0 + 8 * s, k, m0, b);
          tma_load_3d(st + TC_A_PLANE_BYTES, &map_a, full0 + 8 * s, k, m0, g.batch + b);
        }
        if constexpr (B_MN) {
          tma_load_4d(st + 2 * TC_A_PLANE_BYTES, &map_b, full0 + 8 * s, 0, k, n0 >> 5, b);
          tma_load_4d(st + 2 * TC_A_PLANE_BYTES + TC_B_PLANE_BYTES, &map_b, full0 + 8 * s, 0, k, n0 >> 5, g.batch + b);
        } else {
          tma_load_3d(st + 2 * TC_A_PLANE_BYTES, &map_b, full0 + 8 * s, k, n0, b);
          tma_load_3d(st + 2 * TC_A_PLANE_BYTES + TC_B_PLANE_BYTES, &map_b, full0 + 8 * s, k, n0, g.batch + b);
        }
        if (++s == TC_STAGES) {
          s = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && !poisoned) {
      uint32_t phase = 0;
      int s = 0, kb = 0;
      bool ok = true;
      for (int p = 0; p < num_periods && ok; ++p) {
        const int buf = p & 1;
        // the epilogue must have drained this half (two periods ago) before it is overwritten
        if (!mbar_wait(acc_empty0 + 8 * buf, ((p >> 1) & 1) ^ 1, g.wait_limit)) {
          atomicExch(g.error_flag, 4);
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const uint32_t d = tmem_acc + uint32_t(buf * TC_BN);
        const int kb_end = min(kb + TC_PERIOD_KB, nkb);
        bool first = true;
        for (; kb < kb_end; ++kb) {
          if (!mbar_wait(full0 + 8 * s, phase, g.wait_limit)) {
            atomicExch(g.error_flag, 2);
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t st = smem_base + s * TC_STAGE_BYTES;
#pragma unroll
          for (int ks = 0; ks < TC_BK / TC_UMMA_K; ++ks) {
            // one instruction consumes 8 values of k: 32 bytes along a K-major row, 8 rows of 128 bytes
            // of an MN-major tile
            const uint32_t a_off = A_MN ? ks * 1024u : ks * TC_UMMA_K * 4u;
            const uint32_t b_off = B_MN ? ks * 1024u : ks * TC_UMMA_K * 4u;
            const uint32_t pa = st + a_off, pb = st + 2 * TC_A_PLANE_BYTES + b_off;
            const uint64_t a_hi = A_MN ? umma_desc_mn_sw128(pa, g.mn_lbo, g.mn_sbo) : umma_desc_sw64(pa);
            const uint64_t a_lo = A_MN ? umma_desc_mn_sw128(pa + TC_A_PLANE_BYTES, g.mn_lbo, g.mn_sbo)
                                       : umma_desc_sw64(pa + TC_A_PLANE_BYTES);
            const uint64_t b_hi = B_MN ? umma_desc_mn_sw128(pb, g.mn_lbo, g.mn_sbo) : umma_desc_sw64(pb);
            const uint64_t b_lo = B_MN ? umma_desc_mn_sw128(pb + TC_B_PLANE_BYTES, g.mn_lbo, g.mn_sbo)
                                       : umma_desc_sw64(pb + TC_B_PLANE_BYTES);
            // small terms first, the large one last
            umma_tf32_idesc(d, a_hi, b_lo, IDESC, first ? 0u : 1u);
            umma_tf32_idesc(d, a_lo, b_hi, IDESC, 1);
            umma_tf32_idesc(d, a_hi, b_hi, IDESC, 1);
            first = false;
          }
          umma_commit(empty0 + 8 * s);
          if (++s == TC_STAGES) {
            s = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(acc_full0 + 8 * buf);
      }
      if (!ok) { // release the epilogue warps from whatever they wait on
        for (int i = 0; i < 2; ++i)
          asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_full0 + 8 * i) : "memory");
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue, warps 2..9
    const int quad = warp & 3;          // 32-lane group of tensor memory this warp may read
    const int half = (warp - 2) >> 2;   // which 128 of the 256 columns
    float sum[128];
#pragma unroll
    for (int i = 0; i < 128; ++i) sum[i] = 0.0f;
    bool ok = !poisoned;
    for (int p = 0; p < (poisoned ? 0 : num_periods); ++p) {
      const int buf = p & 1;
      if (ok && !mbar_wait(acc_full0 + 8 * buf, (p >> 1) & 1, g.wait_limit)) {
        atomicExch(g.error_flag, 3);
        ok = false;
      }
      if (!ok || *reinterpret_cast<volatile int *>(g.error_flag) != 0) {
        ok = false;
        break;
      }
      tcgen05_fence_after();
      const uint32_t taddr = tmem_acc + (uint32_t(quad * 32) << 16) + uint32_t(buf * TC_BN + half * 128);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(taddr + uint32_t(c * 32), v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int e = 0; e < 32; ++e) sum[c * 32 + e] = sum[c * 32 + e] + __uint_as_float(v[e]);
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty0 + 8 * buf) : "memory");
    }
    const int64_t m = int64_t(m0) + quad * 32 + lane;
    if (g.splits > 1 && !poisoned) {
      // Split-K: leave this CTA's sums in the workspace; whoever draws the tile's last ticket adds the
      // partial sums up in split order (the order never depends on which CTA finishes last).  All eight
      // epilogue warps pass the two barriers whatever happened to them; a warp whose wait ran out says so.
      volatile int *fail_slot = poison_slot + 1;
      volatile unsigned int *ticket_slot = reinterpret_cast<volatile unsigned int *>(poison_slot + 2);
      const int et = int(threadIdx.x) - 64; // 0..255 among the epilogue threads
      const int64_t tile_lin = (int64_t(b) * gridDim.y + tile_m) * (gridDim.x / g.splits) + tile_n;
      float *mine = g.partials + ((tile_lin * g.splits + split) * 32 * 256 + et) * 4;
      if (!ok) *fail_slot = 1;
      if (ok && m < g.M) {
#pragma unroll
        for (int q = 0; q < 32; ++q)
          __stcg(reinterpret_cast<float4 *>(mine + q * 1024), make_float4(sum[4 * q], sum[4 * q + 1], sum[4 * q + 2], sum[4 * q + 3]));
      }
      __threadfence();
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (et == 0) *ticket_slot = (*fail_slot != 0) ? 0xffffffffu : atomicAdd(g.tickets + tile_lin, 1u);
      asm volatile("bar.sync 1, 256;" ::: "memory");
      const unsigned int ticket = *ticket_slot;
      ok = ok && ticket == unsigned(g.splits - 1);
      if (ok) {
        __threadfence();
        if (m < g.M) {
          const float *first = g.partials + (tile_lin * g.splits * 32 * 256 + et) * 4;
#pragma unroll
          for (int q = 0; q < 32; ++q) {
            float4 acc = __ldcg(reinterpret_cast<const float4 *>(first + q * 1024));
            for (int sp = 1; sp < g.splits; ++sp) {
              const float4 v = __ldcg(reinterpret_cast<const float4 *>(first + int64_t(sp) * 32 * 256 * 4 + q * 1024));
              acc.x += v.x;
              acc.y += v.y;
              acc.z += v.z;
              acc.w += v.w;
            }
            sum[4 * q] = acc.x;
            sum[4 * q + 1] = acc.y;
            sum[4 * q + 2] = acc.z;
            sum[4 * q + 3] = acc.w;
          }
        }
        if (et == 0) g.tickets[tile_lin] = 0; // ready for the next launch
      }
    }
    if (ok && m < g.M) {
      float *crow = g.C + (int64_t(b) * g.M + m) * g.N;
      const int64_t n = int64_t(n0) + half * 128;
      if (g.bias) {
        // the second rounded step of x @ W + b: the fp32 product that a separate launch would have
        // stored, plus the bias, rounded once more (every lane reads the same bias word: one broadcast)
#pragma unroll
        for (int i = 0; i < 128; ++i)
          if (n + i < g.N) sum[i] = sum[i] + __ldg(g.bias + (n + i) * g.bias_stride);
      }
#pragma unroll
      for (int q = 0; q < 32; ++q) {
        const int64_t nn = n + 4 * q;
        if (g.c_vec && nn + 3 < g.N) {
          *reinterpret_cast<float4 *>(crow + nn) = make_float4(sum[4 * q], sum[4 * q + 1], sum[4 * q + 2], sum[4 * q + 3]);
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (nn + e < g.N) crow[nn + e] = sum[4 * q + e];
        }
      }
    }
  }

  if (!poisoned && *reinterpret_cast<volatile int *>(g.error_flag) != 0) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) {
    }
  }
  if (g.wait_for_primary_at_end) asm volatile("griddepcontrol.wait;" ::: "memory");
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(512) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------
// Host side
EncodeTiledFn tensor_map_encoder() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    NT_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    if (!p || q != cudaDriverEntryPointSuccess) fail_runtime("cuTensorMapEncodeTiled is not available in this driver.");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}
static EncodeTiledFn encode_fn() { return tensor_map_encoder(); }

// planes: [2 * batch][rows][Kp] fp32, K-major; box = 16 k x box_rows rows.
static CUtensorMap make_map(float *planes, int64_t rows, int64_t Kp, int64_t batch2, uint32_t box_rows) {
  CUtensorMap m;
  cuuint64_t dims[3] = {cuuint64_t(Kp), cuuint64_t(rows), cuuint64_t(batch2)};
  cuuint64_t strides[2] = {cuuint64_t(Kp) * 4, cuuint64_t(rows) * cuuint64_t(Kp) * 4};
  cuuint32_t box[3] = {TC_BK, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult rc = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, planes, dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) fail_runtime("cuTensorMapEncodeTiled failed with code " + std::to_string(int(rc)));
  return m;
}

// Width of the tile panels of the promoted kernel in n-tiles (8 x 256 columns: that slice of a 4096-deep B
// is 67 MB of planes).  NT_GEMM_PANEL overrides it, 0 = off.
static int panel_default() {
  const char *e = getenv("NT_GEMM_PANEL");
  if (e && *e) {
    const int v = atoi(e);
    return v < 0 ? 0 : v;
  }
  return 8;
}
static std::atomic<int> g_tc_panel{panel_default()};

// nt_matmul_pair: the second of two independent products can be launched as the programmatic dependent of the
// first when nothing was launched in between (its operand planes were cache hits) -- then its first CTAs fill the
// SMs that the first product's last wave leaves idle.  g_promoted_seq is the launch count right after the last
// promoted-kernel launch.  Off unless asked for (nt_set_matmul_pair_overlap, NT_GEMM_PAIR_OVERLAP=1): measured on
// the training step it is worth 0.3 % at a 2048-row batch (256 + 512 tiles on 148 SMs), 0.6 % at 4096 rows and
// nothing at 16384 -- under the power cap the SMs that stay busy in a thin last wave clock higher, which already
// recovers most of what the idle ones lose.
static thread_local bool t_pair_first = false, t_pair_second = false;
static thread_local bool t_pair_end_pending = false; // the first product left its profile interval open
static uint64_t g_promoted_seq = ~uint64_t(0);
static int pair_overlap_default() {
  const char *e = getenv("NT_GEMM_PAIR_OVERLAP");
  return (e && *e) ? (atoi(e) != 0) : 0;
}
static std::atomic<int> g_pair_overlap{pair_overlap_default()};
// role: 0 = not in a pair, 1 = first product, 2 = second.  Leaving a pair closes a profile interval the first
// product left open for a second one that never joined it.
void gemm_tc_pair_role(int role) {
  t_pair_first = role == 1;
  t_pair_second = role == 2;
  if (role == 0 && t_pair_end_pending) {
    t_pair_end_pending = false;
    matmul_profile_end();
  }
}
void gemm_tc_set_pair_overlap(bool on) { g_pair_overlap.store(on ? 1 : 0); }

// Split-K tickets: one counter per output tile, zero between launches (the CTA that draws the last ticket of a
// tile resets it).  GEMM launches are ordered on the compute stream, so one array serves them all.
constexpr int64_t TC_MAX_TICKETS = 65536;
static unsigned int *g_tickets = nullptr;
static int max_splits_default() {
  const char *e = getenv("NT_GEMM_SPLITK");
  if (e && *e) {
    const int v = atoi(e);
    return v < 1 ? 1 : (v > 8 ? 8 : v);
  }
  return 8;
}
static std::atomic<int> g_tc_max_splits{max_splits_default()};

static int *g_error_flag = nullptr;
static int *error_flag_ptr();
int *pipeline_error_flag() { return error_flag_ptr(); }
static int *error_flag_ptr() {
  int *&flag = g_error_flag;
  if (!flag) {
    if (is_capturing())
      fail_runtime("gemm_3xtf32: first use inside a graph capture; run the step once eagerly before capturing it.");
    size_t rounded;
    flag = static_cast<int *>(device_alloc(sizeof(int), &rounded));
    NT_CUDA_CHECK(cudaMemsetAsync(flag, 0, sizeof(int), stream()));
  }
  return flag;
}

// Reads (and clears) the device-side error flag of the tensor-core kernel; called after a stream
// synchronisation.  0 = no error.
int gemm_tc_take_error() {
  int *flag = g_error_flag;
  if (!flag) return 0; // the kernel never ran
  int host = 0;
  if (cudaMemcpy(&host, flag, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (host != 0) {
    cudaMemset(flag, 0, sizeof(int));
    if (g_tickets) cudaMemset(g_tickets, 0, size_t(TC_MAX_TICKETS) * 4); // tiles that never completed left theirs behind
  }
  return host;
}

static void launch_split(const float *src, float *planes, int64_t batch, int64_t R, int64_t K, int64_t Kp, int64_t s_b,
                         int64_t s_r, int64_t s_k) {
  SplitArgs a{};
  a.src = src;
  a.hi = planes;
  a.lo = planes + batch * R * Kp;
  a.R = R;
  a.K = K;
  a.Kp = Kp;
  a.s_r = s_r;
  a.s_k = s_k;
  a.s_b = s_b;
  const bool base_al = (reinterpret_cast<uintptr_t>(src) & 15) == 0 && (s_b % 4 == 0);
  a.mode = 0;
  if (s_k == 1 && base_al && s_r % 4 == 0) a.mode = 1;
  else if (s_r == 1 && s_k != 1 && base_al && s_k % 4 == 0) a.mode = 2;
  dim3 grid{unsigned(ceil_div(Kp, 64)), unsigned(ceil_div(R, 64)), unsigned(batch)};
  split_pack<<<grid, 256, 0, stream()>>>(a);
  check_launch("split_pack");
}

void gemm_tc_prepare() {
  static bool configured = false;
  if (!configured) {
    NT_CUDA_CHECK(cudaFuncSetAttribute(gemm_3xtf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(TC_SMEM_BYTES)));
    NT_CUDA_CHECK(cudaFuncSetAttribute(gemm_3xtf32_promoted_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       int(TC_SMEM_BYTES)));
    configured = true;
  }
  error_flag_ptr();
  if (!g_tickets) {
    if (is_capturing())
      fail_runtime("gemm_3xtf32: first use inside a graph capture; run the step once eagerly before capturing it.");
    size_t rounded;
    g_tickets = static_cast<unsigned int *>(device_alloc(size_t(TC_MAX_TICKETS) * 4, &rounded));
    NT_CUDA_CHECK(cudaMemsetAsync(g_tickets, 0, size_t(TC_MAX_TICKETS) * 4, stream()));
  }
}

// One CTA, one thread: the same bounded wait the GEMM pipeline uses, on a barrier that nothing ever
// arrives on.  It must give up after the configured limit, record code 5 and return -- the test of the
// time-out path that needs no fault: the context stays usable and the flag is read at the next
// synchronisation like any pipeline time-out.
__global__ void wait_probe_kernel(int *error_flag, long long limit) {
  __shared__ __align__(8) uint64_t bar;
  const uint32_t b = smem_u32(&bar);
  mbar_init(b, 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  if (!mbar_wait(b, 0, limit)) atomicExch(error_flag, 5);
}

void gemm_tc_wait_probe() {
  int *flag = error_flag_ptr();
  wait_probe_kernel<<<1, 1, 0, stream()>>>(flag, wait_limit_clocks());
  check_launch("wait_probe_kernel");
}

// ---------------------------------------------------------------------------------------------
// Natural-layout operand planes and their cache.
//
// An operand whose matrix has unit stride along one of its two dims is split in the source's own row-major
// order: rows = the strided dim, columns = the unit-stride dim, hi and lo planes [2][batch][R][Cp] with
// Cp = C rounded up to 32 and the padding zeroed.  No transpose on the way: whether the contraction index
// is the column (K-major) or the row (MN-major) of the planes is told to the GEMM kernel instead.  The
// planes are remembered per storage and view geometry: an activation is split once for the forward
// product and found again by the weight-gradient product, a gradient once for both of its products, a
// weight once per update.  An entry is valid while the storage's mutation counter and the epoch (see
// gemm_tc_new_epoch) are the ones it was written under; a stale entry is re-split into the same buffer.
// Inside a graph capture an entry is trusted only if it was split within that same capture, or if it is
// `maintained` -- last written by gemm_tc_refresh, i.e. it belongs to a parameter whose every update re-splits
// it, inside the graph too.  Anything else (an input batch split by an eager warm-up step) is split again
// inside the capture, so that a replay sees whatever the buffer holds by then.
// A storage keeps at most PLANE_ENTRIES_PER_STORAGE entries (views at different offsets of one big tensor
// would otherwise pile up); the least recently used entry that no capture relies on makes room.
struct NatSplitArgs {
  const float *src;
  float *hi, *lo;
  int64_t R, C, Cp, s_r, s_b;
  int vec; // rows of the source may be read 128 bits at a time
};

__global__ void __launch_bounds__(256) split_planes(NatSplitArgs a) {
  const int64_t c = (int64_t(blockIdx.x) * 64 + (threadIdx.x & 63)) * 4;
  if (c >= a.Cp) return;
  const int64_t r0 = int64_t(blockIdx.y) * 16 + (threadIdx.x >> 6);
  const float *src = a.src + int64_t(blockIdx.z) * a.s_b;
  const int64_t plane = int64_t(blockIdx.z) * a.R * a.Cp;
  float4 x[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) { // rows r0, r0 + 4, r0 + 8, r0 + 12: all loads issued before the first use
    const int64_t r = r0 + 4 * i;
    x[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < a.R) {
      const float *p = src + r * a.s_r + c;
      if (a.vec && c + 3 < a.C) {
        x[i] = __ldg(reinterpret_cast<const float4 *>(p));
      } else {
        if (c + 0 < a.C) x[i].x = p[0];
        if (c + 1 < a.C) x[i].y = p[1];
        if (c + 2 < a.C) x[i].z = p[2];
        if (c + 3 < a.C) x[i].w = p[3];
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t r = r0 + 4 * i;
    if (r < a.R) {
      const int64_t idx = plane + r * a.Cp + c;
      const float h0 = split_hi(x[i].x), h1 = split_hi(x[i].y), h2 = split_hi(x[i].z), h3 = split_hi(x[i].w);
      *reinterpret_cast<float4 *>(a.hi + idx) = make_float4(h0, h1, h2, h3);
      *reinterpret_cast<float4 *>(a.lo + idx) =
          make_float4(split_lo(x[i].x, h0), split_lo(x[i].y, h1), split_lo(x[i].z, h2), split_lo(x[i].w, h3));
    }
  }
}

struct PlaneEntry {
  int64_t offset, batch, s_b, R, C, s_r; // the view: element offset, batch count / stride, rows, columns, row stride
  int64_t Cp;
  float *planes;
  size_t rounded;
  uint64_t mutation, epoch;
  int capture = 0;         // id of the capture that last split it, 0 = split eagerly
  bool maintained = false; // last written by gemm_tc_refresh
  uint64_t last_use = 0;   // g_plane_tick of the last look-up that returned it
};
static uint64_t g_plane_tick = 0; // one per look-up; the two operands of a product are consecutive look-ups
constexpr size_t PLANE_ENTRIES_PER_STORAGE = 32;
static std::mutex g_plane_mu;
static std::unordered_map<nt_storage *, std::vector<PlaneEntry>> g_plane_cache;
static uint64_t g_plane_epoch = 1;
static std::atomic<int> g_operand_cache{1};
static std::atomic<uint64_t> g_split_launches{0}, g_split_hits{0};

static void run_split(const nt_storage *s, const PlaneEntry &e) {
  NatSplitArgs a{};
  a.src = static_cast<const float *>(s->data) + e.offset;
  a.hi = e.planes;
  a.lo = e.planes + e.batch * e.R * e.Cp;
  a.R = e.R;
  a.C = e.C;
  a.Cp = e.Cp;
  a.s_r = e.s_r;
  a.s_b = e.s_b;
  a.vec = ((reinterpret_cast<uintptr_t>(a.src) & 15) == 0 && e.s_r % 4 == 0 && e.s_b % 4 == 0) ? 1 : 0;
  dim3 grid{unsigned(ceil_div(e.Cp, 256)), unsigned(ceil_div(e.R, 16)), unsigned(e.batch)};
  split_planes<<<grid, 256, 0, stream()>>>(a);
  check_launch("split_planes");
  g_split_launches.fetch_add(1, std::memory_order_relaxed);
}

// Planes of the view (rows R, columns C with unit stride, row stride s_r, `batch` matrices s_b apart) of
// storage s.  `owned` is set when the caller must free them after its launch (cache off).
static float *natural_planes(nt_storage *s, int64_t offset, int64_t batch, int64_t s_b, int64_t R, int64_t C, int64_t s_r,
                             int64_t *Cp_out, size_t *owned_rounded) {
  const int64_t Cp = ceil_div(C, 32) * 32;
  *Cp_out = Cp;
  *owned_rounded = 0;
  const size_t bytes = size_t(2 * batch * R * Cp) * 4;
  if (!g_operand_cache.load()) {
    PlaneEntry e{offset, batch, s_b, R, C, s_r, Cp, nullptr, 0, 0, 0};
    e.planes = static_cast<float *>(device_alloc(bytes, &e.rounded));
    *owned_rounded = e.rounded;
    run_split(s, e);
    return e.planes;
  }
  const int cid = capture_id();
  std::lock_guard<std::mutex> lk(g_plane_mu);
  const uint64_t tick = ++g_plane_tick;
  auto &list = g_plane_cache[s];
  for (PlaneEntry &e : list) {
    if (e.offset == offset && e.batch == batch && e.s_b == s_b && e.R == R && e.C == C && e.s_r == s_r) {
      const bool current = e.mutation == s->mutation && e.epoch == g_plane_epoch;
      e.last_use = tick;
      if (current && (cid == 0 || e.capture == cid || e.maintained)) {
        g_split_hits.fetch_add(1, std::memory_order_relaxed);
        return e.planes;
      }
      e.mutation = s->mutation;
      e.epoch = g_plane_epoch;
      e.capture = cid;
      e.maintained = false;
      run_split(s, e); // same buffer: a captured graph that reads it keeps reading the right place
      return e.planes;
    }
  }
  if (list.size() >= PLANE_ENTRIES_PER_STORAGE) {
    // least recently used among the entries no capture relies on -- but never the one the previous look-up
    // returned: it may be the other operand of the product being set up, not yet launched
    size_t victim = list.size();
    for (size_t i = 0; i < list.size(); ++i) {
      const PlaneEntry &c = list[i];
      if (c.capture != 0 || c.maintained || c.last_use + 1 >= tick) continue;
      if (victim == list.size() || c.last_use < list[victim].last_use) victim = i;
    }
    if (victim != list.size()) {
      device_free(list[victim].planes, list[victim].rounded); // stream-ordered: earlier readers are already queued
      list.erase(list.begin() + victim);
    }
  }
  PlaneEntry e{offset, batch, s_b, R, C, s_r, Cp, nullptr, 0, s->mutation, g_plane_epoch, cid, false, tick};
  e.planes = static_cast<float *>(device_alloc(bytes, &e.rounded));
  run_split(s, e);
  list.push_back(e);
  return e.planes;
}

// Planes that a producer kernel fills itself while it still holds its output in registers: registers a
// valid entry for the dense [R][C] view of `s` (C a multiple of 32, so the planes index like the output)
// and returns its hi plane (lo follows R * C values later); nullptr when the cache is off.
float *gemm_tc_adopt_planes(nt_storage *s, int64_t R, int64_t C) {
  if (!g_operand_cache.load() || C % 32 != 0) return nullptr;
  const int cid = capture_id();
  std::lock_guard<std::mutex> lk(g_plane_mu);
  auto &list = g_plane_cache[s];
  PlaneEntry e{0, 1, 0, R, C, C, C, nullptr, 0, s->mutation, g_plane_epoch, cid, false};
  e.planes = static_cast<float *>(device_alloc(size_t(2 * R * C) * 4, &e.rounded));
  list.push_back(e);
  return e.planes;
}

void gemm_tc_forget(nt_storage *s) {
  std::vector<PlaneEntry> dead;
  {
    std::lock_guard<std::mutex> lk(g_plane_mu);
    if (g_plane_cache.empty()) return;
    auto it = g_plane_cache.find(s);
    if (it == g_plane_cache.end()) return;
    dead.swap(it->second);
    g_plane_cache.erase(it);
  }
  for (PlaneEntry &e : dead) device_free(e.planes, e.rounded);
}

void gemm_tc_refresh(nt_storage *s) {
  std::lock_guard<std::mutex> lk(g_plane_mu);
  if (g_plane_cache.empty()) return;
  auto it = g_plane_cache.find(s);
  if (it == g_plane_cache.end()) return;
  const int cid = capture_id();
  for (PlaneEntry &e : it->second) {
    e.mutation = s->mutation;
    e.epoch = g_plane_epoch;
    e.capture = cid;
    e.maintained = true;
    run_split(s, e);
  }
}

// For a writer that rewrites a whole dense [R][C] fp32 storage and can write the TF32 planes in the same pass
// (the SGD update): the plane buffer to write, if the storage has exactly one cached view and that view is the
// whole storage with unpadded rows; the caller then calls gemm_tc_mark_refreshed instead of gemm_tc_refresh.
float *gemm_tc_refresh_target(nt_storage *s, int64_t R, int64_t C) {
  if (!g_operand_cache.load() || C % 32 != 0) return nullptr;
  std::lock_guard<std::mutex> lk(g_plane_mu);
  auto it = g_plane_cache.find(s);
  if (it == g_plane_cache.end() || it->second.size() != 1) return nullptr;
  const PlaneEntry &e = it->second.front();
  if (e.offset != 0 || e.batch != 1 || e.R != R || e.C != C || e.s_r != C || e.Cp != C) return nullptr;
  return e.planes;
}
void gemm_tc_mark_refreshed(nt_storage *s) {
  std::lock_guard<std::mutex> lk(g_plane_mu);
  auto it = g_plane_cache.find(s);
  if (it == g_plane_cache.end()) return;
  const int cid = capture_id();
  for (PlaneEntry &e : it->second) {
    e.mutation = s->mutation;
    e.epoch = g_plane_epoch;
    e.capture = cid;
    e.maintained = true;
  }
}

void gemm_tc_new_epoch() {
  std::lock_guard<std::mutex> lk(g_plane_mu);
  g_plane_epoch += 1;
}

void gemm_tc_set_operand_cache(bool on) { g_operand_cache.store(on ? 1 : 0); }
void gemm_tc_set_schedule(int max_splits, int panel) {
  g_tc_max_splits.store(max_splits < 1 ? 1 : (max_splits > 8 ? 8 : max_splits));
  g_tc_panel.store(panel < 0 ? 0 : panel);
}
void gemm_tc_split_stats(uint64_t *launches, uint64_t *hits) {
  *launches = g_split_launches.load();
  *hits = g_split_hits.load();
}

// 4-D map over MN-major planes [2 * batch][R = k][Cp]: {32 m|n, k, (m|n) / 32, plane}; box = 32 x 16 x box_mn/32.
static CUtensorMap make_map_mn(float *planes, int64_t rows_k, int64_t Cp, int64_t batch2, uint32_t box_mn) {
  CUtensorMap m;
  cuuint64_t dims[4] = {32, cuuint64_t(rows_k), cuuint64_t(Cp / 32), cuuint64_t(batch2)};
  cuuint64_t strides[3] = {cuuint64_t(Cp) * 4, 128, cuuint64_t(rows_k) * cuuint64_t(Cp) * 4};
  cuuint32_t box[4] = {32, TC_BK, box_mn / 32, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult rc = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, planes, dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) fail_runtime("cuTensorMapEncodeTiled (MN-major planes) failed with code " + std::to_string(int(rc)));
  return m;
}
// 3-D map over K-major planes [2 * batch][R = m|n][Cp], k extent K (reads past it are zero filled).
static CUtensorMap make_map_k(float *planes, int64_t rows, int64_t K, int64_t Cp, int64_t batch2, uint32_t box_rows) {
  CUtensorMap m;
  cuuint64_t dims[3] = {cuuint64_t(K), cuuint64_t(rows), cuuint64_t(batch2)};
  cuuint64_t strides[2] = {cuuint64_t(Cp) * 4, cuuint64_t(rows) * cuuint64_t(Cp) * 4};
  cuuint32_t box[3] = {TC_BK, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult rc = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, planes, dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) fail_runtime("cuTensorMapEncodeTiled (K-major planes) failed with code " + std::to_string(int(rc)));
  return m;
}

static std::atomic<int> g_promoted{1};
void gemm_tc_set_promoted(bool on) { g_promoted.store(on ? 1 : 0); }

// MN-major tiles as the 4-D map lays them down: [32-wide m|n chunk][16 k rows][128 bytes]
constexpr uint32_t TC_MN_LBO = TC_BK * 128; // next 32 values of m|n
constexpr uint32_t TC_MN_SBO = 4 * 128;     // next swizzle atom (4 rows of k)

template <bool A_MN, bool B_MN>
static void launch_promoted(const CUtensorMap &ma, const CUtensorMap &mb, const TcArgs &g, dim3 grid) {
  static bool configured = false;
  if (!configured) {
    NT_CUDA_CHECK(cudaFuncSetAttribute(gemm_3xtf32_promoted_kernel<A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       int(TC_SMEM_BYTES)));
    configured = true;
  }
  if (!g.wait_for_primary_at_end) {
    gemm_3xtf32_promoted_kernel<A_MN, B_MN><<<grid, 320, TC_SMEM_BYTES, stream()>>>(ma, mb, g);
    return;
  }
  // programmatic dependent launch: this grid's CTAs may start while the previous kernel's last wave still runs
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(320, 1, 1);
  cfg.dynamicSmemBytes = TC_SMEM_BYTES;
  cfg.stream = stream();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  NT_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_3xtf32_promoted_kernel<A_MN, B_MN>, ma, mb, g));
}

// How an operand matrix [P][Q] (strides s_p, s_q) is laid out: unit stride along Q, along P, or neither.
static int unit_dim(int64_t P, int64_t Q, int64_t s_p, int64_t s_q) {
  if (s_q == 1 || Q == 1) return 1; // rows = P, columns = Q
  if (s_p == 1 || P == 1) return 0; // rows = Q, columns = P
  return -1;
}

// The promoted-accumulation kernel over natural-layout planes.  Returns false when an operand has no
// unit-stride matrix dim (the caller then takes the transposing split below).
bool gemm_3xtf32_natural(nt_storage *sa, int64_t a_off, nt_storage *sb, int64_t b_off, float *C, int64_t batch, int64_t M,
                         int64_t N, int64_t K, int64_t a_sb, int64_t a_sm, int64_t a_sk, int64_t b_sb, int64_t b_sk,
                         int64_t b_sn, const float *bias, int64_t bias_stride, bool *bias_done) {
  if (bias_done) *bias_done = false;
  if (!g_promoted.load()) return false;
  if (batch < 1 || batch > 32767 || M < 1 || N < 1 || K < 1) return false;
  if (ceil_div(M, TC_BM) > 65535 || ceil_div(N, TC_BN) > 0x7fffffff) return false;
  if (M >= (int64_t(1) << 31) || N >= (int64_t(1) << 31) || K >= (int64_t(1) << 31)) return false;
  const int ua = unit_dim(M, K, a_sm, a_sk), ub = unit_dim(K, N, b_sk, b_sn);
  if (ua < 0 || ub < 0) return false;
  if (a_sm < 0 || a_sk < 0 || b_sk < 0 || b_sn < 0 || a_sb < 0 || b_sb < 0) return false;
  const bool a_mn = (ua == 0), b_mn = (ub == 1); // A: columns = m; B: columns = n
  // natural rows / columns / row stride of each operand
  const int64_t aR = a_mn ? K : M, aC = a_mn ? M : K, a_sr = a_mn ? a_sk : a_sm;
  const int64_t bR = b_mn ? K : N, bC = b_mn ? N : K, b_sr = b_mn ? b_sk : b_sn;
  if (ceil_div(aR, 16) > 65535 || ceil_div(bR, 16) > 65535) return false; // grid.y of split_planes
  gemm_tc_prepare();
  int64_t aCp = 0, bCp = 0;
  size_t a_owned = 0, b_owned = 0;
  float *pa = natural_planes(sa, a_off, batch, batch > 1 ? a_sb : 0, aR, aC, a_sr, &aCp, &a_owned);
  float *pb = nullptr;
  try {
    pb = natural_planes(sb, b_off, batch, batch > 1 ? b_sb : 0, bR, bC, b_sr, &bCp, &b_owned);
    CUtensorMap map_a = a_mn ? make_map_mn(pa, aR, aCp, 2 * batch, TC_BM) : make_map_k(pa, aR, K, aCp, 2 * batch, TC_BM);
    CUtensorMap map_b = b_mn ? make_map_mn(pb, bR, bCp, 2 * batch, TC_BN) : make_map_k(pb, bR, K, bCp, 2 * batch, TC_BN);
    TcArgs g{};
    g.C = C;
    g.M = M;
    g.N = N;
    g.num_kb = int32_t(ceil_div(K, TC_BK));
    g.batch = int32_t(batch);
    g.c_vec = (N % 4 == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0) ? 1 : 0;
    g.error_flag = error_flag_ptr();
    g.wait_limit = wait_limit_clocks();
    g.mn_lbo = TC_MN_LBO;
    g.mn_sbo = TC_MN_SBO;
    const int64_t tiles_n = ceil_div(N, TC_BN), tiles_m = ceil_div(M, TC_BM);
    {
      const int panel = g_tc_panel.load(std::memory_order_relaxed);
      g.panel = (panel > 0 && tiles_n > panel && tiles_n * tiles_m < (int64_t(1) << 30)) ? panel : 0;
    }
    // Split-K for products that leave most SMs without a tile (a skinny output with a long contraction: 4
    // tiles at 256 x 8192 x 512): up to max_splits CTAs share a tile while tiles x splits still fit one wave.
    // Not for wave quantisation of larger products: measured on the 2048-row training step (256 tiles on 148
    // SMs, 2 waves against 1.75 with four k-quarters) the split costs more than it saves, 10.4 ms per step
    // against 8.3 -- four short pipelines with four epilogues and 134 MB of partial sums per launch.
    size_t part_owned = 0;
    g.splits = 1;
    {
      const int64_t tiles = tiles_m * tiles_n * batch;
      const int sms = sm_count();
      const int max_splits = g_tc_max_splits.load(std::memory_order_relaxed);
      for (int sp = 2; sp <= max_splits && tiles <= TC_MAX_TICKETS; ++sp) {
        const int per = int(ceil_div(ceil_div(int64_t(g.num_kb), int64_t(sp)), int64_t(TC_PERIOD_KB))) * TC_PERIOD_KB;
        if (per < 2 * TC_PERIOD_KB || int64_t(sp - 1) * per >= g.num_kb) continue; // at least 512 of k each, none empty
        if (tiles * sp > sms) break;
        g.splits = sp;
        g.kb_per_split = per;
      }
      if (g.splits > 1) {
        g.partials = static_cast<float *>(device_alloc(size_t(tiles) * g.splits * TC_BM * TC_BN * 4, &part_owned));
        g.tickets = g_tickets;
      }
    }
    g.bias = bias;
    g.bias_stride = bias ? bias_stride : 0;
    if (bias && bias_done) *bias_done = true;
    dim3 grid{unsigned(tiles_n * g.splits), unsigned(tiles_m), unsigned(batch)};
    const bool overlap = g_pair_overlap.load(std::memory_order_relaxed) != 0;
    g.wait_for_primary_at_end = (t_pair_second && overlap && launches_so_far() == g_promoted_seq) ? 1 : 0;
    // the matmul profile times an overlapped pair as one interval of two launches: no event between them
    if (t_pair_end_pending && !g.wait_for_primary_at_end) {
      t_pair_end_pending = false;
      matmul_profile_end();
    }
    if (g.wait_for_primary_at_end && t_pair_end_pending) matmul_profile_extend();
    else matmul_profile_begin();
    if (a_mn && b_mn) launch_promoted<true, true>(map_a, map_b, g, grid);
    else if (a_mn) launch_promoted<true, false>(map_a, map_b, g, grid);
    else if (b_mn) launch_promoted<false, true>(map_a, map_b, g, grid);
    else launch_promoted<false, false>(map_a, map_b, g, grid);
    if (t_pair_first && overlap && matmul_profile_active()) {
      t_pair_end_pending = true; // closed by the second product, or by gemm_tc_pair_role(0)
    } else {
      t_pair_end_pending = false;
      matmul_profile_end();
    }
    if (part_owned) device_free(g.partials, part_owned); // stream-ordered like the operand planes
    check_launch("gemm_3xtf32_promoted_kernel");
    g_promoted_seq = launches_so_far();
  } catch (...) {
    if (a_owned) device_free(pa, a_owned);
    if (b_owned && pb) device_free(pb, b_owned);
    throw;
  }
  if (a_owned) device_free(pa, a_owned);
  if (b_owned) device_free(pb, b_owned);
  return true;
}


// `bias` (N values, element stride bias_stride) is added in the epilogue of the promoted kernel only;
// *bias_done tells the caller whether it was.
bool gemm_3xtf32(const float *A, const float *B, float *C, int64_t batch, int64_t M, int64_t N, int64_t K,
                 int64_t a_sb, int64_t a_sm, int64_t a_sk, int64_t b_sb, int64_t b_sk, int64_t b_sn,
                 const float *bias, int64_t bias_stride, bool *bias_done) {
  if (bias_done) *bias_done = false;
  // limits of one launch / one tensor map
  if (batch < 1 || batch > 32767 || M < 1 || N < 1 || K < 1) return false;
  if (ceil_div(M, TC_BM) > 65535 || ceil_div(N, TC_BN) > 0x7fffffff) return false;
  if (M >= (int64_t(1) << 31) || N >= (int64_t(1) << 31) || K >= (int64_t(1) << 31)) return false;
  gemm_tc_prepare();
  const int64_t Kp = ceil_div(K, 32) * 32;
  size_t ra = 0, rb = 0;
  float *pa = static_cast<float *>(device_alloc(size_t(2 * batch * M * Kp) * 4, &ra));
  float *pb = static_cast<float *>(device_alloc(size_t(2 * batch * N * Kp) * 4, &rb));
  try {
    launch_split(A, pa, batch, M, K, Kp, a_sb, a_sm, a_sk);
    launch_split(B, pb, batch, N, K, Kp, b_sb, b_sn, b_sk);
    CUtensorMap map_a = make_map(pa, M, Kp, 2 * batch, TC_BM);
    CUtensorMap map_b = make_map(pb, N, Kp, 2 * batch, TC_BN);
    TcArgs g{};
    g.C = C;
    g.M = M;
    g.N = N;
    g.num_kb = int32_t(Kp / TC_BK);
    g.batch = int32_t(batch);
    g.c_vec = (N % 4 == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0) ? 1 : 0;
    g.error_flag = error_flag_ptr();
    g.wait_limit = wait_limit_clocks();
    g.bias = nullptr;
    g.bias_stride = 0;
    if (bias && g_promoted.load()) {
      g.bias = bias;
      g.bias_stride = bias_stride;
      if (bias_done) *bias_done = true;
    }
    dim3 grid{unsigned(ceil_div(N, TC_BN)), unsigned(ceil_div(M, TC_BM)), unsigned(batch)};
    matmul_profile_begin();
    if (g_promoted.load())
      gemm_3xtf32_promoted_kernel<false, false><<<grid, 320, TC_SMEM_BYTES, stream()>>>(map_a, map_b, g);
    else
      gemm_3xtf32_kernel<<<grid, 192, TC_SMEM_BYTES, stream()>>>(map_a, map_b, g);
    matmul_profile_end();
    check_launch("gemm_3xtf32_kernel");
  } catch (...) {
    device_free(pa, ra);
    device_free(pb, rb);
    throw;
  }
  device_free(pa, ra);
  device_free(pb, rb);
  return true;
}

} // namespace ntb
