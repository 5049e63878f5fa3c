// Elementwise kernels over the last two collapsed dims when an operand is stored column-major there (a
// transposed view), for large fp32 operands: a persistent, warp-specialised pipeline fed by the copy engine.
//
//   grid      one CTA per SM; a CTA walks 64 x 64 tiles of the output, 4 x 4 tiles (256 x 256 elements) at a
//             time so that every operand, whichever of the two dims it is contiguous along, is read in runs
//             of 1 KB per tile row group.
//   warp 16   lane 0 issues the tile loads: per operand two boxes of 64 rows x 32 values (128 bytes, the
//             128-byte swizzle span), into a ring of 8 stages (one operand) or 5 (two); a column-major
//             operand is loaded through a map whose inner dim is I, so its tile lands as [j][i].
//   warps 0-15 wait for a stage, read both layouts from shared memory (the swizzle makes the [i][j] accesses
//             conflict free and the [j][i] ones 2-way), apply the functor, write the result into one of
//             three output tiles in shared memory; thread 0 hands that tile to the copy engine
//             (cp.async.bulk.tensor store) and releases the stage.
//
// Out-of-range parts of edge tiles are zero-filled on load and clipped on store, so the kernel has no edge
// code.  Every mbarrier wait is bounded; a wait that runs out records code 6 in the device flag, the CTA
// stops issuing, waits (bounded) for loads still in flight and returns.
//
// Same results as the reference's strided elementwise kernels (src/cpp/ops/elementwise.cu, one thread per
// output element through index arithmetic): the functor is applied once per element in both.
#pragma once
#include "nt_core.cuh"
#include "tma.cuh"

namespace ntb {
namespace tile_tma {

constexpr int T = 64;                       // tile edge
constexpr uint32_t HALF_BYTES = 64 * 128;   // one box: 64 rows of 128 bytes
constexpr uint32_t TILE_BYTES = 2 * HALF_BYTES;
constexpr int OUT_BUFS = 3;
constexpr int CONSUMERS = 512;
constexpr int THREADS = CONSUMERS + 32;
// Input ring depth: the loads in flight have to cover the memory latency at full rate (about 64 KB per SM).
__host__ __device__ constexpr int stages_for(int nin) { return nin == 1 ? 8 : 5; }

struct Args {
  int32_t tiles_i, tiles_j;   // tiles along I (second-to-last dim) and J (last dim)
  int32_t group_log2;         // tiles are walked in groups of G x G, G = 1 << group_log2
  int32_t groups_j;           // ceil(tiles_j / G)
  int64_t total;              // G*G * groups_i * groups_j * lead (slots; some fall outside and are skipped)
  int64_t slots_per_lead;     // G*G * groups_i * groups_j
  int32_t col[2];             // operand o is column-major over (I, J)
  long long wait_limit;
  int *error_flag;
};

inline size_t smem_bytes(int nin) { return size_t(stages_for(nin)) * nin * TILE_BYTES + OUT_BUFS * TILE_BYTES + 1024 + 128; }

// slot -> (lead, tile_i, tile_j); false when the slot lies outside the tile grid
__device__ __forceinline__ bool decode(const Args &a, int64_t slot, int &l, int &ti, int &tj) {
  l = int(slot / a.slots_per_lead);
  const int r = int(slot - int64_t(l) * a.slots_per_lead);
  const int gl = a.group_log2;
  const int g = r >> (2 * gl), w = r & ((1 << (2 * gl)) - 1);
  ti = ((g / a.groups_j) << gl) + (w >> gl);
  tj = ((g % a.groups_j) << gl) + (w & ((1 << gl) - 1));
  return ti < a.tiles_i && tj < a.tiles_j;
}

// One warp's share of a tile: 8 rows x 32 columns as 8 steps of 8 x 4 elements.  `rm` / `cm` are this
// thread's byte offsets into a [i][j] / [j][i] tile for step 0; step c flips the 16-byte chunk bits of rm by c
// (the swizzle) and moves cm 4 rows down, flipping its bit 6 on odd steps.
template <class F, int NIN, bool C0, bool C1>
__device__ __forceinline__ void consume(const F &f, const unsigned char *st, unsigned char *ob, uint32_t rm, uint32_t cm) {
  float v0[8], v1[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint32_t r = rm ^ uint32_t(c << 4);
    const uint32_t m = (cm ^ uint32_t((c & 1) << 6)) + uint32_t(c * 512);
    v0[c] = *reinterpret_cast<const float *>(st + (C0 ? m : r));
    if constexpr (NIN == 2) v1[c] = *reinterpret_cast<const float *>(st + TILE_BYTES + (C1 ? m : r));
  }
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    float res;
    if constexpr (NIN == 1) res = f(v0[c]);
    if constexpr (NIN == 2) res = f(v0[c], v1[c]);
    *reinterpret_cast<float *>(ob + (rm ^ uint32_t(c << 4))) = res;
  }
}

template <class F, int NIN>
__global__ void __launch_bounds__(THREADS, 1)
ew_tile_tma(F f, const __grid_constant__ CUtensorMap map_out, const __grid_constant__ CUtensorMap map_in0,
            const __grid_constant__ CUtensorMap map_in1, Args a) {
  constexpr int STAGES = stages_for(NIN);
  extern __shared__ unsigned char raw[];
  const uint32_t base = (smem_u32(raw) + 1023u) & ~1023u;
  unsigned char *aligned = raw + (base - smem_u32(raw));
  const uint32_t in0 = base;                                   // [stage][operand][half][64][32]
  const uint32_t out0 = base + STAGES * NIN * TILE_BYTES;      // [OUT_BUFS][half][64][32]
  const uint32_t bar0 = out0 + OUT_BUFS * TILE_BYTES;          // full[STAGES], empty[STAGES]
  volatile int *flags = reinterpret_cast<volatile int *>(aligned + (bar0 - base) + 8 * 2 * STAGES); // [0] stop, [1] poisoned
  const uint32_t full0 = bar0, empty0 = bar0 + 8 * STAGES;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    flags[0] = 0;
    flags[1] = *reinterpret_cast<volatile int *>(a.error_flag); // an earlier kernel gave up: do nothing
  }
  __syncthreads();
  if (flags[1] != 0) return;

  if (warp == CONSUMERS / 32) {
    // ---------------- producer
    int it = 0;
    bool gave_up = false;
    if (lane == 0) {
      for (int64_t slot = blockIdx.x; slot < a.total; slot += gridDim.x) {
        int l, ti, tj;
        if (!decode(a, slot, l, ti, tj)) continue;
        const int s = it % STAGES, n = it / STAGES;
        if (n > 0 && !mbar_wait(empty0 + 8 * s, uint32_t(n - 1) & 1u, a.wait_limit)) {
          atomicExch(a.error_flag, 6);
          gave_up = true;
          break;
        }
        if (flags[0] != 0) break; // the consumers stopped
        mbar_expect_tx(full0 + 8 * s, NIN * TILE_BYTES);
#pragma unroll
        for (int o = 0; o < NIN; ++o) {
          const CUtensorMap *map = (o == 0) ? &map_in0 : &map_in1;
          const uint32_t dst = in0 + (s * NIN + o) * TILE_BYTES;
          // row-major operand: inner coordinate is j; column-major: inner coordinate is i
          const int x = a.col[o] ? ti * T : tj * T;
          const int y = a.col[o] ? tj * T : ti * T;
          tma_load_3d(dst, map, full0 + 8 * s, x, y, l);
          tma_load_3d(dst + HALF_BYTES, map, full0 + 8 * s, x + 32, y, l);
        }
        ++it;
      }
    }
    __syncwarp();
    __syncthreads(); // every consumer is past its loop
    // Loads still in flight when the consumers stopped early must land before the CTA's shared memory goes.
    if (lane == 0 && (gave_up || flags[0] != 0)) {
      for (int k = (it > STAGES ? it - STAGES : 0); k < it; ++k)
        mbar_wait(full0 + 8 * (k % STAGES), uint32_t(k / STAGES) & 1u, a.wait_limit);
    }
    return;
  }

  // ---------------- consumers: warp w owns rows 8(w%8).. +8 and columns 32(w/8).. +32 of the tile
  const int li = lane >> 2, lj = lane & 3;
  const int i = 8 * (warp & 7) + li;
  const int jh = warp >> 3;
  // [i][j] layout (row-major operands and the output): half j/32, row i, 16-byte chunk ((j%32)/4) ^ (i&7)
  const uint32_t rm = uint32_t(jh) * HALF_BYTES + uint32_t(i) * 128u + uint32_t(lj) * 4u + (uint32_t(li) << 4);
  // [j][i] layout (column-major operands): half i/32, row j, chunk ((i%32)/4) ^ (j&7), word i%4; j = 32jh + 4c + lj
  const uint32_t cm = uint32_t(i >> 5) * HALF_BYTES + uint32_t(i & 3) * 4u + uint32_t(32 * jh + lj) * 128u +
                      ((uint32_t((i & 31) >> 2) ^ uint32_t(lj)) << 4);
  const int colmask = (a.col[0] ? 1 : 0) | ((NIN == 2 && a.col[1]) ? 2 : 0);

  int it = 0;
  for (int64_t slot = blockIdx.x; slot < a.total; slot += gridDim.x) {
    int l, ti, tj;
    if (!decode(a, slot, l, ti, tj)) continue;
    const int s = it % STAGES;
    const uint32_t ob_off = (out0 - base) + uint32_t(it % OUT_BUFS) * TILE_BYTES;
    const bool ok = mbar_wait(full0 + 8 * s, uint32_t(it / STAGES) & 1u, a.wait_limit);
    if (!ok) {
      atomicExch(a.error_flag, 6);
      flags[0] = 1;
    } else {
      const unsigned char *st = aligned + (s * NIN) * TILE_BYTES;
      unsigned char *ob = aligned + ob_off;
      if (colmask == 1) consume<F, NIN, true, false>(f, st, ob, rm, cm);
      else if (colmask == 2) consume<F, NIN, false, true>(f, st, ob, rm, cm);
      else if (colmask == 3) consume<F, NIN, true, true>(f, st, ob, rm, cm);
      else consume<F, NIN, false, false>(f, st, ob, rm, cm);
      fence_proxy_async_smem();
    }
    // the store issued two steps ago read the output tile that the next step writes: it must have drained
    if (tid == 0) tma_store_wait_read<1>();
    asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS) : "memory");
    if (flags[0] != 0) break;
    if (tid == 0) {
      tma_store_3d(&map_out, base + ob_off, tj * T, ti * T, l);
      tma_store_3d(&map_out, base + ob_off + HALF_BYTES, tj * T + 32, ti * T, l);
      tma_store_commit();
      mbar_arrive(empty0 + 8 * s);
    }
    ++it;
  }
  if (tid == 0) tma_store_wait_read<0>();
  __syncthreads(); // pairs with the producer warp's: it may now look at the stop flag
}

// dims/strides in elements; the inner dim has unit stride.
inline CUtensorMap make_map(const void *ptr, int64_t inner, int64_t rows, int64_t lead, int64_t row_stride, int64_t lead_stride) {
  CUtensorMap m;
  cuuint64_t dims[3] = {cuuint64_t(inner), cuuint64_t(rows), cuuint64_t(lead)};
  cuuint64_t strides[2] = {cuuint64_t(row_stride) * 4, cuuint64_t(lead_stride) * 4};
  cuuint32_t box[3] = {32, 64, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult rc = tensor_map_encoder()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void *>(ptr), dims, strides, box, estr,
                                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) fail_runtime("cuTensorMapEncodeTiled (elementwise tile) failed with code " + std::to_string(int(rc)));
  return m;
}

} // namespace tile_tma
} // namespace ntb
