// Elementwise kernels over the last two collapsed dims when an operand is stored column-major there (a
// transposed view), for large fp32 operands: a persistent, warp-specialised pipeline fed by the copy engine.
//
//   grid      one CTA per SM; CTA b takes tiles b, b + grid, ... of a list that walks the 64 x 64 output tiles
//             in groups of 4 x 4 (256 x 256 elements).  The order itself was measured to make no difference
//             (row by row, 2 x 2 ... 16 x 16 groups); the grouping serves the L2 prefetch below, whose boxes
//             cover four tiles side by side along an operand's contiguous dim.
//   warp 16   lane 0 issues the tile loads: per operand two boxes of 64 rows x 32 values (128 bytes, the
//             128-byte swizzle span), into a ring of 8 stages (one operand) or 5 (two); a column-major
//             operand is loaded through a map whose inner dim is I, so its tile lands as [j][i].  It also
//             leaves the tile's coordinates beside the stage, and an end marker after the last tile; with two
//             operands it prefetches into the L2, two rounds ahead, boxes of 64 rows x 1 KB (prefetch_for).
//   warps 0-15 run independently of one another: each waits for a stage, reads its 8 x 32 share of both
//             layouts from shared memory (the swizzle makes the [i][j] accesses conflict free and the
//             [j][i] ones 2-way), releases the stage, applies the functor, writes the results into its own
//             1 KB piece of one of three output tiles and stores that piece itself
//             (cp.async.bulk.tensor store of 8 rows x 32 values).  No CTA-wide barrier in the loop.
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
  int32_t prefetch_rounds;    // the producer prefetches into the L2 this many rounds ahead (0 = off)
  long long wait_limit;
  int *error_flag;
};

inline size_t smem_bytes(int nin) { return size_t(stages_for(nin)) * nin * TILE_BYTES + OUT_BUFS * TILE_BYTES + 1024 + 512; }

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

// The tile loads read 256-byte runs of rows that lie a whole matrix row apart -- a DRAM page per run.  The L2
// prefetch below fetches the same bytes earlier in runs of 1 KB: for the tile the CTA will handle
// `prefetch_rounds` rounds from now, if it is the first of four tiles side by side along the operand's
// contiguous dim, one box of 64 rows x 256 values.  Every CTA strides by the same amount, so each run of
// four has exactly one owner.
template <int NIN>
__device__ __forceinline__ void prefetch_for(const Args &a, int64_t slot, const CUtensorMap *pf0, const CUtensorMap *pf1) {
  int l, ti, tj;
  if (slot >= a.total || !decode(a, slot, l, ti, tj)) return;
#pragma unroll
  for (int o = 0; o < NIN; ++o) {
    const CUtensorMap *map = (o == 0) ? pf0 : pf1;
    if (a.col[o]) {
      if ((ti & 3) == 0) tma_prefetch_l2_3d(map, ti * T, tj * T, l);
    } else {
      if ((tj & 3) == 0) tma_prefetch_l2_3d(map, tj * T, ti * T, l);
    }
  }
}

// One warp's share of a tile: 8 rows x 32 columns as 8 steps of 8 x 4 elements.  `rm` / `cm` are this
// thread's byte offsets into a [i][j] / [j][i] tile for step 0; step c flips the 16-byte chunk bits of rm by c
// (the swizzle) and moves cm 4 rows down, flipping its bit 6 on odd steps.
template <int NIN, bool C0, bool C1>
__device__ __forceinline__ void fetch(const unsigned char *st, uint32_t rm, uint32_t cm, float (&v0)[8], float (&v1)[8]) {
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint32_t r = rm ^ uint32_t(c << 4);
    const uint32_t m = (cm ^ uint32_t((c & 1) << 6)) + uint32_t(c * 512);
    v0[c] = *reinterpret_cast<const float *>(st + (C0 ? m : r));
    if constexpr (NIN == 2) v1[c] = *reinterpret_cast<const float *>(st + TILE_BYTES + (C1 ? m : r));
  }
}

// map_out stores one warp's 8 rows x 32 columns; map_in* load boxes of 64 rows x 32 values; map_pf* are the
// prefetch boxes.
template <class F, int NIN>
__global__ void __launch_bounds__(THREADS, 1)
ew_tile_tma(F f, const __grid_constant__ CUtensorMap map_out, const __grid_constant__ CUtensorMap map_in0,
            const __grid_constant__ CUtensorMap map_in1, const __grid_constant__ CUtensorMap map_pf0,
            const __grid_constant__ CUtensorMap map_pf1, Args a) {
  constexpr int STAGES = stages_for(NIN);
  extern __shared__ unsigned char raw[];
  const uint32_t base = (smem_u32(raw) + 1023u) & ~1023u;
  unsigned char *aligned = raw + (base - smem_u32(raw));
  const uint32_t in0 = base;                                   // [stage][operand][half][64][32]
  const uint32_t out_off = STAGES * NIN * TILE_BYTES;          // [OUT_BUFS][half][64][32]
  const uint32_t bar_off = out_off + OUT_BUFS * TILE_BYTES;    // full[STAGES], empty[STAGES]
  const uint32_t full0 = base + bar_off, empty0 = full0 + 8 * STAGES;
  // per stage: tile_i, tile_j, lead index, valid (0 = no more tiles)
  volatile int4 *coords = reinterpret_cast<volatile int4 *>(aligned + bar_off + 128);
  volatile int *flags = reinterpret_cast<volatile int *>(aligned + bar_off + 128 + 16 * STAGES); // [0] stop, [1] poisoned

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, CONSUMERS / 32);
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
      for (int r = 0; r < a.prefetch_rounds; ++r)
        prefetch_for<NIN>(a, int64_t(blockIdx.x) + int64_t(r) * gridDim.x, &map_pf0, &map_pf1);
      for (int64_t slot = blockIdx.x;; slot += gridDim.x) {
        const bool more = slot < a.total;
        int l = 0, ti = 0, tj = 0;
        if (more) {
          if (a.prefetch_rounds > 0)
            prefetch_for<NIN>(a, slot + int64_t(a.prefetch_rounds) * gridDim.x, &map_pf0, &map_pf1);
          if (!decode(a, slot, l, ti, tj)) continue;
        }
        const int s = it % STAGES, n = it / STAGES;
        if (n > 0 && !mbar_wait(empty0 + 8 * s, uint32_t(n - 1) & 1u, a.wait_limit)) {
          atomicExch(a.error_flag, 6);
          flags[0] = 1;
          gave_up = true;
          break;
        }
        if (flags[0] != 0) break; // a consumer gave up
        coords[s].x = ti;
        coords[s].y = tj;
        coords[s].z = l;
        coords[s].w = more ? 1 : 0;
        if (!more) { // the end marker carries no data
          mbar_arrive(full0 + 8 * s);
          break;
        }
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

  // ---------------- consumers: 16 independent warps; warp w owns rows 8(w%8).. +8 and columns 32(w/8).. +32
  // of every tile, keeps its own ring of three output pieces (1 KB each) and stores them itself.
  const int li = lane >> 2, lj = lane & 3;
  const int i = 8 * (warp & 7) + li;
  const int jh = warp >> 3;
  // [i][j] layout (row-major operands and the output): half j/32, row i, 16-byte chunk ((j%32)/4) ^ (i&7)
  const uint32_t rm = uint32_t(jh) * HALF_BYTES + uint32_t(i) * 128u + uint32_t(lj) * 4u + (uint32_t(li) << 4);
  // [j][i] layout (column-major operands): half i/32, row j, chunk ((i%32)/4) ^ (j&7), word i%4; j = 32jh + 4c + lj
  const uint32_t cm = uint32_t(i >> 5) * HALF_BYTES + uint32_t(i & 3) * 4u + uint32_t(32 * jh + lj) * 128u +
                      ((uint32_t((i & 31) >> 2) ^ uint32_t(lj)) << 4);
  const uint32_t piece = uint32_t(jh) * HALF_BYTES + uint32_t(warp & 7) * 1024u; // this warp's 8 rows in an output tile
  const int colmask = (a.col[0] ? 1 : 0) | ((NIN == 2 && a.col[1]) ? 2 : 0);

  for (int it = 0;; ++it) {
    const int s = it % STAGES;
    // warp-uniform decisions: the lanes poll on their own and must leave the loop together
    if (__any_sync(0xffffffffu, flags[0] != 0)) break;
    if (!__all_sync(0xffffffffu, mbar_wait(full0 + 8 * s, uint32_t(it / STAGES) & 1u, a.wait_limit))) {
      atomicExch(a.error_flag, 6);
      flags[0] = 1;
      break;
    }
    const int ti = coords[s].x, tj = coords[s].y, l = coords[s].z;
    if (coords[s].w == 0) break;
    const unsigned char *st = aligned + (s * NIN) * TILE_BYTES;
    float v0[8], v1[8];
    if (colmask == 1) fetch<NIN, true, false>(st, rm, cm, v0, v1);
    else if (colmask == 2) fetch<NIN, false, true>(st, rm, cm, v0, v1);
    else if (colmask == 3) fetch<NIN, true, true>(st, rm, cm, v0, v1);
    else fetch<NIN, false, false>(st, rm, cm, v0, v1);
    float res[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) { // consuming v0/v1 here makes the loads complete before the stage is released
      if constexpr (NIN == 1) res[c] = f(v0[c]);
      if constexpr (NIN == 2) res[c] = f(v0[c], v1[c]);
    }
    __syncwarp();
    if (lane == 0) {
      mbar_arrive(empty0 + 8 * s);
      tma_store_wait_read<OUT_BUFS - 1>(); // the piece written three tiles ago has been read out
    }
    __syncwarp();
    unsigned char *ob = aligned + out_off + uint32_t(it % OUT_BUFS) * TILE_BYTES;
#pragma unroll
    for (int c = 0; c < 8; ++c) *reinterpret_cast<float *>(ob + (rm ^ uint32_t(c << 4))) = res[c];
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_3d(&map_out, base + out_off + uint32_t(it % OUT_BUFS) * TILE_BYTES + piece, tj * T + 32 * jh,
                   ti * T + 8 * (warp & 7), l);
      tma_store_commit();
    }
  }
  if (lane == 0) tma_store_wait_read<0>();
  __syncthreads(); // pairs with the producer warp's: it may now look at the stop flag
}

// box_rows: 64 for the tile loads, 8 for a warp's store.  prefetch_box: the map of the L2 prefetches (64 rows
// x 256 values, no swizzle) instead.
inline CUtensorMap make_map(const void *ptr, int64_t inner, int64_t rows, int64_t lead, int64_t row_stride, int64_t lead_stride,
                            uint32_t box_rows, bool prefetch_box = false) {
  CUtensorMap m;
  cuuint64_t dims[3] = {cuuint64_t(inner), cuuint64_t(rows), cuuint64_t(lead)};
  cuuint64_t strides[2] = {cuuint64_t(row_stride) * 4, cuuint64_t(lead_stride) * 4};
  cuuint32_t box[3] = {prefetch_box ? 256u : 32u, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult rc = tensor_map_encoder()(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void *>(ptr), dims, strides, box, estr,
                                     CU_TENSOR_MAP_INTERLEAVE_NONE, prefetch_box ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
                                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) fail_runtime("cuTensorMapEncodeTiled (elementwise tile) failed with code " + std::to_string(int(rc)));
  return m;
}

} // namespace tile_tma
} // namespace ntb
