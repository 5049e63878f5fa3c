// Index-array ("fancy") gather and scatter on the device.
//
// The reference implements these two only for CPU storages, one element at a time with std::vector
// coordinate counters (src/cpp/ops/copy_ops.cu:7-83 scatter_to_axes, :85-160 gather_from_axes), and
// its Python layer validates and wraps negative indices by walking the index buffer on the host
// (src/nanotorch/core.py:708-718).  Here both run as one HBM-bound copy kernel:
//
//   - the iteration space is the result shape (gather) or the source shape (scatter); a thread
//     owns UNROLL work items, issues all of its index loads first, then all data loads, then the
//     stores, so two dependent memory latencies are paid once per UNROLL items;
//   - when the innermost iteration dim is a basic (non-indexed) dim that is unit-stride on both
//     sides and everything is 16-byte aligned, a work item is a 16-byte vector, so a row gather
//     x[idx] moves 128 bits per access;
//   - negative indices wrap in the kernel; an optional validation pass over the index arrays
//     reports the first out-of-range value before anything is written (same IndexError as the
//     reference), at the price of one synchronisation -- callers that validated on the host skip it;
//   - scatter with colliding destinations must end with the value the reference's sequential loop
//     writes last.  Unless the caller vouches for unique destinations, a first pass records per
//     destination index tuple the highest source position over the index-array dims (atomicMax) and
//     the copy pass lets only that position write: deterministic and identical to the sequential
//     order.  The table has one entry per destination index tuple -- per row for a row scatter.
#include "elementwise.cuh"

namespace ntb {

constexpr int IX_UNROLL = 4;

struct IndexParams {
  int ndim;     // iteration dims
  int n_fancy;  // index arrays
  int64_t items; // work items (vectors or elements)
  int64_t shape[NT_MAX_DIMS];
  uint32_t div_mul[NT_MAX_DIMS], div_shift[NT_MAX_DIMS];
  int64_t lin_stride[NT_MAX_DIMS];            // linear side: gather output / scatter source
  int64_t ix_stride[NT_MAX_DIMS];             // indexed side, basic dims (0 where the iteration dim is an index dim)
  int64_t ind_stride[NT_MAX_DIMS][NT_MAX_DIMS]; // [p][d]: stride of index array p along iteration dim d
  const int64_t *ind[NT_MAX_DIMS];            // index arrays, advanced by their offsets
  int64_t ind_extent[NT_MAX_DIMS];            // extent of the indexed dim (wrap + range check)
  int64_t ix_fancy_stride[NT_MAX_DIMS];       // stride of the indexed operand along that dim
  // Ordered scatter.  Two source items can only land on the same destination element when they agree on every
  // basic dim, and then their order in the sequential loop is the order of their coordinates on the index-array
  // dims alone.  So the owner table has one entry per destination index tuple (key = sum of index value x
  // key_stride), and the value compared is the item's row-major rank over the index-array dims only
  // (rank_stride is 0 on basic dims): a row scatter keeps one entry per destination row, not per element.
  int64_t rank_stride[NT_MAX_DIMS];
  int64_t key_stride[NT_MAX_DIMS];
  int owner64; // owner entries are 64-bit (2^31 or more positions on the index-array dims)
};

// First out-of-range index seen by a validation pass.
struct IndexError {
  int flag;
  long long value;
  long long extent;
};

// NF > 0: the number of index arrays is known at compile time (their offsets stay in registers).
template <class IDX, int NF, bool WANT_RANK>
__device__ __forceinline__ void ix_offsets(const IndexParams &p, IDX lin, int64_t &lin_off, int64_t &ix_off,
                                           int64_t (&ind_off)[NF > 0 ? NF : NT_MAX_DIMS], int64_t &rank) {
  lin_off = 0;
  ix_off = 0;
  rank = 0;
  const int nf = NF > 0 ? NF : p.n_fancy;
#pragma unroll
  for (int q = 0; q < nf; ++q) ind_off[q] = 0;
  for (int d = p.ndim - 1; d >= 0; --d) {
    IDX ext = IDX(p.shape[d]);
    IDX quo;
    if constexpr (sizeof(IDX) == 4)
      quo = p.div_mul[d] ? (__umulhi(lin, p.div_mul[d]) >> p.div_shift[d]) : lin;
    else
      quo = lin / ext;
    const int64_t r = int64_t(lin - quo * ext);
    lin = quo;
    lin_off += r * p.lin_stride[d];
    ix_off += r * p.ix_stride[d];
    if constexpr (WANT_RANK) rank += r * p.rank_stride[d];
#pragma unroll
    for (int q = 0; q < nf; ++q) ind_off[q] += r * p.ind_stride[q][d];
  }
}

// MODE 0: gather  (to[lin] = from[ix]);  1: scatter (to[ix] = from[lin]);
// MODE 2: scatter ordering pass (owner[key] = max(owner[key], rank + 1));
// MODE 3: scatter copy pass that only lets the recorded owner write.
template <class V, class IDX, int MODE, int NF>
__global__ void __launch_bounds__(256) index_copy(IndexParams p, const V *from, V *to, unsigned long long *owner) {
  const int nf = NF > 0 ? NF : p.n_fancy;
  const int64_t base = (int64_t(blockIdx.x) * IX_UNROLL) * blockDim.x + threadIdx.x;
  constexpr bool ORDERED = MODE == 2 || MODE == 3;
  int64_t lin_off[IX_UNROLL], ix_off[IX_UNROLL], rank[IX_UNROLL], key[IX_UNROLL];
  bool live[IX_UNROLL];
#pragma unroll
  for (int u = 0; u < IX_UNROLL; ++u) {
    const int64_t item = base + int64_t(u) * blockDim.x;
    live[u] = item < p.items;
    key[u] = 0;
    if (live[u]) {
      int64_t ind_off[NF > 0 ? NF : NT_MAX_DIMS];
      ix_offsets<IDX, NF, ORDERED>(p, IDX(item), lin_off[u], ix_off[u], ind_off, rank[u]);
#pragma unroll
      for (int q = 0; q < nf; ++q) {
        long long c = __ldg(p.ind[q] + ind_off[q]);
        const long long ext = p.ind_extent[q];
        if (c < 0) c += ext;
        if (c < 0 || c >= ext) live[u] = false; // reported by the validation pass; never dereferenced
        ix_off[u] += c * p.ix_fancy_stride[q];
        if constexpr (ORDERED) key[u] += c * p.key_stride[q];
      }
    }
  }
  if constexpr (MODE == 2) {
#pragma unroll
    for (int u = 0; u < IX_UNROLL; ++u)
      if (live[u]) {
        if (p.owner64) atomicMax(owner + key[u], static_cast<unsigned long long>(rank[u]) + 1ull);
        else atomicMax(reinterpret_cast<unsigned int *>(owner) + key[u], static_cast<unsigned int>(rank[u]) + 1u);
      }
    return;
  }
  V val[IX_UNROLL];
#pragma unroll
  for (int u = 0; u < IX_UNROLL; ++u) {
    if constexpr (MODE == 3) {
      if (live[u])
        live[u] = p.owner64 ? owner[key[u]] == static_cast<unsigned long long>(rank[u]) + 1ull
                            : reinterpret_cast<const unsigned int *>(owner)[key[u]] == static_cast<unsigned int>(rank[u]) + 1u;
    }
    if (live[u]) val[u] = (MODE == 0) ? from[ix_off[u]] : from[lin_off[u]];
  }
#pragma unroll
  for (int u = 0; u < IX_UNROLL; ++u)
    if (live[u]) {
      if constexpr (MODE == 0)
        to[lin_off[u]] = val[u];
      else
        to[ix_off[u]] = val[u];
    }
}

// One thread per element of one index array view: flags the first value outside [-extent, extent).
struct ValidateParams {
  int ndim;
  int64_t numel;
  int64_t shape[NT_MAX_DIMS], strides[NT_MAX_DIMS];
  const int64_t *data;
  int64_t extent;
};
__global__ void __launch_bounds__(256) index_validate(ValidateParams p, IndexError *err) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= p.numel) return;
  int64_t lin = i, off = 0;
  for (int d = p.ndim - 1; d >= 0; --d) {
    const int64_t q = lin / p.shape[d];
    off += (lin - q * p.shape[d]) * p.strides[d];
    lin = q;
  }
  const long long c = p.data[off];
  if (c < -p.extent || c >= p.extent) {
    if (atomicCAS(&err->flag, 0, 1) == 0) {
      err->value = c < 0 ? c + p.extent : c; // the reference reports the value after wrapping
      err->extent = p.extent;
    }
  }
}

namespace {

struct Plan {
  IndexParams p{};
  int itemsize = 0; // bytes per element
  int vec = 1;      // elements per work item
  const char *lin_base = nullptr; // byte pointers, already advanced by the view offsets
  const char *ix_base = nullptr;
  int64_t key_count = 1;          // destination index tuples: entries of the ordered scatter's owner table
};

[[noreturn]] void fail_index(const std::string &m) { throw Error(NT_ERR_INDEX, m); }

// `lin` is the operand walked linearly (shape = the iteration space), `ix` the operand addressed
// through the index arrays.
Plan make_plan(const char *fname, const int64_t *it_shape, int it_ndim, const int64_t *lin_strides, int64_t lin_offset,
               nt_storage *lin_storage, const nt_view *ix, const int64_t *fancy_dims, int n_fancy,
               const nt_view *fancy_data, const uint8_t *axis_is_fancy, const int64_t *axis_target) {
  const std::string f(fname);
  if (it_ndim < 0 || it_ndim > NT_MAX_DIMS) fail_runtime(f + ": at most 8 dimensions.");
  if (n_fancy < 0 || n_fancy > NT_MAX_DIMS) fail_invalid(f + ": at most 8 index arrays.");
  Plan pl;
  IndexParams &p = pl.p;
  p.ndim = it_ndim;
  p.n_fancy = n_fancy;
  const int ind_ndim = n_fancy ? fancy_data[0].ndim : 0;
  std::vector<int> fancy_of_dim(ix->ndim, -1);
  for (int q = 0; q < n_fancy; ++q) {
    const nt_view &iv = fancy_data[q];
    check_view(&iv, fname);
    if (iv.storage->dtype != NT_INT64) fail_invalid(f + ": index arrays must be Int64.");
    if (iv.storage->device != NT_CUDA) fail_runtime(f + ": requires Cuda.");
    if (iv.ndim != ind_ndim) fail_invalid(f + ": index arrays must share one shape.");
    for (int d = 0; d < ind_ndim; ++d)
      if (iv.shape[d] != fancy_data[0].shape[d]) fail_invalid(f + ": index arrays must share one shape.");
    const int64_t dim = fancy_dims[q];
    if (dim < 0 || dim >= ix->ndim || fancy_of_dim[dim] != -1) fail_invalid(f + ": bad indexed dimension.");
    fancy_of_dim[dim] = q;
    p.ind[q] = static_cast<const int64_t *>(iv.storage->data) + iv.offset;
    p.ind_extent[q] = ix->shape[dim];
    p.ix_fancy_stride[q] = ix->strides[dim];
  }
  std::vector<bool> basic_used(ix->ndim, false), ind_used(ind_ndim > 0 ? ind_ndim : 0, false);
  int64_t items = 1;
  for (int d = 0; d < it_ndim; ++d) {
    p.shape[d] = it_shape[d];
    items *= it_shape[d];
    p.lin_stride[d] = lin_strides[d];
    const int64_t t = axis_target[d];
    if (axis_is_fancy[d]) {
      if (t < 0 || t >= ind_ndim || ind_used[t]) fail_invalid(f + ": bad index-array axis.");
      ind_used[t] = true;
      if (it_shape[d] != fancy_data[0].shape[t]) fail_invalid(f + ": shape does not match the index arrays.");
      for (int q = 0; q < n_fancy; ++q) p.ind_stride[q][d] = fancy_data[q].strides[t];
    } else {
      if (t < 0 || t >= ix->ndim || basic_used[t] || fancy_of_dim[t] != -1) fail_invalid(f + ": bad basic axis.");
      basic_used[t] = true;
      if (it_shape[d] != ix->shape[t]) fail_invalid(f + ": shape does not match the indexed tensor.");
      p.ix_stride[d] = ix->strides[t];
    }
  }
  // a dim of the indexed operand that nothing addresses stays at coordinate 0, as in the reference's
  // zero-initialised counters; it must then have extent >= 1
  p.items = items;
  pl.itemsize = int(dtype_itemsize(ix->storage->dtype));
  pl.lin_base = static_cast<const char *>(lin_storage->data) + lin_offset * pl.itemsize;
  pl.ix_base = static_cast<const char *>(ix->storage->data) + ix->offset * pl.itemsize;
  {
    int64_t acc = 1;
    for (int d = it_ndim - 1; d >= 0; --d) {
      p.rank_stride[d] = axis_is_fancy[d] ? acc : 0;
      if (axis_is_fancy[d]) acc *= it_shape[d];
    }
    acc = 1;
    for (int q = n_fancy - 1; q >= 0; --q) {
      p.key_stride[q] = acc;
      acc *= p.ind_extent[q];
    }
    pl.key_count = acc;
  }
  {
    int64_t positions = 1;
    for (int d = 0; d < it_ndim; ++d)
      if (axis_is_fancy[d]) positions *= it_shape[d];
    p.owner64 = positions >= (int64_t(1) << 31) ? 1 : 0;
  }

  // 16-byte work items when the innermost iteration dim is a basic unit-stride run on both sides
  const int vec = 16 / pl.itemsize;
  if (it_ndim > 0 && items > 0 && !axis_is_fancy[it_ndim - 1]) {
    const int last = it_ndim - 1;
    bool ok = p.lin_stride[last] == 1 && p.ix_stride[last] == 1 && p.shape[last] % vec == 0;
    ok = ok && reinterpret_cast<uintptr_t>(pl.lin_base) % 16 == 0 && reinterpret_cast<uintptr_t>(pl.ix_base) % 16 == 0;
    for (int d = 0; d < last && ok; ++d) ok = p.lin_stride[d] % vec == 0 && p.ix_stride[d] % vec == 0;
    for (int q = 0; q < n_fancy && ok; ++q) ok = p.ix_fancy_stride[q] % vec == 0;
    if (ok) {
      pl.vec = vec;
      p.shape[last] /= vec;
      p.items /= vec;
      for (int d = 0; d < last; ++d) {
        p.lin_stride[d] /= vec;
        p.ix_stride[d] /= vec;
      }
      for (int q = 0; q < n_fancy; ++q) p.ix_fancy_stride[q] /= vec;
    }
  }
  for (int d = 0; d < it_ndim; ++d) ew_fast_divisor(p.shape[d], &p.div_mul[d], &p.div_shift[d]);
  return pl;
}

// Synchronous range check of every index array; throws the reference's IndexError text.
void validate_indices(const nt_view *ix, const int64_t *fancy_dims, int n_fancy, const nt_view *fancy_data) {
  if (n_fancy == 0) return;
  size_t rounded = 0;
  IndexError *err = static_cast<IndexError *>(device_alloc(sizeof(IndexError), &rounded));
  struct Guard {
    void *p;
    size_t r;
    ~Guard() { device_free(p, r); }
  } guard{err, rounded};
  NT_CUDA_CHECK(cudaMemsetAsync(err, 0, sizeof(IndexError), stream()));
  for (int q = 0; q < n_fancy; ++q) {
    const nt_view &iv = fancy_data[q];
    ValidateParams vp{};
    vp.ndim = iv.ndim;
    vp.numel = view_numel(iv);
    for (int d = 0; d < iv.ndim; ++d) {
      vp.shape[d] = iv.shape[d];
      vp.strides[d] = iv.strides[d];
    }
    vp.data = static_cast<const int64_t *>(iv.storage->data) + iv.offset;
    vp.extent = ix->shape[fancy_dims[q]];
    if (vp.numel == 0) continue;
    index_validate<<<unsigned(ceil_div(vp.numel, 256)), 256, 0, stream()>>>(vp, err);
    check_launch("index_validate");
  }
  IndexError host{};
  NT_CUDA_CHECK(cudaMemcpyAsync(&host, err, sizeof(host), cudaMemcpyDeviceToHost, stream()));
  NT_CUDA_CHECK(cudaStreamSynchronize(stream()));
  if (host.flag)
    fail_index("Invalid index " + std::to_string(host.value) + " in axis of len " + std::to_string(host.extent) + ".");
}

template <class V, int MODE> void launch_mode(const Plan &pl, const void *from, void *to, unsigned long long *owner) {
  const int64_t per_block = 256 * IX_UNROLL;
  const int64_t blocks = ceil_div(pl.p.items, per_block);
  if (blocks > 0x7fffffffLL) fail_runtime("index copy: too many elements for one launch.");
  const V *f = static_cast<const V *>(from);
  V *t = static_cast<V *>(to);
  const bool small = pl.p.items < (int64_t(1) << 31);
  if (pl.p.n_fancy == 1) {
    if (small)
      index_copy<V, uint32_t, MODE, 1><<<unsigned(blocks), 256, 0, stream()>>>(pl.p, f, t, owner);
    else
      index_copy<V, uint64_t, MODE, 1><<<unsigned(blocks), 256, 0, stream()>>>(pl.p, f, t, owner);
  } else {
    if (small)
      index_copy<V, uint32_t, MODE, 0><<<unsigned(blocks), 256, 0, stream()>>>(pl.p, f, t, owner);
    else
      index_copy<V, uint64_t, MODE, 0><<<unsigned(blocks), 256, 0, stream()>>>(pl.p, f, t, owner);
  }
  check_launch("index_copy");
}

template <int MODE> void launch_width(const Plan &pl, const void *from, void *to, unsigned long long *owner) {
  switch (pl.itemsize * pl.vec) {
  case 1: return launch_mode<uint8_t, MODE>(pl, from, to, owner);
  case 4: return launch_mode<uint32_t, MODE>(pl, from, to, owner);
  case 8: return launch_mode<unsigned long long, MODE>(pl, from, to, owner);
  case 16: return launch_mode<uint4, MODE>(pl, from, to, owner);
  default: fail_runtime("index copy: unsupported element width.");
  }
}

} // namespace
} // namespace ntb

using namespace ntb;

extern "C" {

int nt_gather_from_axes(const nt_view *x, const int64_t *new_shape, int32_t new_ndim, const int64_t *fancy_dims_in_src,
                        int32_t n_fancy, const nt_view *fancy_dims_data, const uint8_t *out_axis_is_fancy,
                        const int64_t *out_axis_target, uint32_t flags, nt_storage **out) {
  NT_API_BEGIN
  const char *fname = "gather_from_axes";
  check_view(x, fname);
  require_cuda(x, fname);
  if (new_ndim < 0 || new_ndim > NT_MAX_DIMS) fail_runtime("gather_from_axes: at most 8 dimensions.");
  int64_t numel = 1, contig[NT_MAX_DIMS];
  for (int d = new_ndim - 1; d >= 0; --d) {
    if (new_shape[d] < 0) fail_invalid("gather_from_axes: negative extent.");
    contig[d] = numel;
    numel *= new_shape[d];
  }
  StorageRef o(storage_new(numel, x->storage->dtype, NT_CUDA));
  Plan pl = make_plan(fname, new_shape, new_ndim, contig, 0, o.s, x, fancy_dims_in_src, n_fancy, fancy_dims_data,
                      out_axis_is_fancy, out_axis_target);
  if (numel > 0) {
    if (!(flags & NT_INDEX_CHECKED)) validate_indices(x, fancy_dims_in_src, n_fancy, fancy_dims_data);
    launch_width<0>(pl, pl.ix_base, const_cast<char *>(pl.lin_base), nullptr);
  }
  *out = o.release();
  NT_API_END
}

int nt_scatter_to_axes(const nt_view *src, const nt_view *out, const int64_t *fancy_dims_in_src, int32_t n_fancy,
                       const nt_view *fancy_dims_data, const uint8_t *out_axis_is_fancy, const int64_t *out_axis_target,
                       uint32_t flags) {
  NT_API_BEGIN
  const char *fname = "scatter_to_axes";
  check_view(src, fname);
  check_view(out, fname);
  require_cuda(src, fname);
  require_cuda(out, fname);
  require_same_dtype(src, out, fname);
  Plan pl = make_plan(fname, src->shape, src->ndim, src->strides, src->offset, src->storage, out, fancy_dims_in_src,
                      n_fancy, fancy_dims_data, out_axis_is_fancy, out_axis_target);
  if (pl.p.items > 0) {
    if (!(flags & NT_INDEX_CHECKED)) validate_indices(out, fancy_dims_in_src, n_fancy, fancy_dims_data);
    char *to = const_cast<char *>(pl.ix_base);
    if (flags & NT_INDEX_UNIQUE) {
      launch_width<1>(pl, pl.lin_base, to, nullptr);
    } else {
      // one owner entry per destination index tuple (see IndexParams)
      const size_t width = pl.p.owner64 ? 8 : 4;
      const size_t bytes = size_t(pl.key_count > 0 ? pl.key_count : 1) * width;
      size_t rounded = 0;
      auto *scratch = static_cast<char *>(device_alloc(bytes, &rounded));
      struct Guard {
        void *p;
        size_t r;
        ~Guard() { device_free(p, r); }
      } guard{scratch, rounded};
      NT_CUDA_CHECK(cudaMemsetAsync(scratch, 0, bytes, stream()));
      auto *middle = reinterpret_cast<unsigned long long *>(scratch);
      // The ordering pass only needs one item per position on the index-array dims: the same plan with every
      // basic dim shrunk to extent 1 (all items of a row would otherwise hammer one counter).
      Plan order = pl;
      order.p.items = 1;
      for (int d = 0; d < order.p.ndim; ++d) {
        if (order.p.rank_stride[d] == 0) order.p.shape[d] = 1; // a basic dim
        order.p.items *= order.p.shape[d];
        ew_fast_divisor(order.p.shape[d], &order.p.div_mul[d], &order.p.div_shift[d]);
      }
      launch_width<2>(order, pl.lin_base, to, middle);
      launch_width<3>(pl, pl.lin_base, to, middle);
    }
  }
  storage_touch(out->storage);
  NT_API_END
}

} // extern "C"
