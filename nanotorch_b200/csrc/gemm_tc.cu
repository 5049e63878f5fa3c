#include "nt_core.cuh"
namespace ntb {
bool gemm_3xtf32(const float *, const float *, float *, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                 int64_t, int64_t, int64_t) {
  return false;
}
} // namespace ntb
