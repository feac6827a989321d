// Prefill GEMM (M > 32). Returns 1 when a shape is not covered so the caller can fall back to
// the chunked skinny kernel.
#include "common.cuh"

int fb200_qgemm(fb200_device* dev, const fb200_qmatrix* w, const float* x, size_t m, float* y) {
  (void)dev; (void)w; (void)x; (void)m; (void)y;
  return 1;
}
