// Products with weights kept in raw row-major form (F32, F16, Q5_0, Q5_K): the reference's
// Tensor::q_mat_mul dequantises such a matrix and runs a dense matmul
// (fusor-ml/fusor/src/lib.rs:1184-1215). These types are outside the tuned path; one warp forms
// one output with element-wise dequantisation and a fixed-order shuffle reduction.
#include "formats.cuh"

namespace {

__global__ void dense_matmul_kernel(uint32_t type, const uint8_t* __restrict__ w,
                                    const float* __restrict__ x, uint64_t m, uint64_t n, uint64_t k,
                                    float* __restrict__ y) {
  const uint64_t warp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= m * n) return;
  const uint64_t mi = warp / n, ni = warp % n;
  float acc = 0.f;
  for (uint64_t c = lane; c < k; c += 32)
    acc = fmaf(x[mi * k + c], fb::raw_elem(type, w, ni * k + c), acc);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
  if (lane == 0) y[mi * n + ni] = acc;
}

}  // namespace

int fb200_dense_matmul(fb200_device* dev, const fb200_qmatrix* w, const float* x, size_t m, float* y) {
  const uint64_t warps = (uint64_t)m * w->n;
  const uint64_t blocks = (warps * 32 + 255) / 256;
  if (blocks >= (1ull << 31)) return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "dense matmul too large");
  dense_matmul_kernel<<<(unsigned)blocks, 256, 0, dev->stream>>>(w->type, w->data, x, m, w->n, w->k, y);
  FB_LAUNCH_CHECK(dev);
  return FB200_OK;
}
