// Raw GGUF blocks -> tile-interleaved storage, and dequantisation back to row-major f32.
#include "formats.cuh"

namespace {

// One thread per destination byte. Rows beyond N and blocks beyond K are zero (a zero scale
// makes every element of such a block dequantise to 0).
__global__ void repack_kernel(uint32_t type, const uint8_t* __restrict__ raw, uint64_t n,
                              uint64_t row_bytes, int blocks_per_row, int block_bytes,
                              int blocks_per_group, uint8_t* __restrict__ tiled, int ngroups,
                              int tg_bytes, int tile0, uint64_t total) {
  uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  int o = (int)(idx % (uint64_t)tg_bytes);
  uint64_t tgi = idx / (uint64_t)tg_bytes;
  int kg = (int)(tgi % (uint64_t)ngroups);
  uint64_t tile = tgi / (uint64_t)ngroups;
  int row, src;
  fb::tile_src(type, o, &row, &src);
  uint64_t r = (tile + (uint64_t)tile0) * 16 + (uint64_t)row;
  uint8_t v = 0;
  int blk = kg * blocks_per_group + src / block_bytes;
  if (r < n && blk < blocks_per_row)
    v = raw[r * row_bytes + (uint64_t)kg * blocks_per_group * block_bytes + src];
  tiled[idx] = v;
}

// Q5_0 blocks {f16 d, u32 qh, qs[16]} -> Q8_0 blocks {f16 d, i8 q[32]} with q = q5 - 16: the same
// d and the same integers, so (q5 - 16) * d dequantises to the same bits from either form
// (BlockQ5_0::dequantize / BlockQ8_0::dequantize, fusor-ml/gguf/src/lib.rs:1046-1073, 1284-1288).
// One thread per output byte.
__global__ void widen_q5_0_kernel(const uint8_t* __restrict__ q5, uint64_t total, uint8_t* __restrict__ q8) {
  const uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const uint64_t blk = idx / 34;
  const int o = (int)(idx % 34);
  const uint8_t* b = q5 + blk * 22;
  if (o < 2) {
    q8[idx] = b[o];
    return;
  }
  const int i = o - 2, p = i & 15;
  const uint32_t qh = (uint32_t)b[2] | ((uint32_t)b[3] << 8) | ((uint32_t)b[4] << 16) | ((uint32_t)b[5] << 24);
  const int nib = i < 16 ? (b[6 + p] & 0xF) : (b[6 + p] >> 4);
  const int hi = (qh >> i) & 1;
  q8[idx] = (uint8_t)(int8_t)((nib | (hi << 4)) - 16);
}

__global__ void dequant_tiled_kernel(uint32_t type, const uint8_t* __restrict__ tiled, uint64_t n,
                                     uint64_t k, int ngroups, int group_elems, int tg_bytes,
                                     float* __restrict__ out) {
  uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n * k) return;
  uint64_t r = idx / k;
  uint64_t c = idx % k;
  int kg = (int)(c / group_elems), i = (int)(c % group_elems);
  const uint8_t* tg = tiled + ((r >> 4) * (uint64_t)ngroups + kg) * (uint64_t)tg_bytes;
  out[idx] = fb::tile_dequant(type, tg, (int)(r & 15), i);
}

// Rows selected by ids (embedding lookup): out[j, :] = dequant(W[ids[j], :]).
__global__ void dequant_rows_tiled_kernel(uint32_t type, const uint8_t* __restrict__ tiled,
                                          uint64_t n, uint64_t k, int ngroups, int group_elems,
                                          int tg_bytes, const uint32_t* __restrict__ ids,
                                          float* __restrict__ out) {
  uint64_t j = blockIdx.y;
  uint64_t r = ids[j];
  for (uint64_t c = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; c < k;
       c += (uint64_t)gridDim.x * blockDim.x) {
    float v = 0.f;
    if (r < n) {
      int kg = (int)(c / group_elems), i = (int)(c % group_elems);
      const uint8_t* tg = tiled + ((r >> 4) * (uint64_t)ngroups + kg) * (uint64_t)tg_bytes;
      v = fb::tile_dequant(type, tg, (int)(r & 15), i);
    }
    out[j * k + c] = v;
  }
}

__global__ void dequant_raw_kernel(uint32_t type, const uint8_t* __restrict__ raw, uint64_t total,
                                   float* __restrict__ out) {
  uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < total) out[idx] = fb::raw_elem(type, raw, idx);
}

__global__ void dequant_rows_raw_kernel(uint32_t type, const uint8_t* __restrict__ raw, uint64_t n,
                                        uint64_t k, const uint32_t* __restrict__ ids,
                                        float* __restrict__ out) {
  uint64_t j = blockIdx.y;
  uint64_t r = ids[j];
  for (uint64_t c = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; c < k;
       c += (uint64_t)gridDim.x * blockDim.x)
    out[j * k + c] = r < n ? fb::raw_elem(type, raw, r * k + c) : 0.f;
}

}  // namespace

int fb200_launch_repack(fb200_device* dev, uint32_t type, const uint8_t* raw_dev, uint64_t n,
                        uint64_t k, uint8_t* tiled_dev, int ntiles, int ngroups, int tile0) {
  TileGeom g;
  if (!tile_geom(type, &g)) return fb200_fail(dev, FB200_ERR_UNSUPPORTED_DTYPE, "repack: type %u", type);
  uint64_t total = (uint64_t)ntiles * ngroups * g.tg_bytes;
  if (total == 0) return FB200_OK;
  int blocks_per_row = (int)(k / g.block_elems);
  uint64_t row_bytes = (uint64_t)blocks_per_row * g.block_bytes;
  uint64_t nblk = (total + 255) / 256;
  repack_kernel<<<(unsigned)nblk, 256, 0, dev->stream>>>(
      type, raw_dev, n, row_bytes, blocks_per_row, g.block_bytes, g.group_elems / g.block_elems,
      tiled_dev, ngroups, g.tg_bytes, tile0, total);
  FB_LAUNCH_CHECK(dev);
  return FB200_OK;
}

int fb200_launch_widen_q5_0(fb200_device* dev, const uint8_t* q5_dev, uint64_t nblocks, uint8_t* q8_dev) {
  const uint64_t total = nblocks * 34;
  if (total == 0) return FB200_OK;
  widen_q5_0_kernel<<<(unsigned)((total + 255) / 256), 256, 0, dev->stream>>>(q5_dev, total, q8_dev);
  FB_LAUNCH_CHECK(dev);
  return FB200_OK;
}

int fb200_launch_dequantize(fb200_device* dev, const fb200_qmatrix* q, float* out_dev) {
  uint64_t total = q->n * q->k;
  if (total == 0) return FB200_OK;
  uint64_t nblk = (total + 255) / 256;
  if (q->tiled) {
    TileGeom g;
    tile_geom(q->type, &g);
    dequant_tiled_kernel<<<(unsigned)nblk, 256, 0, dev->stream>>>(q->type, q->data, q->n, q->k,
                                                                  q->ngroups, g.group_elems,
                                                                  g.tg_bytes, out_dev);
  } else {
    dequant_raw_kernel<<<(unsigned)nblk, 256, 0, dev->stream>>>(q->type, q->data, total, out_dev);
  }
  FB_LAUNCH_CHECK(dev);
  return FB200_OK;
}

int fb200_launch_dequantize_rows(fb200_device* dev, const fb200_qmatrix* q,
                                 const uint32_t* ids_dev, size_t n_ids, float* out_dev) {
  if (n_ids == 0 || q->k == 0) return FB200_OK;
  dim3 grid((unsigned)((q->k + 255) / 256 > 64 ? 64 : (q->k + 255) / 256), (unsigned)n_ids);
  if (q->tiled) {
    TileGeom g;
    tile_geom(q->type, &g);
    dequant_rows_tiled_kernel<<<grid, 256, 0, dev->stream>>>(q->type, q->data, q->n, q->k,
                                                             q->ngroups, g.group_elems, g.tg_bytes,
                                                             ids_dev, out_dev);
  } else {
    dequant_rows_raw_kernel<<<grid, 256, 0, dev->stream>>>(q->type, q->data, q->n, q->k, ids_dev,
                                                           out_dev);
  }
  FB_LAUNCH_CHECK(dev);
  return FB200_OK;
}
