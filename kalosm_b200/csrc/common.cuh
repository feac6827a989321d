// Internal definitions shared by the translation units of libfusor_b200.so.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

#include "../../include/fusor_b200.h"

// Device handle: one CUDA device, one stream, reusable scratch buffers.
struct fb200_device {
  int ordinal = 0;
  cudaStream_t stream = nullptr;
  bool own_stream = false;
  int sm_count = 148;
  bool pdl = true;  // launch with programmatic stream serialization (FB200_PDL=0 turns it off)
  // side streams (created on first use) for independent products that do not fill the GPU one at a
  // time: forked from `stream` behind fork_ev, joined back through join_ev
  cudaStream_t side_stream[2] = {nullptr, nullptr};
  cudaEvent_t fork_ev = nullptr, join_ev[2] = {nullptr, nullptr};
  char err[512] = {0};  // text of the last error; fixed storage, so failing never allocates
  uint64_t launches = 0;
  // scratch for packed activations (fp16 fragments, group sums, row scales); grown on demand
  void* xpack = nullptr;
  size_t xpack_bytes = 0;
  // partial products of a split-K prefill product
  void* splitk = nullptr;
  size_t splitk_bytes = 0;
  // normalised activations of rms_norm_q_mat_mul when the fused kernel does not apply
  void* normed = nullptr;
  size_t normed_bytes = 0;
  // partial results of the greedy pick over wide rows
  void* argmax_part = nullptr;
  size_t argmax_part_bytes = 0;
  // staging for the *_host entry points
  void* stage = nullptr;
  size_t stage_bytes = 0;
  // device status word (set by kernels that recover from a fault) and its pinned host mirror
  int* status = nullptr;
  int* status_host = nullptr;
  // scratch accounting: bytes currently held by the buffers above, optional cap (0 = none),
  // generation (bumped whenever a scratch buffer moves, so that captured graphs which recorded
  // its address know they are stale), poison mode (new scratch is filled with 0xFF bytes = NaN)
  size_t scratch_total = 0, scratch_limit = 0;
  uint64_t scratch_gen = 0;
  bool poison = false;
  // FB200_TRACE=1: every operation entry point reports its device time (and GB/s of the bytes it
  // must move) on stderr; off inside a stream capture
  bool trace = false, capturing = false;
  int trace_depth = 0;
  cudaEvent_t trace_ev[2] = {nullptr, nullptr};
  // scratch of the fused decode-step kernel: grid barrier word, split-unit partials, counters
  void* fused = nullptr;
  size_t fused_bytes = 0;
  // next epoch of the flagged rows of the fused decode kernel (one per phase executed; never 0,
  // the value of freshly cleared buffers)
  uint32_t ll_epoch = 1;
};

// Quantised (or dense) weight matrix [N, K] in tile-interleaved device storage.
struct fb200_qmatrix {
  fb200_device* dev = nullptr;
  uint32_t type = 0;         // type of the stored blocks: what the kernels dispatch on
  uint32_t source_type = 0;  // type of the GGUF bytes the matrix was built from (differs for Q5_0, stored as Q8_0)
  uint64_t n = 0, k = 0;
  uint64_t raw_nbytes = 0;  // size of the GGUF byte stream this matrix was built from
  // tiled storage
  uint8_t* data = nullptr;
  size_t data_bytes = 0;
  int ntiles = 0;   // ceil(N / 16)
  int ngroups = 0;  // K groups per tile (128 weights for 32-element blocks, 256 for K-quants)
  bool tiled = false;  // false: `data` holds raw row-major bytes (F32/F16/Q5_0/Q5_K)
};

int fb200_fail(fb200_device* dev, int code, const char* fmt, ...);

#define FB_CUDA(dev, expr)                                                              \
  do {                                                                                  \
    cudaError_t e__ = (expr);                                                           \
    if (e__ != cudaSuccess)                                                             \
      return fb200_fail((dev), FB200_ERR_CUDA, "%s: %s (%s:%d)", #expr,                 \
                        cudaGetErrorString(e__), __FILE__, __LINE__);                   \
  } while (0)

#define FB_LAUNCH_CHECK(dev)                                                            \
  do {                                                                                  \
    (dev)->launches++;                                                                  \
    cudaError_t e__ = cudaGetLastError();                                               \
    if (e__ != cudaSuccess)                                                             \
      return fb200_fail((dev), FB200_ERR_CUDA, "kernel launch: %s (%s:%d)",             \
                        cudaGetErrorString(e__), __FILE__, __LINE__);                   \
  } while (0)

// Launches a kernel on the handle's stream, optionally with programmatic stream serialization
// (the kernel may then start while its predecessor is still running and must execute
// griddepcontrol.wait before touching anything the predecessor produces).
template <typename... KArgs, typename... Args>
inline int fb200_launch(fb200_device* dev, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                        bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = dev->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl && dev->pdl) ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
  if (e != cudaSuccess)
    return fb200_fail(dev, FB200_ERR_CUDA, "kernel launch: %s", cudaGetErrorString(e));
  dev->launches++;
  return FB200_OK;
}

// Scope of one operation for the per-operation trace (the counterpart of the reference's
// tracing spans around a forward pass, models/kalosm-llama/src/model/mod.rs:48-74, 112-116): an
// NVTX range named after the operation, and with FB200_TRACE=1 a line on stderr with the
// operation's device time in microseconds and the GB/s of its algorithmic bytes. Timing an
// operation waits for it, so the trace serialises the stream; nested scopes report the outermost.
struct fb200_op_trace {
  fb200_device* dev;
  const char* name;
  double bytes;
  bool timed;
  fb200_op_trace(fb200_device* dev, const char* name, double bytes);
  ~fb200_op_trace();
};

// Makes the handle's device current for the calling thread.
int fb200_bind(fb200_device* dev);
// Synchronises the handle's stream and reads the device status word with it: FB200_ERR_TIMEOUT
// (and the text of fb200_last_error) when a kernel recorded a wait that gave up, else FB200_OK.
int fb200_sync_check(fb200_device* dev);
// Ensures a scratch buffer of at least `bytes` (never shrinks).
int fb200_ensure(fb200_device* dev, void** buf, size_t* cur, size_t bytes);

// ---- geometry of the tiled storage ----------------------------------------------------------
// A tile is 16 consecutive rows of W; a tile-group is the bytes of those rows for one K group.
// Inside a tile-group the quant bytes are ordered so that lane (g = lane / 4, t = lane % 4) of
// a warp reads, with one 16-byte load per 512-byte plane, exactly the bytes it feeds to
// mma.m16n8k16 for rows g (plane h = 0) and g + 8 (plane h = 1).
struct TileGeom {
  int block_elems;  // GGUF block size (32 or 256)
  int block_bytes;  // GGUF block bytes
  int group_elems;  // K elements per tile-group
  int tg_bytes;     // bytes per tile-group = 16 rows * group_elems / block_elems * block_bytes
};

inline bool tile_geom(uint32_t type, TileGeom* g) {
  switch (type) {
    case FB200_Q4_0: *g = {32, 18, 128, 1152}; return true;
    case FB200_Q8_0: *g = {32, 34, 128, 2176}; return true;
    case FB200_Q4_K: *g = {256, 144, 256, 2304}; return true;
    case FB200_Q6_K: *g = {256, 210, 256, 3360}; return true;
    default: return false;
  }
}

inline bool block_geom(uint32_t type, int* elems, int* bytes) {
  switch (type) {
    case FB200_Q4_0: *elems = 32; *bytes = 18; return true;
    case FB200_Q5_0: *elems = 32; *bytes = 22; return true;
    case FB200_Q8_0: *elems = 32; *bytes = 34; return true;
    case FB200_Q4_K: *elems = 256; *bytes = 144; return true;
    case FB200_Q5_K: *elems = 256; *bytes = 176; return true;
    case FB200_Q6_K: *elems = 256; *bytes = 210; return true;
    case FB200_F32: *elems = 1; *bytes = 4; return true;
    case FB200_F16: *elems = 1; *bytes = 2; return true;
    default: return false;
  }
}

// internal launchers (defined in the .cu files)
int fb200_launch_repack(fb200_device* dev, uint32_t type, const uint8_t* raw_dev, uint64_t n,
                        uint64_t k, uint8_t* tiled_dev, int ntiles, int ngroups, int tile0);
int fb200_launch_widen_q5_0(fb200_device* dev, const uint8_t* q5_dev, uint64_t nblocks, uint8_t* q8_dev);
int fb200_launch_dequantize(fb200_device* dev, const fb200_qmatrix* q, float* out_dev);
int fb200_launch_dequantize_rows(fb200_device* dev, const fb200_qmatrix* q,
                                 const uint32_t* ids_dev, size_t n_ids, float* out_dev);
