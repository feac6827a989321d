// C ABI: device handles, tensors, QMatrix and q_mat_mul.
#include <cstdarg>
#include <cstdlib>
#include <cstring>

#include <nvtx3/nvToolsExt.h>

#include "common.cuh"

size_t fb200_xpack_bytes(int mp, uint64_t kp);
bool fb200_q5_covers(const fb200_qmatrix* w);
int fb200_q5_mat_mul(fb200_device* dev, const fb200_qmatrix* w, const float* x, size_t m, float* y, const float* r1,
                     const float* r2, bool r1_is_bias);
int fb200_qgemv_chunk(fb200_device* dev, const fb200_qmatrix* w, const float* x, int mc, float* y,
                      int epi, const float* r1, const float* r2, void* scratch, bool r1_is_bias);
int fb200_dense_matmul(fb200_device* dev, const fb200_qmatrix* w, const float* x, size_t m, float* y);
int fb200_qgemm(fb200_device* dev, const fb200_qmatrix* w, const float* x, size_t m, float* y, bool r1_is_bias,
                const float* r1, const float* r2, int swiglu);
bool fb200_qgemv1_fits(const fb200_qmatrix* w);
int fb200_qgemv1(fb200_device* dev, const fb200_qmatrix* w, const float* x, const float* xres,
                 const float* norm_w, float eps, float* y, int epi, const float* r1, const float* r2);
int fb200_launch_rms_norm(fb200_device* dev, const float* x, const float* res, const float* w,
                          const float* b, float eps, size_t rows, size_t n, float* y);

static thread_local char g_global_err[512] = {0};

// Records the text of an error in fixed storage (the handle's, or a per-thread buffer when there
// is no handle) and returns `code`. No heap allocation on any path, so entry points that promise
// not to allocate may fail through it.
int fb200_fail(fb200_device* dev, int code, const char* fmt, ...) {
  char* dst = dev ? dev->err : g_global_err;
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(dst, 512, fmt, ap);
  va_end(ap);
  return code;
}

fb200_op_trace::fb200_op_trace(fb200_device* d, const char* n, double b) : dev(d), name(n), bytes(b), timed(false) {
  nvtxRangePushA(name);
  if (!dev || !dev->trace || dev->capturing) return;
  if (dev->trace_depth++ == 0 && dev->trace_ev[0]) {
    timed = cudaEventRecord(dev->trace_ev[0], dev->stream) == cudaSuccess;
  }
}

fb200_op_trace::~fb200_op_trace() {
  nvtxRangePop();
  if (!dev || !dev->trace || dev->capturing) return;
  --dev->trace_depth;
  if (!timed) return;
  float ms = 0.f;
  if (cudaEventRecord(dev->trace_ev[1], dev->stream) == cudaSuccess &&
      cudaEventSynchronize(dev->trace_ev[1]) == cudaSuccess &&
      cudaEventElapsedTime(&ms, dev->trace_ev[0], dev->trace_ev[1]) == cudaSuccess) {
    const double us = (double)ms * 1e3;
    if (bytes > 0) fprintf(stderr, "fb200 trace: %-26s %10.2f us %9.1f GB/s\n", name, us, bytes / us / 1e3);
    else fprintf(stderr, "fb200 trace: %-26s %10.2f us\n", name, us);
  }
}

int fb200_bind(fb200_device* dev) {
  if (!dev) return fb200_fail(nullptr, FB200_ERR_INVALID_ARGUMENT, "null device handle");
  FB_CUDA(dev, cudaSetDevice(dev->ordinal));
  return FB200_OK;
}

// Scratch buffers of a handle (packed activations, normalised rows, host staging) replace the
// reference's BufferPool (fusor-ml/tile-ir-runtime/src/buffer_pool.rs:74-260): a buffer only ever
// grows, its bytes count against the handle's optional budget, and in poison mode fresh scratch
// is filled with 0xFF bytes (NaN as f32/f16), the analogue of the pool's poison fill
// (buffer_pool.rs:198-207), so a kernel that reads scratch it never wrote shows up in the result.
int fb200_ensure(fb200_device* dev, void** buf, size_t* cur, size_t bytes) {
  if (*cur >= bytes) return FB200_OK;
  const size_t want = bytes + bytes / 4 + 4096;
  if (dev->scratch_limit && dev->scratch_total - *cur + want > dev->scratch_limit)
    return fb200_fail(dev, FB200_ERR_CAPACITY, "scratch: %zu more bytes would exceed the handle's budget of %zu (in use %zu)",
                      want, dev->scratch_limit, dev->scratch_total);
  if (*buf) {
    FB_CUDA(dev, cudaStreamSynchronize(dev->stream));
    FB_CUDA(dev, cudaFree(*buf));
    dev->scratch_total -= *cur;
    *buf = nullptr;
    *cur = 0;
  }
  dev->scratch_gen++;
  FB_CUDA(dev, cudaMalloc(buf, want));
  *cur = want;
  dev->scratch_total += want;
  if (dev->poison) FB_CUDA(dev, cudaMemsetAsync(*buf, 0xFF, want, dev->stream));
  return FB200_OK;
}

int fb200_sync_check(fb200_device* dev) {
  FB_CUDA(dev, cudaMemcpyAsync(dev->status_host, dev->status, sizeof(int), cudaMemcpyDeviceToHost, dev->stream));
  FB_CUDA(dev, cudaStreamSynchronize(dev->stream));
  if (*dev->status_host != 0)
    return fb200_fail(dev, FB200_ERR_TIMEOUT,
                      "device status %d: a bounded wait inside a kernel gave up, results since then are invalid "
                      "(fb200_device_clear_status resets the word)", *dev->status_host);
  return FB200_OK;
}

extern "C" {

int fb200_device_create(int ordinal, void* stream, fb200_device** out) {
  if (!out) return fb200_fail(nullptr, FB200_ERR_INVALID_ARGUMENT, "out is null");
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || ordinal < 0 || ordinal >= count)
    return fb200_fail(nullptr, FB200_ERR_CUDA, "no CUDA device %d (%s); this backend has no CPU fallback",
                      ordinal, e != cudaSuccess ? cudaGetErrorString(e) : "ordinal out of range");
  fb200_device* d = new fb200_device();
  d->ordinal = ordinal;
  if ((e = cudaSetDevice(ordinal)) != cudaSuccess) {
    delete d;
    return fb200_fail(nullptr, FB200_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(e));
  }
  if (stream) {
    d->stream = (cudaStream_t)stream;
  } else {
    if ((e = cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking)) != cudaSuccess) {
      delete d;
      return fb200_fail(nullptr, FB200_ERR_CUDA, "cudaStreamCreate: %s", cudaGetErrorString(e));
    }
    d->own_stream = true;
  }
  cudaDeviceGetAttribute(&d->sm_count, cudaDevAttrMultiProcessorCount, ordinal);
  if (const char* e = getenv("FB200_PDL")) d->pdl = e[0] != '0';
  if (const char* e = getenv("FB200_POISON")) d->poison = e[0] == '1';
  if (const char* e = getenv("FB200_TRACE")) d->trace = e[0] == '1';
  if (d->trace && (cudaEventCreate(&d->trace_ev[0]) != cudaSuccess || cudaEventCreate(&d->trace_ev[1]) != cudaSuccess))
    d->trace = false;
  if (const char* e = getenv("FB200_SCRATCH_LIMIT")) d->scratch_limit = (size_t)strtoull(e, nullptr, 10);
  if ((e = cudaMalloc(&d->status, sizeof(int))) != cudaSuccess ||
      (e = cudaMemsetAsync(d->status, 0, sizeof(int), d->stream)) != cudaSuccess ||
      (e = cudaMallocHost(&d->status_host, sizeof(int))) != cudaSuccess) {
    if (d->status) cudaFree(d->status);
    delete d;
    return fb200_fail(nullptr, FB200_ERR_CUDA, "status word: %s", cudaGetErrorString(e));
  }
  *d->status_host = 0;
  *out = d;
  return FB200_OK;
}

int fb200_device_destroy(fb200_device* dev) {
  if (!dev) return FB200_OK;
  cudaSetDevice(dev->ordinal);
  cudaStreamSynchronize(dev->stream);
  if (dev->xpack) cudaFree(dev->xpack);
  if (dev->argmax_part) cudaFree(dev->argmax_part);
  if (dev->stage) cudaFree(dev->stage);
  if (dev->normed) cudaFree(dev->normed);
  if (dev->splitk) cudaFree(dev->splitk);
  if (dev->status) cudaFree(dev->status);
  if (dev->status_host) cudaFreeHost(dev->status_host);
  for (cudaEvent_t e : dev->trace_ev) if (e) cudaEventDestroy(e);
  for (cudaStream_t st : dev->side_stream) if (st) cudaStreamDestroy(st);
  for (cudaEvent_t e : dev->join_ev) if (e) cudaEventDestroy(e);
  if (dev->fork_ev) cudaEventDestroy(dev->fork_ev);
  if (dev->fused) cudaFree(dev->fused);
  if (dev->own_stream) cudaStreamDestroy(dev->stream);
  delete dev;
  return FB200_OK;
}

int fb200_device_synchronize(fb200_device* dev) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  return fb200_sync_check(dev);
}

int fb200_device_clear_status(fb200_device* dev) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  FB_CUDA(dev, cudaMemsetAsync(dev->status, 0, sizeof(int), dev->stream));
  FB_CUDA(dev, cudaStreamSynchronize(dev->stream));
  *dev->status_host = 0;
  return FB200_OK;
}

int fb200_device_set_scratch_limit(fb200_device* dev, size_t bytes) {
  if (!dev) return FB200_ERR_INVALID_ARGUMENT;
  dev->scratch_limit = bytes;
  return FB200_OK;
}

int fb200_device_set_poison(fb200_device* dev, int enable) {
  if (!dev) return FB200_ERR_INVALID_ARGUMENT;
  dev->poison = enable != 0;
  return FB200_OK;
}

const char* fb200_last_error(const fb200_device* dev) {
  return dev ? dev->err : g_global_err;
}

uint64_t fb200_launch_count(const fb200_device* dev) { return dev ? dev->launches : 0; }

int fb200_device_status(fb200_device* dev, int* status_out) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  FB_CUDA(dev, cudaMemcpyAsync(status_out, dev->status, sizeof(int), cudaMemcpyDeviceToHost, dev->stream));
  FB_CUDA(dev, cudaStreamSynchronize(dev->stream));
  return FB200_OK;
}

int fb200_malloc(fb200_device* dev, size_t bytes, void** out_dev) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (!out_dev) return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "out_dev is null");
  *out_dev = nullptr;
  if (bytes == 0) return FB200_OK;
  FB_CUDA(dev, cudaMalloc(out_dev, bytes));
  return FB200_OK;
}

int fb200_free(fb200_device* dev, void* ptr_dev) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (!ptr_dev) return FB200_OK;
  FB_CUDA(dev, cudaStreamSynchronize(dev->stream));
  FB_CUDA(dev, cudaFree(ptr_dev));
  return FB200_OK;
}

int fb200_upload(fb200_device* dev, void* dst_dev, const void* src_host, size_t bytes) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (bytes == 0) return FB200_OK;
  FB_CUDA(dev, cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, dev->stream));
  // Pageable sources are staged before the call returns; pinned ones are read asynchronously,
  // so wait: the caller may reuse the buffer right away.
  FB_CUDA(dev, cudaStreamSynchronize(dev->stream));
  return FB200_OK;
}

int fb200_download(fb200_device* dev, void* dst_host, const void* src_dev, size_t bytes) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (bytes)
    FB_CUDA(dev, cudaMemcpyAsync(dst_host, src_dev, bytes, cudaMemcpyDeviceToHost, dev->stream));
  return fb200_sync_check(dev);
}

int fb200_memset(fb200_device* dev, void* dst_dev, int value, size_t bytes) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (bytes) FB_CUDA(dev, cudaMemsetAsync(dst_dev, value, bytes, dev->stream));
  return FB200_OK;
}

// ---- QMatrix -----------------------------------------------------------------------------------

int fb200_qmatrix_from_raw_bytes(fb200_device* dev, const uint64_t* shape, int rank,
                                 const void* bytes_host, size_t nbytes, uint32_t ggml_type,
                                 fb200_qmatrix** out) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (!out) return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "out is null");
  *out = nullptr;
  if (rank != 2 || !shape)
    return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "QMatrix needs a rank-2 shape, got rank %d", rank);
  int be, bb;
  if (!block_geom(ggml_type, &be, &bb))
    return fb200_fail(dev, FB200_ERR_UNSUPPORTED_DTYPE, "unsupported ggml type %u", ggml_type);
  const uint64_t n = shape[0], k = shape[1];
  if (k % (uint64_t)be != 0)
    return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "K = %llu is not a multiple of the block size %d",
                      (unsigned long long)k, be);
  const uint64_t expect = n * (k / be) * (uint64_t)bb;
  if (expect != nbytes)
    return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "shape [%llu, %llu] of type %u needs %llu bytes, got %zu",
                      (unsigned long long)n, (unsigned long long)k, ggml_type,
                      (unsigned long long)expect, nbytes);
  if (n >= (1ull << 31) || k >= (1ull << 31))
    return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "dimension too large");
  fb200_qmatrix* q = new fb200_qmatrix();
  q->dev = dev; q->type = ggml_type; q->source_type = ggml_type; q->n = n; q->k = k; q->raw_nbytes = nbytes;
  // Q5_0 is stored as Q8_0 tiles (the same scale, the 5-bit integer widened to 8 bits: identical
  // values, 34 instead of 22 bytes per block) and takes the Q8_0 kernels
  const bool widen = ggml_type == FB200_Q5_0;
  if (widen) q->type = FB200_Q8_0;
  TileGeom g;
  uint8_t* raw_dev = nullptr;
  uint8_t* wide_dev = nullptr;
  auto cleanup = [&](int code) {
    if (raw_dev) cudaFree(raw_dev);
    if (wide_dev) cudaFree(wide_dev);
    if (q->data) cudaFree(q->data);
    delete q;
    return code;
  };
  if (tile_geom(q->type, &g)) {
    q->tiled = true;
    q->ntiles = (int)((n + 15) / 16);
    q->ngroups = (int)((k + g.group_elems - 1) / g.group_elems);
    q->data_bytes = (size_t)q->ntiles * q->ngroups * g.tg_bytes;
    if (q->data_bytes) {
      cudaError_t e = cudaMalloc(&raw_dev, nbytes ? nbytes : 1);
      if (e == cudaSuccess) e = cudaMalloc(&q->data, q->data_bytes);
      if (e == cudaSuccess && nbytes)
        e = cudaMemcpyAsync(raw_dev, bytes_host, nbytes, cudaMemcpyHostToDevice, dev->stream);
      if (e != cudaSuccess)
        return cleanup(fb200_fail(dev, FB200_ERR_CUDA, "QMatrix upload: %s", cudaGetErrorString(e)));
      if (widen) {
        const uint64_t nblocks = n * (k / 32);
        e = cudaMalloc(&wide_dev, nblocks * 34 ? nblocks * 34 : 1);
        if (e != cudaSuccess)
          return cleanup(fb200_fail(dev, FB200_ERR_CUDA, "QMatrix upload: %s", cudaGetErrorString(e)));
        rc = fb200_launch_widen_q5_0(dev, raw_dev, nblocks, wide_dev);
        if (rc) return cleanup(rc);
      }
      rc = fb200_launch_repack(dev, q->type, widen ? wide_dev : raw_dev, n, k, q->data, q->ntiles, q->ngroups, 0);
      if (rc) return cleanup(rc);
      e = cudaStreamSynchronize(dev->stream);
      if (e != cudaSuccess)
        return cleanup(fb200_fail(dev, FB200_ERR_CUDA, "QMatrix repack: %s", cudaGetErrorString(e)));
      cudaFree(raw_dev);
      raw_dev = nullptr;
      if (wide_dev) cudaFree(wide_dev);
      wide_dev = nullptr;
    }
  } else {
    q->tiled = false;
    q->data_bytes = nbytes;
    if (nbytes) {
      cudaError_t e = cudaMalloc(&q->data, nbytes);
      if (e == cudaSuccess)
        e = cudaMemcpyAsync(q->data, bytes_host, nbytes, cudaMemcpyHostToDevice, dev->stream);
      if (e == cudaSuccess) e = cudaStreamSynchronize(dev->stream);
      if (e != cudaSuccess)
        return cleanup(fb200_fail(dev, FB200_ERR_CUDA, "QMatrix upload: %s", cudaGetErrorString(e)));
    }
  }
  *out = q;
  return FB200_OK;
}

int fb200_qmatrix_free(fb200_qmatrix* q) {
  if (!q) return FB200_OK;
  fb200_device* dev = q->dev;
  int rc = fb200_bind(dev);
  if (rc) return rc;
  cudaStreamSynchronize(dev->stream);
  if (q->data) cudaFree(q->data);
  delete q;
  return FB200_OK;
}

int fb200_qmatrix_shape(const fb200_qmatrix* q, uint64_t* n_out, uint64_t* k_out) {
  if (!q) return FB200_ERR_INVALID_ARGUMENT;
  if (n_out) *n_out = q->n;
  if (k_out) *k_out = q->k;
  return FB200_OK;
}

int fb200_qmatrix_ggml_type(const fb200_qmatrix* q, uint32_t* type_out) {
  if (!q || !type_out) return FB200_ERR_INVALID_ARGUMENT;
  *type_out = q->source_type;
  return FB200_OK;
}

int fb200_qmatrix_nbytes(const fb200_qmatrix* q, uint64_t* nbytes_out) {
  if (!q || !nbytes_out) return FB200_ERR_INVALID_ARGUMENT;
  *nbytes_out = q->raw_nbytes;
  return FB200_OK;
}

int fb200_qmatrix_dequantize(const fb200_qmatrix* q, float* out_dev) {
  if (!q) return FB200_ERR_INVALID_ARGUMENT;
  int rc = fb200_bind(q->dev);
  if (rc) return rc;
  return fb200_launch_dequantize(q->dev, q, out_dev);
}

int fb200_qmatrix_concat_rows(const fb200_qmatrix* const* ms, int n, fb200_qmatrix** out) {
  if (!out) return FB200_ERR_INVALID_ARGUMENT;
  *out = nullptr;
  if (!ms || n <= 0 || !ms[0]) return FB200_ERR_INVALID_ARGUMENT;
  fb200_device* dev = ms[0]->dev;
  int rc = fb200_bind(dev);
  if (rc) return rc;
  uint64_t total_n = 0, raw = 0;
  for (int i = 0; i < n; ++i) {
    if (!ms[i] || ms[i]->dev != dev)
      return fb200_fail(dev, FB200_ERR_DEVICE_MISMATCH, "concat_rows: matrices on different devices");
    if (ms[i]->type != ms[0]->type || ms[i]->source_type != ms[0]->source_type || ms[i]->k != ms[0]->k || !ms[i]->tiled)
      return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "concat_rows: needs one quantised type and one K");
    if (i + 1 < n && ms[i]->n % 16 != 0)
      return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "concat_rows: N of part %d is not a multiple of 16", i);
    total_n += ms[i]->n;
    raw += ms[i]->raw_nbytes;
  }
  fb200_qmatrix* q = new fb200_qmatrix(*ms[0]);
  q->n = total_n;
  q->raw_nbytes = raw;
  q->ntiles = 0;
  q->data_bytes = 0;
  for (int i = 0; i < n; ++i) { q->ntiles += ms[i]->ntiles; q->data_bytes += ms[i]->data_bytes; }
  q->data = nullptr;
  cudaError_t e = cudaMalloc(&q->data, q->data_bytes ? q->data_bytes : 1);
  size_t off = 0;
  for (int i = 0; i < n && e == cudaSuccess; ++i) {
    if (ms[i]->data_bytes)
      e = cudaMemcpyAsync(q->data + off, ms[i]->data, ms[i]->data_bytes, cudaMemcpyDeviceToDevice, dev->stream);
    off += ms[i]->data_bytes;
  }
  if (e != cudaSuccess) {
    if (q->data) cudaFree(q->data);
    delete q;
    return fb200_fail(dev, FB200_ERR_CUDA, "concat_rows: %s", cudaGetErrorString(e));
  }
  *out = q;
  return FB200_OK;
}

// ---- q_mat_mul ---------------------------------------------------------------------------------

int fb200_q_mat_mul(fb200_device* dev, const float* x_dev, size_t m, const fb200_qmatrix* w,
                    float* y_dev, const fb200_epilogue* ep) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (!w || !x_dev || !y_dev) return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "q_mat_mul: null argument");
  if (w->dev != dev)
    return fb200_fail(dev, FB200_ERR_DEVICE_MISMATCH, "q_mat_mul: weight lives on another device handle");
  int epi = ep ? ep->kind : FB200_EPI_NONE;
  if (epi < 0 || epi > 3) return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "q_mat_mul: epilogue kind %d", epi);
  if ((epi == FB200_EPI_RESIDUAL || epi == FB200_EPI_BIAS) && !ep->r1_dev)
    return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "q_mat_mul: residual / bias epilogue without r1");
  // Linear's bias (fusor-ml/fusor/src/layers/linear.rs:93-121) is the residual epilogue with one
  // row shared by all activation rows
  const bool bias = epi == FB200_EPI_BIAS;
  if (bias) {
    if (ep->r2_dev) return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "q_mat_mul: the bias epilogue takes r1 only");
    epi = FB200_EPI_RESIDUAL;
  }
  if (m == 0 || w->n == 0) return FB200_OK;
  fb200_op_trace scope(dev, m == 1 ? "q_mat_mul (1 row)" : m <= 32 ? "q_mat_mul (2..32 rows)" : "q_mat_mul (> 32 rows)",
                       (double)w->raw_nbytes + 4.0 * (double)m * (double)(w->k + w->n));
  if (!w->tiled) {
    if (fb200_q5_covers(w)) {
      if (epi == FB200_EPI_SWIGLU)
        return fb200_fail(dev, FB200_ERR_UNSUPPORTED_DTYPE, "q_mat_mul: no SwiGLU epilogue for Q5_K weights");
      return fb200_q5_mat_mul(dev, w, x_dev, m, y_dev, epi == FB200_EPI_RESIDUAL ? ep->r1_dev : nullptr,
                              epi == FB200_EPI_RESIDUAL ? ep->r2_dev : nullptr, bias);
    }
    if (epi != FB200_EPI_NONE)
      return fb200_fail(dev, FB200_ERR_UNSUPPORTED_DTYPE, "q_mat_mul: epilogues need quantised weights");
    return fb200_dense_matmul(dev, w, x_dev, m, y_dev);
  }
  if (epi == FB200_EPI_SWIGLU && (w->ntiles % 2 != 0 || w->n % 32 != 0))
    return fb200_fail(dev, FB200_ERR_INVALID_SHAPE, "q_mat_mul: SwiGLU needs N = 2F with F a multiple of 16");
  if (m == 1 && fb200_qgemv1_fits(w))
    return fb200_qgemv1(dev, w, x_dev, nullptr, nullptr, 0.f, y_dev, epi, ep ? ep->r1_dev : nullptr,
                        ep ? ep->r2_dev : nullptr);
  if (m > 32) {
    rc = fb200_qgemm(dev, w, x_dev, m, y_dev, bias, epi == FB200_EPI_RESIDUAL ? ep->r1_dev : nullptr,
                     epi == FB200_EPI_RESIDUAL ? ep->r2_dev : nullptr, epi == FB200_EPI_SWIGLU ? 1 : 0);
    if (rc != 1) return rc;  // 1 = shape not covered by the tensor-core GEMM; fall through
  }
  TileGeom g;
  tile_geom(w->type, &g);
  const uint64_t kp = (uint64_t)w->ngroups * g.group_elems;
  rc = fb200_ensure(dev, &dev->xpack, &dev->xpack_bytes, fb200_xpack_bytes(32, kp));
  if (rc) return rc;
  const size_t n_out = epi == FB200_EPI_SWIGLU ? w->n / 2 : w->n;
  for (size_t m0 = 0; m0 < m; m0 += 32) {
    const int mc = (int)((m - m0) < 32 ? (m - m0) : 32);
    rc = fb200_qgemv_chunk(dev, w, x_dev + m0 * w->k, mc, y_dev + m0 * n_out, epi,
                           ep && ep->r1_dev ? ep->r1_dev + (bias ? 0 : m0 * n_out) : nullptr,
                           ep && ep->r2_dev ? ep->r2_dev + m0 * n_out : nullptr, dev->xpack, bias);
    if (rc) return rc;
  }
  return FB200_OK;
}

int fb200_rms_norm_q_mat_mul(fb200_device* dev, const float* x_dev, const float* residual_dev,
                             const float* norm_weight_dev, float eps, size_t m,
                             const fb200_qmatrix* w, float* y_dev, const fb200_epilogue* ep) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (!w || !x_dev || !y_dev || !norm_weight_dev)
    return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "rms_norm_q_mat_mul: null argument");
  if (w->dev != dev)
    return fb200_fail(dev, FB200_ERR_DEVICE_MISMATCH, "rms_norm_q_mat_mul: weight lives on another device handle");
  fb200_epilogue one_row;
  if (ep && ep->kind == FB200_EPI_BIAS && m == 1 && ep->r1_dev && !ep->r2_dev) {
    one_row = {FB200_EPI_RESIDUAL, ep->r1_dev, nullptr};  // one activation row: a bias row is a residual row
    ep = &one_row;
  }
  const int epi = ep ? ep->kind : FB200_EPI_NONE;
  fb200_op_trace scope(dev, "rms_norm + q_mat_mul", (double)w->raw_nbytes + 4.0 * (double)m * (double)(w->k + w->n));
  if (m == 1 && w->tiled && fb200_qgemv1_fits(w) && epi >= 0 && epi <= 2 &&
      !(epi == FB200_EPI_SWIGLU && (w->ntiles % 2 != 0 || w->n % 32 != 0)) &&
      !(epi == FB200_EPI_RESIDUAL && !ep->r1_dev))
    return fb200_qgemv1(dev, w, x_dev, residual_dev, norm_weight_dev, eps, y_dev, epi,
                        ep ? ep->r1_dev : nullptr, ep ? ep->r2_dev : nullptr);
  // general shapes: normalise into scratch, then the plain product
  const size_t bytes = m * w->k * sizeof(float);
  rc = fb200_ensure(dev, &dev->normed, &dev->normed_bytes, bytes);
  if (rc) return rc;
  rc = fb200_launch_rms_norm(dev, x_dev, residual_dev, norm_weight_dev, nullptr, eps, m, w->k,
                             (float*)dev->normed);
  if (rc) return rc;
  return fb200_q_mat_mul(dev, (const float*)dev->normed, m, w, y_dev, ep);
}

int fb200_q_mat_mul_host(fb200_device* dev, const float* x_host, size_t m, const fb200_qmatrix* w,
                         float* y_host) {
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (!w || !x_host || !y_host) return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "q_mat_mul_host: null argument");
  const size_t xb = m * w->k * sizeof(float), yb = m * w->n * sizeof(float);
  const size_t xoff = (xb + 255) & ~(size_t)255;
  rc = fb200_ensure(dev, &dev->stage, &dev->stage_bytes, xoff + yb);
  if (rc) return rc;
  float* xd = (float*)dev->stage;
  float* yd = (float*)((uint8_t*)dev->stage + xoff);
  if (xb) FB_CUDA(dev, cudaMemcpyAsync(xd, x_host, xb, cudaMemcpyHostToDevice, dev->stream));
  rc = fb200_q_mat_mul(dev, xd, m, w, yd, nullptr);
  if (rc) return rc;
  if (yb) FB_CUDA(dev, cudaMemcpyAsync(y_host, yd, yb, cudaMemcpyDeviceToHost, dev->stream));
  FB_CUDA(dev, cudaStreamSynchronize(dev->stream));
  return FB200_OK;
}

}  // extern "C"
