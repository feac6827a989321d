// Tensor-parallel communicator: one rank per GPU, NCCL over NVLink for the two all-reduces per
// layer and the greedy-token exchange of the sharded output head.
//
// The reference has no multi-GPU path; the partition follows the usual split of a transformer
// layer: q/k/v/gate/up by rows, o/down by K, one sum per pair (run_forward in llama.cu).
// NCCL is loaded at run time (dlopen of libnccl.so.2) so that single-GPU users of the library
// do not need it; every entry point fails with FB200_ERR_NCCL when it is missing.
// The communicator also owns the exchange buffer of the fused decode kernel: made here, exported
// as a CUDA IPC handle and mapped by every peer, so that the kernel can store partial rows into
// the peers' memory and poll arrival words without any library call (fused_step.cuh).
#include <dlfcn.h>
#include <nccl.h>

#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "fused_step.cuh"

struct fb200_comm {
  fb200_device* dev = nullptr;
  ncclComm_t nccl = nullptr;
  int rank = 0, size = 1;
  // exchange buffer of the fused decode kernel (layout: see fb200_fused_xchg), mapped by all peers
  uint8_t* xbuf = nullptr;
  uint8_t* peer[8] = {};
  int stride = 0;
  bool attached = false;
  unsigned epoch = 1;  // next exchange number; arrival words start at 0
  // set after a wait inside a kernel gave up: the ranks' epochs and arrival words no longer agree,
  // so every further collective on this communicator is refused until it is made again
  bool broken = false;
};

namespace {

struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

const NcclApi& nccl_api() {
  static NcclApi api = [] {
    NcclApi a;
    // FB200_NCCL_LIB names the library to load instead of the default (a deployment with its own
    // NCCL build; the tests point it at a missing file to see the FB200_ERR_NCCL path)
    const char* named = getenv("FB200_NCCL_LIB");
    void* h = named && named[0] ? dlopen(named, RTLD_NOW | RTLD_GLOBAL) : dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h && !(named && named[0])) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return a;
    a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
    a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
    a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
    a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(dlsym(h, "ncclAllReduce"));
    a.AllGather = reinterpret_cast<decltype(a.AllGather)>(dlsym(h, "ncclAllGather"));
    a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
    a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.AllReduce && a.AllGather && a.GetErrorString;
    return a;
  }();
  return api;
}

int nccl_fail(fb200_device* dev, const char* what, ncclResult_t r) {
  return fb200_fail(dev, FB200_ERR_NCCL, "%s: %s", what, nccl_api().GetErrorString(r));
}

int broken_fail(fb200_comm* c) {
  return fb200_fail(c->dev, FB200_ERR_TIMEOUT,
                    "comm: an exchange timed out earlier; the ranks are out of step, destroy the communicator and make a new one");
}

}  // namespace

// In-place sum over the ranks of buf[n] (f32), on the device handle's stream.
int fb200_comm_all_reduce(fb200_comm* c, float* buf, size_t n) {
  if (c->size == 1 || n == 0) return FB200_OK;
  if (c->broken) return broken_fail(c);
  ncclResult_t r = nccl_api().AllReduce(buf, buf, n, ncclFloat, ncclSum, c->nccl, c->dev->stream);
  if (r != ncclSuccess) return nccl_fail(c->dev, "all_reduce", r);
  return FB200_OK;
}

// out[size][bytes] = every rank's in[bytes].
int fb200_comm_all_gather_bytes(fb200_comm* c, const void* in, void* out, size_t bytes) {
  if (c->broken) return broken_fail(c);
  ncclResult_t r = nccl_api().AllGather(in, out, bytes, ncclChar, c->nccl, c->dev->stream);
  if (r != ncclSuccess) return nccl_fail(c->dev, "all_gather", r);
  return FB200_OK;
}

// Pointers of the peer exchange for a launch that performs `count` exchanges; false when the
// peers have not been attached or a row does not fit a slot.
bool fb200_comm_take_exchange(fb200_comm* c, int row_floats, unsigned count, fb200_fused_xchg* out) {
  if (!c->attached || c->broken || row_floats > c->stride) return false;
  const size_t keys_off = (size_t)2 * c->size * c->stride * 4, flags_off = keys_off + (size_t)2 * c->size * 8;
  for (int r = 0; r < c->size; ++r) {
    out->data[r] = reinterpret_cast<float*>(c->peer[r]);
    out->keys[r] = reinterpret_cast<unsigned long long*>(c->peer[r] + keys_off);
    out->flags[r] = reinterpret_cast<unsigned*>(c->peer[r] + flags_off);
  }
  out->world = c->size; out->me = c->rank; out->stride = c->stride;
  out->poll_limit = FB200_XCHG_POLL_LIMIT;
  out->epoch_base = c->epoch;
  c->epoch += count;
  return true;
}
bool fb200_comm_exchange_ready(const fb200_comm* c, int row_floats) { return c->attached && row_floats <= c->stride; }
void fb200_comm_mark_broken(fb200_comm* c) { if (c) c->broken = true; }

namespace {
__global__ void wait_check_kernel(const unsigned* word, int poll_limit, int* status) {
  if (!fb200_wait_arrival(word, 1u, poll_limit, status)) atomicExch(status, FB200_ERR_TIMEOUT);
}
}  // namespace

int fb200_comm_rank(const fb200_comm* c) { return c->rank; }
int fb200_comm_size(const fb200_comm* c) { return c->size; }
fb200_device* fb200_comm_device(const fb200_comm* c) { return c->dev; }

extern "C" {

int fb200_comm_unique_id(uint8_t* id_out, size_t id_bytes) {
  if (!id_out || id_bytes < sizeof(ncclUniqueId)) return FB200_ERR_INVALID_ARGUMENT;
  if (!nccl_api().ok) return FB200_ERR_NCCL;
  ncclUniqueId id;
  if (nccl_api().GetUniqueId(&id) != ncclSuccess) return FB200_ERR_NCCL;
  memset(id_out, 0, id_bytes);
  memcpy(id_out, &id, sizeof(id));
  return FB200_OK;
}

int fb200_comm_create(fb200_device* dev, int size, int rank, const uint8_t* id, size_t id_bytes, fb200_comm** out) {
  if (!dev || !out) return FB200_ERR_INVALID_ARGUMENT;
  *out = nullptr;
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (size < 1 || rank < 0 || rank >= size || !id || id_bytes < sizeof(ncclUniqueId))
    return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "comm: rank %d of %d", rank, size);
  if (!nccl_api().ok) return fb200_fail(dev, FB200_ERR_NCCL, "comm: libnccl.so.2 could not be loaded");
  ncclUniqueId uid;
  memcpy(&uid, id, sizeof(uid));
  fb200_comm* c = new fb200_comm();
  c->dev = dev; c->rank = rank; c->size = size;
  ncclResult_t r = nccl_api().CommInitRank(&c->nccl, size, uid, rank);
  if (r != ncclSuccess) { delete c; return nccl_fail(dev, "comm init", r); }
  *out = c;
  return FB200_OK;
}

int fb200_comm_exchange_handle(fb200_comm* c, size_t row_floats, uint8_t* handle_out, size_t handle_bytes) {
  if (!c || !handle_out || handle_bytes < sizeof(cudaIpcMemHandle_t)) return FB200_ERR_INVALID_ARGUMENT;
  fb200_device* dev = c->dev;
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (c->size > 8) return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "comm: the peer exchange takes at most 8 ranks");
  if (c->xbuf || row_floats == 0 || row_floats > (1u << 24))
    return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "comm: exchange buffer already made, or bad row size");
  c->stride = (int)((row_floats + 31) / 32 * 32);
  const size_t bytes = (size_t)2 * c->size * c->stride * 4 + (size_t)2 * c->size * 8 + (size_t)c->size * 4 + 256;
  FB_CUDA(dev, cudaMalloc(&c->xbuf, bytes));
  FB_CUDA(dev, cudaMemset(c->xbuf, 0, bytes));
  cudaIpcMemHandle_t h;
  FB_CUDA(dev, cudaIpcGetMemHandle(&h, c->xbuf));
  memset(handle_out, 0, handle_bytes);
  memcpy(handle_out, &h, sizeof(h));
  return FB200_OK;
}

int fb200_comm_exchange_attach(fb200_comm* c, const uint8_t* handles, size_t handle_bytes) {
  if (!c || !handles || handle_bytes < sizeof(cudaIpcMemHandle_t)) return FB200_ERR_INVALID_ARGUMENT;
  fb200_device* dev = c->dev;
  int rc = fb200_bind(dev);
  if (rc) return rc;
  if (!c->xbuf || c->attached) return fb200_fail(dev, FB200_ERR_INVALID_ARGUMENT, "comm: make the exchange handle first, attach once");
  for (int r = 0; r < c->size; ++r) {
    if (r == c->rank) { c->peer[r] = c->xbuf; continue; }
    cudaIpcMemHandle_t h;
    memcpy(&h, handles + (size_t)r * handle_bytes, sizeof(h));
    void* p = nullptr;
    FB_CUDA(dev, cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    c->peer[r] = static_cast<uint8_t*>(p);
  }
  c->attached = true;
  return FB200_OK;
}

int fb200_exchange_wait_check(fb200_device* dev, int poll_limit) {
  if (!dev || poll_limit < 1) return FB200_ERR_INVALID_ARGUMENT;
  int rc = fb200_bind(dev);
  if (rc) return rc;
  unsigned* word = nullptr;
  FB_CUDA(dev, cudaMalloc(&word, 4));
  FB_CUDA(dev, cudaMemsetAsync(word, 0, 4, dev->stream));
  wait_check_kernel<<<1, 1, 0, dev->stream>>>(word, poll_limit, dev->status);
  cudaError_t e = cudaStreamSynchronize(dev->stream);
  cudaFree(word);
  if (e != cudaSuccess) return fb200_fail(dev, FB200_ERR_CUDA, "wait check: %s", cudaGetErrorString(e));
  int st = 0;
  FB_CUDA(dev, cudaMemcpy(&st, dev->status, sizeof(int), cudaMemcpyDeviceToHost));
  if (st == FB200_ERR_TIMEOUT) return fb200_fail(dev, FB200_ERR_TIMEOUT, "the arrival word was not set within %d polls", poll_limit);
  return st;
}

int fb200_comm_destroy(fb200_comm* c) {
  if (!c) return FB200_OK;
  if (c->dev && fb200_bind(c->dev) == FB200_OK) {
    cudaStreamSynchronize(c->dev->stream);
    for (int r = 0; r < c->size; ++r)
      if (c->attached && r != c->rank && c->peer[r]) cudaIpcCloseMemHandle(c->peer[r]);
    if (c->xbuf) cudaFree(c->xbuf);
  }
  if (c->nccl) nccl_api().CommDestroy(c->nccl);
  delete c;
  return FB200_OK;
}

int fb200_comm_all_reduce_sum(fb200_comm* c, float* buf_dev, size_t n) {
  if (!c || !buf_dev) return FB200_ERR_INVALID_ARGUMENT;
  int rc = fb200_bind(c->dev);
  if (rc) return rc;
  return fb200_comm_all_reduce(c, buf_dev, n);
}

}  // extern "C"
