// Receive buffers of the sequence-parallel hand-off: plain cudaMalloc memory on the consumer GPU that the producer
// GPU's process maps through CUDA IPC and then writes with ordinary stores from inside its kernel. These are set-up
// calls (once per process and shape), not part of a forward pass. No TMA descriptor is ever built over such a mapping.
#include <string.h>

#include "lq_common.cuh"

extern "C" int lq_peer_buffer_create(size_t bytes, void** dev_ptr, unsigned char* handle64) {
  if (!dev_ptr || !handle64 || bytes == 0) return lq::fail(LQ_ERR_NULL, "peer_buffer_create: null argument or zero size");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    if (p) cudaFree(p);
    return lq::fail(LQ_ERR_LAUNCH, "peer_buffer_create: %s", cudaGetErrorString(e));
  }
  memcpy(handle64, &h, 64);
  *dev_ptr = p;
  return LQ_OK;
}

extern "C" int lq_peer_buffer_open(const unsigned char* handle64, int owner_device, void** dev_ptr) {
  if (!handle64 || !dev_ptr) return lq::fail(LQ_ERR_NULL, "peer_buffer_open: null argument");
  int me = -1;
  cudaError_t e = cudaGetDevice(&me);
  if (e != cudaSuccess) return lq::fail(LQ_ERR_LAUNCH, "peer_buffer_open: cudaGetDevice: %s", cudaGetErrorString(e));
  if (me != owner_device) {
    int can = 0;
    e = cudaDeviceCanAccessPeer(&can, me, owner_device);
    if (e != cudaSuccess || !can) return lq::fail(LQ_ERR_UNSUPPORTED, "peer_buffer_open: device %d cannot access device %d", me, owner_device);
    e = cudaDeviceEnablePeerAccess(owner_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); e = cudaSuccess; }
    if (e != cudaSuccess) return lq::fail(LQ_ERR_LAUNCH, "peer_buffer_open: cudaDeviceEnablePeerAccess: %s", cudaGetErrorString(e));
  }
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return lq::fail(LQ_ERR_LAUNCH, "peer_buffer_open: cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
  *dev_ptr = p;
  return LQ_OK;
}

extern "C" int lq_peer_buffer_close(void* dev_ptr) {
  if (!dev_ptr) return LQ_OK;
  cudaError_t e = cudaIpcCloseMemHandle(dev_ptr);
  return e == cudaSuccess ? LQ_OK : lq::fail(LQ_ERR_LAUNCH, "peer_buffer_close: %s", cudaGetErrorString(e));
}

extern "C" int lq_peer_buffer_destroy(void* dev_ptr) {
  if (!dev_ptr) return LQ_OK;
  cudaError_t e = cudaFree(dev_ptr);
  return e == cudaSuccess ? LQ_OK : lq::fail(LQ_ERR_LAUNCH, "peer_buffer_destroy: %s", cudaGetErrorString(e));
}
