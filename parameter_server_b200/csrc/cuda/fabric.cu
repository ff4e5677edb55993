// Symmetric heap plumbing: one cudaMalloc'd heap per GPU, exported with CUDA
// IPC so that every rank process maps every peer's heap and the fused kernels
// can load from / store to peer memory directly over NVLink. This takes the
// place of the reference's socket transport (system/van.cc:27-269): there is
// no send/recv, only peer-mapped memory plus release/acquire flags.
#include <string.h>
#include "psb_common.cuh"
#include "psb_cuda.h"

extern "C" int psb_heap_alloc(void** ptr, size_t bytes) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return -(int)e;
  e = cudaMemset(*ptr, 0, bytes);
  return -(int)e;
}
extern "C" int psb_heap_free(void* ptr) { return -(int)cudaFree(ptr); }

// handle_out: 64 bytes (host)
extern "C" int psb_ipc_export(void* ptr, void* handle_out) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return -(int)e;
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}
extern "C" int psb_ipc_open(const void* handle, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return -(int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}
extern "C" int psb_ipc_close(void* ptr) { return -(int)cudaIpcCloseMemHandle(ptr); }
extern "C" int psb_ipc_handle_bytes(void) { return (int)sizeof(cudaIpcMemHandle_t); }

extern "C" int psb_set_device(int dev) { return -(int)cudaSetDevice(dev); }
extern "C" int psb_can_access_peer(int dev, int peer) {
  int ok = 0;
  cudaError_t e = cudaDeviceCanAccessPeer(&ok, dev, peer);
  return e == cudaSuccess ? ok : -(int)e;
}
extern "C" const char* psb_error_string(int neg_code) {
  return cudaGetErrorString((cudaError_t)(-neg_code));
}
