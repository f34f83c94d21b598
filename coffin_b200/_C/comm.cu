// Host helpers for peer memory: device buffers that can be opened by the other ranks of the node
// (CUDA IPC), and the step-epoch kernel.  The handles travel over the CPU control plane; the data
// path afterwards is plain loads/stores on NVLink from inside the compute kernels (tp.cuh).
// Reference role: P2pReduce.__init__ exchanging cudaIpc handles (models/qwen35/ep.py:546-736,
// backends/corex/kernels/p2p_reduce.cu:177-203).
#include <string.h>
#include "tp.cuh"

namespace {
__global__ void epoch_bump_kernel(unsigned* epoch) {
  griddep_launch();
  griddep_wait();
  if (threadIdx.x == 0) *epoch += 1;
}
}  // namespace

CB_EXPORT int cb_peer_alloc(int64_t bytes, void** out) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(p, 0, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  *out = p;
  return 0;
}
CB_EXPORT int cb_peer_free(void* p) { return (int)cudaFree(p); }
CB_EXPORT int cb_ipc_get_handle(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
CB_EXPORT int cb_ipc_open_handle(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return (int)e;
  *out = p;
  return 0;
}
CB_EXPORT int cb_ipc_close_handle(void* p) { return (int)cudaIpcCloseMemHandle(p); }

CB_EXPORT int cb_peer_read_i32(const void* dev, int* out) {
  return (int)cudaMemcpy(out, dev, sizeof(int), cudaMemcpyDeviceToHost);
}

// Advance the step epoch (first kernel of every decode step on every rank).
CB_EXPORT int cb_tp_epoch_bump(void* epoch, void* stream) {
  return (int)cb_launch(epoch_bump_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, (unsigned*)epoch);
}
