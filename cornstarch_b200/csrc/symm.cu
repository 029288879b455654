// Symmetric memory for kernels that read and write peer GPUs directly over NVLink.
//
// Every rank allocates a buffer of the same size with cudaMalloc, exports a CUDA IPC handle, and maps
// the buffers of the other ranks of the node into its own address space; the table of pointers
// (own buffer + peer mappings) is what the fused compute+collective kernels receive.  This small runtime
// replaces, for the fused paths, the NCCL collectives behind ColossalAI's Linear1D_Row / Linear1D_Col
// in the reference (cornstarch/shardformer/policies/llama.py:192-249); NCCL stays for bootstrap, for
// pipeline send/recv and as the measured baseline.
#include "host.h"
#include <string.h>

// Allocate `nbytes` of zeroed device memory on the current device.
CSB_API int csb_symm_alloc(long nbytes, void** out) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)nbytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(p, 0, (size_t)nbytes);
  if (e != cudaSuccess) return (int)e;
  *out = p;
  return 0;
}
CSB_API int csb_symm_free(void* p) { return (int)cudaFree(p); }

// 64-byte IPC handle of an allocation made by csb_symm_alloc.
CSB_API int csb_ipc_export(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
// Map a peer's allocation; enables peer access lazily.
CSB_API int csb_ipc_import(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    fprintf(stderr, "[cornstarch_b200] cudaIpcOpenMemHandle failed: %s\n", cudaGetErrorString(e));
    return (int)e;
  }
  *out = p;
  return 0;
}
CSB_API int csb_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }
CSB_API int csb_ipc_handle_size() { return (int)sizeof(cudaIpcMemHandle_t); }
