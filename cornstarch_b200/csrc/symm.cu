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

// Wait limit of every bounded device-side wait of this library on the CURRENT device, in nanoseconds (0 = back to the
// built-in 2 s).  Stream-ordered with respect to nothing: call it while no kernel of this library is running.
extern "C" int csb_set_wait_ns_attn_fwd(unsigned long long);
extern "C" int csb_set_wait_ns_attn_bwd(unsigned long long);
extern "C" int csb_set_wait_ns_gemm(unsigned long long);
extern "C" int csb_set_wait_ns_grad_reduce(unsigned long long);
CSB_API int csb_set_wait_ns(unsigned long long ns) {
  if (ns == 0) ns = 2000000000ull;
  int e;
  if ((e = csb_set_wait_ns_attn_fwd(ns))) return e;
  if ((e = csb_set_wait_ns_attn_bwd(ns))) return e;
  if ((e = csb_set_wait_ns_gemm(ns))) return e;
  return csb_set_wait_ns_grad_reduce(ns);
}

// Bounds-checked build: first index violation recorded by a kernel since the last call on the CURRENT device
// (0 = none; codes in ptx.cuh), cleared by the call.  The release build always answers 0; csb_bounds_check_enabled()
// tells which build this is.  Both calls synchronise the device.
extern "C" int csb_bounds_status_elementwise();
extern "C" int csb_bounds_status_moe_dispatch();
CSB_API int csb_bounds_status() {
  cudaDeviceSynchronize();
  const int a = csb_bounds_status_elementwise();
  const int b = csb_bounds_status_moe_dispatch();
  return a ? a : b;
}
CSB_API int csb_bounds_check_enabled() {
#ifdef CSB_BOUNDS_CHECK
  return 1;
#else
  return 0;
#endif
}
