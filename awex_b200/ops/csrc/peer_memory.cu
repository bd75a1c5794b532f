// Peer-memory plumbing: export device allocations of this process as CUDA IPC
// handles and map allocations of other processes (same GPU or an NVLink peer).
//
// cudaIpcGetMemHandle identifies a whole cudaMalloc allocation, so a tensor
// inside a caching-allocator segment is published as (handle of the segment,
// byte offset).  The importer opens each distinct segment once and keeps the
// mapping for the lifetime of the registration epoch.
//
// Replaces the reference's per-step pickling of IPC tensors through
// ForkingPickler (awex/util/tensor_util.py:35-183): here handles are exchanged
// once and only re-exported when a base address changes.

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>

namespace {

typedef CUresult (*GetAddressRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);

GetAddressRangeFn address_range_fn() {
  static GetAddressRangeFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &sym, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<GetAddressRangeFn>(sym);
  }
  return fn;
}

}  // namespace

extern "C" {

// base/size of the allocation that contains `ptr`.  Returns 0 on success.
int awex_address_range(uint64_t ptr, uint64_t* base, uint64_t* size) {
  GetAddressRangeFn fn = address_range_fn();
  if (!fn) return -1;
  CUdeviceptr b = 0;
  size_t s = 0;
  CUresult r = fn(&b, &s, static_cast<CUdeviceptr>(ptr));
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  *base = static_cast<uint64_t>(b);
  *size = static_cast<uint64_t>(s);
  return 0;
}

int awex_ipc_handle_bytes() { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }

// Export the allocation starting at `base` (a value returned by awex_address_range).
int awex_ipc_export(uint64_t base, unsigned char* handle_out) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base));
  if (e != cudaSuccess) return static_cast<int>(e);
  std::memcpy(handle_out, &h, sizeof(h));
  return 0;
}

// Map an exported allocation into this process on the current device.
int awex_ipc_open(const unsigned char* handle, uint64_t* mapped) {
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return static_cast<int>(e);
  *mapped = reinterpret_cast<uint64_t>(p);
  return 0;
}

int awex_ipc_close(uint64_t mapped) { return static_cast<int>(cudaIpcCloseMemHandle(reinterpret_cast<void*>(mapped))); }

// Peer access between two devices of ONE process (single-process multi-GPU use).
int awex_enable_peer_access(int device, int peer) {
  int can = 0;
  cudaError_t e = cudaDeviceCanAccessPeer(&can, device, peer);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (!can) return -2;
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(device);
  e = cudaDeviceEnablePeerAccess(peer, 0);
  cudaSetDevice(prev);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return 0;
  }
  return static_cast<int>(e);
}

const char* awex_cuda_error_string(int code) { return cudaGetErrorString(static_cast<cudaError_t>(code)); }

}  // extern "C"
