// Sharing of device memory that was created with the virtual memory management
// API (cuMemCreate + cuMemMap): PyTorch "expandable segments", sleep-mode and
// memory-saver allocators of inference engines.  cudaIpcGetMemHandle refuses
// such memory; the owner instead exports every physical allocation as a POSIX
// file descriptor, the descriptors travel to the other process over a unix
// socket (Python side), and the importer maps them into an address range of its
// own with read/write access for its device.
//
// The reference meets the same wall and documents it as unsupported
// (docs/README.md:91 there); this file has no counterpart in it.
//
// Every entry point returns 0 on success, a CUresult (> 0) when the driver
// refused, or -1 when the driver entry points could not be resolved.  Nothing
// here launches work on the GPU.

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace {

struct DriverApi {
  CUresult (*retain)(CUmemGenericAllocationHandle*, void*) = nullptr;
  CUresult (*export_handle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*import_handle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*release)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*reserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*address_free)(CUdeviceptr, size_t) = nullptr;
  CUresult (*map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*unmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*set_access)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*error_string)(CUresult, const char**) = nullptr;
  bool ok = false;
};

template <typename Fn>
bool resolve(const char* name, Fn* out) {
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &sym, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !sym) return false;
  *out = reinterpret_cast<Fn>(sym);
  return true;
}

const DriverApi& api() {
  static DriverApi a = [] {
    DriverApi d;
    d.ok = resolve("cuMemRetainAllocationHandle", &d.retain) && resolve("cuMemExportToShareableHandle", &d.export_handle) &&
           resolve("cuMemImportFromShareableHandle", &d.import_handle) && resolve("cuMemRelease", &d.release) &&
           resolve("cuMemAddressReserve", &d.reserve) && resolve("cuMemAddressFree", &d.address_free) &&
           resolve("cuMemMap", &d.map) && resolve("cuMemUnmap", &d.unmap) && resolve("cuMemSetAccess", &d.set_access) &&
           resolve("cuGetErrorString", &d.error_string);
    return d;
  }();
  return a;
}

}  // namespace

extern "C" {

// 1 when the driver's virtual-memory entry points are available in this process.
int awex_vmm_available() { return api().ok ? 1 : 0; }

// Export the physical allocation that backs `ptr` as a file descriptor.  The
// allocation must have been created with POSIX file descriptors as a requested
// handle type; the driver refuses otherwise.  The caller owns *fd_out and closes
// it when the importers have taken their copies.
int awex_vmm_export_fd(uint64_t ptr, int* fd_out) {
  const DriverApi& d = api();
  if (!d.ok) return -1;
  CUmemGenericAllocationHandle handle;
  CUresult r = d.retain(&handle, reinterpret_cast<void*>(ptr));
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  int fd = -1;
  r = d.export_handle(&fd, handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  d.release(handle);  // the retain above took a reference; the exported descriptor holds its own
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  *fd_out = fd;
  return 0;
}

// Reserve `total` bytes of address space (aligned to `alignment`, 0: the driver's default).
int awex_vmm_reserve(uint64_t total, uint64_t alignment, uint64_t* va_out) {
  const DriverApi& d = api();
  if (!d.ok) return -1;
  CUdeviceptr va = 0;
  CUresult r = d.reserve(&va, static_cast<size_t>(total), static_cast<size_t>(alignment), 0, 0);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  *va_out = static_cast<uint64_t>(va);
  return 0;
}

// Map the allocation behind `fd` at `va + offset` (`size` bytes, the whole
// allocation) and give `device` read/write access.  The descriptor stays the
// caller's to close; the mapping keeps the memory alive.
int awex_vmm_map_fd(uint64_t va, uint64_t offset, uint64_t size, int fd, int device) {
  const DriverApi& d = api();
  if (!d.ok) return -1;
  CUmemGenericAllocationHandle handle;
  CUresult r = d.import_handle(&handle, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) return static_cast<int>(r);
  const CUdeviceptr at = static_cast<CUdeviceptr>(va + offset);
  r = d.map(at, static_cast<size_t>(size), 0, handle, 0);
  if (r == CUDA_SUCCESS) {
    CUmemAccessDesc access = {};
    access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    access.location.id = device;
    access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    r = d.set_access(at, static_cast<size_t>(size), &access, 1);
    if (r != CUDA_SUCCESS) d.unmap(at, static_cast<size_t>(size));
  }
  d.release(handle);  // the mapping, if made, holds its own reference
  return static_cast<int>(r);
}

// Undo awex_vmm_map_fd for one mapped piece.
int awex_vmm_unmap(uint64_t va, uint64_t offset, uint64_t size) {
  const DriverApi& d = api();
  if (!d.ok) return -1;
  return static_cast<int>(d.unmap(static_cast<CUdeviceptr>(va + offset), static_cast<size_t>(size)));
}

// Give back a reservation whose pieces have all been unmapped.
int awex_vmm_release_range(uint64_t va, uint64_t total) {
  const DriverApi& d = api();
  if (!d.ok) return -1;
  return static_cast<int>(d.address_free(static_cast<CUdeviceptr>(va), static_cast<size_t>(total)));
}

const char* awex_driver_error_string(int code) {
  const DriverApi& d = api();
  const char* text = nullptr;
  if (!d.ok || d.error_string(static_cast<CUresult>(code), &text) != CUDA_SUCCESS || !text) return "unknown driver error";
  return text;
}

}  // extern "C"
