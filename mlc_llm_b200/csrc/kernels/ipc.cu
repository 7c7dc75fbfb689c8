// Fixed-format sharing of a device allocation between two processes of one NVLink box: the exporter
// hands out the 64 raw bytes of a cudaIpcMemHandle_t plus the offset of its tensor inside the
// allocation; the importer maps those bytes and learns how large the mapping really is, so that a
// descriptor which claims a larger pool than was exported is rejected on the host before any kernel
// sees the pointer.  Nothing here interprets serialised code or objects.
//
// Reference counterpart: the KV hand-off of disaggregated serving passes structured transfer metadata
// (cpp/serve/engine_actions/disagg_remote_send.cc:60-120, cpp/serve/data.h kv_append_metadata).
#include "common.cuh"

#include <cstring>

namespace mlcb {

using AddressRangeFn = int (*)(unsigned long long*, size_t*, unsigned long long);

// cuMemGetAddressRange through the runtime's driver entry-point query: no link-time dependency on
// the driver library (the build machine has none).
static AddressRangeFn address_range_fn() {
  static AddressRangeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &res) != cudaSuccess ||
        res != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<AddressRangeFn>(p);
  }();
  return fn;
}

}  // namespace mlcb

// handle64: 64 bytes out.  offset: bytes from the start of the allocation to `ptr`.  alloc_bytes: size
// of the allocation.  The device that owns `ptr` must be current.
MLCB_API int mlcb_ipc_export(const void* ptr, unsigned char* handle64, long long* offset, long long* alloc_bytes) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "descriptor format assumes a 64-byte handle");
  auto range = mlcb::address_range_fn();
  if (range == nullptr) return -2;
  unsigned long long base = 0;
  size_t size = 0;
  if (range(&base, &size, reinterpret_cast<unsigned long long>(ptr)) != 0) return -3;
  cudaIpcMemHandle_t h;
  cudaError_t err = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base));
  if (err != cudaSuccess) {
    cudaGetLastError();
    return static_cast<int>(err);
  }
  std::memcpy(handle64, &h, 64);
  *offset = static_cast<long long>(reinterpret_cast<unsigned long long>(ptr) - base);
  *alloc_bytes = static_cast<long long>(size);
  return 0;
}

// Maps the allocation behind `handle64` into this process (current device = the GPU that will touch
// it).  mapped_bytes = size of the mapping as the driver reports it.
MLCB_API int mlcb_ipc_open(const unsigned char* handle64, void** base, long long* mapped_bytes) {
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, 64);
  void* p = nullptr;
  cudaError_t err = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (err != cudaSuccess) {
    cudaGetLastError();
    return static_cast<int>(err);
  }
  auto range = mlcb::address_range_fn();
  unsigned long long b = 0;
  size_t size = 0;
  if (range == nullptr || range(&b, &size, reinterpret_cast<unsigned long long>(p)) != 0) {
    cudaIpcCloseMemHandle(p);
    return -3;
  }
  *base = p;
  *mapped_bytes = static_cast<long long>(size - (reinterpret_cast<unsigned long long>(p) - b));
  return 0;
}

MLCB_API int mlcb_ipc_close(void* base) {
  cudaError_t err = cudaIpcCloseMemHandle(base);
  if (err != cudaSuccess) cudaGetLastError();
  return static_cast<int>(err);
}
