// Pluggable device allocator with the torch.cuda.memory.CUDAPluggableAllocator ABI.
//
// Role in the reference: csrc/finegrained_alloc/finegrained_allocator.hip:27-56 — a malloc/free pair that
// torch calls for every device allocation, so that the symmetric heap (and everything else) lands in
// memory other GPUs can reach.
//
// Two modes, chosen by the environment variable IRIS_ALLOCATOR_MODE when the first allocation is made:
//   "vmm" (default when the driver offers it): every allocation is its own CUDA virtual-memory-management object,
//          created shareable (POSIX file descriptor) and mapped read/write on its device.  Any tensor torch hands
//          out can then be exported with iris_allocator_export_fd() and mapped by another process of the machine,
//          the way the symmetric heap itself is shared in heap_mode="vmm".  Sizes are rounded up to the
//          allocation granularity (2 MiB on B200).
//   "cudamalloc": plain cudaMalloc / cudaFree; also the fall-back when a VMM step fails.
// Either way the caller's current device is left as it was, failures are reported by returning nullptr (the
// reference exits the process instead, finegrained_allocator.hip:11-16), and LOG_IRIS_ALLOCATOR (any value)
// switches a log line per call on.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/types.h>

#include <mutex>
#include <unordered_map>

namespace {
bool logging_enabled() {
  static const bool on = getenv("LOG_IRIS_ALLOCATOR") != nullptr;
  return on;
}
struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  explicit DeviceGuard(int device) {
    if (cudaGetDevice(&prev) == cudaSuccess && prev != device) switched = cudaSetDevice(device) == cudaSuccess;
  }
  ~DeviceGuard() {
    if (switched) cudaSetDevice(prev);
  }
};

// ---- driver entry points for the VMM mode, resolved once through the runtime (no link against libcuda) ----
struct Vmm {
  bool ok = false;
  decltype(&cuMemCreate) Create = nullptr;
  decltype(&cuMemRelease) Release = nullptr;
  decltype(&cuMemAddressReserve) Reserve = nullptr;
  decltype(&cuMemAddressFree) AddressFree = nullptr;
  decltype(&cuMemMap) Map = nullptr;
  decltype(&cuMemUnmap) Unmap = nullptr;
  decltype(&cuMemSetAccess) SetAccess = nullptr;
  decltype(&cuMemExportToShareableHandle) Export = nullptr;
  decltype(&cuMemGetAllocationGranularity) Granularity = nullptr;
};
Vmm g_vmm;
std::once_flag g_vmm_once;

template <class F>
bool resolve(F& fn, const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess ||
      !p) {
    (void)cudaGetLastError();
    return false;
  }
  fn = reinterpret_cast<F>(p);
  return true;
}

const Vmm& vmm() {
  std::call_once(g_vmm_once, []() {
    const char* mode = getenv("IRIS_ALLOCATOR_MODE");
    if (mode && strcmp(mode, "cudamalloc") == 0) return;
    bool ok = true;
    ok &= resolve(g_vmm.Create, "cuMemCreate");
    ok &= resolve(g_vmm.Release, "cuMemRelease");
    ok &= resolve(g_vmm.Reserve, "cuMemAddressReserve");
    ok &= resolve(g_vmm.AddressFree, "cuMemAddressFree");
    ok &= resolve(g_vmm.Map, "cuMemMap");
    ok &= resolve(g_vmm.Unmap, "cuMemUnmap");
    ok &= resolve(g_vmm.SetAccess, "cuMemSetAccess");
    ok &= resolve(g_vmm.Export, "cuMemExportToShareableHandle");
    ok &= resolve(g_vmm.Granularity, "cuMemGetAllocationGranularity");
    g_vmm.ok = ok;
  });
  return g_vmm;
}

struct Record {
  CUmemGenericAllocationHandle handle;
  size_t bytes;  // mapped size (rounded up)
  int device;
};
std::mutex g_mutex;
std::unordered_map<void*, Record> g_records;  // VMM allocations by base address

void* vmm_malloc(size_t size, int device) {
  const Vmm& v = vmm();
  if (!v.ok) return nullptr;
  if (cudaFree(nullptr) != cudaSuccess) {  // makes sure the device's primary context exists
    (void)cudaGetLastError();
    return nullptr;
  }
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  if (v.Granularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || gran == 0) return nullptr;
  const size_t bytes = (size + gran - 1) / gran * gran;
  CUmemGenericAllocationHandle h;
  if (v.Create(&h, bytes, &prop, 0) != CUDA_SUCCESS) return nullptr;
  CUdeviceptr va = 0;
  if (v.Reserve(&va, bytes, gran, 0, 0) != CUDA_SUCCESS) {
    v.Release(h);
    return nullptr;
  }
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location = prop.location;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (v.Map(va, bytes, 0, h, 0) != CUDA_SUCCESS) {
    v.AddressFree(va, bytes);
    v.Release(h);
    return nullptr;
  }
  if (v.SetAccess(va, bytes, &acc, 1) != CUDA_SUCCESS) {
    v.Unmap(va, bytes);
    v.AddressFree(va, bytes);
    v.Release(h);
    return nullptr;
  }
  void* p = reinterpret_cast<void*>(va);
  std::lock_guard<std::mutex> lock(g_mutex);
  g_records[p] = Record{h, bytes, device};
  return p;
}

// true when `ptr` was a VMM allocation of this plug-in (and is now released)
bool vmm_free(void* ptr) {
  Record r;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = g_records.find(ptr);
    if (it == g_records.end()) return false;
    r = it->second;
    g_records.erase(it);
  }
  const Vmm& v = vmm();
  const CUdeviceptr va = reinterpret_cast<CUdeviceptr>(ptr);
  v.Unmap(va, r.bytes);
  v.AddressFree(va, r.bytes);
  v.Release(r.handle);
  return true;
}
}  // namespace

extern "C" {

void* iris_malloc(ssize_t size, int device, cudaStream_t stream) {
  (void)stream;
  DeviceGuard guard(device);
  void* p = size > 0 ? vmm_malloc((size_t)size, device) : nullptr;
  const char* how = "vmm";
  if (!p) {
    how = "cudaMalloc";
    cudaError_t e = cudaMalloc(&p, (size_t)size);
    if (e != cudaSuccess) {
      fprintf(stderr, "[iris allocator] cudaMalloc(%zd) on device %d failed: %s\n", size, device,
              cudaGetErrorString(e));
      (void)cudaGetLastError();
      return nullptr;
    }
  }
  if (logging_enabled())
    fprintf(stderr, "[iris allocator] malloc %zd bytes on device %d -> %p (%s)\n", size, device, p, how);
  return p;
}

void iris_free(void* ptr, ssize_t size, int device, cudaStream_t stream) {
  (void)stream;
  DeviceGuard guard(device);
  if (!vmm_free(ptr)) {
    cudaError_t e = cudaFree(ptr);
    if (e != cudaSuccess) {
      fprintf(stderr, "[iris allocator] cudaFree(%p) on device %d failed: %s\n", ptr, device, cudaGetErrorString(e));
      (void)cudaGetLastError();
    }
  }
  if (logging_enabled()) fprintf(stderr, "[iris allocator] free %zd bytes on device %d at %p\n", size, device, ptr);
}

// POSIX file descriptor for the allocation that starts at `ptr` (a pointer iris_malloc returned in VMM mode), to be
// passed to another process of the machine and imported there with cuMemImportFromShareableHandle; the caller
// closes it.  *bytes receives the mapped size.  Returns the descriptor, or -1 (not a VMM allocation of this plug-in,
// or the export failed).
int iris_allocator_export_fd(void* ptr, size_t* bytes) {
  Record r;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = g_records.find(ptr);
    if (it == g_records.end()) return -1;
    r = it->second;
  }
  int fd = -1;
  if (vmm().Export(&fd, r.handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS) return -1;
  if (bytes) *bytes = r.bytes;
  return fd;
}

// Number of live VMM allocations (0 in cudamalloc mode).
int iris_allocator_vmm_live(void) {
  std::lock_guard<std::mutex> lock(g_mutex);
  return (int)g_records.size();
}

}  // extern "C"
