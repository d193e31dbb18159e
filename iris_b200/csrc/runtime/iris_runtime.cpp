// Native host runtime: device queries, symmetric-heap memory (cudaMalloc + CUDA IPC, or CUDA virtual
// memory management with POSIX file-descriptor export), peer mapping, and NVLS multicast binding.
//
// Role in the reference: iris/_hip.py:23-131 (ctypes calls into libamdhip64 for hipIpcGetMemHandle,
// hipIpcOpenMemHandle, device count/set, compute-unit count, wall-clock rate).  Here the same services
// are a C ABI in C++ over the CUDA runtime and driver APIs.  The driver entry points are resolved at run
// time through cudaGetDriverEntryPoint so the library loads on machines without a driver.
#include <cuda.h>
#include <cuda_runtime.h>
#include <errno.h>
#include <stdio.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <mutex>

namespace {

thread_local char g_err[512] = "";

int fail_rt(cudaError_t e, const char* what) {
  snprintf(g_err, sizeof(g_err), "%s: %s (%d)", what, cudaGetErrorString(e), (int)e);
  return -(int)e;
}
#define RT_TRY(call)                               \
  do {                                             \
    cudaError_t e_ = (call);                       \
    if (e_ != cudaSuccess) return fail_rt(e_, #call); \
  } while (0)

// ---- driver API, resolved lazily -------------------------------------------------------------
struct Driver {
  bool ok = false;
  decltype(&cuMemCreate) MemCreate = nullptr;
  decltype(&cuMemRelease) MemRelease = nullptr;
  decltype(&cuMemAddressReserve) MemAddressReserve = nullptr;
  decltype(&cuMemAddressFree) MemAddressFree = nullptr;
  decltype(&cuMemMap) MemMap = nullptr;
  decltype(&cuMemUnmap) MemUnmap = nullptr;
  decltype(&cuMemSetAccess) MemSetAccess = nullptr;
  decltype(&cuMemExportToShareableHandle) MemExport = nullptr;
  decltype(&cuMemImportFromShareableHandle) MemImport = nullptr;
  decltype(&cuMemGetAllocationGranularity) MemGranularity = nullptr;
  decltype(&cuMulticastCreate) McCreate = nullptr;
  decltype(&cuMulticastAddDevice) McAddDevice = nullptr;
  decltype(&cuMulticastBindMem) McBindMem = nullptr;
  decltype(&cuMulticastUnbind) McUnbind = nullptr;
  decltype(&cuMulticastGetGranularity) McGranularity = nullptr;
  decltype(&cuDeviceGetAttribute) DeviceGetAttribute = nullptr;
  decltype(&cuGetErrorString) GetErrorString = nullptr;
};
Driver g_drv;
std::once_flag g_drv_once;

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

const Driver& drv() {
  std::call_once(g_drv_once, []() {
    bool ok = true;
    ok &= resolve(g_drv.MemCreate, "cuMemCreate");
    ok &= resolve(g_drv.MemRelease, "cuMemRelease");
    ok &= resolve(g_drv.MemAddressReserve, "cuMemAddressReserve");
    ok &= resolve(g_drv.MemAddressFree, "cuMemAddressFree");
    ok &= resolve(g_drv.MemMap, "cuMemMap");
    ok &= resolve(g_drv.MemUnmap, "cuMemUnmap");
    ok &= resolve(g_drv.MemSetAccess, "cuMemSetAccess");
    ok &= resolve(g_drv.MemExport, "cuMemExportToShareableHandle");
    ok &= resolve(g_drv.MemImport, "cuMemImportFromShareableHandle");
    ok &= resolve(g_drv.MemGranularity, "cuMemGetAllocationGranularity");
    ok &= resolve(g_drv.DeviceGetAttribute, "cuDeviceGetAttribute");
    ok &= resolve(g_drv.GetErrorString, "cuGetErrorString");
    // Multicast entry points are optional (older drivers).
    resolve(g_drv.McCreate, "cuMulticastCreate");
    resolve(g_drv.McAddDevice, "cuMulticastAddDevice");
    resolve(g_drv.McBindMem, "cuMulticastBindMem");
    resolve(g_drv.McUnbind, "cuMulticastUnbind");
    resolve(g_drv.McGranularity, "cuMulticastGetGranularity");
    g_drv.ok = ok;
  });
  return g_drv;
}

int fail_drv(CUresult r, const char* what) {
  const char* s = nullptr;
  if (g_drv.GetErrorString) g_drv.GetErrorString(r, &s);
  snprintf(g_err, sizeof(g_err), "%s: %s (%d)", what, s ? s : "?", (int)r);
  return -(int)r - 100000;
}
#define DRV_TRY(call)                                  \
  do {                                                 \
    CUresult r_ = (call);                              \
    if (r_ != CUDA_SUCCESS) return fail_drv(r_, #call); \
  } while (0)

CUmemAllocationProp device_prop(int device) {
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

}  // namespace

extern "C" {

const char* iris_rt_last_error() { return g_err; }

int iris_rt_device_count() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return n;
}

int iris_rt_set_device(int device) {
  RT_TRY(cudaSetDevice(device));
  RT_TRY(cudaFree(0));  // make sure the primary context exists before any driver call
  return 0;
}

int iris_rt_get_device() {
  int d = -1;
  if (cudaGetDevice(&d) != cudaSuccess) return -1;
  return d;
}

// Number of streaming multiprocessors (the reference's get_cu_count, iris/_hip.py:78-87).
int iris_rt_sm_count(int device) {
  int v = 0;
  RT_TRY(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device));
  return v;
}

// Rate in kHz of the timer that iris::globaltimer() reads (the reference's get_wall_clock_rate,
// iris/_hip.py:107-114).  %globaltimer counts nanoseconds.
int iris_rt_wall_clock_rate_khz(int /*device*/) { return 1000000; }

int iris_rt_can_access_peer(int device, int peer) {
  int v = 0;
  if (cudaDeviceCanAccessPeer(&v, device, peer) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return v;
}

// Enable direct access from `device` (current) to `peer`; already-enabled is not an error.
int iris_rt_enable_peer(int device, int peer) {
  RT_TRY(cudaSetDevice(device));
  cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    (void)cudaGetLastError();
    return 0;
  }
  if (e != cudaSuccess) return fail_rt(e, "cudaDeviceEnablePeerAccess");
  return 0;
}

// ---- cudaMalloc + CUDA IPC path ----------------------------------------------------------------
int iris_rt_malloc(int device, uint64_t bytes, void** out) {
  RT_TRY(cudaSetDevice(device));
  RT_TRY(cudaMalloc(out, bytes));
  return 0;
}
int iris_rt_free(void* p) {
  RT_TRY(cudaFree(p));
  return 0;
}
int iris_rt_memset(void* p, int value, uint64_t bytes) {
  RT_TRY(cudaMemset(p, value, bytes));
  return 0;
}
int iris_rt_ipc_handle_size() { return (int)sizeof(cudaIpcMemHandle_t); }
int iris_rt_ipc_get_handle(void* p, void* out_handle) {
  cudaIpcMemHandle_t h;
  RT_TRY(cudaIpcGetMemHandle(&h, p));
  memcpy(out_handle, &h, sizeof(h));
  return 0;
}
int iris_rt_ipc_open_handle(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  RT_TRY(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}
int iris_rt_ipc_close_handle(void* p) {
  RT_TRY(cudaIpcCloseMemHandle(p));
  return 0;
}

int iris_rt_memcpy_h2d(void* dst, const void* src, uint64_t bytes) {
  RT_TRY(cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice));
  return 0;
}
int iris_rt_memcpy_d2h(void* dst, const void* src, uint64_t bytes) {
  RT_TRY(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost));
  return 0;
}
int iris_rt_device_synchronize() {
  RT_TRY(cudaDeviceSynchronize());
  return 0;
}

// ---- virtual-memory-management path ------------------------------------------------------------
int iris_rt_vmm_supported(int device) {
  const Driver& d = drv();
  if (!d.ok) return 0;
  int v = 0;
  if (d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, device) !=
      CUDA_SUCCESS)
    return 0;
  return v;
}

int iris_rt_multicast_supported(int device) {
  const Driver& d = drv();
  if (!d.ok || !d.McCreate) return 0;
  int v = 0;
  if (d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device) != CUDA_SUCCESS) return 0;
  return v;
}

// Allocation granularity for heaps on `device`; heap sizes must be multiples of it.
int64_t iris_rt_vmm_granularity(int device) {
  const Driver& d = drv();
  if (!d.ok) return -1;
  CUmemAllocationProp prop = device_prop(device);
  size_t g = 0;
  if (d.MemGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS) return -1;
  return (int64_t)g;
}

// Create physical memory on `device`; returns the generic allocation handle and a POSIX fd for export.
int iris_rt_vmm_create(int device, uint64_t bytes, uint64_t* out_handle, int* out_fd) {
  const Driver& d = drv();
  if (!d.ok) {
    snprintf(g_err, sizeof(g_err), "CUDA driver entry points unavailable");
    return -1;
  }
  RT_TRY(cudaSetDevice(device));
  RT_TRY(cudaFree(0));
  CUmemAllocationProp prop = device_prop(device);
  CUmemGenericAllocationHandle h;
  DRV_TRY(d.MemCreate(&h, bytes, &prop, 0));
  int fd = -1;
  CUresult r = d.MemExport(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    d.MemRelease(h);
    return fail_drv(r, "cuMemExportToShareableHandle");
  }
  *out_handle = (uint64_t)h;
  *out_fd = fd;
  return 0;
}

int iris_rt_vmm_import(int fd, uint64_t* out_handle) {
  const Driver& d = drv();
  CUmemGenericAllocationHandle h;
  DRV_TRY(d.MemImport(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
  *out_handle = (uint64_t)h;
  return 0;
}

int iris_rt_vmm_release(uint64_t handle) {
  DRV_TRY(drv().MemRelease((CUmemGenericAllocationHandle)handle));
  return 0;
}

int iris_rt_vmm_reserve(uint64_t bytes, uint64_t alignment, uint64_t* out_va) {
  CUdeviceptr va = 0;
  DRV_TRY(drv().MemAddressReserve(&va, bytes, alignment, 0, 0));
  *out_va = (uint64_t)va;
  return 0;
}

int iris_rt_vmm_address_free(uint64_t va, uint64_t bytes) {
  DRV_TRY(drv().MemAddressFree((CUdeviceptr)va, bytes));
  return 0;
}

// Map `handle` at `va` and give `device` read/write access.
int iris_rt_vmm_map(uint64_t va, uint64_t bytes, uint64_t handle, int device) {
  const Driver& d = drv();
  DRV_TRY(d.MemMap((CUdeviceptr)va, bytes, 0, (CUmemGenericAllocationHandle)handle, 0));
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  CUresult r = d.MemSetAccess((CUdeviceptr)va, bytes, &acc, 1);
  if (r != CUDA_SUCCESS) {
    d.MemUnmap((CUdeviceptr)va, bytes);
    return fail_drv(r, "cuMemSetAccess");
  }
  return 0;
}

int iris_rt_vmm_unmap(uint64_t va, uint64_t bytes) {
  DRV_TRY(drv().MemUnmap((CUdeviceptr)va, bytes));
  return 0;
}

// ---- NVLS multicast ----------------------------------------------------------------------------
int64_t iris_rt_multicast_granularity(int num_devices, uint64_t bytes) {
  const Driver& d = drv();
  if (!d.McGranularity) return -1;
  CUmulticastObjectProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.numDevices = (unsigned)num_devices;
  prop.size = bytes;
  prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t g = 0;
  if (d.McGranularity(&g, &prop, CU_MULTICAST_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS) return -1;
  return (int64_t)g;
}

// Rank 0 creates the multicast object and exports it as an fd.
int iris_rt_multicast_create(int num_devices, uint64_t bytes, uint64_t* out_handle, int* out_fd) {
  const Driver& d = drv();
  if (!d.McCreate) {
    snprintf(g_err, sizeof(g_err), "multicast entry points unavailable");
    return -1;
  }
  CUmulticastObjectProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.numDevices = (unsigned)num_devices;
  prop.size = bytes;
  prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  CUmemGenericAllocationHandle h;
  DRV_TRY(d.McCreate(&h, &prop));
  int fd = -1;
  CUresult r = d.MemExport(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) {
    d.MemRelease(h);
    return fail_drv(r, "cuMemExportToShareableHandle(multicast)");
  }
  *out_handle = (uint64_t)h;
  *out_fd = fd;
  return 0;
}

int iris_rt_multicast_add_device(uint64_t mc_handle, int device) {
  DRV_TRY(drv().McAddDevice((CUmemGenericAllocationHandle)mc_handle, (CUdevice)device));
  return 0;
}

int iris_rt_multicast_bind(uint64_t mc_handle, uint64_t mem_handle, uint64_t bytes) {
  DRV_TRY(drv().McBindMem((CUmemGenericAllocationHandle)mc_handle, 0, (CUmemGenericAllocationHandle)mem_handle, 0,
                          bytes, 0));
  return 0;
}

int iris_rt_multicast_unbind(uint64_t mc_handle, int device, uint64_t bytes) {
  DRV_TRY(drv().McUnbind((CUmemGenericAllocationHandle)mc_handle, (CUdevice)device, 0, bytes));
  return 0;
}

// ---- file-descriptor passing between the ranks of one machine (SCM_RIGHTS) -----------------------
// The receiver binds an abstract-namespace Unix datagram socket named `name`; the sender addresses it.
int iris_rt_fd_listen(const char* name) {
  int s = socket(AF_UNIX, SOCK_DGRAM, 0);
  if (s < 0) {
    snprintf(g_err, sizeof(g_err), "socket: %s", strerror(errno));
    return -1;
  }
  struct sockaddr_un addr;
  memset(&addr, 0, sizeof(addr));
  addr.sun_family = AF_UNIX;
  size_t len = strlen(name);
  if (len > sizeof(addr.sun_path) - 2) len = sizeof(addr.sun_path) - 2;
  memcpy(addr.sun_path + 1, name, len);  // leading NUL: abstract namespace, no file to clean up
  if (bind(s, (struct sockaddr*)&addr, (socklen_t)(offsetof(struct sockaddr_un, sun_path) + 1 + len)) != 0) {
    snprintf(g_err, sizeof(g_err), "bind(%s): %s", name, strerror(errno));
    close(s);
    return -1;
  }
  return s;
}

int iris_rt_fd_send(const char* name, int fd_to_send, int tag) {
  int s = socket(AF_UNIX, SOCK_DGRAM, 0);
  if (s < 0) return -1;
  struct sockaddr_un addr;
  memset(&addr, 0, sizeof(addr));
  addr.sun_family = AF_UNIX;
  size_t len = strlen(name);
  if (len > sizeof(addr.sun_path) - 2) len = sizeof(addr.sun_path) - 2;
  memcpy(addr.sun_path + 1, name, len);
  struct msghdr msg;
  memset(&msg, 0, sizeof(msg));
  struct iovec iov;
  iov.iov_base = &tag;
  iov.iov_len = sizeof(tag);
  char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  msg.msg_name = &addr;
  msg.msg_namelen = (socklen_t)(offsetof(struct sockaddr_un, sun_path) + 1 + len);
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  struct cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd_to_send, sizeof(int));
  ssize_t n = sendmsg(s, &msg, 0);
  int rc = 0;
  if (n < 0) {
    snprintf(g_err, sizeof(g_err), "sendmsg(%s): %s", name, strerror(errno));
    rc = -1;
  }
  close(s);
  return rc;
}

// Receive one fd on listening socket `s`; waits at most timeout_ms.  Returns the fd (>= 0) and the tag.
int iris_rt_fd_recv(int s, int timeout_ms, int* out_tag) {
  struct timeval tv;
  tv.tv_sec = timeout_ms / 1000;
  tv.tv_usec = (timeout_ms % 1000) * 1000;
  setsockopt(s, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
  struct msghdr msg;
  memset(&msg, 0, sizeof(msg));
  int tag = -1;
  struct iovec iov;
  iov.iov_base = &tag;
  iov.iov_len = sizeof(tag);
  char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  ssize_t n = recvmsg(s, &msg, 0);
  if (n < 0) {
    snprintf(g_err, sizeof(g_err), "recvmsg: %s", strerror(errno));
    return -1;
  }
  struct cmsghdr* c = CMSG_FIRSTHDR(&msg);
  if (!c || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS) {
    snprintf(g_err, sizeof(g_err), "recvmsg: no descriptor in message");
    return -1;
  }
  int fd = -1;
  memcpy(&fd, CMSG_DATA(c), sizeof(int));
  if (out_tag) *out_tag = tag;
  return fd;
}

int iris_rt_fd_close(int fd) { return close(fd); }

}  // extern "C"
