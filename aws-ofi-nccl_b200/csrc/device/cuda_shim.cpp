#include "b200net/cuda_shim.h"

#include <cuda.h>
#include <dlfcn.h>

#include <cerrno>
#include <cstring>
#include <mutex>

#include "b200net/log.h"

namespace b200net::cuda {

namespace {
struct Api {
  void* lib = nullptr;
  bool ok = false;
  int ndev = 0;
  CUresult (*GetProcAddress)(const char*, void**, int, cuuint64_t, CUdriverProcAddressQueryResult*) = nullptr;
  CUresult (*Init)(unsigned) = nullptr;
  CUresult (*DeviceGetCount)(int*) = nullptr;
  CUresult (*DeviceGet)(CUdevice*, int) = nullptr;
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
  CUresult (*DeviceGetP2PAttribute)(int*, CUdevice_P2PAttribute, CUdevice, CUdevice) = nullptr;
  CUresult (*DeviceGetPCIBusId)(char*, int, CUdevice) = nullptr;
  CUresult (*DeviceGetUuid)(CUuuid*, CUdevice) = nullptr;
  CUresult (*PointerGetAttribute)(void*, CUpointer_attribute, CUdeviceptr) = nullptr;
  CUresult (*MemGetAddressRange)(CUdeviceptr*, size_t*, CUdeviceptr) = nullptr;
  CUresult (*IpcGetMemHandle)(CUipcMemHandle*, CUdeviceptr) = nullptr;
  CUresult (*IpcOpenMemHandle)(CUdeviceptr*, CUipcMemHandle, unsigned) = nullptr;
  CUresult (*IpcCloseMemHandle)(CUdeviceptr) = nullptr;
  CUresult (*CtxGetCurrent)(CUcontext*) = nullptr;
  CUresult (*CtxSetCurrent)(CUcontext) = nullptr;
  CUresult (*DevicePrimaryCtxRetain)(CUcontext*, CUdevice) = nullptr;
  CUresult (*StreamCreate)(CUstream*, unsigned) = nullptr;
  CUresult (*StreamCreateWithPriority)(CUstream*, unsigned, int) = nullptr;
  CUresult (*CtxGetStreamPriorityRange)(int*, int*) = nullptr;
  CUresult (*StreamDestroy)(CUstream) = nullptr;
  CUresult (*StreamSynchronize)(CUstream) = nullptr;
  CUresult (*EventCreate)(CUevent*, unsigned) = nullptr;
  CUresult (*EventDestroy)(CUevent) = nullptr;
  CUresult (*EventRecord)(CUevent, CUstream) = nullptr;
  CUresult (*EventQuery)(CUevent) = nullptr;
  CUresult (*MemcpyAsync)(CUdeviceptr, CUdeviceptr, size_t, CUstream) = nullptr;
  CUresult (*ModuleLoadData)(CUmodule*, const void*) = nullptr;
  CUresult (*ModuleUnload)(CUmodule) = nullptr;
  CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
  CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream,
                           void**, void**) = nullptr;
  CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
  CUresult (*MemHostAlloc)(void**, size_t, unsigned) = nullptr;
  CUresult (*MemFreeHost)(void*) = nullptr;
  CUresult (*MemHostRegister)(void*, size_t, unsigned) = nullptr;
  CUresult (*MemHostUnregister)(void*) = nullptr;
  CUresult (*CtxSynchronize)() = nullptr;
  CUresult (*MemAlloc)(CUdeviceptr*, size_t) = nullptr;
  CUresult (*MemFree)(CUdeviceptr) = nullptr;
  CUresult (*MemsetD8)(CUdeviceptr, unsigned char, size_t) = nullptr;
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*MemRetainAllocationHandle)(CUmemGenericAllocationHandle*, void*) = nullptr;
  CUresult (*CtxGetDevice)(CUdevice*) = nullptr;
  CUresult (*MemGetHandleForAddressRange)(void*, CUdeviceptr, size_t, CUmemRangeHandleType, unsigned long long) = nullptr;
  CUresult (*FlushGPUDirectRDMAWrites)(CUflushGPUDirectRDMAWritesTarget, CUflushGPUDirectRDMAWritesScope) = nullptr;
};
Api g;
std::once_flag g_once;
int g_init_rc = -ENOSYS;

template <typename F>
bool sym(F& fn, const char* name, bool required = true) {
  void* p = nullptr;
  CUdriverProcAddressQueryResult q;
  if (g.GetProcAddress && g.GetProcAddress(name, &p, 12000, CU_GET_PROC_ADDRESS_DEFAULT, &q) == CUDA_SUCCESS && p) {
    fn = reinterpret_cast<F>(p);
    return true;
  }
  fn = nullptr;
  return !required;
}

void do_init() {
  for (const char* name : {"libcuda.so.1", "libcuda.so"}) {
    g.lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
    if (g.lib) break;
  }
  if (!g.lib) return;
  g.GetProcAddress = reinterpret_cast<decltype(g.GetProcAddress)>(dlsym(g.lib, "cuGetProcAddress_v2"));
  if (!g.GetProcAddress) return;
  bool ok = true;
  ok &= sym(g.Init, "cuInit");
  ok &= sym(g.DeviceGetCount, "cuDeviceGetCount");
  ok &= sym(g.DeviceGet, "cuDeviceGet");
  ok &= sym(g.DeviceGetAttribute, "cuDeviceGetAttribute");
  ok &= sym(g.DeviceGetP2PAttribute, "cuDeviceGetP2PAttribute");
  ok &= sym(g.DeviceGetPCIBusId, "cuDeviceGetPCIBusId");
  ok &= sym(g.DeviceGetUuid, "cuDeviceGetUuid");
  ok &= sym(g.PointerGetAttribute, "cuPointerGetAttribute");
  ok &= sym(g.MemGetAddressRange, "cuMemGetAddressRange");
  ok &= sym(g.IpcGetMemHandle, "cuIpcGetMemHandle");
  ok &= sym(g.IpcOpenMemHandle, "cuIpcOpenMemHandle");
  ok &= sym(g.IpcCloseMemHandle, "cuIpcCloseMemHandle");
  ok &= sym(g.CtxGetCurrent, "cuCtxGetCurrent");
  ok &= sym(g.CtxSetCurrent, "cuCtxSetCurrent");
  ok &= sym(g.DevicePrimaryCtxRetain, "cuDevicePrimaryCtxRetain");
  ok &= sym(g.StreamCreate, "cuStreamCreate");
  sym(g.StreamCreateWithPriority, "cuStreamCreateWithPriority", false);
  sym(g.CtxGetStreamPriorityRange, "cuCtxGetStreamPriorityRange", false);
  ok &= sym(g.StreamDestroy, "cuStreamDestroy");
  ok &= sym(g.StreamSynchronize, "cuStreamSynchronize");
  ok &= sym(g.EventCreate, "cuEventCreate");
  ok &= sym(g.EventDestroy, "cuEventDestroy");
  ok &= sym(g.EventRecord, "cuEventRecord");
  ok &= sym(g.EventQuery, "cuEventQuery");
  ok &= sym(g.MemcpyAsync, "cuMemcpyAsync");
  sym(g.ModuleLoadData, "cuModuleLoadData", false);
  sym(g.ModuleUnload, "cuModuleUnload", false);
  sym(g.ModuleGetFunction, "cuModuleGetFunction", false);
  sym(g.LaunchKernel, "cuLaunchKernel", false);
  sym(g.FuncSetAttribute, "cuFuncSetAttribute", false);
  sym(g.MemHostAlloc, "cuMemHostAlloc", false);
  sym(g.MemFreeHost, "cuMemFreeHost", false);
  sym(g.MemHostRegister, "cuMemHostRegister", false);
  sym(g.MemHostUnregister, "cuMemHostUnregister", false);
  sym(g.CtxSynchronize, "cuCtxSynchronize", false);
  ok &= sym(g.MemAlloc, "cuMemAlloc");
  ok &= sym(g.MemFree, "cuMemFree");
  ok &= sym(g.MemsetD8, "cuMemsetD8");
  ok &= sym(g.MemCreate, "cuMemCreate");
  ok &= sym(g.MemRelease, "cuMemRelease");
  ok &= sym(g.MemGetAllocationGranularity, "cuMemGetAllocationGranularity");
  ok &= sym(g.MemAddressReserve, "cuMemAddressReserve");
  ok &= sym(g.MemAddressFree, "cuMemAddressFree");
  ok &= sym(g.MemMap, "cuMemMap");
  ok &= sym(g.MemUnmap, "cuMemUnmap");
  ok &= sym(g.MemSetAccess, "cuMemSetAccess");
  ok &= sym(g.MemExportToShareableHandle, "cuMemExportToShareableHandle");
  sym(g.MemImportFromShareableHandle, "cuMemImportFromShareableHandle", false);
  sym(g.MemRetainAllocationHandle, "cuMemRetainAllocationHandle", false);
  sym(g.CtxGetDevice, "cuCtxGetDevice", false);
  sym(g.MemGetHandleForAddressRange, "cuMemGetHandleForAddressRange", false);
  sym(g.FlushGPUDirectRDMAWrites, "cuFlushGPUDirectRDMAWrites", false);
  if (!ok) return;
  if (g.Init(0) != CUDA_SUCCESS) return;
  if (g.DeviceGetCount(&g.ndev) != CUDA_SUCCESS || g.ndev <= 0) return;
  g.ok = true;
  g_init_rc = 0;
}

inline int rc_of(CUresult r) { return r == CUDA_SUCCESS ? 0 : -(10000 + static_cast<int>(r)); }
}  // namespace

int init() {
  std::call_once(g_once, do_init);
  return g_init_rc;
}
bool available() { return init() == 0; }
int device_count() { return available() ? g.ndev : 0; }

int pointer_info(const void* ptr, int* device, void** alloc_base, size_t* alloc_size, bool* is_vmm) {
  if (!available()) return -ENOSYS;
  unsigned mem_type = 0;
  if (g.PointerGetAttribute(&mem_type, CU_POINTER_ATTRIBUTE_MEMORY_TYPE, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS ||
      mem_type != CU_MEMORYTYPE_DEVICE)
    return -EINVAL;
  int ord = 0;
  if (g.PointerGetAttribute(&ord, CU_POINTER_ATTRIBUTE_DEVICE_ORDINAL, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS) return -EINVAL;
  CUdeviceptr base = 0;
  size_t size = 0;
  if (g.MemGetAddressRange(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS) return -EINVAL;
  if (device) *device = ord;
  if (alloc_base) *alloc_base = reinterpret_cast<void*>(base);
  if (alloc_size) *alloc_size = size;
  if (is_vmm) {
    int legacy_ok = 0;  // IPC-capable legacy allocation?
    *is_vmm = g.PointerGetAttribute(&legacy_ok, CU_POINTER_ATTRIBUTE_IS_LEGACY_CUDA_IPC_CAPABLE, base) != CUDA_SUCCESS || !legacy_ok;
  }
  return 0;
}

bool is_host_pointer(const void* ptr) {
  if (!available()) return true;
  unsigned mem_type = 0;
  const CUresult r = g.PointerGetAttribute(&mem_type, CU_POINTER_ATTRIBUTE_MEMORY_TYPE, reinterpret_cast<CUdeviceptr>(ptr));
  return r != CUDA_SUCCESS || mem_type != CU_MEMORYTYPE_DEVICE;
}

int host_device_alias(const void* host_ptr, void** device_ptr) {
  if (!available()) return -ENOSYS;
  CUdeviceptr d = 0;
  if (g.PointerGetAttribute(&d, CU_POINTER_ATTRIBUTE_DEVICE_POINTER, reinterpret_cast<CUdeviceptr>(host_ptr)) != CUDA_SUCCESS || !d)
    return -EINVAL;
  *device_ptr = reinterpret_cast<void*>(d);
  return 0;
}

int ipc_get_handle(void* alloc_base, uint8_t out[64]) {
  if (!available()) return -ENOSYS;
  CUipcMemHandle h;
  const CUresult r = g.IpcGetMemHandle(&h, reinterpret_cast<CUdeviceptr>(alloc_base));
  if (r != CUDA_SUCCESS) return rc_of(r);
  static_assert(sizeof(h) == 64, "IPC handles are 64 bytes");
  memcpy(out, &h, 64);
  return 0;
}
int ipc_open(const uint8_t handle[64], void** mapped) {
  if (!available()) return -ENOSYS;
  CUipcMemHandle h;
  memcpy(&h, handle, 64);
  CUdeviceptr p = 0;
  const CUresult r = g.IpcOpenMemHandle(&p, h, CU_IPC_MEM_LAZY_ENABLE_PEER_ACCESS);
  if (r != CUDA_SUCCESS) return rc_of(r);
  *mapped = reinterpret_cast<void*>(p);
  return 0;
}
int ipc_close(void* mapped) { return available() ? rc_of(g.IpcCloseMemHandle(reinterpret_cast<CUdeviceptr>(mapped))) : -ENOSYS; }

int ctx_get_current(Context* ctx) {
  if (!available()) return -ENOSYS;
  CUcontext c = nullptr;
  const CUresult r = g.CtxGetCurrent(&c);
  *ctx = c;
  return rc_of(r);
}
int ctx_set_current(Context ctx) { return available() ? rc_of(g.CtxSetCurrent(static_cast<CUcontext>(ctx))) : -ENOSYS; }
int ensure_primary_ctx(int device) {
  if (!available()) return -ENOSYS;
  CUcontext cur = nullptr;
  if (g.CtxGetCurrent(&cur) == CUDA_SUCCESS && cur) return 0;
  CUdevice d;
  CUresult r = g.DeviceGet(&d, device);
  if (r != CUDA_SUCCESS) return rc_of(r);
  CUcontext c = nullptr;
  r = g.DevicePrimaryCtxRetain(&c, d);
  if (r != CUDA_SUCCESS) return rc_of(r);
  return rc_of(g.CtxSetCurrent(c));
}

int stream_create(Stream* s) {
  if (!available()) return -ENOSYS;
  CUstream st = nullptr;
  const CUresult r = g.StreamCreate(&st, CU_STREAM_NON_BLOCKING);
  *s = st;
  return rc_of(r);
}
int stream_create_high_priority(Stream* s) {
  if (!available()) return -ENOSYS;
  int least = 0, greatest = 0;
  if (!g.StreamCreateWithPriority || !g.CtxGetStreamPriorityRange || g.CtxGetStreamPriorityRange(&least, &greatest) != CUDA_SUCCESS)
    return stream_create(s);
  CUstream st = nullptr;
  const CUresult r = g.StreamCreateWithPriority(&st, CU_STREAM_NON_BLOCKING, greatest);
  if (r != CUDA_SUCCESS) return stream_create(s);
  *s = st;
  return 0;
}
int stream_destroy(Stream s) { return available() ? rc_of(g.StreamDestroy(static_cast<CUstream>(s))) : -ENOSYS; }
int stream_synchronize(Stream s) { return available() ? rc_of(g.StreamSynchronize(static_cast<CUstream>(s))) : -ENOSYS; }
int event_create(Event* e) {
  if (!available()) return -ENOSYS;
  CUevent ev = nullptr;
  const CUresult r = g.EventCreate(&ev, CU_EVENT_DISABLE_TIMING);
  *e = ev;
  return rc_of(r);
}
int event_destroy(Event e) { return available() ? rc_of(g.EventDestroy(static_cast<CUevent>(e))) : -ENOSYS; }
int event_record(Event e, Stream s) {
  return available() ? rc_of(g.EventRecord(static_cast<CUevent>(e), static_cast<CUstream>(s))) : -ENOSYS;
}
int event_query(Event e) {
  if (!available()) return -ENOSYS;
  const CUresult r = g.EventQuery(static_cast<CUevent>(e));
  if (r == CUDA_SUCCESS) return 0;
  if (r == CUDA_ERROR_NOT_READY) return 1;
  return rc_of(r);
}
int module_load_data(const void* image, void** module) {
  if (!available() || !g.ModuleLoadData) return -ENOSYS;
  CUmodule m = nullptr;
  const int rc = rc_of(g.ModuleLoadData(&m, image));
  *module = m;
  return rc;
}
int module_unload(void* module) {
  return (available() && g.ModuleUnload) ? rc_of(g.ModuleUnload(static_cast<CUmodule>(module))) : -ENOSYS;
}
int module_get_function(void* module, const char* name, void** fn) {
  if (!available() || !g.ModuleGetFunction) return -ENOSYS;
  CUfunction f = nullptr;
  const int rc = rc_of(g.ModuleGetFunction(&f, static_cast<CUmodule>(module), name));
  *fn = f;
  return rc;
}
int func_set_max_dynamic_smem(void* fn, int bytes) {
  if (!available() || !g.FuncSetAttribute) return -ENOSYS;
  return rc_of(g.FuncSetAttribute(static_cast<CUfunction>(fn), CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, bytes));
}
int launch_kernel(void* fn, unsigned grid, unsigned block, unsigned smem_bytes, Stream s, void** args) {
  if (!available() || !g.LaunchKernel) return -ENOSYS;
  return rc_of(g.LaunchKernel(static_cast<CUfunction>(fn), grid, 1, 1, block, 1, 1, smem_bytes, static_cast<CUstream>(s), args,
                              nullptr));
}
int host_alloc(void** ptr, size_t bytes) {
  if (!available() || !g.MemHostAlloc) return -ENOSYS;
  return rc_of(g.MemHostAlloc(ptr, bytes, CU_MEMHOSTALLOC_PORTABLE | CU_MEMHOSTALLOC_DEVICEMAP));
}
int host_free(void* ptr) { return (available() && g.MemFreeHost) ? rc_of(g.MemFreeHost(ptr)) : -ENOSYS; }
int host_register(void* ptr, size_t bytes) {
  if (!available() || !g.MemHostRegister) return -ENOSYS;
  return rc_of(g.MemHostRegister(ptr, bytes, CU_MEMHOSTREGISTER_PORTABLE | CU_MEMHOSTREGISTER_DEVICEMAP));
}
int host_unregister(void* ptr) { return (available() && g.MemHostUnregister) ? rc_of(g.MemHostUnregister(ptr)) : -ENOSYS; }

int memcpy_async(void* dst, const void* src, size_t n, Stream s) {
  if (!available()) return -ENOSYS;
  return rc_of(g.MemcpyAsync(reinterpret_cast<CUdeviceptr>(dst), reinterpret_cast<CUdeviceptr>(src), n, static_cast<CUstream>(s)));
}

int mem_alloc(void** ptr, size_t bytes) {
  if (!available()) return -ENOSYS;
  CUdeviceptr p = 0;
  CUresult r = g.MemAlloc(&p, bytes);
  if (r != CUDA_SUCCESS) return rc_of(r);
  r = g.MemsetD8(p, 0, bytes);
  // The fill runs on the legacy default stream and may still be in flight when the call returns;
  // the callers go on to use the memory on non-blocking streams, which do not wait for that stream.
  if (r == CUDA_SUCCESS && g.CtxSynchronize) r = g.CtxSynchronize();
  if (r != CUDA_SUCCESS) {
    g.MemFree(p);
    return rc_of(r);
  }
  *ptr = reinterpret_cast<void*>(p);
  return 0;
}
int mem_free(void* ptr) { return available() ? rc_of(g.MemFree(reinterpret_cast<CUdeviceptr>(ptr))) : -ENOSYS; }

int vmm_alloc(int device, size_t bytes, void** ptr, size_t* rounded, uint64_t* handle_out) {
  if (!available()) return -ENOSYS;
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  CUresult r = g.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM);
  if (r != CUDA_SUCCESS) return rc_of(r);
  const size_t sz = (bytes + gran - 1) / gran * gran;
  CUmemGenericAllocationHandle h;
  r = g.MemCreate(&h, sz, &prop, 0);
  if (r != CUDA_SUCCESS) return rc_of(r);
  CUdeviceptr va = 0;
  r = g.MemAddressReserve(&va, sz, 0, 0, 0);
  if (r != CUDA_SUCCESS) { g.MemRelease(h); return rc_of(r); }
  r = g.MemMap(va, sz, 0, h, 0);
  if (r != CUDA_SUCCESS) { g.MemAddressFree(va, sz); g.MemRelease(h); return rc_of(r); }
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location = prop.location;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = g.MemSetAccess(va, sz, &acc, 1);
  if (r != CUDA_SUCCESS) { g.MemUnmap(va, sz); g.MemAddressFree(va, sz); g.MemRelease(h); return rc_of(r); }
  *ptr = reinterpret_cast<void*>(va);
  *rounded = sz;
  *handle_out = h;
  return 0;
}
int vmm_free(void* ptr, size_t rounded, uint64_t handle) {
  if (!available()) return -ENOSYS;
  g.MemUnmap(reinterpret_cast<CUdeviceptr>(ptr), rounded);
  g.MemAddressFree(reinterpret_cast<CUdeviceptr>(ptr), rounded);
  return rc_of(g.MemRelease(handle));
}
int vmm_export_fd(uint64_t handle, int* fd) {
  if (!available()) return -ENOSYS;
  return rc_of(g.MemExportToShareableHandle(fd, handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
}
int vmm_export_range(void* alloc_base, int* fd) {
  if (!available() || !g.MemRetainAllocationHandle) return -ENOTSUP;
  CUmemGenericAllocationHandle h;
  CUresult r = g.MemRetainAllocationHandle(&h, alloc_base);
  if (r != CUDA_SUCCESS) return rc_of(r);
  r = g.MemExportToShareableHandle(fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  g.MemRelease(h);   // the retain took a reference of its own
  return rc_of(r);
}
int vmm_import_map(int fd, size_t bytes, void** mapped) {
  if (!available() || !g.MemImportFromShareableHandle || !g.CtxGetDevice) return -ENOTSUP;
  CUdevice dev;
  CUresult r = g.CtxGetDevice(&dev);
  if (r != CUDA_SUCCESS) return rc_of(r);
  CUmemGenericAllocationHandle h;
  r = g.MemImportFromShareableHandle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) return rc_of(r);
  CUdeviceptr va = 0;
  r = g.MemAddressReserve(&va, bytes, 0, 0, 0);
  if (r != CUDA_SUCCESS) { g.MemRelease(h); return rc_of(r); }
  r = g.MemMap(va, bytes, 0, h, 0);
  g.MemRelease(h);   // the mapping keeps the allocation alive
  if (r != CUDA_SUCCESS) { g.MemAddressFree(va, bytes); return rc_of(r); }
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = g.MemSetAccess(va, bytes, &acc, 1);
  if (r != CUDA_SUCCESS) { g.MemUnmap(va, bytes); g.MemAddressFree(va, bytes); return rc_of(r); }
  *mapped = reinterpret_cast<void*>(va);
  return 0;
}
int vmm_unmap(void* mapped, size_t bytes) {
  if (!available()) return -ENOSYS;
  const CUresult r = g.MemUnmap(reinterpret_cast<CUdeviceptr>(mapped), bytes);
  g.MemAddressFree(reinterpret_cast<CUdeviceptr>(mapped), bytes);
  return rc_of(r);
}
int get_dmabuf_fd(void* ptr, size_t size, int* fd, uint64_t* offset) {
  if (!available() || !g.MemGetHandleForAddressRange) return -ENOTSUP;
  const uintptr_t page = 4096;
  const uintptr_t start = reinterpret_cast<uintptr_t>(ptr) & ~(page - 1);
  const uintptr_t end = (reinterpret_cast<uintptr_t>(ptr) + size + page - 1) & ~(page - 1);
  const CUresult r = g.MemGetHandleForAddressRange(fd, start, end - start, CU_MEM_RANGE_HANDLE_TYPE_DMA_BUF_FD, 0);
  if (r != CUDA_SUCCESS) return -ENOTSUP;
  if (offset) *offset = reinterpret_cast<uintptr_t>(ptr) - start;
  return 0;
}
bool dmabuf_supported(int device) {
  if (!available()) return false;
  int v = 0;
  CUdevice d;
  if (g.DeviceGet(&d, device) != CUDA_SUCCESS) return false;
  return g.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_DMA_BUF_SUPPORTED, d) == CUDA_SUCCESS && v;
}
int flush_gpudirect_rdma_writes() {
  if (!available() || !g.FlushGPUDirectRDMAWrites) return -ENOTSUP;
  return rc_of(g.FlushGPUDirectRDMAWrites(CU_FLUSH_GPU_DIRECT_RDMA_WRITES_TARGET_CURRENT_CTX, CU_FLUSH_GPU_DIRECT_RDMA_WRITES_TO_OWNER));
}
int p2p_attribute(int attr, int src_dev, int dst_dev, int* value) {
  if (!available()) return -ENOSYS;
  CUdevice a, b;
  if (g.DeviceGet(&a, src_dev) != CUDA_SUCCESS || g.DeviceGet(&b, dst_dev) != CUDA_SUCCESS) return -EINVAL;
  return rc_of(g.DeviceGetP2PAttribute(value, static_cast<CUdevice_P2PAttribute>(attr), a, b));
}
int device_attribute(int attr, int dev, int* value) {
  if (!available()) return -ENOSYS;
  CUdevice d;
  if (g.DeviceGet(&d, dev) != CUDA_SUCCESS) return -EINVAL;
  return rc_of(g.DeviceGetAttribute(value, static_cast<CUdevice_attribute>(attr), d));
}
int device_pci_bus_id(int dev, char* out, int len) {
  if (!available()) return -ENOSYS;
  CUdevice d;
  if (g.DeviceGet(&d, dev) != CUDA_SUCCESS) return -EINVAL;
  return rc_of(g.DeviceGetPCIBusId(out, len, d));
}
int device_uuid(int dev, uint8_t out[16]) {
  if (!available()) return -ENOSYS;
  CUdevice d;
  if (g.DeviceGet(&d, dev) != CUDA_SUCCESS) return -EINVAL;
  CUuuid u;
  const CUresult r = g.DeviceGetUuid(&u, d);
  if (r == CUDA_SUCCESS) memcpy(out, u.bytes, 16);
  return rc_of(r);
}

}  // namespace b200net::cuda
