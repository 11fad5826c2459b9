// CUDA driver access for the host plugin. The plugin links against no CUDA library: libcuda.so.1
// is dlopen()ed at init and every entry point is resolved by name, so the same shared object loads
// on a machine without a GPU (host-memory transport only)
// (reference: src/nccl_ofi_cuda.cpp — driver API only, resolved at run time; :481-568 VMM
// allocation; :453 dma-buf export; :252 GPUDirect flush).
#pragma once
#include <cstddef>
#include <cstdint>

namespace b200net::cuda {

using Stream = void*;
using Event = void*;
using Context = void*;

// Loads the driver and calls cuInit. 0 on success, -ENOSYS when there is no driver or no device.
int init();
bool available();
int device_count();

// Pointer classification. Returns 0 and fills the outputs if `ptr` is device memory.
int pointer_info(const void* ptr, int* device, void** alloc_base, size_t* alloc_size, bool* is_vmm);
bool is_host_pointer(const void* ptr);
// The address at which kernels of the current device can read page-locked host memory (memory
// from the driver's host allocators or registered with it). -EINVAL for pageable memory.
int host_device_alias(const void* host_ptr, void** device_ptr);

// Legacy IPC (cudaMalloc-style allocations): 64-byte handles.
int ipc_get_handle(void* alloc_base, uint8_t out[64]);
int ipc_open(const uint8_t handle[64], void** mapped);
int ipc_close(void* mapped);

// Context handling: the proxy thread that calls into the plugin may have no current context.
int ctx_get_current(Context* ctx);
int ctx_set_current(Context ctx);
int ensure_primary_ctx(int device);

int stream_create(Stream* s);
// A non-blocking stream of the greatest priority the device offers.
int stream_create_high_priority(Stream* s);
int stream_destroy(Stream s);
int event_create(Event* e);
int event_destroy(Event e);
int event_record(Event e, Stream s);
int event_query(Event e);  // 0 done, 1 not yet, <0 error
int memcpy_async(void* dst, const void* src, size_t n, Stream s);  // unified addressing: any direction
int stream_synchronize(Stream s);

// Kernels from an embedded image: load into the current context, look up, launch.
int module_load_data(const void* image, void** module);
int module_unload(void* module);
int module_get_function(void* module, const char* name, void** fn);
// Raises the dynamic shared memory a kernel may be launched with (above the 48 KiB default).
int func_set_max_dynamic_smem(void* fn, int bytes);
int launch_kernel(void* fn, unsigned grid, unsigned block, unsigned smem_bytes, Stream s, void** args);
// Page-locked host memory that the GPU can write (portable, mapped).
int host_alloc(void** ptr, size_t bytes);
int host_free(void* ptr);
// Page-locks memory the caller already owns (whole pages), so asynchronous copies from and to it
// do not pass through the driver's staging buffer; -ENOSYS when the driver does not offer it.
int host_register(void* ptr, size_t bytes);
int host_unregister(void* ptr);

// Plain device allocation (IPC-exportable with ipc_get_handle), zero-filled.
int mem_alloc(void** ptr, size_t bytes);
int mem_free(void* ptr);

// VMM allocation that can be exported to peers as a POSIX fd (granularity rounded).
int vmm_alloc(int device, size_t bytes, void** ptr, size_t* rounded, uint64_t* handle_out);
int vmm_free(void* ptr, size_t rounded, uint64_t handle);
int vmm_export_fd(uint64_t handle, int* fd);
// Peer access to somebody else's allocation of the virtual-memory API (NCCL's own buffers are
// such): the owner exports the allocation behind a mapped range as a POSIX fd, the peer (once it
// holds a duplicate of that fd) imports it, maps it and enables access for its current device.
int vmm_export_range(void* alloc_base, int* fd);
int vmm_import_map(int fd, size_t bytes, void** mapped);
int vmm_unmap(void* mapped, size_t bytes);
// dma-buf descriptor of an address range (for regMrDmaBuf users); -ENOTSUP when unsupported.
int get_dmabuf_fd(void* ptr, size_t size, int* fd, uint64_t* offset);
bool dmabuf_supported(int device);
// Orders earlier remote writes before later reads of the GPU; -ENOTSUP when not offered.
int flush_gpudirect_rdma_writes();
// NVLink topology of the box.
int p2p_attribute(int attr, int src_dev, int dst_dev, int* value);
int device_attribute(int attr, int dev, int* value);
int device_pci_bus_id(int dev, char* out, int len);
int device_uuid(int dev, uint8_t out[16]);

}  // namespace b200net::cuda
