// Buffers for the functional tests: host memory, or, with FUNC_NET_DEVICE=1, device memory.
// Included after the test has defined g_rank.
//
// Three modes:
//   host    plain malloc; data() == host().
//   view    the stand-in driver is on the library path (CPU runs): buffers come from it and are
//           registered as NCCL_PTR_CUDA, so the plugin's IPC mapping, copy-kernel and eager-pack
//           paths run. data() is not accessible to host code (a stray dereference faults); host()
//           is a second mapping of the same bytes, so to_device() / from_device() have nothing to do.
//   mirror  a real driver (a GPU box), or the stand-in with FUNC_NET_MIRROR=1: data() is device
//           memory, host() a separate host copy; to_device() pushes the host copy before the
//           plugin is given the buffer, from_device() fetches it before the test checks it.
//           FUNC_NET_VMM=1 makes the device memory a cuMemCreate allocation (as NCCL's buffers are).
// A test written against host() + to_device() + from_device() runs unchanged in all three.
#pragma once
#include <dlfcn.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include "b200net/cuda_shim.h"
#include "nccl_abi.h"

using FakeAllocFn = int (*)(void**, size_t);
using FakeFreeFn = int (*)(void*);
using FakeViewFn = void* (*)(void*);
static FakeViewFn g_dev_view = nullptr;
static FakeAllocFn g_dev_alloc = nullptr;
static FakeFreeFn g_dev_free = nullptr;

enum TestBufMode { BUF_HOST = 0, BUF_VIEW = 1, BUF_MIRROR = 2 };
static int device_mode_kind() {
  static int mode = -1;
  if (mode < 0) {
    mode = BUF_HOST;
    if (getenv("FUNC_NET_DEVICE") && atoi(getenv("FUNC_NET_DEVICE"))) {
      void* h = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
      if (h) {
        g_dev_alloc = reinterpret_cast<FakeAllocFn>(dlsym(h, "fake_cuda_mem_alloc"));
        g_dev_free = reinterpret_cast<FakeFreeFn>(dlsym(h, "fake_cuda_mem_free"));
        g_dev_view = reinterpret_cast<FakeViewFn>(dlsym(h, "fake_cuda_host_view"));
      }
      const bool stand_in = g_dev_alloc && g_dev_free && g_dev_view;
      const bool want_mirror = getenv("FUNC_NET_MIRROR") && atoi(getenv("FUNC_NET_MIRROR"));
      if (stand_in && !want_mirror) {
        mode = BUF_VIEW;
      } else if (b200net::cuda::available()) {
        // one GPU per rank where there are several, so that payloads cross NVLink
        const int count = b200net::cuda::device_count();
        const char* pick = getenv("FUNC_NET_GPU");
        const int ordinal = pick ? atoi(pick) : (count > 0 ? g_rank % count : 0);
        if (b200net::cuda::ensure_primary_ctx(ordinal) == 0) mode = BUF_MIRROR;
      }
      if (mode == BUF_HOST) fprintf(stderr, "[rank %d] FUNC_NET_DEVICE set but no usable driver was found: host buffers\n", g_rank);
    }
  }
  return mode;
}
static bool device_mode() { return device_mode_kind() != BUF_HOST; }

struct TestBuf {
  uint8_t* p = nullptr;   // the address given to the plugin
  uint8_t* h = nullptr;   // where the test itself reads and writes the bytes
  size_t n = 0;
  bool dev = false;
  bool mirror = false;
  size_t vmm_rounded = 0;     // mirror mode with FUNC_NET_VMM=1: the buffer is a cuMemCreate allocation
  uint64_t vmm_handle = 0;
  uint8_t* data() { return p; }
  uint8_t* host() { return h; }
  size_t size() const { return n; }
  // host() -> data(): call after filling, before the plugin (or a peer) may read or overwrite the buffer
  int to_device(size_t off = 0, size_t len = ~size_t{0}) { return copy(true, off, len); }
  // data() -> host(): call before checking what arrived
  int from_device(size_t off = 0, size_t len = ~size_t{0}) { return copy(false, off, len); }

 private:
  int copy(bool push, size_t off, size_t len) {
    if (!mirror || off >= n) return 0;
    if (len > n - off) len = n - off;
    static b200net::cuda::Stream st = nullptr;
    if (!st && b200net::cuda::stream_create(&st) != 0) return 1;
    const int rc = push ? b200net::cuda::memcpy_async(p + off, h + off, len, st) : b200net::cuda::memcpy_async(h + off, p + off, len, st);
    return rc != 0 || b200net::cuda::stream_synchronize(st) != 0;
  }
};

static int buf_alloc(TestBuf* b, size_t n, bool want_device = true) {
  b->n = n;
  const int kind = want_device ? device_mode_kind() : BUF_HOST;
  b->dev = kind != BUF_HOST;
  b->mirror = kind == BUF_MIRROR;
  if (kind == BUF_VIEW) {
    void* p = nullptr;
    if (g_dev_alloc(&p, n) != 0) return 1;
    b->p = static_cast<uint8_t*>(p);
    b->h = static_cast<uint8_t*>(g_dev_view(p));
  } else if (kind == BUF_MIRROR) {
    void* p = nullptr;
    if (getenv("FUNC_NET_VMM") && atoi(getenv("FUNC_NET_VMM"))) {
      // the way NCCL allocates its own buffers: create, reserve, map (exportable as a descriptor)
      const int count = b200net::cuda::device_count();
      const char* pick = getenv("FUNC_NET_GPU");
      const int ordinal = pick ? atoi(pick) : (count > 0 ? g_rank % count : 0);
      if (b200net::cuda::vmm_alloc(ordinal, n, &p, &b->vmm_rounded, &b->vmm_handle) != 0) return 1;
    } else if (b200net::cuda::mem_alloc(&p, n) != 0) {
      return 1;
    }
    b->p = static_cast<uint8_t*>(p);
    b->h = static_cast<uint8_t*>(calloc(1, n));
    if (!b->h) return 1;
  } else {
    b->p = b->h = static_cast<uint8_t*>(malloc(n));
  }
  return b->p ? 0 : 1;
}
static void buf_free(TestBuf* b) {
  if (!b->p) return;
  if (b->mirror) {
    if (b->vmm_rounded) b200net::cuda::vmm_free(b->p, b->vmm_rounded, b->vmm_handle);
    else b200net::cuda::mem_free(b->p);
    b->vmm_rounded = 0;
    free(b->h);
  } else if (b->dev) {
    g_dev_free(b->p);
  } else {
    free(b->p);
  }
  b->p = b->h = nullptr;
}
static int buf_type() { return device_mode() ? NCCL_PTR_CUDA : NCCL_PTR_HOST; }
static int buf_type(const TestBuf& b) { return b.dev ? NCCL_PTR_CUDA : NCCL_PTR_HOST; }
