// Buffers for the functional tests: host memory, or, with FUNC_NET_DEVICE=1, "device" memory.
// Included after the test has defined g_rank.
#pragma once
#include <dlfcn.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include "nccl_abi.h"

// "Device" buffers for CPU runs: with FUNC_NET_DEVICE=1 and the stand-in driver on the library
// path (it serves device memory out of POSIX shared memory), buffers come from the driver and are
// registered as NCCL_PTR_CUDA, so the plugin's IPC mapping, copy-kernel and eager-pack paths run.
// The address handed to the plugin is not accessible to host code (a stray dereference faults);
// the test fills and checks the bytes through host().
struct TestBuf {
  uint8_t* p = nullptr;   // the address given to the plugin
  uint8_t* h = nullptr;   // where the test itself reads and writes the same bytes
  size_t n = 0;
  bool dev = false;
  uint8_t* data() { return p; }
  uint8_t* host() { return h; }
  size_t size() const { return n; }
};
using FakeAllocFn = int (*)(void**, size_t);
using FakeFreeFn = int (*)(void*);
using FakeViewFn = void* (*)(void*);
static FakeViewFn g_dev_view = nullptr;
static FakeAllocFn g_dev_alloc = nullptr;
static FakeFreeFn g_dev_free = nullptr;
static bool device_mode() {
  static int mode = -1;
  if (mode < 0) {
    mode = 0;
    if (getenv("FUNC_NET_DEVICE") && atoi(getenv("FUNC_NET_DEVICE"))) {
      void* h = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
      if (h) {
        g_dev_alloc = reinterpret_cast<FakeAllocFn>(dlsym(h, "fake_cuda_mem_alloc"));
        g_dev_free = reinterpret_cast<FakeFreeFn>(dlsym(h, "fake_cuda_mem_free"));
        g_dev_view = reinterpret_cast<FakeViewFn>(dlsym(h, "fake_cuda_host_view"));
      }
      mode = (g_dev_alloc && g_dev_free && g_dev_view) ? 1 : 0;
      if (!mode) fprintf(stderr, "[rank %d] FUNC_NET_DEVICE set but the stand-in driver is not on the library path\n", g_rank);
    }
  }
  return mode == 1;
}
static int buf_alloc(TestBuf* b, size_t n, bool want_device = true) {
  b->n = n;
  b->dev = want_device && device_mode();
  if (b->dev) {
    void* p = nullptr;
    if (g_dev_alloc(&p, n) != 0) return 1;
    b->p = static_cast<uint8_t*>(p);
    b->h = static_cast<uint8_t*>(g_dev_view(p));
  } else {
    b->p = b->h = static_cast<uint8_t*>(malloc(n));
  }
  return b->p ? 0 : 1;
}
static void buf_free(TestBuf* b) {
  if (!b->p) return;
  if (b->dev) g_dev_free(b->p);
  else free(b->p);
  b->p = nullptr;
}
static int buf_type() { return device_mode() ? NCCL_PTR_CUDA : NCCL_PTR_HOST; }
static int buf_type(const TestBuf& b) { return b.dev ? NCCL_PTR_CUDA : NCCL_PTR_HOST; }
