// The helper thread that opens peers' device allocations, against the stand-in driver (run with it
// on the library path): a mapping that arrives within the wait is handed to the caller, who closes
// it; one that is abandoned while the open is still running is closed by the helper itself, so no
// mapping outlives its owner either way; a handle that cannot be opened reports an error.
#include <dlfcn.h>
#include <unistd.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <thread>

#include "b200net/cuda_shim.h"
#include "b200net/ipc_mapper.h"
#include "test_util.h"
using namespace b200net;

int main() {
  if (!cuda::available()) {
    fprintf(stderr, "no driver on the library path: nothing to test\n");
    return 0;
  }
  void* drv = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
  auto live = drv ? reinterpret_cast<int (*)()>(dlsym(drv, "fake_cuda_live_peer_mappings")) : nullptr;
  if (!live) {
    fprintf(stderr, "a real driver is loaded: this test needs the stand-in\n");
    return 0;
  }
  CHECK_EQ(cuda::ensure_primary_ctx(0), 0);
  cuda::Context ctx = nullptr;
  CHECK_EQ(cuda::ctx_get_current(&ctx), 0);
  void* mem = nullptr;
  CHECK_EQ(cuda::mem_alloc(&mem, 1 << 16), 0);
  uint8_t handle[64];
  CHECK_EQ(cuda::ipc_get_handle(mem, handle), 0);

  // 1. the open finishes within the wait: state 1, the owner closes
  auto job = IpcMapper::instance().submit(handle, ctx);
  CHECK(job != nullptr);
  CHECK_EQ(IpcMapper::wait(*job, 2000000), 1);
  CHECK(job->mapped != nullptr);
  CHECK_EQ(live(), 1);
  CHECK(job->abandon());            // mapped: the caller has to close it
  CHECK_EQ(cuda::ipc_close(job->mapped), 0);
  CHECK_EQ(live(), 0);

  // 2. a slow open, abandoned while it runs: the helper closes the mapping when it arrives
  setenv("FAKE_CUDA_IPC_OPEN_DELAY_MS", "200", 1);
  job = IpcMapper::instance().submit(handle, ctx);
  CHECK_EQ(IpcMapper::wait(*job, 1000), 0);   // still running after a millisecond
  CHECK(!job->abandon());                      // nothing for the caller to close
  for (int i = 0; i < 300 && job->state.load() == 2 && live() == 0; ++i) std::this_thread::sleep_for(std::chrono::milliseconds(2));
  std::this_thread::sleep_for(std::chrono::milliseconds(400));
  CHECK_EQ(live(), 0);                          // opened, seen as abandoned, closed again
  CHECK_EQ(job->state.load(), 2);

  // 3. a slow open that the owner waits out in a second wait
  job = IpcMapper::instance().submit(handle, ctx);
  CHECK_EQ(IpcMapper::wait(*job, 1000), 0);
  CHECK_EQ(IpcMapper::wait(*job, 2000000), 1);
  CHECK(job->abandon());
  CHECK_EQ(cuda::ipc_close(job->mapped), 0);
  unsetenv("FAKE_CUDA_IPC_OPEN_DELAY_MS");

  // 4. a handle that names nothing: negative state, nothing mapped
  uint8_t bogus[64];
  memset(bogus, 0x5A, sizeof(bogus));
  job = IpcMapper::instance().submit(bogus, ctx);
  CHECK(IpcMapper::wait(*job, 2000000) < 0);
  CHECK(!job->abandon());
  CHECK_EQ(live(), 0);

  CHECK_EQ(cuda::mem_free(mem), 0);
  printf("ok\n");
  return 0;
}
