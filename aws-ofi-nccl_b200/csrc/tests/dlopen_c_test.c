/* A plain C program must be able to dlopen() the plugin and find its tables: no unresolved C++
 * runtime symbols, C-compatible ABI header (reference: tests/unit/dlopen_c_test.c). */
#include <dlfcn.h>
#include <stdio.h>
#include <string.h>

#include "../include/nccl_abi.h"

int main(int argc, char** argv) {
  const char* so = argc > 1 ? argv[1] : "./libnccl-net-ofi-b200.so";
  void* h = dlopen(so, RTLD_NOW | RTLD_LOCAL);
  if (!h) {
    fprintf(stderr, "dlopen failed: %s\n", dlerror());
    return 1;
  }
  const char* syms[] = {"ncclNetPlugin_v6", "ncclNetPlugin_v7", "ncclNetPlugin_v8", "ncclNetPlugin_v9",
                        "ncclNetPlugin_v10", "ncclNetPlugin_v11", "ncclNetPlugin_v12"};
  for (unsigned i = 0; i < sizeof(syms) / sizeof(syms[0]); ++i) {
    if (!dlsym(h, syms[i])) {
      fprintf(stderr, "missing symbol %s\n", syms[i]);
      return 1;
    }
  }
  ncclNet_v11_t* net = (ncclNet_v11_t*)dlsym(h, "ncclNetPlugin_v11");
  if (!net->name || !net->init || !net->devices || !net->isend || !net->irecv || !net->test || !net->finalize) {
    fprintf(stderr, "incomplete table\n");
    return 1;
  }
  printf("ok %s\n", net->name);
  dlclose(h);
  return 0;
}
