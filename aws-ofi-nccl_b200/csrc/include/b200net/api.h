// Validated C-level API under the ABI tables: argument checks, errno -> ncclResult_t mapping,
// exception containment, per-thread endpoint lookup (reference: src/nccl_ofi_api.cpp,
// include/nccl_ofi_api.h:30-75).
#pragma once
#include <cerrno>

#include "b200net/net.h"
#include "nccl_abi.h"

namespace b200net::api {

inline ncclResult_t to_nccl(int rc) {
  if (rc >= 0) return ncclSuccess;
  switch (-rc) {
    case EINVAL: case EMSGSIZE: return ncclInvalidArgument;
    case ENOTSUP: case EPROTO: return ncclInvalidUsage;
    case ENOMEM: case ENOSPC: case EIO: case EFAULT: return ncclSystemError;
    case ENOTCONN: case ECONNABORTED: case EHOSTUNREACH: case ETIMEDOUT: case ECONNRESET: return ncclRemoteError;
    default: return ncclSystemError;
  }
}

ncclResult_t init(ncclDebugLogger_t log_fn);
ncclResult_t fini();
ncclResult_t devices(int* ndev);
ncclResult_t get_properties(int dev, Properties* props);
ncclResult_t listen(int dev, void* handle, void** lcomm);
ncclResult_t connect(int dev, void* handle, void** scomm, int traffic_class);
ncclResult_t accept(void* lcomm, void** rcomm);
ncclResult_t reg_mr(void* comm, void* data, size_t size, int type, void** mhandle);
ncclResult_t reg_mr_dmabuf(void* comm, void* data, size_t size, int type, uint64_t offset, int fd, void** mhandle);
ncclResult_t dereg_mr(void* comm, void* mhandle);
ncclResult_t isend(void* scomm, void* data, size_t size, int tag, void* mhandle, void** request);
ncclResult_t irecv(void* rcomm, int n, void** data, size_t* sizes, int* tags, void** mhandles, void** request,
                   bool optional_completion = false);
ncclResult_t iflush(void* rcomm, int n, void** data, int* sizes, void** mhandles, void** request);
ncclResult_t test(void* request, int* done, int* sizes);
ncclResult_t close_send(void* scomm);
ncclResult_t close_recv(void* rcomm);
ncclResult_t close_listen(void* lcomm);

}  // namespace b200net::api
