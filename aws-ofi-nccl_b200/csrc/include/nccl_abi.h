// NCCL plugin ABI in one header: the structures NCCL reads after dlsym() of
//   ncclNetPlugin_v6..v12, ncclTunerPlugin_v2/v3/v5/v6, ncclGinPlugin_v11/v13/v14, ncclRmaPlugin_v14/v15.
// Field order and types are fixed by NCCL (reference keeps per-version copies under
// 3rd-party/nccl/cuda/include/nccl/); everything here is plain C so a C program can include it.
#ifndef B200NET_NCCL_ABI_H_
#define B200NET_NCCL_ABI_H_

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- results, logging ------------------------------------------------------------------ */
typedef enum {
  ncclSuccess = 0, ncclUnhandledCudaError = 1, ncclSystemError = 2, ncclInternalError = 3,
  ncclInvalidArgument = 4, ncclInvalidUsage = 5, ncclRemoteError = 6
} ncclResult_t;

typedef enum { NCCL_LOG_NONE = 0, NCCL_LOG_VERSION = 1, NCCL_LOG_WARN = 2, NCCL_LOG_INFO = 3,
               NCCL_LOG_ABORT = 4, NCCL_LOG_TRACE = 5 } ncclDebugLogLevel;
typedef enum { NCCL_INIT = 1, NCCL_COLL = 2, NCCL_P2P = 4, NCCL_SHM = 8, NCCL_NET = 16, NCCL_GRAPH = 32,
               NCCL_TUNING = 64, NCCL_ENV = 128, NCCL_ALLOC = 256, NCCL_CALL = 512, NCCL_ALL = ~0 } ncclDebugLogSubSys;
typedef void (*ncclDebugLogger_t)(ncclDebugLogLevel level, unsigned long flags, const char* file, int line,
                                  const char* fmt, ...);
typedef ncclResult_t (*ncclProfilerCallback_t)(void** eHandle, int type, void* pHandle, int64_t pluginId, void* extData);

/* ---- element types / reductions (collnet + tuner signatures mention them) -------------- */
typedef enum { ncclInt8 = 0, ncclChar = 0, ncclUint8 = 1, ncclInt32 = 2, ncclInt = 2, ncclUint32 = 3, ncclInt64 = 4,
               ncclUint64 = 5, ncclFloat16 = 6, ncclHalf = 6, ncclFloat32 = 7, ncclFloat = 7, ncclFloat64 = 8,
               ncclDouble = 8, ncclBfloat16 = 9 } ncclDataType_t;
typedef enum { ncclSum = 0, ncclProd = 1, ncclMax = 2, ncclMin = 3, ncclAvg = 4, ncclNumOps = 5,
               ncclMaxRedOp = 0x7fffffff } ncclRedOp_t;

/* ---- net constants ------------------------------------------------------------------------ */
#define NCCL_NET_HANDLE_MAXSIZE 128
#define NCCL_NET_MAX_REQUESTS 32
#define NCCL_PTR_HOST 0x1
#define NCCL_PTR_CUDA 0x2
#define NCCL_PTR_DMABUF 0x4
#define NCCL_NET_OPTIONAL_RECV_COMPLETION 0x1
#define NCCL_NET_MULTI_REQUEST 0x2
#define NCCL_NET_MR_FLAG_FORCE_SO (1 << 0)
#define NCCL_NET_MR_FLAG_SIGNAL_NEVER_RESET (1 << 1)
#define NCCL_NET_SIGNAL_OP_INC 0x1
#define NCCL_NET_SIGNAL_OP_ADD 0x2
#define NCCL_NET_TRAFFIC_CLASS_UNDEF (-1)
#define NCCL_NET_ATTR_UNDEF (-1)
#define NCCL_GIN_MAX_CONNECTIONS 4

typedef enum {
  NCCL_NET_DEVICE_HOST = 0, NCCL_NET_DEVICE_UNPACK = 1, NCCL_NET_DEVICE_GIN_PROXY = 2,
  NCCL_NET_DEVICE_GIN_GDAKI = 3, NCCL_NET_DEVICE_GIN_GPI = 4, NCCL_NET_DEVICE_GIN_EFA_GDA = 5
} ncclNetDeviceType;
#define NCCL_NET_DEVICE_INVALID_VERSION 0x0

typedef struct {
  ncclNetDeviceType netDeviceType;
  int netDeviceVersion;
  void* handle;
  size_t size;
  int needsProxyProgress;
} ncclNetDeviceHandle_t;

/* ---- property structs, one per ABI generation ------------------------------------------- */
typedef struct { int ndevs; int devs[4]; } ncclNetVDeviceProps_v9_t;   /* v9, v10, v11 */
typedef struct { int ndevs; int devs[8]; } ncclNetVDeviceProps_v12_t;
typedef struct { int trafficClass; } ncclNetCommConfig_t;              /* v10, v11, v12 */

typedef struct {
  char* name; char* pciPath; uint64_t guid; int ptrSupport; int speed; int port; float latency;
  int maxComms; int maxRecvs;
} ncclNetProperties_v6_t;
typedef struct {
  char* name; char* pciPath; uint64_t guid; int ptrSupport; int speed; int port; float latency;
  int maxComms; int maxRecvs; ncclNetDeviceType netDeviceType; int netDeviceVersion;
} ncclNetProperties_v7_t;
typedef struct {
  char* name; char* pciPath; uint64_t guid; int ptrSupport; int regIsGlobal; int speed; int port; float latency;
  int maxComms; int maxRecvs; ncclNetDeviceType netDeviceType; int netDeviceVersion;
} ncclNetProperties_v8_t;
typedef struct {
  char* name; char* pciPath; uint64_t guid; int ptrSupport; int regIsGlobal; int forceFlush; int speed; int port;
  float latency; int maxComms; int maxRecvs; ncclNetDeviceType netDeviceType; int netDeviceVersion;
  ncclNetVDeviceProps_v9_t vProps; size_t maxP2pBytes; size_t maxCollBytes;
} ncclNetProperties_v9_t;
typedef ncclNetProperties_v9_t ncclNetProperties_v10_t;
typedef struct {
  char* name; char* pciPath; uint64_t guid; int ptrSupport; int regIsGlobal; int forceFlush; int speed; int port;
  float latency; int maxComms; int maxRecvs; ncclNetDeviceType netDeviceType; int netDeviceVersion;
  ncclNetVDeviceProps_v9_t vProps; size_t maxP2pBytes; size_t maxCollBytes; int maxMultiRequestSize;
} ncclNetProperties_v11_t;
typedef struct {
  char* name; char* pciPath; uint64_t guid; int ptrSupport; int regIsGlobal; int forceFlush; int speed; int port;
  float latency; int maxComms; int maxRecvs; ncclNetDeviceType netDeviceType; int netDeviceVersion;
  ncclNetVDeviceProps_v12_t vProps; size_t maxP2pBytes; size_t maxCollBytes; int maxMultiRequestSize;
  int16_t railId; int16_t planeId;
} ncclNetProperties_v12_t;

typedef struct { int32_t maxConcurrentPeers, minConcurrentPeers, maxFlowsPerPeer, minFlowsPerPeer; } ncclNetCommAttr_t;
typedef struct { ncclNetCommAttr_t sendCommAttr, recvCommAttr; uint32_t op, algo, proto; } ncclNetAttr_t;

/* ---- ncclNet function tables ---------------------------------------------------------------- */
#define B200NET_NET_COMMON_TAIL_V6                                                                              \
  ncclResult_t (*regMrDmaBuf)(void* comm, void* data, size_t size, int type, uint64_t offset, int fd, void** mhandle); \
  ncclResult_t (*deregMr)(void* comm, void* mhandle);

typedef struct {
  const char* name;
  ncclResult_t (*init)(ncclDebugLogger_t logFunction);
  ncclResult_t (*devices)(int* ndev);
  ncclResult_t (*getProperties)(int dev, ncclNetProperties_v6_t* props);
  ncclResult_t (*listen)(int dev, void* handle, void** listenComm);
  ncclResult_t (*connect)(int dev, void* handle, void** sendComm);
  ncclResult_t (*accept)(void* listenComm, void** recvComm);
  ncclResult_t (*regMr)(void* comm, void* data, int size, int type, void** mhandle);
  B200NET_NET_COMMON_TAIL_V6
  ncclResult_t (*isend)(void* sendComm, void* data, int size, int tag, void* mhandle, void** request);
  ncclResult_t (*irecv)(void* recvComm, int n, void** data, int* sizes, int* tags, void** mhandles, void** request);
  ncclResult_t (*iflush)(void* recvComm, int n, void** data, int* sizes, void** mhandles, void** request);
  ncclResult_t (*test)(void* request, int* done, int* sizes);
  ncclResult_t (*closeSend)(void* sendComm);
  ncclResult_t (*closeRecv)(void* recvComm);
  ncclResult_t (*closeListen)(void* listenComm);
} ncclNet_v6_t;

typedef struct {
  const char* name;
  ncclResult_t (*init)(ncclDebugLogger_t logFunction);
  ncclResult_t (*devices)(int* ndev);
  ncclResult_t (*getProperties)(int dev, ncclNetProperties_v7_t* props);
  ncclResult_t (*listen)(int dev, void* handle, void** listenComm);
  ncclResult_t (*connect)(int dev, void* handle, void** sendComm, ncclNetDeviceHandle_t** sendDevComm);
  ncclResult_t (*accept)(void* listenComm, void** recvComm, ncclNetDeviceHandle_t** recvDevComm);
  ncclResult_t (*regMr)(void* comm, void* data, int size, int type, void** mhandle);
  B200NET_NET_COMMON_TAIL_V6
  ncclResult_t (*isend)(void* sendComm, void* data, int size, int tag, void* mhandle, void** request);
  ncclResult_t (*irecv)(void* recvComm, int n, void** data, int* sizes, int* tags, void** mhandles, void** request);
  ncclResult_t (*iflush)(void* recvComm, int n, void** data, int* sizes, void** mhandles, void** request);
  ncclResult_t (*test)(void* request, int* done, int* sizes);
  ncclResult_t (*closeSend)(void* sendComm);
  ncclResult_t (*closeRecv)(void* recvComm);
  ncclResult_t (*closeListen)(void* listenComm);
  ncclResult_t (*getDeviceMr)(void* comm, void* mhandle, void** dptr_mhandle);
  ncclResult_t (*irecvConsumed)(void* recvComm, int n, void* request);
} ncclNet_v7_t;

typedef struct {
  const char* name;
  ncclResult_t (*init)(ncclDebugLogger_t logFunction);
  ncclResult_t (*devices)(int* ndev);
  ncclResult_t (*getProperties)(int dev, ncclNetProperties_v8_t* props);
  ncclResult_t (*listen)(int dev, void* handle, void** listenComm);
  ncclResult_t (*connect)(int dev, void* handle, void** sendComm, ncclNetDeviceHandle_t** sendDevComm);
  ncclResult_t (*accept)(void* listenComm, void** recvComm, ncclNetDeviceHandle_t** recvDevComm);
  ncclResult_t (*regMr)(void* comm, void* data, size_t size, int type, void** mhandle);
  B200NET_NET_COMMON_TAIL_V6
  ncclResult_t (*isend)(void* sendComm, void* data, int size, int tag, void* mhandle, void** request);
  ncclResult_t (*irecv)(void* recvComm, int n, void** data, int* sizes, int* tags, void** mhandles, void** request);
  ncclResult_t (*iflush)(void* recvComm, int n, void** data, int* sizes, void** mhandles, void** request);
  ncclResult_t (*test)(void* request, int* done, int* sizes);
  ncclResult_t (*closeSend)(void* sendComm);
  ncclResult_t (*closeRecv)(void* recvComm);
  ncclResult_t (*closeListen)(void* listenComm);
  ncclResult_t (*getDeviceMr)(void* comm, void* mhandle, void** dptr_mhandle);
  ncclResult_t (*irecvConsumed)(void* recvComm, int n, void* request);
} ncclNet_v8_t;

typedef struct {
  const char* name;
  ncclResult_t (*init)(ncclDebugLogger_t logFunction);
  ncclResult_t (*devices)(int* ndev);
  ncclResult_t (*getProperties)(int dev, ncclNetProperties_v9_t* props);
  ncclResult_t (*listen)(int dev, void* handle, void** listenComm);
  ncclResult_t (*connect)(int dev, void* handle, void** sendComm, ncclNetDeviceHandle_t** sendDevComm);
  ncclResult_t (*accept)(void* listenComm, void** recvComm, ncclNetDeviceHandle_t** recvDevComm);
  ncclResult_t (*regMr)(void* comm, void* data, size_t size, int type, void** mhandle);
  B200NET_NET_COMMON_TAIL_V6
  ncclResult_t (*isend)(void* sendComm, void* data, size_t size, int tag, void* mhandle, void** request);
  ncclResult_t (*irecv)(void* recvComm, int n, void** data, size_t* sizes, int* tags, void** mhandles, void** request);
  ncclResult_t (*iflush)(void* recvComm, int n, void** data, int* sizes, void** mhandles, void** request);
  ncclResult_t (*test)(void* request, int* done, int* sizes);
  ncclResult_t (*closeSend)(void* sendComm);
  ncclResult_t (*closeRecv)(void* recvComm);
  ncclResult_t (*closeListen)(void* listenComm);
  ncclResult_t (*getDeviceMr)(void* comm, void* mhandle, void** dptr_mhandle);
  ncclResult_t (*irecvConsumed)(void* recvComm, int n, void* request);
  ncclResult_t (*makeVDevice)(int* d, ncclNetVDeviceProps_v9_t* props);
} ncclNet_v9_t;

typedef struct {
  const char* name;
  ncclResult_t (*init)(ncclDebugLogger_t logFunction, ncclProfilerCallback_t profFunction);
  ncclResult_t (*devices)(int* ndev);
  ncclResult_t (*getProperties)(int dev, ncclNetProperties_v10_t* props);
  ncclResult_t (*listen)(int dev, void* handle, void** listenComm);
  ncclResult_t (*connect)(int dev, ncclNetCommConfig_t* config, void* handle, void** sendComm,
                          ncclNetDeviceHandle_t** sendDevComm);
  ncclResult_t (*accept)(void* listenComm, void** recvComm, ncclNetDeviceHandle_t** recvDevComm);
  ncclResult_t (*regMr)(void* comm, void* data, size_t size, int type, void** mhandle);
  B200NET_NET_COMMON_TAIL_V6
  ncclResult_t (*isend)(void* sendComm, void* data, size_t size, int tag, void* mhandle, void* phandle, void** request);
  ncclResult_t (*irecv)(void* recvComm, int n, void** data, size_t* sizes, int* tags, void** mhandles, void** phandles,
                        void** request);
  ncclResult_t (*iflush)(void* recvComm, int n, void** data, int* sizes, void** mhandles, void** request);
  ncclResult_t (*test)(void* request, int* done, int* sizes);
  ncclResult_t (*closeSend)(void* sendComm);
  ncclResult_t (*closeRecv)(void* recvComm);
  ncclResult_t (*closeListen)(void* listenComm);
  ncclResult_t (*getDeviceMr)(void* comm, void* mhandle, void** dptr_mhandle);
  ncclResult_t (*irecvConsumed)(void* recvComm, int n, void* request);
  ncclResult_t (*makeVDevice)(int* d, ncclNetVDeviceProps_v9_t* props);
} ncclNet_v10_t;

#define B200NET_NET_V11_BODY(PROPS_T, VPROPS_T)                                                                          \
  const char* name;                                                                                                      \
  ncclResult_t (*init)(void** ctx, uint64_t commId, ncclNetCommConfig_t* config, ncclDebugLogger_t logFunction,          \
                       ncclProfilerCallback_t profFunction);                                                             \
  ncclResult_t (*devices)(int* ndev);                                                                                    \
  ncclResult_t (*getProperties)(int dev, PROPS_T* props);                                                                \
  ncclResult_t (*listen)(void* ctx, int dev, void* handle, void** listenComm);                                           \
  ncclResult_t (*connect)(void* ctx, int dev, void* handle, void** sendComm, ncclNetDeviceHandle_t** sendDevComm);       \
  ncclResult_t (*accept)(void* listenComm, void** recvComm, ncclNetDeviceHandle_t** recvDevComm);                        \
  ncclResult_t (*regMr)(void* comm, void* data, size_t size, int type, void** mhandle);                                  \
  B200NET_NET_COMMON_TAIL_V6                                                                                             \
  ncclResult_t (*isend)(void* sendComm, void* data, size_t size, int tag, void* mhandle, void* phandle, void** request); \
  ncclResult_t (*irecv)(void* recvComm, int n, void** data, size_t* sizes, int* tags, void** mhandles, void** phandles,  \
                        void** request);                                                                                 \
  ncclResult_t (*iflush)(void* recvComm, int n, void** data, int* sizes, void** mhandles, void** request);               \
  ncclResult_t (*test)(void* request, int* done, int* sizes);                                                            \
  ncclResult_t (*closeSend)(void* sendComm);                                                                             \
  ncclResult_t (*closeRecv)(void* recvComm);                                                                             \
  ncclResult_t (*closeListen)(void* listenComm);                                                                         \
  ncclResult_t (*getDeviceMr)(void* comm, void* mhandle, void** dptr_mhandle);                                           \
  ncclResult_t (*irecvConsumed)(void* recvComm, int n, void* request);                                                   \
  ncclResult_t (*makeVDevice)(int* d, VPROPS_T* props);                                                                  \
  ncclResult_t (*finalize)(void* ctx);                                                                                   \
  ncclResult_t (*setNetAttr)(void* ctx, ncclNetAttr_t* netAttr);

typedef struct { B200NET_NET_V11_BODY(ncclNetProperties_v11_t, ncclNetVDeviceProps_v9_t) } ncclNet_v11_t;
typedef struct { B200NET_NET_V11_BODY(ncclNetProperties_v12_t, ncclNetVDeviceProps_v12_t) } ncclNet_v12_t;

/* ---- GIN (GPU-initiated networking) ---------------------------------------------------------- */
typedef struct { int nSignals, nCounters, nContexts, queueDepth, trafficClass; } ncclGinConfig_v13_t;
typedef struct { int nSignals, nCounters, nContexts, queueDepth, trafficClass, backendVersion, rankStride; } ncclGinConfig_v14_t;
typedef struct { bool supportsStrongSignals; bool supportsVASignals; } ncclGinProperties_v14_t;

#define B200NET_GIN_MR_FNS                                                                                                \
  ncclResult_t (*regMrSym)(void* collComm, void* data, size_t size, int type, uint64_t mrFlags, void** mhandle,          \
                           void** ginHandle);                                                                            \
  ncclResult_t (*regMrSymDmaBuf)(void* collComm, void* data, size_t size, int type, uint64_t offset, int fd,             \
                                 uint64_t mrFlags, void** mhandle, void** ginHandle);                                    \
  ncclResult_t (*deregMrSym)(void* collComm, void* mhandle);                                                             \
  ncclResult_t (*destroyContext)(void* ginCtx);                                                                          \
  ncclResult_t (*closeColl)(void* collComm);                                                                             \
  ncclResult_t (*closeListen)(void* listenComm);

typedef struct {
  const char* name;
  ncclResult_t (*init)(void** ctx, uint64_t commId, ncclDebugLogger_t logFunction);
  ncclResult_t (*devices)(int* ndev);
  ncclResult_t (*getProperties)(int dev, ncclNetProperties_v11_t* props);
  ncclResult_t (*listen)(void* ctx, int dev, void* handle, void** listenComm);
  ncclResult_t (*connect)(void* ctx, void* handles[], int nranks, int rank, void* listenComm, void** collComm);
  ncclResult_t (*createContext)(void* collComm, int nSignals, int nCounters, void** ginCtx,
                                ncclNetDeviceHandle_t** devHandle);
  B200NET_GIN_MR_FNS
  ncclResult_t (*iput)(void* collComm, uint64_t srcOff, void* srcMhandle, size_t size, uint64_t dstOff,
                       void* dstMhandle, uint32_t rank, void** request);
  ncclResult_t (*iputSignal)(void* collComm, uint64_t srcOff, void* srcMhandle, size_t size, uint64_t dstOff,
                             void* dstMhandle, uint32_t rank, uint64_t signalOff, void* signalMhandle,
                             uint64_t signalValue, uint32_t signalOp, void** request);
  ncclResult_t (*test)(void* collComm, void* request, int* done);
  ncclResult_t (*ginProgress)(void* collComm);
  ncclResult_t (*queryLastError)(void* ginCtx, bool* hasError);
  ncclResult_t (*finalize)(void* ctx);
} ncclGin_v11_t;

typedef struct {
  const char* name;
  ncclResult_t (*init)(void** ctx, uint64_t commId, ncclDebugLogger_t logFunction);
  ncclResult_t (*devices)(int* ndev);
  ncclResult_t (*getProperties)(int dev, ncclNetProperties_v12_t* props);
  ncclResult_t (*listen)(void* ctx, int dev, void* handle, void** listenComm);
  ncclResult_t (*connect)(void* ctx, void* handles[], int nranks, int rank, void* listenComm, void** collComm);
  ncclResult_t (*createContext)(void* collComm, ncclGinConfig_v13_t* config, void** ginCtx,
                                ncclNetDeviceHandle_t** devHandle);
  B200NET_GIN_MR_FNS
  ncclResult_t (*iput)(void* ginCtx, int context, uint64_t srcOff, void* srcMhandle, size_t size, uint64_t dstOff,
                       void* dstMhandle, uint32_t rank, void** request);
  ncclResult_t (*iputSignal)(void* ginCtx, int context, uint64_t srcOff, void* srcMhandle, size_t size,
                             uint64_t dstOff, void* dstMhandle, uint32_t rank, uint64_t signalOff,
                             void* signalMhandle, uint64_t signalValue, uint32_t signalOp, void** request);
  ncclResult_t (*iget)(void* ginCtx, int context, uint64_t remoteOff, void* remoteMhandle, size_t size,
                       uint64_t localOff, void* localMhandle, uint32_t rank, void** request);
  ncclResult_t (*iflush)(void* ginCtx, int context, void* mhandle, uint32_t rank, void** request);
  ncclResult_t (*test)(void* collComm, void* request, int* done);
  ncclResult_t (*ginProgress)(void* ginCtx);
  ncclResult_t (*queryLastError)(void* ginCtx, bool* hasError);
  ncclResult_t (*finalize)(void* ctx);
} ncclGin_v13_t;

typedef struct {
  const char* name;
  ncclResult_t (*init)(void** ctx, uint64_t commId, ncclDebugLogger_t logFunction);
  ncclResult_t (*devices)(int* ndev);
  ncclResult_t (*getGinProperties)(ncclGinProperties_v14_t* ginProps);
  ncclResult_t (*getProperties)(int dev, ncclNetProperties_v12_t* props);
  ncclResult_t (*listen)(void* ctx, int dev, void* handle, void** listenComm);
  ncclResult_t (*connect)(void* ctx, void* handles[], int nranks, int rank, void* listenComm, void** collComm);
  ncclResult_t (*createContext)(void* collComm, ncclGinConfig_v14_t* config, void** ginCtx,
                                ncclNetDeviceHandle_t** devHandle);
  B200NET_GIN_MR_FNS
  ncclResult_t (*ginProgress)(void* ginCtx);
  ncclResult_t (*queryLastError)(void* ginCtx, bool* hasError);
  ncclResult_t (*finalize)(void* ctx);
} ncclGin_v14_t;

/* ---- RMA (host-initiated put/get/signal) ------------------------------------------------------ */
typedef struct { int nContexts, trafficClass, rankStride; } ncclRmaConfig_t;
enum ncclRmaOptFlags { ncclRmaOptFlagsDefault = 0, ncclRmaOptFlagsAggregateRequests = (1 << 0) };

#define B200NET_RMA_HEAD                                                                                                  \
  const char* name;                                                                                                      \
  ncclResult_t (*init)(void** ctx, uint64_t commId, ncclDebugLogger_t logFunction);                                      \
  ncclResult_t (*devices)(int* ndev);                                                                                    \
  ncclResult_t (*getProperties)(int dev, ncclNetProperties_v12_t* props);                                                \
  ncclResult_t (*listen)(void* ctx, int dev, void* handle, void** listenComm);                                           \
  ncclResult_t (*connect)(void* ctx, void* handles[], int nranks, int rank, void* listenComm, void** collComm);          \
  ncclResult_t (*createContext)(void* collComm, ncclRmaConfig_t* config, void** rmaCtx);                                 \
  ncclResult_t (*regMrSym)(void* collComm, void* data, size_t size, int type, uint64_t mrFlags, void** mhandle);         \
  ncclResult_t (*regMrSymDmaBuf)(void* collComm, void* data, size_t size, int type, uint64_t offset, int fd,             \
                                 uint64_t mrFlags, void** mhandle);                                                      \
  ncclResult_t (*deregMrSym)(void* collComm, void* mhandle);                                                             \
  ncclResult_t (*destroyContext)(void* rmaCtx);                                                                          \
  ncclResult_t (*closeColl)(void* collComm);                                                                             \
  ncclResult_t (*closeListen)(void* listenComm);
#define B200NET_RMA_TAIL                                                                                                  \
  ncclResult_t (*iflush)(void* rmaCtx, int context, void* mhandle, uint32_t rank, void** request);                       \
  ncclResult_t (*test)(void* collComm, void* request, int* done);                                                        \
  ncclResult_t (*rmaProgress)(void* rmaCtx);                                                                             \
  ncclResult_t (*queryLastError)(void* rmaCtx, bool* hasError);                                                          \
  ncclResult_t (*finalize)(void* ctx);

typedef struct {
  B200NET_RMA_HEAD
  ncclResult_t (*iput)(void* rmaCtx, int context, uint64_t srcOff, void* srcMhandle, size_t size, uint64_t dstOff,
                       void* dstMhandle, uint32_t rank, void** request);
  ncclResult_t (*iputSignal)(void* rmaCtx, int context, uint64_t srcOff, void* srcMhandle, size_t size,
                             uint64_t dstOff, void* dstMhandle, uint32_t rank, uint64_t signalOff,
                             void* signalMhandle, uint64_t signalValue, uint32_t signalOp, bool isStrongSignal,
                             void** request);
  ncclResult_t (*iget)(void* rmaCtx, int context, uint64_t remoteOff, void* remoteMhandle, size_t size,
                       uint64_t localOff, void* localMhandle, uint32_t rank, void** request);
  B200NET_RMA_TAIL
} ncclRma_v14_t;

typedef struct {
  B200NET_RMA_HEAD
  ncclResult_t (*iput)(void* rmaCtx, int context, uint64_t srcOff, void* srcMhandle, size_t size, uint64_t dstOff,
                       void* dstMhandle, uint32_t rank, uint32_t optFlags, void** request);
  ncclResult_t (*iputSignal)(void* rmaCtx, int context, uint64_t srcOff, void* srcMhandle, size_t size,
                             uint64_t dstOff, void* dstMhandle, uint32_t rank, uint64_t signalOff,
                             void* signalMhandle, uint64_t signalValue, uint32_t signalOp, bool isStrongSignal,
                             uint32_t optFlags, void** request);
  ncclResult_t (*iget)(void* rmaCtx, int context, uint64_t remoteOff, void* remoteMhandle, size_t size,
                       uint64_t localOff, void* localMhandle, uint32_t rank, uint32_t optFlags, void** request);
  B200NET_RMA_TAIL
} ncclRma_v15_t;

/* ---- tuner ----------------------------------------------------------------------------------- */
typedef enum { ncclFuncBroadcast = 0, ncclFuncReduce = 1, ncclFuncAllGather = 2, ncclFuncReduceScatter = 3,
               ncclFuncAllReduce = 4, ncclFuncSendRecv = 5, ncclFuncSend = 6, ncclFuncRecv = 7, ncclNumFuncs = 8 } ncclFunc_t;
#define NCCL_NUM_FUNCTIONS 5
#define NCCL_NUM_ALGORITHMS 7
#define NCCL_ALGO_UNDEF (-1)
#define NCCL_ALGO_TREE 0
#define NCCL_ALGO_RING 1
#define NCCL_ALGO_COLLNET_DIRECT 2
#define NCCL_ALGO_COLLNET_CHAIN 3
#define NCCL_ALGO_NVLS 4
#define NCCL_ALGO_NVLS_TREE 5
#define NCCL_ALGO_PAT 6
#define NCCL_NUM_PROTOCOLS 3
#define NCCL_PROTO_UNDEF (-1)
#define NCCL_PROTO_LL 0
#define NCCL_PROTO_LL128 1
#define NCCL_PROTO_SIMPLE 2
#define NCCL_ALGO_PROTO_IGNORE (-1.0f)

typedef struct { int nNvlDomains, minRanksPerNvlDomain, maxRanksPerNvlDomain; } ncclNvlDomainInfo_t;
typedef struct {
  double baseLatencies[7][3];
  double hwLatencies[3][7][3];
  double llMaxBws[4][3];
  double perChMaxRingLL128Bws[4][3];
  double perChMaxTreeLL128Bws[4][3];
  double perChMaxTreeBws[4][3];
  double perChMaxNVLSTreeBws[4][3];
} ncclTunerConstants_t;

typedef struct {
  const char* name;
  ncclResult_t (*init)(size_t nRanks, size_t nNodes, ncclDebugLogger_t logFunction, void** context);
  ncclResult_t (*getCollInfo)(void* context, ncclFunc_t collType, size_t nBytes, int collNetSupport, int nvlsSupport,
                              int numPipeOps, int* algorithm, int* protocol, int* nChannels);
  ncclResult_t (*destroy)(void* context);
} ncclTuner_v2_t;
typedef struct {
  const char* name;
  ncclResult_t (*init)(size_t nRanks, size_t nNodes, ncclDebugLogger_t logFunction, void** context);
  ncclResult_t (*getCollInfo)(void* context, ncclFunc_t collType, size_t nBytes, int numPipeOps, float** collCostTable,
                              int numAlgo, int numProto, int* nChannels);
  ncclResult_t (*destroy)(void* context);
} ncclTuner_v3_t;
typedef struct {
  const char* name;
  ncclResult_t (*init)(size_t nRanks, size_t nNodes, ncclDebugLogger_t logFunction, void** context);
  ncclResult_t (*getCollInfo)(void* context, ncclFunc_t collType, size_t nBytes, int numPipeOps, float** collCostTable,
                              int numAlgo, int numProto, int regBuff, int* nChannels);
  ncclResult_t (*destroy)(void* context);
} ncclTuner_v4_t;
typedef struct {
  const char* name;
  ncclResult_t (*init)(void** ctx, uint64_t commId, size_t nRanks, size_t nNodes, ncclDebugLogger_t logFunction,
                       ncclNvlDomainInfo_t* nvlDomainInfo, ncclTunerConstants_t* constants);
  ncclResult_t (*getCollInfo)(void* context, ncclFunc_t collType, size_t nBytes, int numPipeOps, float** collCostTable,
                              int numAlgo, int numProto, int regBuff, int* nChannels);
  ncclResult_t (*finalize)(void* context);
} ncclTuner_v5_t;
typedef struct {
  const char* name;
  ncclResult_t (*init)(void** ctx, uint64_t commId, size_t nRanks, size_t nNodes, ncclDebugLogger_t logFunction,
                       ncclNvlDomainInfo_t* nvlDomainInfo, ncclTunerConstants_t* constants);
  ncclResult_t (*getCollInfo)(void* context, ncclFunc_t collType, size_t nBytes, int numPipeOps, float** collCostTable,
                              int numAlgo, int numProto, int regBuff, int* nChannels);
  ncclResult_t (*finalize)(void* context);
  ncclResult_t (*getChunkSize)(void* context, ncclFunc_t collType, size_t nBytes, int algo, int proto, int nChannels,
                               size_t* chunkSize);
} ncclTuner_v6_t;

#ifdef __cplusplus
}
#endif
#endif /* B200NET_NCCL_ABI_H_ */
