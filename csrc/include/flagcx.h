/*
 * flagcx.h -- public C interface of the B200-native FlagCX-compatible
 * collective library.
 *
 * Symbol names, enumerator values and struct sizes follow the FlagCX 0.13
 * public header (flagcx/include/flagcx.h in the FlagCX project) so that a
 * program written against FlagCX links against this library unchanged.
 * Everything behind the symbols is a different design: one process per GPU,
 * a CUDA-VMM symmetric heap mapped into every local peer, and collectives
 * that are single sm_100a kernels reading and writing peer memory over
 * NVLink.  Host buffers (or a host without a GPU) take the TCP socket path.
 */
#ifndef FLAGCX_H_
#define FLAGCX_H_

#include <stddef.h>
#include <stdint.h>

#define FLAGCX_VERSION_MAJOR 0
#define FLAGCX_VERSION_MINOR 13
#define FLAGCX_VERSION_PATCH 0
#define FLAGCX_VERSION_CODE                                                    \
  (FLAGCX_VERSION_MAJOR * 10000 + FLAGCX_VERSION_MINOR * 100 +                 \
   FLAGCX_VERSION_PATCH)

#ifdef __cplusplus
extern "C" {
#endif

/* ---- result codes ------------------------------------------------------ */
typedef enum {
  flagcxSuccess = 0,
  flagcxUnhandledDeviceError = 1,
  flagcxSystemError = 2,
  flagcxInternalError = 3,
  flagcxInvalidArgument = 4,
  flagcxInvalidUsage = 5,
  flagcxRemoteError = 6,
  flagcxInProgress = 7,
  flagcxUnhandledCCLError = 8,
  flagcxNotSupported = 9,
  flagcxNumResults = 10
} flagcxResult_t;

/* ---- element types ----------------------------------------------------- */
typedef enum {
  flagcxInt8 = 0,
  flagcxChar = 0,
  flagcxUint8 = 1,
  flagcxInt32 = 2,
  flagcxInt = 2,
  flagcxUint32 = 3,
  flagcxInt64 = 4,
  flagcxUint64 = 5,
  flagcxFloat16 = 6,
  flagcxHalf = 6,
  flagcxFloat32 = 7,
  flagcxFloat = 7,
  flagcxFloat64 = 8,
  flagcxDouble = 8,
  flagcxBfloat16 = 9,
  flagcxNumTypes = 10
} flagcxDataType_t;

/* ---- reductions -------------------------------------------------------- */
typedef enum { flagcxNumRedOps_dummy = 5 } flagcxRedOp_dummy_t;
typedef enum {
  flagcxSum = 0,
  flagcxProd = 1,
  flagcxMax = 2,
  flagcxMin = 3,
  flagcxAvg = 4,
  flagcxRedNoOp = 5,
  flagcxNumRedOps = 5,
  flagcxMaxRedOp = 0x7fffffff >> (32 - 8 * sizeof(flagcxRedOp_dummy_t))
} flagcxRedOp_t;

/* Size in bytes of one element of `dtype` (0 for an unknown type). */
size_t getFlagcxDataTypeSize(flagcxDataType_t dtype);

/* ---- operation tags (used by the tuner and by statistics) --------------- */
typedef enum {
  flagcxCommOpSend = 0,
  flagcxCommOpRecv = 1,
  flagcxCommOpBroadcast = 2,
  flagcxCommOpGather = 3,
  flagcxCommOpScatter = 4,
  flagcxCommOpReduce = 5,
  flagcxCommOpAllReduce = 6,
  flagcxCommOpAllGather = 7,
  flagcxCommOpReduceScatter = 8,
  flagcxCommOpAlltoAll = 9,
  flagcxCommOpAlltoAllv = 10,
  flagcxCommNoOp = 11,
  flagcxNumCommOps = 12
} flagcxCommOp_t;

typedef enum {
  flagcxMemcpyHostToDevice = 0,
  flagcxMemcpyDeviceToHost = 1,
  flagcxMemcpyDeviceToDevice = 2
} flagcxMemcpyType_t;

typedef enum {
  flagcxMemHost = 0, /* pinned host memory */
  flagcxMemDevice = 1,
  flagcxMemManaged = 2
} flagcxMemType_t;

typedef enum {
  flagcxEventDefault = 0,
  flagcxEventDisableTiming = 1
} flagcxEventType_t;

typedef enum {
  FLAGCX_VENDOR_NVIDIA = 0,
  FLAGCX_VENDOR_ILUVATAR_COREX = 1,
  FLAGCX_VENDOR_MLU = 2,
  FLAGCX_VENDOR_METAX = 3,
} flagcxVendorType;

/* ---- handles ----------------------------------------------------------- */
#define FLAGCX_UNIQUE_ID_BYTES 256
typedef struct {
  char internal[FLAGCX_UNIQUE_ID_BYTES];
} flagcxUniqueId;
typedef flagcxUniqueId *flagcxUniqueId_t;

typedef struct flagcxComm *flagcxComm_t;
typedef struct flagcxStream *flagcxStream_t;
typedef struct flagcxEvent *flagcxEvent_t;
typedef struct flagcxIpcMemHandle *flagcxIpcMemHandle_t;
struct flagcxInnerWindow;
typedef struct flagcxInnerWindow *flagcxInnerWindow_t;
struct flagcxSymWindow;
typedef struct flagcxSymWindow *flagcxSymWindow_t;
struct flagcxWindow;
typedef struct flagcxWindow *flagcxWindow_t;

typedef struct {
  flagcxStream_t stream;
  flagcxEvent_t event;
  void **argList;
} flagcxFuncArgs;

/*
 * Runtime function table.  On a GPU host the entries drive the CUDA runtime;
 * on a host without a GPU they operate on a "host device" (malloc/memcpy,
 * streams and events that complete immediately) so the same caller code runs.
 */
struct flagcxDeviceHandle {
  flagcxResult_t (*deviceSynchronize)();
  flagcxResult_t (*deviceMemcpy)(void *dst, void *src, size_t size, flagcxMemcpyType_t type,
      flagcxStream_t stream);
  flagcxResult_t (*deviceMemset)(void *ptr, int value, size_t size, flagcxMemType_t type,
      flagcxStream_t stream);
  flagcxResult_t (*deviceMalloc)(void **ptr, size_t size, flagcxMemType_t type, flagcxStream_t stream);
  flagcxResult_t (*deviceFree)(void *ptr, flagcxMemType_t type, flagcxStream_t stream);
  flagcxResult_t (*setDevice)(int dev);
  flagcxResult_t (*getDevice)(int *dev);
  flagcxResult_t (*getDeviceCount)(int *count);
  flagcxResult_t (*getVendor)(char *vendor);
  flagcxResult_t (*hostGetDevicePointer)(void **pDevice, void *pHost);
  flagcxResult_t (*streamCreate)(flagcxStream_t *stream);
  flagcxResult_t (*streamDestroy)(flagcxStream_t stream);
  flagcxResult_t (*streamCopy)(flagcxStream_t *newStream, void *oldStream);
  flagcxResult_t (*streamFree)(flagcxStream_t stream);
  flagcxResult_t (*streamSynchronize)(flagcxStream_t stream);
  flagcxResult_t (*streamQuery)(flagcxStream_t stream);
  flagcxResult_t (*streamWaitEvent)(flagcxStream_t stream, flagcxEvent_t event);
  flagcxResult_t (*eventCreate)(flagcxEvent_t *event, flagcxEventType_t eventType);
  flagcxResult_t (*eventDestroy)(flagcxEvent_t event);
  flagcxResult_t (*eventRecord)(flagcxEvent_t event, flagcxStream_t stream);
  flagcxResult_t (*eventSynchronize)(flagcxEvent_t event);
  flagcxResult_t (*eventQuery)(flagcxEvent_t event);
  flagcxResult_t (*eventElapsedTime)(float *ms, flagcxEvent_t start, flagcxEvent_t end);
  flagcxResult_t (*ipcMemHandleCreate)(flagcxIpcMemHandle_t *handle, size_t *size);
  flagcxResult_t (*ipcMemHandleGet)(flagcxIpcMemHandle_t handle, void *devPtr);
  flagcxResult_t (*ipcMemHandleOpen)(flagcxIpcMemHandle_t handle, void **devPtr);
  flagcxResult_t (*ipcMemHandleClose)(void *devPtr);
  flagcxResult_t (*ipcMemHandleFree)(flagcxIpcMemHandle_t handle);
};
typedef struct flagcxDeviceHandle *flagcxDeviceHandle_t;

flagcxResult_t flagcxDeviceHandleInit(flagcxDeviceHandle_t *devHandle);
flagcxResult_t flagcxDeviceHandleFree(flagcxDeviceHandle_t devHandle);

/* Older entry points kept for source compatibility. */
struct flagcxHandlerGroup {
  flagcxUniqueId_t uniqueId;
  flagcxComm_t comm;
  flagcxDeviceHandle_t devHandle;
};
typedef struct flagcxHandlerGroup *flagcxHandlerGroup_t;
flagcxResult_t flagcxHandleInit(flagcxHandlerGroup_t *handler);
flagcxResult_t flagcxHandleFree(flagcxHandlerGroup_t handler);

/* ---- memory ------------------------------------------------------------ */
typedef enum {
  flagcxMemCCL = 0,   /* CUDA-VMM allocation that can be shared with peers */
  flagcxMemSHMEM = 1, /* accepted, served by the same VMM allocator */
} flagcxMemAllocator_t;

#define FLAGCX_WIN_DEFAULT 0x00
#define FLAGCX_WIN_COLL_SYMMETRIC 0x01

#ifdef __cplusplus
#define FLAGCX_DEFAULT_ALLOCATOR = flagcxMemCCL
#else
#define FLAGCX_DEFAULT_ALLOCATOR
#endif

/* Allocate / free peer-shareable device memory (2 MiB granularity). On a host
 * without a GPU this returns page-aligned host memory. */
flagcxResult_t flagcxMemAlloc(void **ptr, size_t size, flagcxMemAllocator_t allocator FLAGCX_DEFAULT_ALLOCATOR);
flagcxResult_t flagcxMemFree(void *ptr, flagcxMemAllocator_t allocator FLAGCX_DEFAULT_ALLOCATOR);

/* Local registration: remembers [buff, buff+size) so that later collectives on
 * it can skip the staging copy once a window covers it. */
flagcxResult_t flagcxCommRegister(const flagcxComm_t comm, void *buff, size_t size, void **handle,
    flagcxMemAllocator_t allocator FLAGCX_DEFAULT_ALLOCATOR);
flagcxResult_t flagcxCommDeregister(const flagcxComm_t comm, void *handle,
    flagcxMemAllocator_t allocator FLAGCX_DEFAULT_ALLOCATOR);

/* Collective: every rank passes a buffer of the same size obtained from
 * flagcxMemAlloc; afterwards every local peer has it mapped and collectives
 * whose arguments fall inside the window run without staging. */
flagcxResult_t flagcxCommWindowRegister(flagcxComm_t comm, void *buff, size_t size, flagcxWindow_t *win,
    int winFlags, flagcxMemAllocator_t allocator FLAGCX_DEFAULT_ALLOCATOR);
flagcxResult_t flagcxCommWindowDeregister(flagcxComm_t comm, flagcxWindow_t win,
    flagcxMemAllocator_t allocator FLAGCX_DEFAULT_ALLOCATOR);

/* ---- communicator life cycle -------------------------------------------- */
flagcxResult_t flagcxIsHomoComm(flagcxComm_t comm, int *isHomo);
flagcxResult_t flagcxGetVersion(int *version);
flagcxResult_t flagcxGetUniqueId(flagcxUniqueId_t uniqueId);
flagcxResult_t flagcxCommInitRank(flagcxComm_t *comm, int nranks, flagcxUniqueId_t commId, int rank);
flagcxResult_t flagcxCommFinalize(flagcxComm_t comm);
flagcxResult_t flagcxCommDestroy(flagcxComm_t comm);
/* Abort raises a flag that every device-side wait of this communicator polls,
 * so kernels in flight return with an error status instead of spinning. */
flagcxResult_t flagcxCommAbort(flagcxComm_t comm);
flagcxResult_t flagcxCommResume(flagcxComm_t comm);
flagcxResult_t flagcxCommSuspend(flagcxComm_t comm);
const char *flagcxGetErrorString(flagcxResult_t result);
const char *flagcxGetLastError(flagcxComm_t comm);
/* Reports a device-side wait that ran out of time, an abort, or a socket
 * failure seen by the watchdog thread since the communicator was created. */
flagcxResult_t flagcxCommGetAsyncError(flagcxComm_t comm, flagcxResult_t *asyncError);
flagcxResult_t flagcxCommCount(const flagcxComm_t comm, int *count);
flagcxResult_t flagcxCommGetDeviceNumber(const flagcxComm_t comm, int *device);
flagcxResult_t flagcxCommUserRank(const flagcxComm_t comm, int *rank);

/* ---- collectives --------------------------------------------------------- */
flagcxResult_t flagcxBarrier(flagcxComm_t comm, flagcxStream_t stream);
flagcxResult_t flagcxReduce(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype,
    flagcxRedOp_t op, int root, flagcxComm_t comm, flagcxStream_t stream);
flagcxResult_t flagcxGather(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype,
    int root, flagcxComm_t comm, flagcxStream_t stream);
flagcxResult_t flagcxScatter(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype,
    int root, flagcxComm_t comm, flagcxStream_t stream);
flagcxResult_t flagcxBroadcast(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype,
    int root, flagcxComm_t comm, flagcxStream_t stream);
flagcxResult_t flagcxAllReduce(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype,
    flagcxRedOp_t op, flagcxComm_t comm, flagcxStream_t stream);
flagcxResult_t flagcxReduceScatter(const void *sendbuff, void *recvbuff, size_t recvcount,
    flagcxDataType_t datatype, flagcxRedOp_t op, flagcxComm_t comm, flagcxStream_t stream);
flagcxResult_t flagcxAllGather(const void *sendbuff, void *recvbuff, size_t sendcount,
    flagcxDataType_t datatype, flagcxComm_t comm, flagcxStream_t stream);
flagcxResult_t flagcxAlltoAll(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype,
    flagcxComm_t comm, flagcxStream_t stream);
flagcxResult_t flagcxAlltoAllv(const void *sendbuff, size_t *sendcounts, size_t *sdispls, void *recvbuff,
    size_t *recvcounts, size_t *rdispls, flagcxDataType_t datatype, flagcxComm_t comm, flagcxStream_t stream);
flagcxResult_t flagcxSend(const void *sendbuff, size_t count, flagcxDataType_t datatype, int peer,
    flagcxComm_t comm, flagcxStream_t stream);
flagcxResult_t flagcxRecv(void *recvbuff, size_t count, flagcxDataType_t datatype, int peer, flagcxComm_t comm,
    flagcxStream_t stream);

/* ---- one-sided host API --------------------------------------------------- */
/* Collective registration of a data buffer (index returned in call order: the
 * first registered buffer is memory region 0, the next 1, ...). */
flagcxResult_t flagcxOneSideRegister(flagcxComm_t comm, void *buff, size_t size);
flagcxResult_t flagcxOneSideSignalRegister(const flagcxComm_t comm, void *buff, size_t size, int ptrType);
flagcxResult_t flagcxOneSideStagingRegister(const flagcxComm_t comm, void *buff, size_t size);
flagcxResult_t flagcxOneSideStagingDeregister(const flagcxComm_t comm);
flagcxResult_t flagcxGet(flagcxComm_t comm, int peer, size_t srcOffset, size_t dstOffset, size_t size,
    int srcMrIdx, int dstMrIdx);
flagcxResult_t flagcxPut(flagcxComm_t comm, int peer, size_t srcOffset, size_t dstOffset, size_t size,
    int srcMrIdx, int dstMrIdx);
flagcxResult_t flagcxBatchPut(flagcxComm_t comm, int peer, const size_t *srcOffsets, const size_t *dstOffsets,
    const size_t *sizes, const int *srcMrIdxs, const int *dstMrIdxs, size_t count);
flagcxResult_t flagcxPutSignal(const void *localbuff, size_t count, flagcxDataType_t datatype, int peer,
    flagcxWindow_t peerWin, size_t peerWinOffset, unsigned int flags, flagcxComm_t comm,
    flagcxStream_t stream);
flagcxResult_t flagcxSignal(int peer, unsigned int flags, flagcxComm_t comm, flagcxStream_t stream);
typedef struct {
  uint64_t opCnt; /* how many signals to wait for from `peer` */
  int peer;
} flagcxWaitSignalDesc_t;
flagcxResult_t flagcxWaitSignal(int nDesc, const flagcxWaitSignalDesc_t *signalDescs, flagcxComm_t comm,
    flagcxStream_t stream);
flagcxResult_t flagcxReadCounter(flagcxComm_t comm, uint64_t *count);
flagcxResult_t flagcxWaitCounter(flagcxComm_t comm, uint64_t target);

/* ---- grouping -------------------------------------------------------------- */
/* Operations issued between Start and End are queued and launched together:
 * all queued sends/receives become one direct-write kernel. */
flagcxResult_t flagcxGroupStart(flagcxComm_t comm);
flagcxResult_t flagcxGroupEnd(flagcxComm_t comm);

#ifdef __cplusplus
}
#endif
#endif /* FLAGCX_H_ */
