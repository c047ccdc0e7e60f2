/*
 * flagcx_net.h -- network adaptor interface (host-side, two-sided).
 *
 * The library ships one adaptor, "socket" (TCP, several striped connections per
 * peer).  A shared object named by FLAGCX_NET_ADAPTOR_PLUGIN may export the
 * symbol flagcxNetAdaptorPlugin_v1 of this type to replace it.  Same role and
 * same entry-point vocabulary as flagcxNetAdaptor in the FlagCX project
 * (flagcx/adaptor/include/flagcx_net_adaptor.h); the one-sided entries are
 * optional and may be NULL.
 */
#ifndef FLAGCX_NET_H_
#define FLAGCX_NET_H_
#include "flagcx.h"

#ifdef __cplusplus
extern "C" {
#endif

#define FLAGCX_NET_HANDLE_BYTES 128

typedef struct {
  char name[64];
  int speedMbps;
  int maxComms;
  int supportsDeviceMemory; /* 0: host pointers only */
} flagcxNetProperties_t;

struct flagcxNetAdaptor_v1 {
  const char *name;
  flagcxResult_t (*init)();
  flagcxResult_t (*devices)(int *ndev);
  flagcxResult_t (*getProperties)(int dev, void *props);
  /* handle: FLAGCX_NET_HANDLE_BYTES written by listen, consumed by connect */
  flagcxResult_t (*listen)(int dev, void *handle, void **listenComm);
  flagcxResult_t (*connect)(int dev, void *handle, void **sendComm);
  flagcxResult_t (*accept)(void *listenComm, void **recvComm);
  flagcxResult_t (*closeSend)(void *sendComm);
  flagcxResult_t (*closeRecv)(void *recvComm);
  flagcxResult_t (*closeListen)(void *listenComm);
  flagcxResult_t (*regMr)(void *comm, void *data, size_t size, int type,
                          int mrFlags, void **mhandle);
  flagcxResult_t (*regMrDmaBuf)(void *comm, void *data, size_t size, int type,
                                uint64_t offset, int fd, int mrFlags,
                                void **mhandle);
  flagcxResult_t (*deregMr)(void *comm, void *mhandle);
  flagcxResult_t (*isend)(void *sendComm, void *data, size_t size, int tag,
                          void *mhandle, void *phandle, void **request);
  flagcxResult_t (*irecv)(void *recvComm, int n, void **data, size_t *sizes,
                          int *tags, void **mhandles, void **phandles,
                          void **request);
  flagcxResult_t (*iflush)(void *recvComm, int n, void **data, int *sizes,
                           void **mhandles, void **request);
  /* done=1 releases the request; sizes[0] receives the byte count */
  flagcxResult_t (*test)(void *request, int *done, int *sizes);
  flagcxResult_t (*iput)(void *sendComm, uint64_t srcOff, uint64_t dstOff,
                         size_t size, int srcRank, int dstRank,
                         void **srcHandles, void **dstHandles, void **request);
  flagcxResult_t (*iget)(void *sendComm, uint64_t srcOff, uint64_t dstOff,
                         size_t size, int srcRank, int dstRank,
                         void **srcHandles, void **dstHandles, void **request);
  flagcxResult_t (*iputSignal)(void *sendComm, uint64_t srcOff, uint64_t dstOff,
                               size_t size, int srcRank, int dstRank,
                               void **srcHandles, void **dstHandles,
                               uint64_t signalOff, void **signalHandles,
                               uint64_t signalValue, void **request);
  flagcxResult_t (*getDevFromName)(char *name, int *dev);
};

#define FLAGCX_NET_ADAPTOR_PLUGIN_SYMBOL_V1 flagcxNetAdaptorPlugin_v1

/* The adaptor in use (built-in socket adaptor unless a plugin was loaded). */
const struct flagcxNetAdaptor_v1 *flagcxGetNetAdaptor(void);

#ifdef __cplusplus
}
#endif
#endif
