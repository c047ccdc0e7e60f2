/* flagcx_p2p.h -- point-to-point transfer engine between processes that are NOT members of
 * one communicator: the prefill and decode workers of a disaggregated serving stack
 * handing KV-cache blocks to each other, a parameter server, a checkpoint loader.
 *
 * Same job as the P2P engine of the FlagCX project (flagcx/include/flagcx_p2p.h there:
 * engine, connections, memory regions, serialisable descriptors, one-sided read / write,
 * vectors of them, notifications, addressing a peer's memory by its virtual address).
 * That engine moves data with RDMA verbs; this one is built for one NVSwitch machine:
 *
 *   - device memory of a peer process on the same machine is mapped through its CUDA IPC
 *     handle the first time a descriptor names it, and a read or write is then ONE
 *     cudaMemcpyAsync on the caller's stream: the DMA engines move the bytes over NVLink at
 *     the peer-copy rate, no SM and no host thread touches them, and the owner takes no part;
 *   - host memory, and any memory of a process on another machine, goes through the owner:
 *     the request travels over the connection's TCP socket and the owner's service thread
 *     copies (slow path, for control data and tests without a GPU);
 *   - notifications are small messages queued at the receiver.
 *
 * Every blocking call has a deadline (FLAGCX_SOCKET_TIMEOUT_MS) and returns an error code
 * when the peer has gone away.  All functions return flagcxSuccess or an error code.
 */
#ifndef FLAGCX_P2P_H_
#define FLAGCX_P2P_H_

#include <stddef.h>
#include <stdint.h>

#include "flagcx.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct flagcxP2pEngine *flagcxP2pEngine_t;
typedef struct flagcxP2pConn *flagcxP2pConn_t;
typedef uint64_t flagcxP2pMr_t;

#define FLAGCX_P2P_DESC_BYTES 128
#define FLAGCX_P2P_MAX_NOTIF_BYTES 4096

/* Names a range of registered memory of some engine.  Plain bytes: send it to whoever
 * should read or write that range, by any channel (a notification, an RPC, a file). */
typedef struct {
  unsigned char bytes[FLAGCX_P2P_DESC_BYTES];
} flagcxP2pDesc_t;

/* ---- engine ------------------------------------------------------------------------- */
/* cudaDevice: the GPU whose memory this engine registers, or -1 for host memory only.
 * The engine listens on an ephemeral TCP port of every interface. */
flagcxResult_t flagcxP2pEngineCreate(int cudaDevice, flagcxP2pEngine_t *engine);
flagcxResult_t flagcxP2pEngineDestroy(flagcxP2pEngine_t engine);
flagcxResult_t flagcxP2pEngineGetPort(flagcxP2pEngine_t engine, int *port);
/* "ip:port" a peer passes to flagcxP2pEngineConnect. */
flagcxResult_t flagcxP2pEngineGetMetadata(flagcxP2pEngine_t engine, char *buf, size_t len);

/* ---- connections -------------------------------------------------------------------- */
flagcxResult_t flagcxP2pEngineConnect(flagcxP2pEngine_t engine, const char *ipPort, flagcxP2pConn_t *conn);
/* The next connection a peer has opened to this engine; timeoutMs < 0 waits for ever,
 * flagcxInProgress when none arrived in time. */
flagcxResult_t flagcxP2pEngineAccept(flagcxP2pEngine_t engine, flagcxP2pConn_t *conn, int timeoutMs);
/* The engine's connection to the peer listening at "ip:port": opened on the first call,
 * returned from a cache afterwards.  The engine closes it at flagcxP2pEngineDestroy; destroying it
 * earlier also takes it out of the cache. */
flagcxResult_t flagcxP2pEngineGetConn(flagcxP2pEngine_t engine, const char *ipPort, flagcxP2pConn_t *conn);
flagcxResult_t flagcxP2pConnDestroy(flagcxP2pConn_t conn);
/* 1 when the peer runs on this machine (device memory is reached directly). */
flagcxResult_t flagcxP2pConnIsLocal(flagcxP2pConn_t conn, int *isLocal);
/* CUDA device of the peer engine (-1: host only). */
flagcxResult_t flagcxP2pConnPeerDevice(flagcxP2pConn_t conn, int *device);

/* ---- memory ------------------------------------------------------------------------- */
/* Registers [data, data+size): device memory from cudaMalloc (a torch tensor's storage
 * included) or ordinary host memory.  Must stay allocated until it is deregistered. */
flagcxResult_t flagcxP2pEngineReg(flagcxP2pEngine_t engine, void *data, size_t size, flagcxP2pMr_t *mr);
flagcxResult_t flagcxP2pEngineDereg(flagcxP2pEngine_t engine, flagcxP2pMr_t mr);
/* Descriptor of [addr, addr+len) inside region mr. */
flagcxResult_t flagcxP2pEngineMakeDesc(flagcxP2pEngine_t engine, flagcxP2pMr_t mr, const void *addr, size_t len,
                                       flagcxP2pDesc_t *desc);
/* Descriptor of a range of the PEER's memory given its address in the peer's address space
 * (the peer must have registered a region that contains it). */
flagcxResult_t flagcxP2pConnLookup(flagcxP2pConn_t conn, uint64_t remoteAddr, size_t len, flagcxP2pDesc_t *desc);

/* ---- one-sided transfers ------------------------------------------------------------ */
/* local: any host or device pointer of this process (need not be registered).  stream:
 * where a device-to-device transfer is queued; NULL = the call returns when the data has
 * arrived.  Transfers that go through the owner are always complete on return. */
flagcxResult_t flagcxP2pWrite(flagcxP2pConn_t conn, const void *local, const flagcxP2pDesc_t *remote, size_t bytes,
                              flagcxStream_t stream);
flagcxResult_t flagcxP2pRead(flagcxP2pConn_t conn, void *local, const flagcxP2pDesc_t *remote, size_t bytes,
                             flagcxStream_t stream);
flagcxResult_t flagcxP2pWriteVector(flagcxP2pConn_t conn, int n, const void *const *locals, const flagcxP2pDesc_t *remotes,
                                    const size_t *bytes, flagcxStream_t stream);
flagcxResult_t flagcxP2pReadVector(flagcxP2pConn_t conn, int n, void *const *locals, const flagcxP2pDesc_t *remotes,
                                   const size_t *bytes, flagcxStream_t stream);

/* ---- notifications ------------------------------------------------------------------ */
flagcxResult_t flagcxP2pSendNotif(flagcxP2pConn_t conn, const void *msg, size_t len);
/* flagcxInProgress when nothing arrived within timeoutMs. */
flagcxResult_t flagcxP2pRecvNotif(flagcxP2pConn_t conn, void *buf, size_t capacity, size_t *len, int timeoutMs);

#ifdef __cplusplus
}
#endif
#endif /* FLAGCX_P2P_H_ */
