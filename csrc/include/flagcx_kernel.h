/*
 * flagcx_kernel.h -- host entry points of the device API: create the handles that
 * user kernels receive (flagcxDevComm, flagcxDevMem from flagcx_device.cuh).
 *
 * Same names and roles as flagcx/include/flagcx_kernel_internal.h:132-163 in the
 * FlagCX project.  The handles here are thin: a device communicator is a view of
 * the communicator's barrier inboxes and signal pads, a device memory handle is
 * the peer-pointer table of a registered window.
 */
#ifndef FLAGCX_KERNEL_H_
#define FLAGCX_KERNEL_H_
#include "flagcx.h"

#ifdef __cplusplus
extern "C" {
#endif

struct flagcxDevCommRequirements {
  bool intraMulticast;
  int barrierCount;
  int intraBarrierCount;
  int interBarrierCount;
  int intraLLA2ABlockCount;
  int intraLLA2ASlotCount;
  bool interForceEnable;
  int interContextCount;
  int interSignalCount;
  int interCounterCount;
};
#define FLAGCX_DEV_COMM_REQUIREMENTS_INITIALIZER {false, 0, 0, 0, 0, 0, false, 4, 0, 0}

typedef enum {
  flagcxNetTypeNone = 0,
  flagcxNetTypeProxy = 2,
  flagcxNetTypeGdaki = 3,
} flagcxNetType_t;

struct flagcxCommProperties {
  int rank;
  int nRanks;
  int deviceId;
  bool vendorDeviceApiSupport;
  bool multicastSupport;
  flagcxNetType_t netType;
};
typedef struct flagcxCommProperties flagcxCommProperties_t;

typedef struct flagcxDevCommInternal *flagcxDevComm_t;
typedef struct flagcxDevMemInternal *flagcxDevMem_t;

/* Validates the requirements against the communicator's fixed pads (barrier slots
 * 256..511 are the caller's, FLAGCX_MAX_SIGNALS signals, FLAGCX_MAX_COUNTERS
 * counters) and returns a handle. */
flagcxResult_t flagcxDevCommCreate(flagcxComm_t comm, const struct flagcxDevCommRequirements *reqs,
                                   flagcxDevComm_t *devComm);
flagcxResult_t flagcxDevCommDestroy(flagcxComm_t comm, flagcxDevComm_t devComm);
/* buff must lie in a window (win, or one found by address); collective only when
 * the window still has to be created (win == NULL and buff not yet registered). */
flagcxResult_t flagcxDevMemCreate(flagcxComm_t comm, void *buff, size_t size, flagcxWindow_t win,
                                  flagcxDevMem_t *devMem);
flagcxResult_t flagcxDevMemDestroy(flagcxComm_t comm, flagcxDevMem_t devMem);

/* Copies of the POD structs (struct flagcxDevComm / flagcxDevMem) for passing to
 * kernels by value ... */
flagcxResult_t flagcxDevCommGetStruct(flagcxDevComm_t devComm, void *out, size_t outBytes);
flagcxResult_t flagcxDevMemGetStruct(flagcxDevMem_t devMem, void *out, size_t outBytes);
/* ... or device-resident copies for callers that can only pass pointers. */
flagcxResult_t flagcxDevCommGetDevicePtr(flagcxDevComm_t devComm, void **devPtr);
flagcxResult_t flagcxDevCommFreeDevicePtr(flagcxDevComm_t devComm);
flagcxResult_t flagcxDevMemGetDevicePtr(flagcxDevMem_t devMem, void **devPtr);
flagcxResult_t flagcxDevMemFreeDevicePtr(flagcxDevMem_t devMem);

flagcxResult_t flagcxCommQueryProperties(flagcxComm_t comm, flagcxCommProperties_t *props);

#ifdef __cplusplus
}
#endif
#endif
