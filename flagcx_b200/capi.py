"""ctypes binding of libflagcx.so.

Plays the role of the FlagCX inter-service wrapper
(plugin/interservice/flagcx_wrapper.py in the FlagCX project): Python code and the
tests drive the C API directly.  Works on hosts without a GPU (socket path).

The library is looked for in ``flagcx_b200/lib``; ``flagcx_b200.build.build()``
compiles it.  Nothing falls back silently: a missing library raises.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence

import numpy as np

_LIB_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib")
# FLAGCX_LIBRARY selects another build of the library (sanitizer or bounds-checking builds)
LIB_PATH = os.environ.get("FLAGCX_LIBRARY") or os.path.join(_LIB_DIR, "libflagcx.so")

# ---- enums (flagcx.h) --------------------------------------------------------
flagcxSuccess = 0
flagcxUnhandledDeviceError = 1
flagcxSystemError = 2
flagcxInternalError = 3
flagcxInvalidArgument = 4
flagcxInvalidUsage = 5
flagcxRemoteError = 6
flagcxInProgress = 7
flagcxNotSupported = 9

INT8, UINT8, INT32, UINT32, INT64, UINT64, HALF, FLOAT, DOUBLE, BFLOAT16 = range(10)
NUM_TYPES = 10
SUM, PROD, MAX, MIN, AVG = range(5)

OP_SEND, OP_RECV, OP_BROADCAST, OP_GATHER, OP_SCATTER, OP_REDUCE, OP_ALLREDUCE, \
    OP_ALLGATHER, OP_REDUCESCATTER, OP_ALLTOALL, OP_ALLTOALLV = range(11)

ALGO_AUTO = -1
(ALGO_ONESHOT, ALGO_TWOSHOT, ALGO_NVLS_ONESHOT, ALGO_NVLS_TWOSHOT, ALGO_PUSH, ALGO_PULL, ALGO_NVLS, ALGO_LL, ALGO_RING,
 ALGO_COPY_ENGINE) = range(10)

WIN_DEFAULT = 0
WIN_COLL_SYMMETRIC = 1

_NP_TO_DT = {
    np.dtype(np.int8): INT8, np.dtype(np.uint8): UINT8, np.dtype(np.int32): INT32,
    np.dtype(np.uint32): UINT32, np.dtype(np.int64): INT64, np.dtype(np.uint64): UINT64,
    np.dtype(np.float16): HALF, np.dtype(np.float32): FLOAT, np.dtype(np.float64): DOUBLE,
}
DT_SIZE = {INT8: 1, UINT8: 1, INT32: 4, UINT32: 4, INT64: 8, UINT64: 8, HALF: 2, FLOAT: 4, DOUBLE: 8, BFLOAT16: 2}


def np_dtype_code(dt) -> int:
    return _NP_TO_DT[np.dtype(dt)]


class UniqueId(C.Structure):
    _fields_ = [("internal", C.c_char * 256)]


class FusedOpts(C.Structure):
    _fields_ = [("scale", C.c_float), ("outDtype", C.c_int), ("residual", C.c_void_p),
                ("algo", C.c_int), ("nCtas", C.c_int)]


class OpStats(C.Structure):
    _fields_ = [("calls", C.c_uint64), ("bytes", C.c_uint64), ("lastAlgo", C.c_int),
                ("lastCtas", C.c_int), ("lastMs", C.c_float)]


class UserBufferStats(C.Structure):
    """Counters of the on-demand export of user buffers (flagcxCommUserBufferStats)."""
    _fields_ = [("enabled", C.c_int), ("hits", C.c_uint64), ("exports", C.c_uint64), ("refused", C.c_uint64),
                ("stale", C.c_uint64), ("peerOpened", C.c_uint64), ("peerClosed", C.c_uint64)]


class WaitSignalDesc(C.Structure):
    _fields_ = [("opCnt", C.c_uint64), ("peer", C.c_int)]


class CudaStream(C.Structure):
    """struct flagcxStream { cudaStream_t base; }"""
    _fields_ = [("base", C.c_void_p)]


class FlagcxError(RuntimeError):
    def __init__(self, code: int, what: str, detail: str = ""):
        self.code = code
        super().__init__(f"{what} failed with {code}: {detail}")


_lib: Optional[C.CDLL] = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(
                f"{LIB_PATH} is missing; build it with `python -c 'import flagcx_b200.build as b; b.build()'` "
                "or `make -C csrc -j`")
        _lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
        _lib.flagcxGetErrorString.restype = C.c_char_p
        _lib.flagcxGetLastError.restype = C.c_char_p
        _lib.flagcxGetLastError.argtypes = [C.c_void_p]
        _lib.getFlagcxDataTypeSize.restype = C.c_size_t
    return _lib


def check(code: int, what: str, comm=None) -> None:
    if code != flagcxSuccess:
        l = lib()
        detail = l.flagcxGetErrorString(code).decode()
        last = l.flagcxGetLastError(comm).decode() if comm is not None else ""
        raise FlagcxError(code, what, f"{detail}; {last}")


def _ptr(x) -> C.c_void_p:
    """Address of a numpy array, torch tensor, int or None."""
    if x is None:
        return C.c_void_p(0)
    if isinstance(x, int):
        return C.c_void_p(x)
    if isinstance(x, np.ndarray):
        return C.c_void_p(x.ctypes.data)
    if hasattr(x, "data_ptr"):
        return C.c_void_p(x.data_ptr())
    raise TypeError(type(x))


def _sizes(v: Sequence[int]):
    return (C.c_size_t * len(v))(*[int(i) for i in v])


def get_unique_id() -> UniqueId:
    uid = UniqueId()
    check(lib().flagcxGetUniqueId(C.byref(uid)), "flagcxGetUniqueId")
    return uid


def unique_id_bytes(uid: UniqueId) -> bytes:
    return bytes(C.string_at(C.addressof(uid), 256))


def unique_id_from_bytes(b: bytes) -> UniqueId:
    uid = UniqueId()
    C.memmove(C.addressof(uid), b, 256)
    return uid


class Stream:
    """Wraps a raw cudaStream_t value (0 = default stream) as a flagcxStream_t."""

    def __init__(self, cuda_stream: int = 0):
        self._s = CudaStream(C.c_void_p(cuda_stream))

    @property
    def handle(self):
        return C.byref(self._s)


def _stream_arg(stream):
    if stream is None:
        return None
    if isinstance(stream, Stream):
        return stream.handle
    if isinstance(stream, int):
        s = Stream(stream)
        _stream_arg._keep = s  # keep alive until the next call
        return s.handle
    if hasattr(stream, "cuda_stream"):  # torch.cuda.Stream
        s = Stream(stream.cuda_stream)
        _stream_arg._keep = s
        return s.handle
    raise TypeError(type(stream))


class Comm:
    """One rank of a communicator."""

    def __init__(self, handle: C.c_void_p, owns: bool = True):
        self.h = handle
        self.owns = owns

    # -- construction ----------------------------------------------------------
    @classmethod
    def init_rank(cls, nranks: int, uid: UniqueId, rank: int) -> "Comm":
        h = C.c_void_p()
        check(lib().flagcxCommInitRank(C.byref(h), nranks, C.byref(uid), rank), "flagcxCommInitRank")
        return cls(h)

    @classmethod
    def emu_world(cls, nranks: int, device: int = 0):
        arr = (C.c_void_p * nranks)()
        check(lib().flagcxEmuWorldCreate(nranks, device, arr), "flagcxEmuWorldCreate")
        return [cls(C.c_void_p(arr[i]), owns=False) for i in range(nranks)]

    @staticmethod
    def emu_world_destroy(comms):
        check(lib().flagcxEmuWorldDestroy(comms[0].h), "flagcxEmuWorldDestroy")

    def destroy(self):
        if self.h and self.owns:
            check(lib().flagcxCommDestroy(self.h), "flagcxCommDestroy")
        self.h = None

    def abort(self):
        if self.h:
            lib().flagcxCommAbort(self.h)
            if self.owns:
                self.h = None

    # -- queries ------------------------------------------------------------------
    def _int(self, fn) -> int:
        v = C.c_int()
        check(getattr(lib(), fn)(self.h, C.byref(v)), fn, self.h)
        return v.value

    @property
    def rank(self): return self._int("flagcxCommUserRank")
    @property
    def nranks(self): return self._int("flagcxCommCount")
    @property
    def device_path(self): return bool(self._int("flagcxCommIsDevicePath"))
    @property
    def has_multicast(self): return bool(self._int("flagcxCommHasMulticast"))

    def async_error(self) -> int:
        v = C.c_int()
        check(lib().flagcxCommGetAsyncError(self.h, C.byref(v)), "flagcxCommGetAsyncError")
        return v.value

    def last_error(self) -> str:
        return lib().flagcxGetLastError(self.h).decode()

    def set_wait_timeout_ms(self, ms: int):
        check(lib().flagcxCommSetWaitTimeoutMs(self.h, ms), "flagcxCommSetWaitTimeoutMs", self.h)

    def trace_enable(self, capacity: int):
        """Keep the last `capacity` collective calls in a ring (0: off)."""
        check(lib().flagcxCommTraceEnable(self.h, int(capacity)), "flagcxCommTraceEnable", self.h)

    def trace_dump(self, path: str):
        """Write the ring as JSON (synchronises the recorded CUDA events)."""
        check(lib().flagcxCommTraceDump(self.h, path.encode()), "flagcxCommTraceDump", self.h)

    def stats(self, op: int) -> OpStats:
        s = OpStats()
        check(lib().flagcxCommGetStats(self.h, op, C.byref(s)), "flagcxCommGetStats", self.h)
        return s

    def user_buffer_stats(self) -> UserBufferStats:
        s = UserBufferStats()
        check(lib().flagcxCommUserBufferStats(self.h, C.byref(s)), "flagcxCommUserBufferStats", self.h)
        return s

    # -- collectives (buffers: numpy arrays, torch tensors or raw addresses) ---------
    def all_reduce(self, send, recv, count, dtype, op=SUM, stream=None):
        check(lib().flagcxAllReduce(_ptr(send), _ptr(recv), C.c_size_t(count), dtype, op, self.h, _stream_arg(stream)),
              "flagcxAllReduce", self.h)

    def all_reduce_fused(self, send, recv, count, dtype, op=SUM, scale=1.0, out_dtype=NUM_TYPES, residual=None,
                         algo=ALGO_AUTO, nctas=0, stream=None):
        o = FusedOpts(scale, out_dtype, _ptr(residual), algo, nctas)
        check(lib().flagcxAllReduceFused(_ptr(send), _ptr(recv), C.c_size_t(count), dtype, op, C.byref(o), self.h,
                                         _stream_arg(stream)), "flagcxAllReduceFused", self.h)

    def reduce_scatter(self, send, recv, recvcount, dtype, op=SUM, stream=None):
        check(lib().flagcxReduceScatter(_ptr(send), _ptr(recv), C.c_size_t(recvcount), dtype, op, self.h,
                                        _stream_arg(stream)), "flagcxReduceScatter", self.h)

    def reduce_scatter_fused(self, send, recv, recvcount, dtype, op=SUM, scale=1.0, out_dtype=NUM_TYPES,
                             residual=None, algo=ALGO_AUTO, nctas=0, stream=None):
        o = FusedOpts(scale, out_dtype, _ptr(residual), algo, nctas)
        check(lib().flagcxReduceScatterFused(_ptr(send), _ptr(recv), C.c_size_t(recvcount), dtype, op, C.byref(o),
                                             self.h, _stream_arg(stream)), "flagcxReduceScatterFused", self.h)

    def all_gather(self, send, recv, sendcount, dtype, stream=None, algo=ALGO_AUTO, nctas=0):
        if algo != ALGO_AUTO or nctas:
            check(lib().flagcxAllGatherEx(_ptr(send), _ptr(recv), C.c_size_t(sendcount), dtype, algo, nctas, self.h,
                                          _stream_arg(stream)), "flagcxAllGatherEx", self.h)
        else:
            check(lib().flagcxAllGather(_ptr(send), _ptr(recv), C.c_size_t(sendcount), dtype, self.h,
                                        _stream_arg(stream)), "flagcxAllGather", self.h)

    def broadcast(self, send, recv, count, dtype, root, stream=None):
        check(lib().flagcxBroadcast(_ptr(send), _ptr(recv), C.c_size_t(count), dtype, root, self.h,
                                    _stream_arg(stream)), "flagcxBroadcast", self.h)

    def reduce(self, send, recv, count, dtype, op, root, stream=None):
        check(lib().flagcxReduce(_ptr(send), _ptr(recv), C.c_size_t(count), dtype, op, root, self.h,
                                 _stream_arg(stream)), "flagcxReduce", self.h)

    def gather(self, send, recv, count, dtype, root, stream=None):
        check(lib().flagcxGather(_ptr(send), _ptr(recv), C.c_size_t(count), dtype, root, self.h,
                                 _stream_arg(stream)), "flagcxGather", self.h)

    def scatter(self, send, recv, count, dtype, root, stream=None):
        check(lib().flagcxScatter(_ptr(send), _ptr(recv), C.c_size_t(count), dtype, root, self.h,
                                  _stream_arg(stream)), "flagcxScatter", self.h)

    def all_to_all(self, send, recv, count, dtype, stream=None):
        check(lib().flagcxAlltoAll(_ptr(send), _ptr(recv), C.c_size_t(count), dtype, self.h, _stream_arg(stream)),
              "flagcxAlltoAll", self.h)

    def all_to_allv(self, send, scounts, sdispls, recv, rcounts, rdispls, dtype, stream=None):
        check(lib().flagcxAlltoAllv(_ptr(send), _sizes(scounts), _sizes(sdispls), _ptr(recv), _sizes(rcounts),
                                    _sizes(rdispls), dtype, self.h, _stream_arg(stream)), "flagcxAlltoAllv", self.h)

    def send(self, buf, count, dtype, peer, stream=None):
        check(lib().flagcxSend(_ptr(buf), C.c_size_t(count), dtype, peer, self.h, _stream_arg(stream)),
              "flagcxSend", self.h)

    def recv(self, buf, count, dtype, peer, stream=None):
        check(lib().flagcxRecv(_ptr(buf), C.c_size_t(count), dtype, peer, self.h, _stream_arg(stream)),
              "flagcxRecv", self.h)

    def group_start(self):
        check(lib().flagcxGroupStart(self.h), "flagcxGroupStart", self.h)

    def group_end(self):
        check(lib().flagcxGroupEnd(self.h), "flagcxGroupEnd", self.h)

    def barrier(self, stream=None):
        check(lib().flagcxBarrier(self.h, _stream_arg(stream)), "flagcxBarrier", self.h)

    # -- memory ---------------------------------------------------------------------------
    def window_register(self, ptr, size: int, flags: int = WIN_COLL_SYMMETRIC) -> C.c_void_p:
        w = C.c_void_p()
        check(lib().flagcxCommWindowRegister(self.h, _ptr(ptr), C.c_size_t(size), C.byref(w), flags, 0),
              "flagcxCommWindowRegister", self.h)
        return w

    def window_deregister(self, win):
        check(lib().flagcxCommWindowDeregister(self.h, win, 0), "flagcxCommWindowDeregister", self.h)

    # -- tuner -------------------------------------------------------------------------------
    def tune(self, op, dtype, min_bytes, max_bytes, iters=10):
        check(lib().flagcxTunerTune(self.h, op, dtype, C.c_size_t(min_bytes), C.c_size_t(max_bytes), iters),
              "flagcxTunerTune", self.h)

    def tuner_save(self, path: str):
        check(lib().flagcxTunerSave(self.h, path.encode()), "flagcxTunerSave", self.h)

    def tuner_load(self, path: str):
        check(lib().flagcxTunerLoad(self.h, path.encode()), "flagcxTunerLoad", self.h)

    def tuner_query(self, op, nbytes, registered=True):
        a, n = C.c_int(), C.c_int()
        check(lib().flagcxTunerQuery(self.h, op, C.c_size_t(nbytes), int(registered), C.byref(a), C.byref(n)),
              "flagcxTunerQuery", self.h)
        return a.value, n.value


def mem_alloc(size: int) -> int:
    p = C.c_void_p()
    check(lib().flagcxMemAlloc(C.byref(p), C.c_size_t(size), 0), "flagcxMemAlloc")
    return p.value


def mem_free(ptr: int) -> None:
    check(lib().flagcxMemFree(C.c_void_p(ptr), 0), "flagcxMemFree")


def window_peer_pointer(win, peer: int, offset: int = 0) -> int:
    p = C.c_void_p()
    check(lib().flagcxWindowGetPeerPointer(win, peer, C.c_size_t(offset), C.byref(p)), "flagcxWindowGetPeerPointer")
    return p.value


def host_reduce(dst: np.ndarray, src: np.ndarray, dtype: int, op: int) -> None:
    check(lib().flagcxHostReduce(_ptr(dst), _ptr(src), C.c_size_t(dst.size), dtype, op), "flagcxHostReduce")
