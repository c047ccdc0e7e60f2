"""Point-to-point transfer engine (csrc/include/flagcx_p2p.h): one-sided reads and writes
between processes that share no communicator, e.g. prefill and decode workers exchanging
KV-cache blocks.  Device memory of a peer on the same machine is reached through a CUDA IPC
mapping with one ``cudaMemcpyAsync`` per transfer (DMA engines over NVLink); host memory
and remote machines go through the owner's service thread.

    eng = P2pEngine(device=0)                 # on both sides
    mr = eng.register(kv_cache)               # a torch tensor, numpy array or (address, bytes)
    desc = eng.describe(mr, kv_cache[3])      # bytes: hand them to the peer (notification, RPC, ...)

    conn = eng.connect(peer_metadata)         # "ip:port" from the peer's eng.metadata
    conn.write(local_block, desc)             # one-sided: the owner's process takes no part
    conn.notify(b"block 3 written")
"""
from __future__ import annotations

import ctypes as C

from flagcx_b200 import capi

DESC_BYTES = 128
MAX_NOTIF_BYTES = 4096


class _Desc(C.Structure):
    _fields_ = [("bytes", C.c_ubyte * DESC_BYTES)]


def _span(x):
    """(address, nbytes) of a torch tensor, numpy array, (address, nbytes) pair or bytes-like."""
    if isinstance(x, tuple):
        return int(x[0]), int(x[1])
    if hasattr(x, "data_ptr"):
        assert x.is_contiguous(), "tensor must be contiguous"
        return x.data_ptr(), x.numel() * x.element_size()
    if hasattr(x, "ctypes"):
        return x.ctypes.data, x.nbytes
    raise TypeError(f"cannot take the address of {type(x)}")


def _desc_arg(desc) -> _Desc:
    d = _Desc()
    b = bytes(desc)
    assert len(b) == DESC_BYTES, "a descriptor is 128 bytes"
    C.memmove(C.addressof(d), b, DESC_BYTES)
    return d


class P2pConn:
    def __init__(self, handle, engine: "P2pEngine"):
        self.h, self.engine = handle, engine

    @property
    def is_local(self) -> bool:
        v = C.c_int()
        capi.check(capi.lib().flagcxP2pConnIsLocal(self.h, C.byref(v)), "flagcxP2pConnIsLocal")
        return bool(v.value)

    @property
    def peer_device(self) -> int:
        v = C.c_int()
        capi.check(capi.lib().flagcxP2pConnPeerDevice(self.h, C.byref(v)), "flagcxP2pConnPeerDevice")
        return v.value

    def lookup(self, remote_addr: int, nbytes: int) -> bytes:
        """Descriptor of a range of the peer's registered memory, by its address over there."""
        d = _Desc()
        capi.check(capi.lib().flagcxP2pConnLookup(self.h, C.c_uint64(remote_addr), C.c_size_t(nbytes), C.byref(d)),
                   "flagcxP2pConnLookup")
        return bytes(d.bytes)

    def write(self, local, desc, nbytes: int | None = None, stream=None) -> None:
        addr, n = _span(local)
        d = _desc_arg(desc)
        capi.check(capi.lib().flagcxP2pWrite(self.h, C.c_void_p(addr), C.byref(d), C.c_size_t(n if nbytes is None else nbytes),
                                             capi._stream_arg(stream)), "flagcxP2pWrite")

    def read(self, local, desc, nbytes: int | None = None, stream=None) -> None:
        addr, n = _span(local)
        d = _desc_arg(desc)
        capi.check(capi.lib().flagcxP2pRead(self.h, C.c_void_p(addr), C.byref(d), C.c_size_t(n if nbytes is None else nbytes),
                                            capi._stream_arg(stream)), "flagcxP2pRead")

    def _vector(self, fn, name, locals_, descs, stream):
        n = len(locals_)
        assert n == len(descs)
        spans = [_span(x) for x in locals_]
        ptrs = (C.c_void_p * n)(*[s[0] for s in spans])
        sizes = (C.c_size_t * n)(*[s[1] for s in spans])
        ds = (_Desc * n)(*[_desc_arg(d) for d in descs])
        capi.check(fn(self.h, n, ptrs, ds, sizes, capi._stream_arg(stream)), name)

    def write_vector(self, locals_, descs, stream=None) -> None:
        self._vector(capi.lib().flagcxP2pWriteVector, "flagcxP2pWriteVector", locals_, descs, stream)

    def read_vector(self, locals_, descs, stream=None) -> None:
        self._vector(capi.lib().flagcxP2pReadVector, "flagcxP2pReadVector", locals_, descs, stream)

    def notify(self, msg: bytes) -> None:
        capi.check(capi.lib().flagcxP2pSendNotif(self.h, msg, C.c_size_t(len(msg))), "flagcxP2pSendNotif")

    def recv_notification(self, timeout_ms: int = -1) -> bytes | None:
        """The next notification, or None when none arrived in time."""
        buf = C.create_string_buffer(MAX_NOTIF_BYTES)
        n = C.c_size_t()
        code = capi.lib().flagcxP2pRecvNotif(self.h, buf, C.c_size_t(MAX_NOTIF_BYTES), C.byref(n), timeout_ms)
        if code == capi.flagcxInProgress:
            return None
        capi.check(code, "flagcxP2pRecvNotif")
        return buf.raw[: n.value]

    def close(self) -> None:
        if self.h:
            capi.check(capi.lib().flagcxP2pConnDestroy(self.h), "flagcxP2pConnDestroy")
            self.h = None


class P2pEngine:
    def __init__(self, device: int = -1):
        h = C.c_void_p()
        capi.check(capi.lib().flagcxP2pEngineCreate(device, C.byref(h)), "flagcxP2pEngineCreate")
        self.h, self.device = h, device

    @property
    def port(self) -> int:
        v = C.c_int()
        capi.check(capi.lib().flagcxP2pEngineGetPort(self.h, C.byref(v)), "flagcxP2pEngineGetPort")
        return v.value

    @property
    def metadata(self) -> str:
        buf = C.create_string_buffer(128)
        capi.check(capi.lib().flagcxP2pEngineGetMetadata(self.h, buf, C.c_size_t(128)), "flagcxP2pEngineGetMetadata")
        return buf.value.decode()

    def connect(self, ip_port: str) -> P2pConn:
        c = C.c_void_p()
        capi.check(capi.lib().flagcxP2pEngineConnect(self.h, ip_port.encode(), C.byref(c)), "flagcxP2pEngineConnect")
        return P2pConn(c, self)

    def get_conn(self, ip_port: str) -> P2pConn:
        """The engine's cached connection to that peer (opened on first use; owned by the engine)."""
        c = C.c_void_p()
        capi.check(capi.lib().flagcxP2pEngineGetConn(self.h, ip_port.encode(), C.byref(c)), "flagcxP2pEngineGetConn")
        return P2pConn(c, self)

    def accept(self, timeout_ms: int = -1) -> P2pConn | None:
        c = C.c_void_p()
        code = capi.lib().flagcxP2pEngineAccept(self.h, C.byref(c), timeout_ms)
        if code == capi.flagcxInProgress:
            return None
        capi.check(code, "flagcxP2pEngineAccept")
        return P2pConn(c, self)

    def register(self, mem) -> int:
        addr, n = _span(mem)
        mr = C.c_uint64()
        capi.check(capi.lib().flagcxP2pEngineReg(self.h, C.c_void_p(addr), C.c_size_t(n), C.byref(mr)), "flagcxP2pEngineReg")
        return mr.value

    def deregister(self, mr: int) -> None:
        capi.check(capi.lib().flagcxP2pEngineDereg(self.h, C.c_uint64(mr)), "flagcxP2pEngineDereg")

    def describe(self, mr: int, mem) -> bytes:
        """Descriptor of `mem`, a tensor / array / (address, nbytes) pair inside region `mr`."""
        addr, n = _span(mem)
        d = _Desc()
        capi.check(capi.lib().flagcxP2pEngineMakeDesc(self.h, C.c_uint64(mr), C.c_void_p(addr), C.c_size_t(n), C.byref(d)),
                   "flagcxP2pEngineMakeDesc")
        return bytes(d.bytes)

    def close(self) -> None:
        if self.h:
            capi.check(capi.lib().flagcxP2pEngineDestroy(self.h), "flagcxP2pEngineDestroy")
            self.h = None
