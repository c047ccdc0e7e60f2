"""Device-API conformance: pointers, SymPtr, barrier, put/get/putValue, signals, counters,
shadows, cooperative groups, teams, resets and a bounded wait -- kernels from
csrc/tests/device_api_kernels.cu run over an emulated world on one GPU."""
import ctypes as C
import os
import subprocess

import pytest
import torch

from flagcx_b200 import capi

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "csrc", "tests", "device_api_kernels.cu")
LIB = os.path.join(ROOT, "csrc", "tests", "libflagcx_devtest.so")


def _testlib():
    from flagcx_b200.build import build_devtest
    assert build_devtest() == LIB  # rebuilt when its source or a device header is newer
    lib = C.CDLL(LIB)
    lib.fcxDevTestLaunch.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
    return lib


class World:
    def __init__(self, n, n_words=256, timeout_ms=None):
        self.lib = _testlib()
        self.n, self.n_words = n, n_words
        self.comms = capi.Comm.emu_world(n, 0)
        if timeout_ms:
            for c in self.comms:
                c.set_wait_timeout_ms(timeout_ms)
        self.bufs = [torch.zeros(n_words, dtype=torch.int64, device="cuda") for _ in range(n)]
        wins = [self.comms[r].window_register(self.bufs[r], n_words * 8) for r in range(n)]
        cb, mb = C.c_int(), C.c_int()
        self.lib.fcxDevTestSizes(C.byref(cb), C.byref(mb))
        comm_bytes, mem_bytes = bytearray(), bytearray()
        self.handles = []
        for r in range(n):
            dc, dm = C.c_void_p(), C.c_void_p()
            capi.check(capi.lib().flagcxDevCommCreate(self.comms[r].h, None, C.byref(dc)), "flagcxDevCommCreate")
            capi.check(capi.lib().flagcxDevMemCreate(self.comms[r].h, C.c_void_p(self.bufs[r].data_ptr()),
                                                    C.c_size_t(n_words * 8), wins[r], C.byref(dm)), "flagcxDevMemCreate")
            b1, b2 = C.create_string_buffer(cb.value), C.create_string_buffer(mb.value)
            capi.check(capi.lib().flagcxDevCommGetStruct(dc, b1, C.c_size_t(cb.value)), "flagcxDevCommGetStruct")
            capi.check(capi.lib().flagcxDevMemGetStruct(dm, b2, C.c_size_t(mb.value)), "flagcxDevMemGetStruct")
            comm_bytes += b1.raw
            mem_bytes += b2.raw
            self.handles.append((dc, dm))
        self.d_comms = torch.frombuffer(comm_bytes, dtype=torch.uint8).cuda()
        self.d_mems = torch.frombuffer(mem_bytes, dtype=torch.uint8).cuda()
        self.results = torch.zeros(n * 64, dtype=torch.int64, device="cuda")

    def run(self, which, iterations=1):
        self.results.zero_()
        rc = self.lib.fcxDevTestLaunch(which, self.d_comms.data_ptr(), self.d_mems.data_ptr(), self.results.data_ptr(),
                                       self.n, self.n_words, iterations, None)
        assert rc == 0, rc
        torch.cuda.synchronize()
        return self.results.view(self.n, 64).cpu()

    def close(self):
        for r, (dc, dm) in enumerate(self.handles):
            capi.lib().flagcxDevMemDestroy(self.comms[r].h, dm)
            capi.lib().flagcxDevCommDestroy(self.comms[r].h, dc)
        capi.Comm.emu_world_destroy(self.comms)


@pytest.fixture(params=[2, 4, 8])
def world(request):
    w = World(request.param)
    yield w
    w.close()


def test_pointers_and_symptr(world):
    res = world.run(1)
    assert bool((res[:, 0] == 1).all())
    for r in range(world.n):
        assert world.bufs[r][: world.n].tolist() == [1000 + p for p in range(world.n)]


def test_barrier_orders_a_ring_of_updates(world):
    iters = 2 * world.n
    res = world.run(2, iters)
    assert bool((res[:, 0] == 1).all())
    # the token started at rank 0 with value 1 and moved one hop per iteration
    final = [int(b[0]) for b in world.bufs]
    assert final[iters % world.n] == 1 + iters and sum(1 for v in final if v) == 1


def test_put_with_signal_and_counter(world):
    half = world.n_words // 2
    for call in (1, 2):  # signals and counters accumulate across launches
        res = world.run(3, call)
        assert bool((res[:, 0] == 1).all()), res[:, :3]
        assert bool((res[:, 1] >= call).all()) and bool((res[:, 2] == call).all())
    for r in range(world.n):
        prev = (r - 1) % world.n
        want = torch.arange(half) + prev * 100000
        assert torch.equal(world.bufs[r][half:].cpu(), want)


def test_putvalue_signal_add_and_shadows(world):
    res = world.run(4)
    assert bool((res[:, 0] == 1).all())
    assert bool((res[:, 1] == 6).all())  # shadow followed two rounds of +3
    for r in range(world.n):
        prev = (r - 1) % world.n
        assert world.bufs[r][10:12].tolist() == [7000 + prev * 10, 7000 + prev * 10 + 1]


def test_get_with_a_warp(world):
    half = world.n_words // 2
    res = world.run(5)
    assert bool((res[:, 0] == 1).all())
    for r in range(world.n):
        prev = (r - 1) % world.n
        assert torch.equal(world.bufs[r][half:].cpu(), torch.arange(half) + prev * 100000 + 50000)


def test_cooperative_groups_and_tile_signal(world):
    for call in (1, 2):
        res = world.run(6, call)
        assert bool((res[:, 0] == 1).all())


def test_teams_device_and_host(world):
    res = world.run(7)
    assert bool((res[:, 0] == 1).all())
    assert world.lib.fcxDevTestTeamsHost() == 0


def test_reset_signals_and_counters(world):
    world.run(3, 1)
    world.run(4)
    res = world.run(8)
    assert bool((res[:, 0] == 1).all())


def test_c_linkage_wrappers(world):
    """flagcx_device_c.cuh: put with remote signal and local counter, get, putValue with
    signal, shadows, flush and the split barrier, called by their extern "C" names."""
    for _ in range(2):  # the kernel resets its signals and counters, so it can run again
        res = world.run(10)
        assert bool((res[:, 0] == 1).all()), res[:, 0]
    half = world.n_words // 2
    for r in range(world.n):
        prev = (r - 1) % world.n
        assert torch.equal(world.bufs[r][half:2 * half - 1].cpu(), (torch.arange(half) + prev * 100000)[:half - 1])
        assert int(world.bufs[r][world.n_words - 1]) == 0xabc000 + prev


def test_unsatisfied_wait_returns_false_and_reports():
    w = World(2, timeout_ms=150)
    try:
        res = w.run(9)
        assert bool((res[:, 0] == 0).all())
        assert w.comms[0].async_error() == capi.flagcxRemoteError
        assert "timed out" in w.comms[0].last_error()
        assert float(torch.ones(4, device="cuda").sum()) == 4.0  # context still healthy
    finally:
        w.close()


def test_one_sided_host_api_put_get_signal_counter():
    """flagcxOneSideRegister / Put / Get / BatchPut / ReadCounter / WaitCounter / PutSignal /
    Signal / WaitSignal between two emulated ranks."""
    L = capi.lib()
    comms = capi.Comm.emu_world(2, 0)
    try:
        nbytes = 1 << 16
        bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
        bufs[0][:4096] = torch.arange(4096, device="cuda") % 251
        bufs[1][:4096] = (torch.arange(4096, device="cuda") * 7) % 253
        for r in range(2):
            capi.check(L.flagcxOneSideRegister(comms[r].h, C.c_void_p(bufs[r].data_ptr()), C.c_size_t(nbytes)), "register")
        sz = C.c_size_t
        capi.check(L.flagcxPut(comms[0].h, 1, sz(0), sz(8192), sz(1024), 0, 0), "put")
        capi.check(L.flagcxWaitCounter(comms[0].h, C.c_uint64(1)), "waitCounter")
        assert torch.equal(bufs[1][8192:8192 + 1024], bufs[0][:1024])
        capi.check(L.flagcxGet(comms[1].h, 0, sz(1024), sz(16384), sz(512), 0, 0), "get")
        capi.check(L.flagcxWaitCounter(comms[1].h, C.c_uint64(1)), "waitCounter")
        assert torch.equal(bufs[1][16384:16384 + 512], bufs[0][1024:1536])
        offs = (C.c_size_t * 2)(0, 2048)
        dsts = (C.c_size_t * 2)(20480, 24576)
        sizes = (C.c_size_t * 2)(256, 256)
        mrs = (C.c_int * 2)(0, 0)
        capi.check(L.flagcxBatchPut(comms[0].h, 1, offs, dsts, sizes, mrs, mrs, sz(2)), "batchPut")
        capi.check(L.flagcxWaitCounter(comms[0].h, C.c_uint64(3)), "waitCounter")
        cnt = C.c_uint64()
        capi.check(L.flagcxReadCounter(comms[0].h, C.byref(cnt)), "readCounter")
        assert cnt.value == 3
        assert torch.equal(bufs[1][24576:24576 + 256], bufs[0][2048:2304])
        # put with signal into a registered window, the receiver waits on its stream
        wins = [comms[r].window_register(bufs[r], nbytes) for r in range(2)]
        src = torch.full((2048,), 9, dtype=torch.uint8, device="cuda")
        capi.check(L.flagcxPutSignal(C.c_void_p(src.data_ptr()), sz(2048), capi.UINT8, 1, wins[0], sz(32768), 0,
                                     comms[0].h, None), "putSignal")
        capi.check(L.flagcxSignal(1, 0, comms[0].h, None), "signal")
        desc = capi.WaitSignalDesc(2, 0)
        capi.check(L.flagcxWaitSignal(1, C.byref(desc), comms[1].h, None), "waitSignal")
        torch.cuda.synchronize()
        assert comms[1].async_error() == 0, comms[1].last_error()
        assert bool((bufs[1][32768:32768 + 2048] == 9).all())
        # out-of-range requests are refused
        assert L.flagcxPut(comms[0].h, 1, sz(0), sz(nbytes), sz(16), 0, 0) == capi.flagcxInvalidArgument
        assert L.flagcxPut(comms[0].h, 1, sz(0), sz(0), sz(16), 3, 0) == capi.flagcxInvalidArgument
    finally:
        torch.cuda.synchronize()
        capi.Comm.emu_world_destroy(comms)


def test_requirements_are_validated():
    comms = capi.Comm.emu_world(2, 0)
    try:
        class Reqs(C.Structure):
            _fields_ = [("intraMulticast", C.c_bool), ("barrierCount", C.c_int), ("intraBarrierCount", C.c_int),
                        ("interBarrierCount", C.c_int), ("intraLLA2ABlockCount", C.c_int), ("intraLLA2ASlotCount", C.c_int),
                        ("interForceEnable", C.c_bool), ("interContextCount", C.c_int), ("interSignalCount", C.c_int),
                        ("interCounterCount", C.c_int)]
        dc = C.c_void_p()
        too_many = Reqs(False, 100000, 0, 0, 0, 0, False, 4, 0, 0)
        assert capi.lib().flagcxDevCommCreate(comms[0].h, C.byref(too_many), C.byref(dc)) == capi.flagcxInvalidArgument
        wants_mc = Reqs(True, 1, 1, 0, 0, 0, False, 4, 0, 0)
        assert capi.lib().flagcxDevCommCreate(comms[0].h, C.byref(wants_mc), C.byref(dc)) == capi.flagcxNotSupported
        fine = Reqs(False, 4, 4, 0, 0, 0, False, 4, 8, 8)
        assert capi.lib().flagcxDevCommCreate(comms[0].h, C.byref(fine), C.byref(dc)) == 0
        capi.lib().flagcxDevCommDestroy(comms[0].h, dc)
    finally:
        capi.Comm.emu_world_destroy(comms)
