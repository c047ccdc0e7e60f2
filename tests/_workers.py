"""Rank bodies for the multi-process tests (imported by name in spawned children)."""
import os
import time

import numpy as np

from flagcx_b200 import capi

NP_TYPES = {
    capi.INT8: np.int8, capi.UINT8: np.uint8, capi.INT32: np.int32, capi.UINT32: np.uint32,
    capi.INT64: np.int64, capi.UINT64: np.uint64, capi.HALF: np.float16, capi.FLOAT: np.float32,
    capi.DOUBLE: np.float64,
}


def seeded(rank, n, dtype_code):
    """Values uniform in [-1, 1) from seed=rank (small integers for integer types)."""
    rng = np.random.default_rng(rank)
    npdt = NP_TYPES[dtype_code]
    if np.issubdtype(npdt, np.floating):
        return rng.uniform(-1, 1, n).astype(npdt)
    if np.issubdtype(npdt, np.unsignedinteger):
        return rng.integers(0, 3, n).astype(npdt)
    return rng.integers(-2, 3, n).astype(npdt)


def np_reduce(arrs, op):
    acc = np.stack(arrs).astype(np.float64)
    if op == capi.SUM:
        return acc.sum(0)
    if op == capi.PROD:
        return acc.prod(0)
    if op == capi.MAX:
        return acc.max(0)
    if op == capi.MIN:
        return acc.min(0)
    if op == capi.AVG:
        return acc.sum(0) / len(arrs)
    raise ValueError(op)


def rel_err(got, ref):
    got = np.asarray(got, np.float64)
    return float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), 1.0)))


def host_collectives(rank, n, uid, count, dtype_code):
    """Host-buffer collectives: allreduce / allgather / reducescatter / alltoall / send-recv
    on host buffers, checked against numpy."""
    comm = capi.Comm.init_rank(n, capi.unique_id_from_bytes(uid), rank)
    assert comm.rank == rank and comm.nranks == n
    xs = [seeded(r, count, dtype_code) for r in range(n)]
    x = xs[rank]
    out = {}
    ar = np.empty_like(x)
    comm.all_reduce(x, ar, count, dtype_code, capi.SUM)
    out["allreduce"] = rel_err(ar, np_reduce(xs, capi.SUM))
    ag = np.empty(count * n, x.dtype)
    comm.all_gather(x, ag, count, dtype_code)
    out["allgather"] = float(not np.array_equal(ag, np.concatenate(xs)))
    per = count // n
    rs = np.empty(per, x.dtype)
    comm.reduce_scatter(x, rs, per, dtype_code, capi.SUM)
    out["reducescatter"] = rel_err(rs, np_reduce([a[: per * n] for a in xs], capi.SUM)[rank * per:(rank + 1) * per])
    a2a = np.empty(per * n, x.dtype)
    comm.all_to_all(x, a2a, per, dtype_code)
    exp = np.concatenate([xs[p][rank * per:(rank + 1) * per] for p in range(n)])
    out["alltoall"] = float(not np.array_equal(a2a, exp))
    # ring send/recv inside a group
    nxt, prv = (rank + 1) % n, (rank - 1 + n) % n
    got = np.empty_like(x)
    comm.group_start()
    comm.send(x, count, dtype_code, nxt)
    comm.recv(got, count, dtype_code, prv)
    comm.group_end()
    out["sendrecv"] = float(not np.array_equal(got, xs[prv]))
    comm.barrier()
    comm.destroy()
    return out


def host_collectives_through_plugin(rank, n, uid, count, plugin_path):
    """The host collectives with FLAGCX_NET_ADAPTOR_PLUGIN set: results as usual, and the
    plugin's own counters show that it carried the traffic."""
    import ctypes
    out = host_collectives(rank, n, uid, count, capi.FLOAT)
    plug = ctypes.CDLL(plugin_path)  # same object the library loaded
    sent, recvd, msgs = ctypes.c_uint64(), ctypes.c_uint64(), ctypes.c_uint64()
    plug.flagcxNetExampleCounters(ctypes.byref(sent), ctypes.byref(recvd), ctypes.byref(msgs))
    out["plugin_bytes_sent"] = int(sent.value)
    out["plugin_messages"] = int(msgs.value)
    return out


def nccl_shim_program(rank, n, uid, shim_path, count):
    """What a program written against NCCL does, through the preloadable stand-in:
    init from a 128-byte id, all-reduce, all-gather, a grouped ring send/recv."""
    import ctypes as C

    class NcclUniqueId(C.Structure):
        _fields_ = [("internal", C.c_char * 128)]

    capi.lib()  # libflagcx.so resident (the shim links against it)
    nccl = C.CDLL(shim_path)
    nccl.ncclCommInitRank.argtypes = [C.POINTER(C.c_void_p), C.c_int, NcclUniqueId, C.c_int]
    nccl.ncclGetErrorString.restype = C.c_char_p
    nid = NcclUniqueId()
    C.memmove(C.byref(nid), uid[:128], 128)  # (a c_char array field reads back as a copy)
    assert not any(uid[128:]), "the bootstrap id must fit NCCL's 128 bytes"
    comm = C.c_void_p()
    rc = nccl.ncclCommInitRank(C.byref(comm), n, nid, rank)
    assert rc == 0, nccl.ncclGetErrorString(rc)
    got_rank, got_n = C.c_int(-1), C.c_int(-1)
    assert nccl.ncclCommUserRank(comm, C.byref(got_rank)) == 0 and nccl.ncclCommCount(comm, C.byref(got_n)) == 0
    assert (got_rank.value, got_n.value) == (rank, n)
    NCCL_FLOAT, NCCL_SUM = 7, 0
    xs = [seeded(r, count, capi.FLOAT) for r in range(n)]
    x, out = xs[rank], {}
    ar = np.empty_like(x)
    p = lambda a: C.c_void_p(a.ctypes.data)  # noqa: E731
    assert nccl.ncclAllReduce(p(x), p(ar), C.c_size_t(count), NCCL_FLOAT, NCCL_SUM, comm, None) == 0
    out["allreduce"] = rel_err(ar, np_reduce(xs, capi.SUM))
    ag = np.empty(count * n, np.float32)
    assert nccl.ncclAllGather(p(x), p(ag), C.c_size_t(count), NCCL_FLOAT, comm, None) == 0
    out["allgather"] = float(not np.array_equal(ag, np.concatenate(xs)))
    got = np.empty_like(x)
    assert nccl.ncclGroupStart() == 0
    assert nccl.ncclSend(p(x), C.c_size_t(count), NCCL_FLOAT, (rank + 1) % n, comm, None) == 0
    assert nccl.ncclRecv(p(got), C.c_size_t(count), NCCL_FLOAT, (rank - 1) % n, comm, None) == 0
    assert nccl.ncclGroupEnd() == 0
    out["sendrecv"] = float(not np.array_equal(got, xs[(rank - 1) % n]))
    assert nccl.ncclAllReduce(p(x), p(ar), C.c_size_t(count), 11, NCCL_SUM, comm, None) == 4  # fp8: invalid argument
    assert nccl.ncclCommDestroy(comm) == 0
    return out


def host_all_ops(rank, n, uid, count):
    """Every collective, several dtypes and reductions, odd counts."""
    comm = capi.Comm.init_rank(n, capi.unique_id_from_bytes(uid), rank)
    worst = 0.0
    for dt in (capi.FLOAT, capi.DOUBLE, capi.INT32, capi.INT64, capi.UINT8, capi.HALF):
        xs = [seeded(r, count, dt) for r in range(n)]
        x = xs[rank]
        for op in (capi.SUM, capi.PROD, capi.MAX, capi.MIN, capi.AVG):
            if op == capi.AVG and not np.issubdtype(x.dtype, np.floating):
                continue
            ar = np.empty_like(x)
            comm.all_reduce(x, ar, count, dt, op)
            tol_scale = 1e-2 if dt == capi.HALF else 1.0
            worst = max(worst, rel_err(ar, np_reduce(xs, op)) * tol_scale)
            root = (n - 1) if n > 1 else 0
            rd = np.zeros_like(x)
            comm.reduce(x, rd, count, dt, op, root)
            if rank == root:
                worst = max(worst, rel_err(rd, np_reduce(xs, op)) * tol_scale)
        # in place
        ip = x.copy()
        comm.all_reduce(ip, ip, count, dt, capi.MAX)
        worst = max(worst, rel_err(ip, np_reduce(xs, capi.MAX)))
        root = 0
        b = x.copy() if rank == root else np.zeros_like(x)
        comm.broadcast(b, b, count, dt, root)
        assert np.array_equal(b, xs[root]), "broadcast"
        g = np.zeros(count * n, x.dtype)
        comm.gather(x, g, count, dt, root)
        if rank == root:
            assert np.array_equal(g, np.concatenate(xs)), "gather"
        src = np.concatenate(xs) if rank == root else np.zeros(count * n, x.dtype)
        sc = np.zeros(count, x.dtype)
        comm.scatter(src, sc, count, dt, root)
        assert np.array_equal(sc, xs[rank]), "scatter"
    # alltoallv with rank-dependent counts
    dt = capi.FLOAT
    scounts = [(rank + p) % 5 + 1 for p in range(n)]
    rcounts = [(p + rank) % 5 + 1 for p in range(n)]
    sdispls = np.concatenate([[0], np.cumsum(scounts)[:-1]]).tolist()
    rdispls = np.concatenate([[0], np.cumsum(rcounts)[:-1]]).tolist()
    send = (np.arange(sum(scounts)) + 1000 * rank).astype(np.float32)
    recv = np.zeros(sum(rcounts), np.float32)
    comm.all_to_allv(send, scounts, sdispls, recv, rcounts, rdispls, dt)
    for p in range(n):
        pc = [(p + q) % 5 + 1 for q in range(n)]
        pd = np.concatenate([[0], np.cumsum(pc)[:-1]])
        exp = (np.arange(pd[rank], pd[rank] + pc[rank]) + 1000 * p).astype(np.float32)
        assert np.array_equal(recv[rdispls[p]:rdispls[p] + rcounts[p]], exp), "alltoallv"
    comm.destroy()
    return worst


def rank_that_dies(rank, n, uid, victim):
    """Failure on the host: one rank exits before the collective; the others must get
    an error code back (not hang)."""
    comm = capi.Comm.init_rank(n, capi.unique_id_from_bytes(uid), rank)
    x = np.ones(1 << 16, np.float32)
    out = np.empty_like(x)
    comm.all_reduce(x, out, x.size, capi.FLOAT, capi.SUM)  # connections are up now
    if rank == victim:
        os._exit(0)
    time.sleep(0.3)
    try:
        comm.all_reduce(x, out, x.size, capi.FLOAT, capi.SUM)
    except capi.FlagcxError as e:
        return e.code
    return 0


def survivors_rebuild_a_smaller_communicator(rank, n, uid, victim, path):
    """Elastic recovery on the host: a rank exits, the others see an error code, destroy the
    communicator, agree on a new unique id (the lowest survivor creates it and publishes it
    through a file) and carry on with n-1 ranks."""
    comm = capi.Comm.init_rank(n, capi.unique_id_from_bytes(uid), rank)
    x = np.full(1 << 12, float(rank + 1), np.float32)
    out = np.empty_like(x)
    comm.all_reduce(x, out, x.size, capi.FLOAT, capi.SUM)
    assert out[0] == n * (n + 1) / 2
    if rank == victim:
        os._exit(0)
    time.sleep(0.3)
    try:
        comm.all_reduce(x, out, x.size, capi.FLOAT, capi.SUM)
        return {"error": 0}
    except capi.FlagcxError as e:
        code = e.code
    try:
        comm.abort()
    except Exception:
        pass
    survivors = [r for r in range(n) if r != victim]
    new_rank = survivors.index(rank)
    if new_rank == 0:
        with open(path + ".tmp", "wb") as f:
            f.write(capi.unique_id_bytes(capi.get_unique_id()))
        os.replace(path + ".tmp", path)
    deadline = time.time() + 30
    while not os.path.exists(path):
        assert time.time() < deadline
        time.sleep(0.05)
    comm2 = capi.Comm.init_rank(len(survivors), capi.unique_id_from_bytes(open(path, "rb").read()), new_rank)
    comm2.all_reduce(x, out, x.size, capi.FLOAT, capi.SUM)
    want = float(sum(r + 1 for r in survivors))
    ok = bool(np.all(out == want))
    comm2.destroy()
    return {"error": code, "recovered": ok, "new_world": len(survivors)}


def rank_that_is_late(rank, n, uid, late, delay_s):
    """Failure on the host without a dead process: one rank reaches the collective only
    after the others' deadline has passed.  The punctual ranks get an error code when their
    deadline runs out; the late rank gets one too when it finally calls (its peers have given
    up), and nobody hangs."""
    comm = capi.Comm.init_rank(n, capi.unique_id_from_bytes(uid), rank)
    x = np.ones(1 << 14, np.float32)
    out = np.empty_like(x)
    comm.all_reduce(x, out, x.size, capi.FLOAT, capi.SUM)  # connections are up now
    if rank == late:
        time.sleep(delay_s)
    t0 = time.time()
    try:
        comm.all_reduce(x, out, x.size, capi.FLOAT, capi.SUM)
        code = 0
    except capi.FlagcxError as e:
        code = e.code
    return {"code": code, "seconds": time.time() - t0}


def rank_that_never_joins(rank, n, uid):
    """Rank n-1 never calls flagcxCommInitRank: the others time out with an error."""
    if rank == n - 1:
        return "absent"
    try:
        capi.Comm.init_rank(n, capi.unique_id_from_bytes(uid), rank)
    except capi.FlagcxError as e:
        return e.code
    return 0


def wrong_unique_id(rank, n, uid):
    bad = bytearray(uid)
    bad[0] ^= 0xFF  # corrupt the magic
    try:
        capi.Comm.init_rank(n, capi.unique_id_from_bytes(bytes(bad)), rank)
    except capi.FlagcxError as e:
        return e.code
    return 0


def mismatched_sizes(rank, n, uid):
    """Ranks disagree on the message size: the receiver sees a size error, not garbage."""
    comm = capi.Comm.init_rank(n, capi.unique_id_from_bytes(uid), rank)
    code = 0
    try:
        if rank == 0:
            comm.send(np.ones(1000, np.float32), 1000, capi.FLOAT, 1)
        elif rank == 1:
            comm.recv(np.empty(10, np.float32), 10, capi.FLOAT, 0)
    except capi.FlagcxError as e:
        code = e.code
    return code


def comm_id_env(rank, n, uid_unused):
    """Rendezvous through FLAGCX_COMM_ID instead of a shared unique id."""
    uid = capi.get_unique_id()  # every rank builds the same id from the environment
    comm = capi.Comm.init_rank(n, uid, rank)
    x = np.full(8, rank + 1, np.float64)
    out = np.empty_like(x)
    comm.all_reduce(x, out, 8, capi.DOUBLE, capi.SUM)
    comm.destroy()
    return float(out[0])


# ---------------------------------------------------------------------------
# multi-GPU ranks (one process per GPU)
# ---------------------------------------------------------------------------
def _torch_seeded(rank, count, tdt):
    import torch
    g = torch.Generator().manual_seed(rank)
    return (torch.rand(count, generator=g, dtype=torch.float64) * 2 - 1).to(tdt)


def gpu_collectives(rank, n, uid, count, registered):
    """Every device collective on real peers; registered (zero-copy) or staged."""
    import torch
    from flagcx_b200.utils.symm import SymmetricBuffer
    torch.cuda.set_device(rank)
    comm = capi.Comm.init_rank(n, capi.unique_id_from_bytes(uid), rank)
    assert comm.device_path, "expected the NVLink device path"
    worst = {}
    bufs = []

    def alloc(numel, tdt):
        if registered:
            b = SymmetricBuffer(comm, numel * torch.empty((), dtype=tdt).element_size())
            bufs.append(b)
            return b.view(tdt, numel)
        return torch.empty(numel, dtype=tdt, device="cuda")

    for dt, tdt, tol in ((capi.FLOAT, torch.float32, 1e-6), (capi.BFLOAT16, torch.bfloat16, 2 ** -7 * n)):
        cpu = [_torch_seeded(r, count * n, tdt) for r in range(n)]
        ref = torch.stack([c.to(torch.float64) for c in cpu]).sum(0)
        x = alloc(count * n, tdt)
        x.copy_(cpu[rank])
        for algo in (capi.ALGO_ONESHOT, capi.ALGO_TWOSHOT):
            out = alloc(count * n, tdt)
            comm.all_reduce_fused(x, out, count * n, dt, capi.SUM, algo=algo)
            torch.cuda.synchronize()
            err = ((out.cpu().to(torch.float64) - ref).abs() / ref.abs().clamp(min=1)).max().item()
            worst[f"allreduce{algo}_{dt}"] = err / tol
        rs = alloc(count, tdt)
        comm.reduce_scatter(x, rs, count, dt, capi.SUM)
        torch.cuda.synchronize()
        err = ((rs.cpu().to(torch.float64) - ref[rank * count:(rank + 1) * count]).abs()
               / ref[rank * count:(rank + 1) * count].abs().clamp(min=1)).max().item()
        worst[f"reducescatter_{dt}"] = err / tol
        for algo in (capi.ALGO_PUSH, capi.ALGO_PULL):
            ag = alloc(count * n, tdt)
            ag.zero_()
            comm.all_gather(x[:count], ag, count, dt, algo=algo)
            torch.cuda.synchronize()
            want = torch.cat([c[:count] for c in cpu])
            worst[f"allgather{algo}_{dt}"] = float(not torch.equal(ag.cpu(), want))
        aa = alloc(count * n, tdt)
        comm.all_to_all(x, aa, count, dt)
        torch.cuda.synchronize()
        want = torch.cat([cpu[p][rank * count:(rank + 1) * count] for p in range(n)])
        worst[f"alltoall_{dt}"] = float(not torch.equal(aa.cpu(), want))
        bc = alloc(count, tdt)
        bc.copy_(cpu[rank][:count])
        comm.broadcast(bc, bc, count, dt, n - 1)
        torch.cuda.synchronize()
        worst[f"broadcast_{dt}"] = float(not torch.equal(bc.cpu(), cpu[n - 1][:count]))
    # grouped ring exchange on plain tensors
    big = (5 << 20) // 4 + 3
    src = torch.full((big,), float(rank), device="cuda")
    dst = torch.empty(big, device="cuda")
    comm.group_start()
    comm.send(src, big, capi.FLOAT, (rank + 1) % n)
    comm.recv(dst, big, capi.FLOAT, (rank - 1) % n)
    comm.group_end()
    torch.cuda.synchronize()
    worst["sendrecv"] = float(not bool((dst == float((rank - 1) % n)).all()))
    comm.barrier()
    assert comm.async_error() == 0, comm.last_error()
    for b in bufs:
        b.free()
    comm.destroy()
    return worst


def gpu_user_buffers_under_skew(rank, n, uid, rounds):
    """Ordinary torch tensors (nothing registered by the caller), ranks with different
    allocation histories, one rank held back by compute before every collective: a small
    all-reduce directly followed by a large all-reduce / reduce-scatter / all-gather,
    exact results every round.  Runs with on-demand export of user buffers (the default)
    and, with FLAGCX_USER_BUFFER_EXPORT=0, through the staging window."""
    import torch
    torch.cuda.set_device(rank)
    comm = capi.Comm.init_rank(n, capi.unique_id_from_bytes(uid), rank)
    assert comm.device_path, "expected the NVLink device path"
    exporting = bool(comm.user_buffer_stats().enabled)
    import flagcx_b200.torch_backend as tb
    tb.follow_torch_allocator(comm)  # segments freed by empty_cache() below are unmapped at the peers first
    # different allocation histories: segments and offsets differ between the ranks
    ballast = [torch.empty((rank + 1) * (3 << 20) + 4096 * i, dtype=torch.uint8, device="cuda") for i in range(rank + 2)]
    small_n, big_n, per = 1024, (6 << 20) + 16 * n, (1 << 20)
    busy = torch.randn(2048, 2048, device="cuda")
    bad = []
    for it in range(rounds):
        # integers small enough that every sum is exact in fp32
        small = torch.full((small_n,), float(rank + it), device="cuda")
        big = (torch.arange(big_n, device="cuda", dtype=torch.float32) % 1000) + rank
        rs_in = (torch.arange(per * n, device="cuda", dtype=torch.float32) % 512) * (rank + 1)
        rs_out = torch.empty(per, device="cuda")
        ag_out = torch.empty(per * n, device="cuda")
        if it % n == rank:  # this round's straggler
            for _ in range(20):
                busy = (busy @ busy).clamp_(-1, 1)
        comm.all_reduce(small, small, small_n, capi.FLOAT, capi.SUM)
        comm.all_reduce(big, big, big_n, capi.FLOAT, capi.SUM)
        comm.all_reduce(small, small, small_n, capi.FLOAT, capi.SUM)
        comm.reduce_scatter(rs_in, rs_out, per, capi.FLOAT, capi.SUM)
        comm.all_gather(rs_out, ag_out, per, capi.FLOAT)
        torch.cuda.synchronize()
        base = sum(range(n))
        want_small = float((n * it + base) * n)
        if not bool((small == want_small).all()):
            bad.append(("small", it))
        want_big = (torch.arange(big_n, device="cuda", dtype=torch.float32) % 1000) * n + base
        if not torch.equal(big, want_big):
            bad.append(("big", it))
        tri = n * (n + 1) // 2
        want_rs = (torch.arange(per * n, device="cuda", dtype=torch.float32) % 512) * tri
        if not torch.equal(rs_out, want_rs[rank * per:(rank + 1) * per]):
            bad.append(("reduce_scatter", it))
        if not torch.equal(ag_out, want_rs):
            bad.append(("all_gather", it))
        if it % 3 == 2:  # hand the segments back so that addresses get reused by new allocations
            del small, big, rs_in, rs_out, ag_out, want_big, want_rs
            torch.cuda.empty_cache()
    st = comm.user_buffer_stats()
    assert comm.async_error() == 0, comm.last_error()
    comm.barrier()
    del ballast
    tb.unfollow_torch_allocator(comm)
    comm.destroy()
    return {"bad": bad, "exporting": exporting, "exports": int(st.exports), "hits": int(st.hits),
            "refused": int(st.refused), "stale": int(st.stale)}


def gpu_nvls_collectives(rank, n, uid, count):
    """The multimem (NVLink SHARP) kernels on registered windows: all-reduce one- and
    two-shot, reduce-scatter, all-gather, against fp64 sums of the same seeded inputs.
    Every rank stays alive until all of them have unbound their memory."""
    import torch
    from flagcx_b200.utils.symm import SymmetricBuffer
    torch.cuda.set_device(rank)
    comm = capi.Comm.init_rank(n, capi.unique_id_from_bytes(uid), rank)
    if not comm.has_multicast:
        comm.destroy()
        return {"skipped": 1.0}
    worst, bufs = {}, []

    def alloc(numel, tdt):
        b = SymmetricBuffer(comm, max(numel * torch.empty((), dtype=tdt).element_size(), 1 << 21))
        bufs.append(b)
        return b.view(tdt, numel)

    try:
        for dt, tdt, tol in ((capi.FLOAT, torch.float32, 1e-6), (capi.BFLOAT16, torch.bfloat16, 2 ** -7 * n)):
            cpu = [_torch_seeded(r, count * n, tdt) for r in range(n)]
            ref = torch.stack([c.to(torch.float64) for c in cpu]).sum(0)
            x = alloc(count * n, tdt)
            x.copy_(cpu[rank])
            for algo in (capi.ALGO_NVLS_ONESHOT, capi.ALGO_NVLS_TWOSHOT):
                out = alloc(count * n, tdt)
                out.zero_()
                comm.all_reduce_fused(x, out, count * n, dt, capi.SUM, algo=algo)
                torch.cuda.synchronize()
                if comm.stats(capi.OP_ALLREDUCE).lastAlgo != algo:
                    worst[f"allreduce{algo}_{dt}_fell_back"] = 2.0  # the multimem kernel did not run
                err = ((out.cpu().to(torch.float64) - ref).abs() / ref.abs().clamp(min=1)).max().item()
                worst[f"allreduce{algo}_{dt}"] = err / tol
            rs = alloc(count, tdt)
            comm.reduce_scatter_fused(x, rs, count, dt, capi.SUM, algo=capi.ALGO_NVLS)
            torch.cuda.synchronize()
            if comm.stats(capi.OP_REDUCESCATTER).lastAlgo != capi.ALGO_NVLS:
                worst[f"reducescatter_{dt}_fell_back"] = 2.0
            sl = ref[rank * count:(rank + 1) * count]
            worst[f"reducescatter_{dt}"] = ((rs.cpu().to(torch.float64) - sl).abs() / sl.abs().clamp(min=1)).max().item() / tol
            ag = alloc(count * n, tdt)
            ag.zero_()
            comm.all_gather(x[:count], ag, count, dt, algo=capi.ALGO_NVLS)
            torch.cuda.synchronize()
            if comm.stats(capi.OP_ALLGATHER).lastAlgo != capi.ALGO_NVLS:
                worst[f"allgather_{dt}_fell_back"] = 2.0
            worst[f"allgather_{dt}"] = float(not torch.equal(ag.cpu(), torch.cat([c[:count] for c in cpu])))
        if comm.async_error() != 0:
            worst["device_error"] = 2.0
    finally:
        # nobody leaves while a peer's memory is still bound to the multicast object
        for b in bufs:
            b.free()
        comm.destroy()
    return worst


def gpu_copy_engine_collectives(rank, n, uid, count, rounds):
    """All-gather into a window with the data moved by the copy engines (two one-CTA barrier
    kernels around n peer copies): exact results over several rounds that reuse the same
    output buffer with changing contents, out of place and in place, while one rank is
    slowed down by extra work in its stream."""
    import torch
    from flagcx_b200.utils.symm import SymmetricBuffer
    torch.cuda.set_device(rank)
    comm = capi.Comm.init_rank(n, capi.unique_id_from_bytes(uid), rank)
    worst = {}
    buf = SymmetricBuffer(comm, count * n * 2)
    out = buf.view(torch.bfloat16, count * n)
    src = torch.empty(count, dtype=torch.bfloat16, device="cuda")
    ballast = torch.randn(2048, 2048, device="cuda")
    try:
        for it in range(rounds):
            if rank == it % n:  # a straggler: its peers reach the collective long before it
                for _ in range(20):
                    ballast = (ballast @ ballast).clamp_(-1, 1)
            in_place = it % 2 == 1
            val = lambda r: float((r + 1) * 8 + it % 7)
            if in_place:
                mine = out[rank * count:(rank + 1) * count]
                mine.fill_(val(rank))
            else:
                mine = src
                mine.fill_(val(rank))
            comm.all_gather(mine, out, count, capi.BFLOAT16, algo=capi.ALGO_COPY_ENGINE)
            if comm.stats(capi.OP_ALLGATHER).lastAlgo != capi.ALGO_COPY_ENGINE:
                worst["fell_back"] = 2.0
            got = out.view(n, count).float()
            want = torch.tensor([val(r) for r in range(n)], device="cuda")[:, None].expand(n, count)
            if not torch.equal(got, want):
                worst[f"round{it}"] = 2.0
        # reduce-scatter: peer copies into the owners' staging areas, then a local reduce.
        # Plain torch tensors on both sides; a block larger than a staging slot (several
        # chunks) and a small odd one; exact small-integer sums; average fused in.
        for it, cnt in enumerate((count * 3 + 40, 1000, count * 3 + 40)):
            if rank == (it + 1) % n:
                for _ in range(20):
                    ballast = (ballast @ ballast).clamp_(-1, 1)
            x = torch.empty(n, cnt, dtype=torch.float32, device="cuda")
            for blk in range(n):
                x[blk].fill_(float(rank + 1 + blk + it))
            y = torch.zeros(cnt, dtype=torch.float32, device="cuda")
            comm.reduce_scatter_fused(x, y, cnt, capi.FLOAT, capi.AVG if it == 2 else capi.SUM, algo=capi.ALGO_COPY_ENGINE, nctas=8)
            if comm.stats(capi.OP_REDUCESCATTER).lastAlgo != capi.ALGO_COPY_ENGINE:
                worst["rs_fell_back"] = 2.0
            want = float(sum(r + 1 + rank + it for r in range(n)))
            if it == 2:
                want /= n
            if not torch.equal(y, torch.full_like(y, want)):
                worst[f"rs_round{it}"] = 2.0
        torch.cuda.synchronize()
        if comm.async_error() != 0:
            worst["device_error"] = 2.0
    finally:
        torch.cuda.synchronize()
        comm.barrier()
        buf.free()
        comm.destroy()
    return worst


def gpu_two_level(rank, n, uid, per_node):
    """A machine split into nodes of `per_node` ranks (FLAGCX_HOSTID per rank, set by the
    test): all-reduce and all-gather take the two-level route (NVLink kernels inside a
    node, host network between), everything else the flat host route."""
    import torch
    torch.cuda.set_device(rank)
    comm = capi.Comm.init_rank(n, capi.unique_id_from_bytes(uid), rank)
    assert not comm.device_path, "the split must take the communicator off the single-domain device path"
    worst = {}
    for dt, tdt, tol in ((capi.FLOAT, torch.float32, 1e-6), (capi.BFLOAT16, torch.bfloat16, 2 ** -7 * n)):
        for count in (3, 1000, 70003, (1 << 20) + 8):
            cpu = [_torch_seeded(r, count, tdt) for r in range(n)]
            ref = torch.stack([c.to(torch.float64) for c in cpu]).sum(0)
            x = cpu[rank].cuda()
            out = torch.empty_like(x)
            comm.all_reduce(x, out, count, dt, capi.SUM)
            torch.cuda.synchronize()
            err = ((out.cpu().to(torch.float64) - ref).abs() / ref.abs().clamp(min=1)).max().item()
            worst[f"allreduce_{dt}_{count}"] = err / tol
            comm.all_reduce(x, x, count, dt, capi.AVG)  # in place
            torch.cuda.synchronize()
            err = ((x.cpu().to(torch.float64) - ref / n).abs() / (ref / n).abs().clamp(min=1)).max().item()
            worst[f"allreduce_avg_{dt}_{count}"] = err / tol
            ag = torch.zeros(count * n, dtype=tdt, device="cuda")
            comm.all_gather(cpu[rank].cuda(), ag, count, dt)
            torch.cuda.synchronize()
            worst[f"allgather_{dt}_{count}"] = float(not torch.equal(ag.cpu(), torch.cat(cpu)))
    # an operation without a two-level route: flat host path
    cnt = 4099
    cpu = [_torch_seeded(r, cnt * n, torch.float32) for r in range(n)]
    rs = torch.empty(cnt, device="cuda")
    comm.reduce_scatter(cpu[rank].cuda(), rs, cnt, capi.FLOAT, capi.SUM)
    torch.cuda.synchronize()
    ref = torch.stack(cpu).to(torch.float64).sum(0)[rank * cnt:(rank + 1) * cnt]
    worst["reducescatter_flat"] = ((rs.cpu().to(torch.float64) - ref).abs().max().item()) / 1e-5
    comm.destroy()
    return worst


def gpu_peer_never_launches(rank, n, uid):
    """One rank skips the collective: the others' kernels give up after the time limit
    and report a remote error; nobody hangs and no GPU faults."""
    import torch
    torch.cuda.set_device(rank)
    comm = capi.Comm.init_rank(n, capi.unique_id_from_bytes(uid), rank)
    comm.set_wait_timeout_ms(300)
    x = torch.ones(4096, device="cuda")
    code = 0
    if rank != n - 1:
        comm.all_reduce(x, x, x.numel(), capi.FLOAT, capi.SUM)
        torch.cuda.synchronize()
        code = comm.async_error()
        healthy = float((torch.ones(8, device="cuda") * 3).sum()) == 24.0
        assert healthy
    # leave between steps, with nothing in flight; abort skips the closing handshake
    comm.abort()
    return code


# ---------------------------------------------------------------------------
# torch.distributed backend "flagcx"
# ---------------------------------------------------------------------------
def torch_backend_ops(rank, n, uid_unused, port, use_cuda):
    """Every ProcessGroup operation against values computed by hand."""
    import torch
    import torch.distributed as dist
    import flagcx_b200.torch_backend  # noqa: F401  (registers "flagcx")
    if use_cuda:
        torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank) if use_cuda else torch.device("cpu")
    dist.init_process_group("flagcx", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=n)
    try:
        t = torch.full((1000,), float(rank + 1), device=dev)
        dist.all_reduce(t)
        assert torch.all(t == n * (n + 1) / 2), "allreduce"
        t = torch.full((1000,), float(rank + 1), device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert torch.all(t == n), "allreduce max"
        t = torch.full((64,), float(rank), device=dev)
        dist.broadcast(t, src=n - 1)
        assert torch.all(t == n - 1), "broadcast"
        outs = [torch.empty(16, device=dev) for _ in range(n)]
        dist.all_gather(outs, torch.full((16,), float(rank), device=dev))
        assert all(torch.all(outs[r] == r) for r in range(n)), "allgather"
        flat = torch.empty(16 * n, device=dev)
        dist.all_gather_into_tensor(flat, torch.full((16,), float(rank), device=dev))
        assert torch.equal(flat, torch.arange(n, device=dev).repeat_interleave(16).float()), "allgather base"
        rs = torch.empty(8, device=dev)
        dist.reduce_scatter_tensor(rs, torch.arange(8 * n, device=dev).float())
        assert torch.equal(rs, torch.arange(8 * rank, 8 * rank + 8, device=dev).float() * n), "reduce_scatter base"
        rs2 = torch.empty(8, device=dev)
        dist.reduce_scatter(rs2, [torch.full((8,), float(p), device=dev) for p in range(n)])
        assert torch.all(rs2 == rank * n), "reduce_scatter list"
        red = torch.full((32,), 2.0, device=dev)
        dist.reduce(red, dst=0)
        if rank == 0:
            assert torch.all(red == 2.0 * n), "reduce"
        a2a_in = torch.arange(4 * n, device=dev).float() + 100 * rank
        a2a_out = torch.empty(4 * n, device=dev)
        dist.all_to_all_single(a2a_out, a2a_in)
        want = torch.cat([torch.arange(4 * rank, 4 * rank + 4, device=dev).float() + 100 * p for p in range(n)])
        assert torch.equal(a2a_out, want), "alltoall base"
        # uneven splits -> alltoallv
        in_splits = [(rank + p) % 3 + 1 for p in range(n)]
        out_splits = [(p + rank) % 3 + 1 for p in range(n)]
        src = torch.arange(sum(in_splits), device=dev).float() + 1000 * rank
        dst = torch.empty(sum(out_splits), device=dev)
        dist.all_to_all_single(dst, src, out_splits, in_splits)
        off = 0
        for p in range(n):
            ps = [(p + q) % 3 + 1 for q in range(n)]
            start = sum(ps[:rank])
            want = torch.arange(start, start + ps[rank], device=dev).float() + 1000 * p
            assert torch.equal(dst[off:off + out_splits[p]], want), "alltoallv"
            off += out_splits[p]
        gl = [torch.empty(4, device=dev) for _ in range(n)] if rank == 0 else None
        dist.gather(torch.full((4,), float(rank), device=dev), gl, dst=0)
        if rank == 0:
            assert all(torch.all(gl[r] == r) for r in range(n)), "gather"
        sc = torch.empty(4, device=dev)
        dist.scatter(sc, [torch.full((4,), float(p * 3), device=dev) for p in range(n)] if rank == 0 else None, src=0)
        assert torch.all(sc == rank * 3), "scatter"
        # p2p ring through batch_isend_irecv (coalesced into one group launch)
        sendt = torch.full((2048,), float(rank), device=dev)
        recvt = torch.empty(2048, device=dev)
        ops = [dist.P2POp(dist.isend, sendt, (rank + 1) % n), dist.P2POp(dist.irecv, recvt, (rank - 1) % n)]
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        if use_cuda:
            torch.cuda.synchronize()
        assert torch.all(recvt == (rank - 1) % n), "batch_isend_irecv"
        dist.barrier()
        if use_cuda:
            torch.cuda.synchronize()
    finally:
        dist.destroy_process_group()
    return "ok"


def torch_backend_options(rank, n, uid_unused, port):
    """pg_options of the backend: with enable_tuner every collective's (operation, bytes)
    is recorded; bool tensors reduce as logical or / and."""
    import torch
    import torch.distributed as dist
    import flagcx_b200.torch_backend as tb
    dist.init_process_group("flagcx", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=n,
                            pg_options=tb.Options(enable_tuner=True, tune_group_idx=3))
    try:
        dev = torch.device("cpu")
        t = torch.ones(1000)
        dist.all_reduce(t)
        dist.all_reduce(torch.ones(50))
        dist.all_reduce(torch.ones(1000))  # same size again: one tune object
        flat = torch.empty(16 * n)
        dist.all_gather_into_tensor(flat, torch.ones(16))
        objs = tb.tune_objects(dist.group.WORLD, dev)
        assert (capi.OP_ALLREDUCE, 4000) in objs and (capi.OP_ALLREDUCE, 200) in objs, objs
        assert (capi.OP_ALLGATHER, 64 * n) in objs and len(objs) == 3, objs
        b = torch.tensor([rank == 0, False, True])
        dist.all_reduce(b)  # sum of bools: logical or
        assert b.tolist() == [True, False, True], b
        b = torch.tensor([rank == 0, False, True])
        dist.all_reduce(b, op=dist.ReduceOp.PRODUCT)  # logical and
        assert b.tolist() == [False, False, True], b
        dist.barrier()
    finally:
        dist.destroy_process_group()
    return "ok"


def tp_fused(rank, n, uid, M, N, K):
    """all-gather->GEMM and GEMM->reduce-scatter against torch on gathered operands."""
    import torch
    from flagcx_b200.parallel.tp import AllGatherGemm, GemmReduceScatter
    torch.cuda.set_device(rank)
    comm = capi.Comm.init_rank(n, capi.unique_id_from_bytes(uid), rank)
    rows = M // n

    def seeded(seed, shape):
        g = torch.Generator().manual_seed(seed)
        return (torch.randn(*shape, generator=g) * 0.5).to(torch.bfloat16)

    out = {}
    # column-parallel: X sharded by rows, every rank its own W
    xs = [seeded(10 + r, (rows, K)) for r in range(n)]
    w = seeded(100 + rank, (N, K)).cuda()
    agg = AllGatherGemm(comm, M, N, K)
    for it in range(3):  # several calls: flags are epochs, buffers are reused
        agg.shard.copy_(xs[rank].cuda() * (it + 1))
        d = agg(w)
        torch.cuda.synchronize()
        ref = (torch.cat(xs).float().cuda() * (it + 1)) @ w.float().T
        err = ((d.float() - ref).abs() / (ref.abs().mean() + ref.abs())).max().item()
        out["ag_gemm"] = max(out.get("ag_gemm", 0.0), err)
    agg.close()
    # row-parallel: every rank a K-slice; the sum over ranks is scattered by rows
    xk = [seeded(200 + r, (M, K)) for r in range(n)]
    wk = [seeded(300 + r, (N, K)) for r in range(n)]
    grs = GemmReduceScatter(comm, M, N, K)
    for it in range(3):
        o = grs(xk[rank].cuda(), wk[rank].cuda())
        torch.cuda.synchronize()
        ref = sum((xk[r].float() @ wk[r].float().T) for r in range(n))[rank * rows:(rank + 1) * rows].cuda()
        err = ((o.float() - ref).abs() / (ref.abs().mean() + ref.abs())).max().item()
        out["gemm_rs"] = max(out.get("gemm_rs", 0.0), err)
    grs.close()
    assert comm.async_error() == 0, comm.last_error()
    comm.destroy()
    return out


def fsdp_losses(rank, n, uid_unused, port, steps):
    """Tiny Llama through the sharding engine on n GPUs, same batch on every rank."""
    import torch
    import torch.distributed as dist
    from flagcx_b200 import ops
    from flagcx_b200.models.llama import LlamaConfig, build_units
    from flagcx_b200.parallel.fsdp import ShardedModel
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    comm = None
    if n > 1:
        import flagcx_b200.torch_backend as tb
        dist.init_process_group("flagcx", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=n)
        comm = tb.comm_of(dist.group.WORLD, dev)
    cfg = LlamaConfig.tiny()
    ops.assume_unit_loss_grad = True
    model = ShardedModel(build_units(cfg), comm, rank, n, dev, lr=1e-3)
    g = torch.Generator().manual_seed(7)
    tok = torch.randint(0, cfg.vocab, (257,), generator=g).to(dev)
    losses = [round(float(model.train_step(tok[:-1], tok[1:])), 4) for _ in range(steps)]
    if comm is not None:
        assert comm.async_error() == 0, comm.last_error()
    model.close()
    if n > 1:
        dist.barrier()
        dist.destroy_process_group()
    return losses


def torch_fsdp2_losses(rank, n, uid_unused, port, backend):
    """torch's own FSDP (fully_shard) on GPUs over the given backend: per-step losses."""
    import torch
    import torch.distributed as dist
    import torch.nn as nn
    from torch.distributed.fsdp import fully_shard
    import flagcx_b200.torch_backend  # noqa: F401
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group(backend, init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=n)
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(256, 512, bias=False), nn.GELU(), nn.Linear(512, 512, bias=False), nn.GELU(),
                          nn.Linear(512, 64, bias=False)).to(dev).to(torch.bfloat16)
    for layer in model:
        if isinstance(layer, nn.Linear):
            fully_shard(layer)
    fully_shard(model)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
    g = torch.Generator().manual_seed(50 + rank)
    losses = []
    for _ in range(5):
        x = torch.randn(32, 256, generator=g).to(dev).to(torch.bfloat16)
        y = torch.randn(32, 64, generator=g).to(dev).to(torch.bfloat16)
        loss = (model(x).float() - y.float()).pow(2).mean()
        loss.backward()
        opt.step()
        opt.zero_grad()
        t = loss.detach().clone()
        dist.all_reduce(t)
        losses.append(round(float(t) / n, 4))
    torch.cuda.synchronize()
    dist.destroy_process_group()
    return losses


def torch_ddp_parity(rank, n, uid_unused, port, backend, use_cuda):
    """A small model under DistributedDataParallel: returns the losses so that the
    parent can compare backends."""
    import torch
    import torch.distributed as dist
    import flagcx_b200.torch_backend  # noqa: F401
    if use_cuda:
        torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank) if use_cuda else torch.device("cpu")
    dist.init_process_group(backend, init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=n)
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.Tanh(), torch.nn.Linear(64, 8)).to(dev)
    ddp = torch.nn.parallel.DistributedDataParallel(model, device_ids=[rank] if use_cuda else None)
    opt = torch.optim.SGD(ddp.parameters(), lr=0.05)
    losses = []
    g = torch.Generator().manual_seed(100 + rank)
    for _ in range(5):
        x = torch.randn(16, 32, generator=g).to(dev)
        y = torch.randn(16, 8, generator=g).to(dev)
        loss = torch.nn.functional.mse_loss(ddp(x), y)
        opt.zero_grad()
        loss.backward()
        opt.step()
        t = loss.detach().clone()
        dist.all_reduce(t)
        losses.append(float(t) / n)
    dist.destroy_process_group()
    return losses


# ---------------------------------------------------------------------------
# pipeline parallelism
# ---------------------------------------------------------------------------
def _pp_stage_module(stage, width):
    import torch
    g = torch.Generator().manual_seed(100 + stage)
    lin = torch.nn.Linear(width, width)
    with torch.no_grad():
        lin.weight.copy_(torch.randn(width, width, generator=g) * 0.3)
        lin.bias.copy_(torch.randn(width, generator=g) * 0.1)
    return torch.nn.Sequential(lin, torch.nn.Tanh())


def pp_1f1b(rank, n, uid, n_micro, width, use_cuda=False):
    """1F1B over n stages (CPU tensors, or one GPU per stage) against the same model run
    in one process."""
    import torch
    from flagcx_b200.parallel.pp import PipelineStage
    if use_cuda:
        torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank) if use_cuda else torch.device("cpu")
    comm = capi.Comm.init_rank(n, capi.unique_id_from_bytes(uid), rank)
    batch = 4
    g = torch.Generator().manual_seed(7)
    xs = [torch.randn(batch, width, generator=g) for _ in range(n_micro)]
    ts = [torch.randn(batch, width, generator=g) for _ in range(n_micro)]
    stage = PipelineStage(comm, _pp_stage_module(rank, width).to(dev), None if rank == 0 else (batch, width),
                          (batch, width), device=dev)
    loss = stage.run_1f1b(xs if rank == 0 else None, n_micro,
                          (lambda y, i: ((y - ts[i].to(dev)) ** 2).mean() / n_micro) if rank == n - 1 else None)
    if use_cuda:
        torch.cuda.synchronize()
    # reference: the whole model here
    full = [_pp_stage_module(s, width) for s in range(n)]
    ref_loss = 0.0
    for i in range(n_micro):
        y = xs[i]
        for m in full:
            y = m(y)
        l = ((y - ts[i]) ** 2).mean() / n_micro
        l.backward()
        ref_loss += float(l)
    mine, ref = stage.module[0], full[rank][0]
    out = {"grad_w": float((mine.weight.grad.cpu() - ref.weight.grad).abs().max()),
           "grad_b": float((mine.bias.grad.cpu() - ref.bias.grad).abs().max())}
    if rank == n - 1:
        out["loss"] = abs(loss - ref_loss)
    comm.barrier()
    comm.destroy()
    return out


def host_random_stress(rank, n, uid, rounds, seed):
    """Random operations, sizes and per-rank delays on the host path: every rank draws the
    same schedule from `seed` and its own sleeps from (seed, rank)."""
    comm = capi.Comm.init_rank(n, capi.unique_id_from_bytes(uid), rank)
    plan = np.random.default_rng(seed)
    jitter = np.random.default_rng(seed * 1000 + rank)
    worst = 0.0
    for it in range(rounds):
        op = int(plan.integers(0, 5))
        count = int(plan.integers(1, 40000))
        root = int(plan.integers(0, n))
        xs = [np.random.default_rng(seed + 17 * it + r).uniform(-1, 1, count * n).astype(np.float32) for r in range(n)]
        x = xs[rank]
        time.sleep(float(jitter.uniform(0, 0.004)))
        if op == 0:
            out = np.empty_like(x)
            comm.all_reduce(x, out, x.size, capi.FLOAT, capi.SUM)
            worst = max(worst, rel_err(out, np_reduce(xs, capi.SUM)))
        elif op == 1:
            out = np.empty(count * n, np.float32)
            comm.all_gather(x[:count], out, count, capi.FLOAT)
            worst = max(worst, float(not np.array_equal(out, np.concatenate([a[:count] for a in xs]))))
        elif op == 2:
            out = np.empty(count, np.float32)
            comm.reduce_scatter(x, out, count, capi.FLOAT, capi.SUM)
            worst = max(worst, rel_err(out, np_reduce(xs, capi.SUM)[rank * count:(rank + 1) * count]))
        elif op == 3:
            out = np.empty(count * n, np.float32)
            comm.all_to_all(x, out, count, capi.FLOAT)
            want = np.concatenate([xs[p][rank * count:(rank + 1) * count] for p in range(n)])
            worst = max(worst, float(not np.array_equal(out, want)))
        else:
            buf = x[:count].copy()
            comm.broadcast(buf, buf, count, capi.FLOAT, root)
            worst = max(worst, float(not np.array_equal(buf, xs[root][:count])))
    comm.barrier()
    comm.destroy()
    return worst


def gpu_buffers_over_sockets(rank, n, uid):
    """Device buffers on ranks that may not use NVLink (FLAGCX_FORCE_HOST=1): staged through
    pinned memory over the host path.  No kernel of one rank waits for another, so the
    ranks may share a GPU."""
    import torch
    torch.cuda.set_device(0)
    comm = capi.Comm.init_rank(n, capi.unique_id_from_bytes(uid), rank)
    assert not comm.device_path
    count = 100003
    xs = [_torch_seeded(r, count, torch.float32) for r in range(n)]
    x = xs[rank].cuda()
    out = torch.empty_like(x)
    comm.all_reduce(x, out, count, capi.FLOAT, capi.SUM)
    torch.cuda.synchronize()
    ref = torch.stack(xs).double().sum(0)
    worst = {"allreduce": float(((out.cpu().double() - ref).abs() / ref.abs().clamp(min=1)).max())}
    comm.all_reduce(x, x, count, capi.FLOAT, capi.SUM)  # in place
    torch.cuda.synchronize()
    worst["allreduce_inplace"] = float(((x.cpu().double() - ref).abs() / ref.abs().clamp(min=1)).max())
    ag = torch.empty(count * n, device="cuda")
    comm.all_gather(xs[rank].cuda(), ag, count, capi.FLOAT)
    torch.cuda.synchronize()
    worst["allgather"] = float(not torch.equal(ag.cpu(), torch.cat(xs)))
    comm.barrier()
    comm.destroy()
    return worst


# ---------------------------------------------------------------------------
# sequence / context parallelism
# ---------------------------------------------------------------------------
def sp_ulysses_and_ring(rank, n, uid, S, H, D, use_cuda=False):
    """Ulysses re-sharding and ring attention (CPU tensors, or one GPU per rank) against
    full attention."""
    import torch
    from flagcx_b200.parallel.sp import Ulysses, ring_attention
    if use_cuda:
        torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank) if use_cuda else torch.device("cpu")
    comm = capi.Comm.init_rank(n, capi.unique_id_from_bytes(uid), rank)
    g = torch.Generator().manual_seed(11)
    q, k, v = (torch.randn(S, H, D, generator=g).to(dev) for _ in range(3))
    s = S // n
    mine = slice(rank * s, (rank + 1) * s)
    out = {}
    u = Ulysses(comm)
    heads = u.seq_to_heads(q[mine].contiguous())
    h = H // n
    out["seq_to_heads"] = float((heads - q[:, rank * h:(rank + 1) * h]).abs().max())
    out["roundtrip"] = float((u.heads_to_seq(heads) - q[mine]).abs().max())

    def full_attention(causal):
        sc = torch.einsum("shd,thd->hst", q, k) / D ** 0.5
        if causal:
            sc = sc.masked_fill(~torch.ones(S, S, dtype=torch.bool, device=dev).tril(), -float("inf"))
        return torch.einsum("hst,thd->shd", sc.softmax(-1), v)

    for causal in (False, True):
        got = ring_attention(comm, q[mine].contiguous(), k[mine].contiguous(), v[mine].contiguous(), causal=causal)
        out[f"ring_causal{int(causal)}"] = float((got - full_attention(causal)[mine]).abs().max())
    comm.barrier()
    comm.destroy()
    return out


def p2p_engine_pair(rank, n, uid_unused, path, use_cuda):
    """Two processes that share no communicator: rank 0 owns a registered buffer, rank 1
    writes and reads it one-sidedly (whole, by looked-up address, as a vector), both trade
    notifications; bad ranges come back as error codes."""
    import json
    import os
    import time
    from flagcx_b200.p2p import P2pEngine
    N = 1 << 20
    if use_cuda:
        import torch
        ndev = torch.cuda.device_count()
        dev = rank % ndev
        torch.cuda.set_device(dev)
        zeros = lambda k: torch.zeros(k, dtype=torch.uint8, device="cuda")
        pattern = lambda k, seed: ((torch.arange(k, device="cuda", dtype=torch.int64) * (seed * 2 + 1) + seed) % 251).to(torch.uint8)
        equal = lambda a, b: bool(torch.equal(a, b))
        addr = lambda t: t.data_ptr()
        eng = P2pEngine(dev)
    else:
        zeros = lambda k: np.zeros(k, np.uint8)
        pattern = lambda k, seed: ((np.arange(k, dtype=np.int64) * (seed * 2 + 1) + seed) % 251).astype(np.uint8)
        equal = lambda a, b: bool(np.array_equal(a, b))
        addr = lambda t: t.ctypes.data
        eng = P2pEngine(-1)
    out = {}
    if rank == 0:
        buf = zeros(N)
        mr = eng.register(buf)
        with open(path + ".tmp", "w") as f:
            json.dump({"meta": eng.metadata, "desc": eng.describe(mr, buf).hex(), "addr": addr(buf)}, f)
        os.replace(path + ".tmp", path)
        conn = eng.accept(60000)
        assert conn is not None, "nobody connected"
        assert conn.recv_notification(60000) == b"whole buffer written"
        if use_cuda:
            torch.cuda.synchronize()
        out["whole_write"] = float(not equal(buf, pattern(N, 1)))
        conn.notify(b"checked")  # the writer goes on only now: the next writes change the buffer
        assert conn.recv_notification(60000) == b"pieces written"
        want = pattern(N, 1)
        want[4096:4096 + 100] = pattern(100, 2)
        for i in range(3):
            want[65536 * (i + 1): 65536 * (i + 1) + 1000 + i] = pattern(1000 + i, 3 + i)
        if use_cuda:
            torch.cuda.synchronize()
        out["piece_writes"] = float(not equal(buf, want))
        buf[:] = pattern(N, 9)
        if use_cuda:
            torch.cuda.synchronize()
        conn.notify(b"read me")
        assert conn.recv_notification(60000) == b"bye"
        out["is_local"] = float(not conn.is_local)
        conn.close()
        eng.deregister(mr)
    else:
        deadline = time.time() + 60
        while not os.path.exists(path):
            assert time.time() < deadline, "the owner never published its metadata"
            time.sleep(0.05)
        info = json.load(open(path))
        desc = bytes.fromhex(info["desc"])
        conn = eng.connect(info["meta"])
        conn.write(pattern(N, 1), desc)
        conn.notify(b"whole buffer written")
        assert conn.recv_notification(60000) == b"checked"
        small = conn.lookup(info["addr"] + 4096, 100)  # by the owner's virtual address
        conn.write(pattern(100, 2), small)
        pieces = [pattern(1000 + i, 3 + i) for i in range(3)]
        conn.write_vector(pieces, [conn.lookup(info["addr"] + 65536 * (i + 1), 1000 + i) for i in range(3)])
        conn.notify(b"pieces written")
        assert conn.recv_notification(60000) == b"read me"
        got = zeros(N)
        conn.read(got, desc)
        if use_cuda:
            torch.cuda.synchronize()
        out["whole_read"] = float(not equal(got, pattern(N, 9)))
        parts = [zeros(512), zeros(700)]
        conn.read_vector(parts, [conn.lookup(info["addr"] + 10, 512), conn.lookup(info["addr"] + N - 700, 700)])
        out["vector_read"] = float(not (equal(parts[0], pattern(N, 9)[10:522]) and equal(parts[1], pattern(N, 9)[N - 700:])))
        # errors, not faults: a range outside every registered region, more bytes than the descriptor covers
        for name, fn in (("lookup_outside", lambda: conn.lookup(info["addr"] + N - 10, 100)),
                         ("write_too_long", lambda: conn.write(zeros(200), small, nbytes=200))):
            try:
                fn()
                out[name] = 2.0
            except capi.FlagcxError:
                out[name] = 0.0
        # the connection still works afterwards
        conn.read(parts[0], conn.lookup(info["addr"], 512))
        out["after_errors"] = float(not equal(parts[0], pattern(N, 9)[:512]))
        assert conn.recv_notification(10) is None  # nothing pending: times out cleanly
        out["is_local"] = float(not conn.is_local)
        conn.notify(b"bye")
        conn.close()
    eng.close()
    return out


def p2p_engine_owner_dies(rank, n, uid_unused, path):
    """Failure on the host: the owner of the memory exits after the first transfer.  The
    initiator's next calls come back with an error code within the socket deadline."""
    import json
    import os
    import time
    from flagcx_b200.p2p import P2pEngine
    eng = P2pEngine(-1)
    if rank == 0:
        buf = np.zeros(1 << 16, np.uint8)
        mr = eng.register(buf)
        with open(path + ".tmp", "w") as f:
            json.dump({"meta": eng.metadata, "desc": eng.describe(mr, buf).hex()}, f)
        os.replace(path + ".tmp", path)
        conn = eng.accept(60000)
        assert conn.recv_notification(60000) == b"first done"
        os._exit(0)  # no goodbye, no socket shutdown by the library
    deadline = time.time() + 60
    while not os.path.exists(path):
        assert time.time() < deadline
        time.sleep(0.05)
    info = json.load(open(path))
    conn = eng.connect(info["meta"])
    src = np.ones(1 << 16, np.uint8)
    conn.write(src, bytes.fromhex(info["desc"]))
    conn.notify(b"first done")
    time.sleep(0.5)
    out = {}
    t0 = time.time()
    for name, fn in (("write", lambda: conn.write(src, bytes.fromhex(info["desc"]))),
                     ("notify", lambda: conn.notify(b"anyone?")),
                     ("read", lambda: conn.read(src, bytes.fromhex(info["desc"])))):
        try:
            fn()
            out[name] = 0
        except capi.FlagcxError as e:
            out[name] = e.code
    out["seconds"] = time.time() - t0
    conn.close()
    eng.close()
    return out

