"""Single-GPU tier: every collective kernel, run as an emulated world (all ranks in
one cooperative launch, see flagcxEmuWorldCreate) and compared with a plain PyTorch
fp64/fp32 reference computed from the same seeded inputs."""
import os

import pytest
import torch

from flagcx_b200 import capi

pytestmark = pytest.mark.gpu

TORCH_DT = {
    capi.FLOAT: torch.float32, capi.BFLOAT16: torch.bfloat16, capi.HALF: torch.float16,
    capi.DOUBLE: torch.float64, capi.INT32: torch.int32, capi.INT64: torch.int64,
    capi.UINT8: torch.uint8, capi.INT8: torch.int8,
}
_worlds = {}


def world(n):
    if n not in _worlds:
        _worlds[n] = capi.Comm.emu_world(n, 0)
    return _worlds[n]


@pytest.fixture(scope="module", autouse=True)
def _teardown():
    yield
    torch.cuda.synchronize()
    for comms in _worlds.values():
        capi.Comm.emu_world_destroy(comms)
    _worlds.clear()


def make_inputs(n, count, dt, lo=-1.0, hi=1.0):
    tdt = TORCH_DT[dt]
    xs = []
    for r in range(n):
        g = torch.Generator().manual_seed(r)
        if tdt.is_floating_point:
            x = torch.rand(count, generator=g, dtype=torch.float64) * (hi - lo) + lo
        elif tdt == torch.uint8:
            x = torch.randint(0, 3, (count,), generator=g)
        else:
            x = torch.randint(-2, 3, (count,), generator=g)
        xs.append(x.to(tdt).cuda())
    return xs


def reference(xs, op):
    acc = torch.stack([x.cpu().to(torch.float64) for x in xs])
    if op == capi.SUM:
        return acc.sum(0)
    if op == capi.AVG:
        return acc.sum(0) / len(xs)
    if op == capi.PROD:
        return acc.prod(0)
    if op == capi.MAX:
        return acc.max(0).values
    return acc.min(0).values


def tol(dt, n):
    return {capi.BFLOAT16: 2 ** -7, capi.HALF: 2 ** -10}.get(dt, 1e-6 if dt == capi.FLOAT else 1e-12) * max(1, n // 2)


def check_close(got, ref, dt, n, what):
    got = got.cpu().to(torch.float64)
    if not TORCH_DT[dt].is_floating_point:
        assert torch.equal(got, ref), what
        return
    err = ((got - ref).abs() / ref.abs().clamp(min=1.0)).max().item()
    assert err <= tol(dt, n), f"{what}: rel err {err}"


def assert_no_device_error(comms):
    for c in comms:
        assert c.async_error() == capi.flagcxSuccess, c.last_error()


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("algo", [capi.ALGO_ONESHOT, capi.ALGO_TWOSHOT])
@pytest.mark.parametrize("dt", [capi.FLOAT, capi.BFLOAT16, capi.HALF])
@pytest.mark.parametrize("count", [1, 7, 4099, (1 << 18) + 3])
def test_allreduce_sum(n, algo, dt, count):
    comms = world(n)
    xs = make_inputs(n, count, dt)
    outs = [torch.empty_like(x) for x in xs]
    for r in range(n):
        comms[r].all_reduce_fused(xs[r], outs[r], count, dt, capi.SUM, algo=algo)
    torch.cuda.synchronize()
    assert_no_device_error(comms)
    ref = reference(xs, capi.SUM)
    for r in range(n):
        check_close(outs[r], ref, dt, n, f"rank {r}")
    # every rank must hold bit-identical results
    for r in range(1, n):
        assert torch.equal(outs[r], outs[0])


@pytest.mark.parametrize("dt", [capi.FLOAT, capi.DOUBLE, capi.INT32, capi.INT64, capi.UINT8, capi.INT8, capi.BFLOAT16])
@pytest.mark.parametrize("op", [capi.SUM, capi.PROD, capi.MAX, capi.MIN, capi.AVG])
def test_allreduce_all_ops_and_types(dt, op):
    n, count = 3, 1031
    comms = world(n)
    xs = make_inputs(n, count, dt)
    outs = [torch.empty_like(x) for x in xs]
    for r in range(n):
        comms[r].all_reduce(xs[r], outs[r], count, dt, op)
    torch.cuda.synchronize()
    assert_no_device_error(comms)
    ref = reference(xs, op)
    if not TORCH_DT[dt].is_floating_point:
        if op == capi.AVG:
            ref = torch.stack([x.cpu().to(torch.int64) for x in xs]).sum(0)
            ref = torch.div(ref, n, rounding_mode="trunc").to(torch.float64)
        wrapped = ref.to(torch.int64).to(TORCH_DT[dt]).to(torch.float64)
        for r in range(n):
            assert torch.equal(outs[r].cpu().to(torch.float64), wrapped), (dt, op, r)
    else:
        for r in range(n):
            check_close(outs[r], ref, dt, n, f"op {op} rank {r}")


@pytest.mark.parametrize("n", [2, 8])
def test_allreduce_in_place_and_large(n):
    count = (3 << 20) + 8
    comms = world(n)
    xs = make_inputs(n, count, capi.BFLOAT16)
    ref = reference(xs, capi.SUM)
    for r in range(n):
        comms[r].all_reduce(xs[r], xs[r], count, capi.BFLOAT16, capi.SUM)
    torch.cuda.synchronize()
    assert_no_device_error(comms)
    for r in range(n):
        check_close(xs[r], ref, capi.BFLOAT16, n, f"in-place rank {r}")


@pytest.mark.parametrize("n", [2, 4])
@pytest.mark.parametrize("algo", [capi.ALGO_ONESHOT, capi.ALGO_TWOSHOT])
def test_allreduce_fused_scale_cast_residual(n, algo):
    """bf16 in, 1/world scale, fp32 out, residual add -- all inside the collective."""
    count = 70001
    comms = world(n)
    xs = make_inputs(n, count, capi.BFLOAT16)
    res = torch.rand(count, dtype=torch.float32).cuda()
    outs = [torch.empty(count, dtype=torch.float32, device="cuda") for _ in range(n)]
    for r in range(n):
        comms[r].all_reduce_fused(xs[r], outs[r], count, capi.BFLOAT16, capi.SUM, scale=1.0 / n,
                                  out_dtype=capi.FLOAT, residual=res, algo=algo)
    torch.cuda.synchronize()
    assert_no_device_error(comms)
    ref = reference(xs, capi.SUM) / n + res.cpu().to(torch.float64)
    # one-shot: fp32 accumulation, single rounding to fp32.  two-shot: the reduced, scaled
    # slice crosses NVLink in the input type, so it is rounded once to bf16 before widening.
    bound = 1e-5 if algo == capi.ALGO_ONESHOT else 2 ** -8
    for r in range(n):
        err = (outs[r].cpu().to(torch.float64) - ref).abs().max().item()
        assert err < bound, err
        assert torch.equal(outs[r], outs[0]), "ranks must agree bit for bit"


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("count", [8 * 1024 * 8, 100003])
def test_allreduce_two_shot_with_widening_result(n, count):
    """fp16/bf16 in, fp32 out over the two-shot path, with and without a residual, also
    from buffers that are not 16-byte aligned."""
    comms = world(n)
    for dt in (capi.BFLOAT16, capi.HALF):
        for shift in (0, 1):
            xs = [x[shift:] for x in make_inputs(n, count + shift, dt)]
            res = torch.rand(count + shift, dtype=torch.float32).cuda()[shift:]
            for use_res in (False, True):
                outs = [torch.zeros(count + shift, dtype=torch.float32, device="cuda")[shift:] for _ in range(n)]
                for r in range(n):
                    comms[r].all_reduce_fused(xs[r], outs[r], count, dt, capi.SUM, scale=0.5, out_dtype=capi.FLOAT,
                                              residual=res if use_res else None, algo=capi.ALGO_TWOSHOT)
                torch.cuda.synchronize()
                assert_no_device_error(comms)
                ref = reference(xs, capi.SUM) * 0.5
                for r in range(n):
                    got = outs[r].cpu().to(torch.float64) - (res.cpu().to(torch.float64) if use_res else 0)
                    err = ((got - ref).abs() / ref.abs().clamp(min=1.0)).max().item()
                    assert err <= tol(dt, n), (dt, shift, use_res, err)
                    assert torch.equal(outs[r], outs[0])


@pytest.mark.parametrize("n", [2, 3, 8])
@pytest.mark.parametrize("dt", [capi.FLOAT, capi.BFLOAT16, capi.DOUBLE, capi.INT8])
def test_small_messages_without_barrier(n, dt):
    """The LL path (data and flag in one store, no barrier): every count from 1 to 257,
    out of place and in place, several operations back to back so that both slot
    parities are reused, plus the largest message a slot holds."""
    comms = world(n)
    es = torch.empty((), dtype=TORCH_DT[dt]).element_size()
    counts = list(range(1, 258, 1 if dt == capi.BFLOAT16 else 7)) + [65536 // es]
    for count in counts:
        xs = make_inputs(n, count + 1, dt)
        ref = reference([x[1:] for x in xs], capi.SUM)
        if not TORCH_DT[dt].is_floating_point:
            ref = ref.to(torch.int64).to(TORCH_DT[dt]).to(torch.float64)
        outs = [torch.zeros_like(x) for x in xs]
        for r in range(n):  # views one element into the allocation: not 8-byte aligned for small types
            comms[r].all_reduce_fused(xs[r][1:], outs[r][1:], count, dt, capi.SUM, algo=capi.ALGO_LL)
        for r in range(n):  # in place
            comms[r].all_reduce_fused(xs[r][1:], xs[r][1:], count, dt, capi.SUM, algo=capi.ALGO_LL)
        torch.cuda.synchronize()
        assert_no_device_error(comms)
        assert comms[0].stats(capi.OP_ALLREDUCE).lastAlgo == capi.ALGO_LL
        for r in range(n):
            check_close(outs[r][1:], ref, dt, n, f"LL count {count} rank {r}")
            assert torch.equal(xs[r][1:], outs[r][1:]), "in place"
            assert torch.equal(outs[r], outs[0])
            assert float(outs[r][0]) == 0.0, "wrote before the buffer"


@pytest.mark.parametrize("n", [2, 3, 4, 8])
@pytest.mark.parametrize("exchange", [False, True])
def test_ring_algorithms(n, exchange):
    """Ring all-reduce, reduce-scatter and all-gather (n-1 neighbour-to-neighbour steps)
    against the fp64 reference, odd and large counts, several calls in a row (the step
    flags only ever count up)."""
    if exchange:
        os.environ["FLAGCX_EMU_EXCHANGE"] = "1"
    try:
        comms = world(n)
        for dt in (capi.FLOAT, capi.BFLOAT16):
            for count in (5, 4099, (1 << 17) + 40):
                xs = make_inputs(n, count * n, dt)
                ref = reference(xs, capi.SUM)
                outs = [torch.zeros_like(x) for x in xs]
                for r in range(n):
                    comms[r].all_reduce_fused(xs[r], outs[r], count * n, dt, capi.SUM, algo=capi.ALGO_RING)
                rs = [torch.zeros(count, dtype=TORCH_DT[dt], device="cuda") for _ in range(n)]
                for r in range(n):
                    comms[r].reduce_scatter_fused(xs[r], rs[r], count, dt, capi.AVG, algo=capi.ALGO_RING)
                ag = [torch.zeros(count * n, dtype=TORCH_DT[dt], device="cuda") for _ in range(n)]
                for r in range(n):
                    comms[r].all_gather(rs[r], ag[r], count, dt, algo=capi.ALGO_RING)
                torch.cuda.synchronize()
                assert_no_device_error(comms)
                assert comms[0].stats(capi.OP_ALLREDUCE).lastAlgo == capi.ALGO_RING
                assert comms[0].stats(capi.OP_REDUCESCATTER).lastAlgo == capi.ALGO_RING
                for r in range(n):
                    # partial sums travel in the element type: one rounding per hop
                    check_close(outs[r], ref, dt, 4 * n, f"ring allreduce n={n} count={count} rank {r}")
                    assert torch.equal(outs[r], outs[0]), "ranks must agree bit for bit"
                    check_close(rs[r], ref[r * count:(r + 1) * count] / n, dt, 4 * n, f"ring reduce-scatter rank {r}")
                    assert torch.equal(ag[r], torch.cat(rs)), f"ring allgather rank {r}"
    finally:
        if exchange:
            del os.environ["FLAGCX_EMU_EXCHANGE"]


@pytest.mark.parametrize("n", [2, 4, 8])
def test_small_reduce_scatter_and_alltoall_without_barrier(n):
    comms = world(n)
    for dt in (capi.FLOAT, capi.BFLOAT16):
        for count in (1, 3, 257, 1024):
            xs = make_inputs(n, count * n, dt)
            ref = reference(xs, capi.SUM)
            rs = [torch.zeros(count, dtype=TORCH_DT[dt], device="cuda") for _ in range(n)]
            aa = [torch.zeros(count * n, dtype=TORCH_DT[dt], device="cuda") for _ in range(n)]
            for _ in range(2):  # both slot parities
                for r in range(n):
                    comms[r].reduce_scatter_fused(xs[r], rs[r], count, dt, capi.SUM, algo=capi.ALGO_LL)
                for r in range(n):
                    comms[r].all_to_all(xs[r], aa[r], count, dt)  # small blocks: the heuristic's own choice
            torch.cuda.synchronize()
            assert_no_device_error(comms)
            assert comms[0].stats(capi.OP_REDUCESCATTER).lastAlgo == capi.ALGO_LL
            assert comms[0].stats(capi.OP_ALLTOALL).lastAlgo == capi.ALGO_LL
            for r in range(n):
                check_close(rs[r], ref[r * count:(r + 1) * count], dt, n, f"LL reduce-scatter count {count} rank {r}")
                assert torch.equal(aa[r], torch.cat([xs[p][r * count:(r + 1) * count] for p in range(n)])), "LL alltoall"


def test_small_allgather_without_barrier():
    n = 4
    comms = world(n)
    for count in (1, 3, 64, 1001, 8192):
        xs = [x for x in make_inputs(n, count, capi.BFLOAT16)]
        outs = [torch.zeros(count * n, dtype=torch.bfloat16, device="cuda") for _ in range(n)]
        for r in range(n):
            comms[r].all_gather(xs[r], outs[r], count, capi.BFLOAT16, algo=capi.ALGO_LL)
        torch.cuda.synchronize()
        assert_no_device_error(comms)
        assert comms[0].stats(capi.OP_ALLGATHER).lastAlgo == capi.ALGO_LL
        for r in range(n):
            assert torch.equal(outs[r], torch.cat(xs)), (count, r)


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("dt", [capi.FLOAT, capi.BFLOAT16])
@pytest.mark.parametrize("count", [5, 1000, 65536 + 8])
def test_reduce_scatter_and_allgather(n, dt, count):
    comms = world(n)
    xs = make_inputs(n, count * n, dt)
    outs = [torch.empty(count, dtype=TORCH_DT[dt], device="cuda") for _ in range(n)]
    for r in range(n):
        comms[r].reduce_scatter(xs[r], outs[r], count, dt, capi.SUM)
    torch.cuda.synchronize()
    assert_no_device_error(comms)
    ref = reference(xs, capi.SUM)
    for r in range(n):
        check_close(outs[r], ref[r * count:(r + 1) * count], dt, n, f"reduce-scatter rank {r}")
    # allgather, both directions of data movement
    for algo in (capi.ALGO_PUSH, capi.ALGO_PULL):
        gath = [torch.zeros(count * n, dtype=TORCH_DT[dt], device="cuda") for _ in range(n)]
        for r in range(n):
            comms[r].all_gather(outs[r], gath[r], count, dt, algo=algo)
        torch.cuda.synchronize()
        assert_no_device_error(comms)
        want = torch.cat(outs)
        for r in range(n):
            assert torch.equal(gath[r], want), f"allgather algo {algo} rank {r}"


def test_reduce_scatter_fused_average_to_fp32():
    n, count = 4, 12345
    comms = world(n)
    xs = make_inputs(n, count * n, capi.BFLOAT16)
    outs = [torch.empty(count, dtype=torch.float32, device="cuda") for _ in range(n)]
    for r in range(n):
        comms[r].reduce_scatter_fused(xs[r], outs[r], count, capi.BFLOAT16, capi.AVG, out_dtype=capi.FLOAT)
    torch.cuda.synchronize()
    assert_no_device_error(comms)
    ref = reference(xs, capi.AVG)
    for r in range(n):
        err = (outs[r].cpu().to(torch.float64) - ref[r * count:(r + 1) * count]).abs().max().item()
        assert err < 1e-5, err


@pytest.mark.parametrize("n", [2, 4, 8])
def test_rooted_and_alltoall(n):
    comms = world(n)
    count, dt = 3001, capi.FLOAT
    xs = make_inputs(n, count * n, dt)
    root = n - 1
    # broadcast
    bs = [xs[r][:count].clone() for r in range(n)]
    for r in range(n):
        comms[r].broadcast(bs[r], bs[r], count, dt, root)
    # reduce
    rd = [torch.zeros(count, device="cuda") for _ in range(n)]
    for r in range(n):
        comms[r].reduce(xs[r], rd[r], count, dt, capi.MAX, root)
    # gather
    ga = [torch.zeros(count * n, device="cuda") for _ in range(n)]
    for r in range(n):
        comms[r].gather(xs[r], ga[r], count, dt, root)
    # scatter
    sc = [torch.zeros(count, device="cuda") for _ in range(n)]
    for r in range(n):
        comms[r].scatter(xs[r], sc[r], count, dt, root)
    # alltoall
    aa = [torch.zeros(count * n, device="cuda") for _ in range(n)]
    for r in range(n):
        comms[r].all_to_all(xs[r], aa[r], count, dt)
    torch.cuda.synchronize()
    assert_no_device_error(comms)
    for r in range(n):
        assert torch.equal(bs[r], xs[root][:count]), "broadcast"
        assert torch.equal(sc[r], xs[root][r * count:(r + 1) * count]), "scatter"
        want = torch.cat([xs[p][r * count:(r + 1) * count] for p in range(n)])
        assert torch.equal(aa[r], want), "alltoall"
    assert torch.equal(rd[root], torch.stack([x[:count] for x in xs]).max(0).values), "reduce"
    assert torch.equal(ga[root], torch.cat([x[:count] for x in xs])), "gather"


def test_alltoallv_and_grouped_sendrecv():
    n = 4
    comms = world(n)
    counts = [[(r + p) % 4 * 100 + 3 for p in range(n)] for r in range(n)]  # counts[r][p]: r -> p
    sends, recvs, sd, rd = [], [], [], []
    for r in range(n):
        sc, rc = counts[r], [counts[p][r] for p in range(n)]
        sd.append([sum(sc[:i]) for i in range(n)])
        rd.append([sum(rc[:i]) for i in range(n)])
        sends.append((torch.arange(sum(sc), dtype=torch.float32) + 10000 * r).cuda())
        recvs.append(torch.zeros(sum(rc), device="cuda"))
    for r in range(n):
        comms[r].all_to_allv(sends[r], counts[r], sd[r], recvs[r], [counts[p][r] for p in range(n)], rd[r], capi.FLOAT)
    torch.cuda.synchronize()
    assert_no_device_error(comms)
    for r in range(n):
        for p in range(n):
            want = sends[p][sd[p][r]:sd[p][r] + counts[p][r]]
            assert torch.equal(recvs[r][rd[r][p]:rd[r][p] + counts[p][r]], want)
    # ring exchange through the point-to-point kernel, message larger than one slot chunk
    big = (5 << 20) // 4 + 17
    xs = make_inputs(n, big, capi.FLOAT)
    got = [torch.zeros(big, device="cuda") for _ in range(n)]
    for r in range(n):
        comms[r].group_start()
        comms[r].send(xs[r], big, capi.FLOAT, (r + 1) % n)
        comms[r].recv(got[r], big, capi.FLOAT, (r - 1) % n)
        comms[r].group_end()
    torch.cuda.synchronize()
    assert_no_device_error(comms)
    for r in range(n):
        assert torch.equal(got[r], xs[(r - 1) % n])


def test_staged_paths_for_unregistered_buffers():
    """Same kernels with the copy-in/copy-out staging that unregistered buffers take."""
    os.environ["FLAGCX_EMU_FORCE_STAGING"] = "1"
    try:
        n = 4
        comms = world(n)
        count = (1 << 20) + 24
        for dt in (capi.FLOAT, capi.BFLOAT16):
            xs = make_inputs(n, count, dt)
            ref = reference(xs, capi.SUM)
            for algo in (capi.ALGO_ONESHOT, capi.ALGO_TWOSHOT):
                outs = [torch.empty_like(x) for x in xs]
                for r in range(n):
                    comms[r].all_reduce_fused(xs[r], outs[r], count, dt, capi.SUM, algo=algo)
                torch.cuda.synchronize()
                assert_no_device_error(comms)
                for r in range(n):
                    check_close(outs[r], ref, dt, n, f"staged algo {algo} rank {r}")
        per = 50000
        xs = make_inputs(n, per * n, capi.FLOAT)
        rs = [torch.empty(per, device="cuda") for _ in range(n)]
        for r in range(n):
            comms[r].reduce_scatter(xs[r], rs[r], per, capi.FLOAT, capi.SUM)
        ag = [torch.empty(per * n, device="cuda") for _ in range(n)]
        for r in range(n):
            comms[r].all_gather(rs[r], ag[r], per, capi.FLOAT)
        aa = [torch.empty(per * n, device="cuda") for _ in range(n)]
        for r in range(n):
            comms[r].all_to_all(xs[r], aa[r], per, capi.FLOAT)
        bc = [xs[r][:per].clone() for r in range(n)]
        for r in range(n):
            comms[r].broadcast(bc[r], bc[r], per, capi.FLOAT, 1)
        torch.cuda.synchronize()
        assert_no_device_error(comms)
        ref = reference(xs, capi.SUM)
        for r in range(n):
            check_close(rs[r], ref[r * per:(r + 1) * per], capi.FLOAT, n, "staged reduce-scatter")
            assert torch.equal(ag[r], torch.cat(rs)), "staged allgather"
            assert torch.equal(aa[r], torch.cat([xs[p][r * per:(r + 1) * per] for p in range(n)])), "staged alltoall"
            assert torch.equal(bc[r], xs[1][:per]), "staged broadcast"
    finally:
        del os.environ["FLAGCX_EMU_FORCE_STAGING"]


def _all_collectives_once(n, count, dt, shift):
    """Every collective on fresh buffers that start `shift` elements into their allocation."""
    comms = world(n)
    tdt = TORCH_DT[dt]

    def buf(numel, fill=None):
        t = torch.zeros(numel + shift, dtype=tdt, device="cuda")[shift:]
        if fill is not None:
            t.copy_(fill)
        return t

    xs = [buf(count * n, x) for x in make_inputs(n, count * n, dt)]
    ref = reference(xs, capi.SUM)
    # all-reduce: one-shot out of place, two-shot out of place and in place
    for algo, inplace in ((capi.ALGO_ONESHOT, False), (capi.ALGO_TWOSHOT, False), (capi.ALGO_TWOSHOT, True)):
        ins = [buf(count * n, x) for x in xs]
        outs = ins if inplace else [buf(count * n) for _ in range(n)]
        for r in range(n):
            comms[r].all_reduce_fused(ins[r], outs[r], count * n, dt, capi.SUM, algo=algo)
        torch.cuda.synchronize()
        assert_no_device_error(comms)
        for r in range(n):
            check_close(outs[r], ref, dt, n, f"allreduce algo {algo} inplace {inplace} rank {r}")
    rs = [buf(count) for _ in range(n)]
    for r in range(n):
        comms[r].reduce_scatter(xs[r], rs[r], count, dt, capi.SUM)
    torch.cuda.synchronize()
    for r in range(n):
        check_close(rs[r], ref[r * count:(r + 1) * count], dt, n, f"reduce-scatter rank {r}")
    for algo in (capi.ALGO_PUSH, capi.ALGO_PULL):
        ag = [buf(count * n) for _ in range(n)]
        for r in range(n):
            comms[r].all_gather(rs[r], ag[r], count, dt, algo=algo)
        torch.cuda.synchronize()
        for r in range(n):
            assert torch.equal(ag[r], torch.cat(rs)), f"allgather algo {algo} rank {r}"
    # all-gather in place: the input is the rank's own block of the output
    ag = [buf(count * n) for _ in range(n)]
    for r in range(n):
        ag[r][r * count:(r + 1) * count].copy_(rs[r])
        comms[r].all_gather(ag[r][r * count:(r + 1) * count], ag[r], count, dt)
    torch.cuda.synchronize()
    for r in range(n):
        assert torch.equal(ag[r], torch.cat(rs)), f"in-place allgather rank {r}"
    aa = [buf(count * n) for _ in range(n)]
    for r in range(n):
        comms[r].all_to_all(xs[r], aa[r], count, dt)
    root = n - 1
    bc = [buf(count, xs[r][:count]) for r in range(n)]
    for r in range(n):
        comms[r].broadcast(bc[r], bc[r], count, dt, root)
    rd = [buf(count) for _ in range(n)]
    for r in range(n):
        comms[r].reduce(xs[r], rd[r], count, dt, capi.SUM, root)
    ga = [buf(count * n) for _ in range(n)]
    for r in range(n):
        comms[r].gather(xs[r], ga[r], count, dt, root)
    sc = [buf(count) for _ in range(n)]
    for r in range(n):
        comms[r].scatter(xs[r], sc[r], count, dt, root)
    torch.cuda.synchronize()
    assert_no_device_error(comms)
    for r in range(n):
        assert torch.equal(aa[r], torch.cat([xs[p][r * count:(r + 1) * count] for p in range(n)])), "alltoall"
        assert torch.equal(bc[r], xs[root][:count]), "broadcast"
        assert torch.equal(sc[r], xs[root][r * count:(r + 1) * count]), "scatter"
    check_close(rd[root], reference([x[:count] for x in xs], capi.SUM), dt, n, "reduce")
    assert torch.equal(ga[root], torch.cat([x[:count] for x in xs])), "gather"


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("shift", [0, 1])
def test_pointer_exchange_for_buffers_outside_windows(n, shift):
    """Buffers that are not inside a symmetric window: every rank tells its peers inside
    the kernel where its buffer is (the path ordinary torch tensors take between
    processes).  shift=1 starts every buffer off a 16-byte boundary."""
    os.environ["FLAGCX_EMU_EXCHANGE"] = "1"
    try:
        _all_collectives_once(n, 3001, capi.FLOAT, shift)
        _all_collectives_once(n, 777, capi.BFLOAT16, shift)
    finally:
        del os.environ["FLAGCX_EMU_EXCHANGE"]


def test_pointer_exchange_alltoallv():
    os.environ["FLAGCX_EMU_EXCHANGE"] = "1"
    try:
        n = 4
        comms = world(n)
        counts = [[(r * 3 + p) % 5 * 64 + (1 if (r + p) % 2 else 0) for p in range(n)] for r in range(n)]
        sends, recvs, sd, rd = [], [], [], []
        for r in range(n):
            sc, rc = counts[r], [counts[p][r] for p in range(n)]
            sd.append([sum(sc[:i]) for i in range(n)])
            rd.append([sum(rc[:i]) for i in range(n)])
            sends.append((torch.arange(sum(sc), dtype=torch.float32) + 10000 * r).cuda())
            recvs.append(torch.zeros(sum(rc), device="cuda"))
        for _ in range(3):  # consecutive launches alternate the pad parity
            for r in range(n):
                comms[r].all_to_allv(sends[r], counts[r], sd[r], recvs[r], [counts[p][r] for p in range(n)], rd[r],
                                     capi.FLOAT)
        torch.cuda.synchronize()
        assert_no_device_error(comms)
        for r in range(n):
            for p in range(n):
                want = sends[p][sd[p][r]:sd[p][r] + counts[p][r]]
                assert torch.equal(recvs[r][rd[r][p]:rd[r][p] + counts[p][r]], want)
    finally:
        del os.environ["FLAGCX_EMU_EXCHANGE"]


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("exchange", [False, True])
def test_bulk_copy_engine_paths(n, exchange):
    """The large-message paths (one thread per CTA driving bulk copies through a ring of
    shared-memory stages; reduce inputs fetched by bulk loads), forced at small sizes."""
    env = {"FLAGCX_BULK_COPY_MIN_BYTES": "65536", "FLAGCX_BULK_ALLREDUCE_MIN_BYTES": "65536"}
    if exchange:
        env["FLAGCX_EMU_EXCHANGE"] = "1"
    os.environ.update(env)
    try:
        comms = world(n)
        for dt, count in ((capi.BFLOAT16, (1 << 19) + 8 * n), (capi.FLOAT, 3 * (1 << 17))):
            xs = make_inputs(n, count * n, dt)
            ref = reference(xs, capi.SUM)
            outs = [torch.empty_like(x) for x in xs]
            for r in range(n):
                comms[r].all_reduce_fused(xs[r], outs[r], count * n, dt, capi.SUM, algo=capi.ALGO_TWOSHOT)
            rs = [torch.empty(count, dtype=TORCH_DT[dt], device="cuda") for _ in range(n)]
            for r in range(n):
                comms[r].reduce_scatter(xs[r], rs[r], count, dt, capi.SUM)
            ag = [torch.zeros(count * n, dtype=TORCH_DT[dt], device="cuda") for _ in range(n)]
            for r in range(n):
                comms[r].all_gather(rs[r], ag[r], count, dt, algo=capi.ALGO_PUSH)
            aa = [torch.zeros(count * n, dtype=TORCH_DT[dt], device="cuda") for _ in range(n)]
            for r in range(n):
                comms[r].all_to_all(xs[r], aa[r], count, dt)
            bc = [xs[r][:count * n].clone() for r in range(n)]
            for r in range(n):
                comms[r].broadcast(bc[r], bc[r], count * n, dt, 0)
            torch.cuda.synchronize()
            assert_no_device_error(comms)
            for r in range(n):
                check_close(outs[r], ref, dt, n, f"two-shot rank {r}")
                check_close(rs[r], ref[r * count:(r + 1) * count], dt, n, f"reduce-scatter rank {r}")
                assert torch.equal(ag[r], torch.cat(rs)), f"allgather rank {r}"
                assert torch.equal(aa[r], torch.cat([xs[p][r * count:(r + 1) * count] for p in range(n)])), "alltoall"
                assert torch.equal(bc[r], xs[0]), "broadcast"
    finally:
        for k in env:
            del os.environ[k]


def test_barrier_and_stats():
    n = 8
    comms = world(n)
    for r in range(n):
        comms[r].barrier()
    torch.cuda.synchronize()
    assert_no_device_error(comms)
    st = comms[0].stats(capi.OP_ALLREDUCE)
    assert st.calls > 0 and st.bytes > 0 and st.lastCtas >= 1


def test_wait_that_nobody_satisfies_times_out_cleanly():
    """A device-side wait on a signal no rank ever raises must give up after the
    communicator's time limit and report it, leaving the GPU usable."""
    comms = capi.Comm.emu_world(2, 0)
    try:
        comms[0].set_wait_timeout_ms(200)
        desc = capi.WaitSignalDesc(1, 1)
        capi.check(capi.lib().flagcxWaitSignal(1, capi.C.byref(desc), comms[0].h, None), "flagcxWaitSignal")
        torch.cuda.synchronize()
        assert comms[0].async_error() == capi.flagcxRemoteError
        assert "timed out" in comms[0].last_error()
        # the context is still healthy
        x = torch.ones(1024, device="cuda")
        assert float((x * 2).sum()) == 2048.0
    finally:
        capi.Comm.emu_world_destroy(comms)
