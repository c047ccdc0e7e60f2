"""CPU tier: collectives on host buffers over the TCP bootstrap + socket adaptor,
checked against numpy, and host-side failure detection.  No GPU needed."""
import socket

import numpy as np
import pytest

from flagcx_b200 import capi
from tests._mp import run_ranks


def test_version_and_error_strings():
    v = capi.C.c_int()
    capi.check(capi.lib().flagcxGetVersion(capi.C.byref(v)), "flagcxGetVersion")
    assert v.value == 1300
    assert b"invalid argument" in capi.lib().flagcxGetErrorString(capi.flagcxInvalidArgument)
    assert capi.lib().getFlagcxDataTypeSize(capi.BFLOAT16) == 2
    assert capi.lib().getFlagcxDataTypeSize(capi.DOUBLE) == 8


@pytest.mark.parametrize("shm", [0, 1])
def test_world2_fp32_1mi_elements_matches_numpy(shm):
    """The headline CPU configuration: world_size=2, fp32, 1,048,576 elements, seed=rank,
    1e-6 relative error.  shm=0: over the socket adaptor; shm=1: over the shared-memory
    rings that ranks of one machine use by default."""
    res = run_ranks(2, "host_collectives", 1 << 20, capi.FLOAT, env={"FLAGCX_HOST_SHM": shm})
    for rank, errs in res.items():
        for name, e in errs.items():
            assert e <= 1e-6, (rank, name, e)


@pytest.mark.parametrize("shm", [0, 1])
@pytest.mark.parametrize("n", [1, 3, 4])
def test_other_world_sizes(n, shm):
    res = run_ranks(n, "host_collectives", 12 * 1024, capi.DOUBLE, env={"FLAGCX_HOST_SHM": shm})
    for errs in res.values():
        assert all(e <= 1e-12 for e in errs.values()), errs


@pytest.mark.parametrize("shm", [0, 1])
def test_every_op_dtype_and_reduction(shm):
    res = run_ranks(3, "host_all_ops", 1237, env={"FLAGCX_HOST_SHM": shm})
    assert all(w <= 1e-5 for w in res.values()), res


def test_multi_socket_striping_and_helper_threads():
    env = {"FLAGCX_NSOCKS_PERTHREAD": 2, "FLAGCX_SOCKET_NTHREADS": 2, "FLAGCX_SOCKET_STRIPE_MIN": 4096,
           "FLAGCX_HOST_SHM": 0}
    res = run_ranks(2, "host_collectives", 1 << 18, capi.FLOAT, env=env)
    for errs in res.values():
        assert all(e <= 1e-6 for e in errs.values()), errs


def test_net_adaptor_plugin_carries_the_host_collectives():
    """csrc/plugin/net_example.cc, built here, replaces the socket adaptor
    (role of adaptor_plugin/net in the FlagCX project)."""
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    subprocess.run(["make", "-C", os.path.join(root, "csrc"), "plugin-example"], check=True, capture_output=True)
    plugin = os.path.join(root, "flagcx_b200", "lib", "libflagcx_net_example.so")
    count = 50000
    res = run_ranks(3, "host_collectives_through_plugin", count, plugin,
                    env={"FLAGCX_NET_ADAPTOR_PLUGIN": plugin}, timeout=120)
    for rank, out in res.items():
        assert out["plugin_bytes_sent"] >= count * 4 and out["plugin_messages"] > 0, (rank, out)
        errs = {k: v for k, v in out.items() if not k.startswith("plugin_") and v > 1e-5}
        assert not errs, (rank, errs)


def test_comm_id_environment_rendezvous():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    res = run_ranks(3, "comm_id_env", env={"FLAGCX_COMM_ID": f"127.0.0.1:{port}"})
    assert all(v == 6.0 for v in res.values()), res


# ---- failure detection on the host ---------------------------------------------------
@pytest.mark.parametrize("shm", [0, 1])
def test_dead_rank_gives_an_error_not_a_hang(shm):
    res = run_ranks(3, "rank_that_dies", 1, env={"FLAGCX_SOCKET_TIMEOUT_MS": 3000, "FLAGCX_HOST_SHM": shm},
                    expect_dead=(1,), timeout=60)
    assert set(res) == {0, 2}
    assert all(code in (capi.flagcxRemoteError, capi.flagcxSystemError) for code in res.values()), res


@pytest.mark.parametrize("shm", [0, 1])
def test_late_rank_costs_a_deadline_not_a_hang(shm):
    res = run_ranks(3, "rank_that_is_late", 2, 4.0, env={"FLAGCX_SOCKET_TIMEOUT_MS": 1500, "FLAGCX_HOST_SHM": shm},
                    timeout=90)
    for r in (0, 1):  # gave up when their deadline ran out, well before the late rank arrived
        assert res[r]["code"] in (capi.flagcxRemoteError, capi.flagcxSystemError), res
        assert res[r]["seconds"] < 3.9, res
    # the late rank finds nobody waiting: an error (or, if its part needed no peer any more, success), never a hang
    assert res[2]["code"] in (0, capi.flagcxRemoteError, capi.flagcxSystemError), res
    assert res[2]["seconds"] < 10, res


def test_survivors_destroy_and_rebuild_a_smaller_communicator(tmp_path):
    res = run_ranks(3, "survivors_rebuild_a_smaller_communicator", 1, str(tmp_path / "new_id"),
                    env={"FLAGCX_SOCKET_TIMEOUT_MS": 3000}, expect_dead=(1,), timeout=90)
    assert set(res) == {0, 2}
    for r in res.values():
        assert r["error"] in (capi.flagcxRemoteError, capi.flagcxSystemError) and r["recovered"] and r["new_world"] == 2, res


def test_absent_rank_times_out_at_init():
    res = run_ranks(2, "rank_that_never_joins", env={"FLAGCX_SOCKET_TIMEOUT_MS": 1500}, timeout=60)
    assert res[1] == "absent"
    assert res[0] in (capi.flagcxRemoteError, capi.flagcxSystemError), res


def test_corrupt_unique_id_is_rejected():
    res = run_ranks(1, "wrong_unique_id")
    assert res[0] == capi.flagcxInvalidArgument


@pytest.mark.parametrize("shm", [0, 1])
def test_mismatched_message_sizes_are_detected(shm):
    res = run_ranks(2, "mismatched_sizes", env={"FLAGCX_SOCKET_TIMEOUT_MS": 3000, "FLAGCX_HOST_SHM": shm}, timeout=60)
    assert res[1] in (capi.flagcxInternalError, capi.flagcxRemoteError, capi.flagcxSystemError), res


# ---- host reductions (unit level) -------------------------------------------------------
@pytest.mark.parametrize("op,fn", [(capi.SUM, np.add), (capi.PROD, np.multiply), (capi.MAX, np.maximum),
                                   (capi.MIN, np.minimum)])
@pytest.mark.parametrize("dt", [np.int8, np.uint8, np.int32, np.uint32, np.int64, np.uint64, np.float32, np.float64])
def test_host_reduce_matches_numpy(op, fn, dt):
    rng = np.random.default_rng(1)
    a = rng.integers(1, 5, 1001).astype(dt)
    b = rng.integers(1, 5, 1001).astype(dt)
    want = fn(a, b)
    capi.host_reduce(a, b, capi.np_dtype_code(dt), op)
    assert np.array_equal(a, want)


def test_host_reduce_half_and_bfloat16_round_to_nearest_even():
    rng = np.random.default_rng(2)
    a = rng.uniform(-4, 4, 4096).astype(np.float16)
    b = rng.uniform(-4, 4, 4096).astype(np.float16)
    want = (a.astype(np.float32) + b.astype(np.float32)).astype(np.float16)
    capi.host_reduce(a, b, capi.HALF, capi.SUM)
    assert np.array_equal(a, want)
    # bf16 stored as the upper half of an fp32
    x = rng.uniform(-4, 4, 4096).astype(np.float32)
    y = rng.uniform(-4, 4, 4096).astype(np.float32)
    xb = (x.view(np.uint32) >> 16).astype(np.uint16)
    yb = (y.view(np.uint32) >> 16).astype(np.uint16)
    xf = (xb.astype(np.uint32) << 16).view(np.float32)
    yf = (yb.astype(np.uint32) << 16).view(np.float32)
    s = (xf + yf).view(np.uint32)
    rounded = ((s + 0x7FFF + ((s >> 16) & 1)) >> 16).astype(np.uint16)
    capi.host_reduce(xb, yb, capi.BFLOAT16, capi.SUM)
    assert np.array_equal(xb, rounded)


def test_trace_ring_records_calls_and_dumps_json(tmp_path):
    """Role of the event-record ring behind the FlagCX tuner's Start/StopProfiling."""
    import json
    comm = capi.Comm.init_rank(1, capi.get_unique_id(), 0)
    comm.trace_enable(4)
    x = np.arange(1000, dtype=np.float32)
    y = np.empty_like(x)
    for _ in range(6):  # more calls than slots: the ring keeps the last four
        comm.all_reduce(x, y, x.size, capi.FLOAT, capi.SUM)
    comm.all_gather(x, y, x.size, capi.FLOAT)
    path = str(tmp_path / "trace.json")
    comm.trace_dump(path)
    doc = json.load(open(path))
    recs = doc["records"]
    assert doc["rank"] == 0 and len(recs) == 4
    assert [r["seq"] for r in recs] == [3, 4, 5, 6]
    assert recs[-1]["op"].lower().replace("_", "") == "allgather" and recs[0]["bytes"] == 4000
    assert all(r["route"] == "host" and r["host_us"] > 0 for r in recs)
    comm.trace_enable(0)
    with pytest.raises(capi.FlagcxError):
        comm.trace_dump(path)
    comm.destroy()


def test_nccl_stand_in_runs_an_nccl_program_on_this_library():
    """csrc/shim/nccl_shim.cc (role of plugin/nccl in the FlagCX project)."""
    import ctypes
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    subprocess.run(["make", "-C", os.path.join(root, "csrc"), "nccl-shim"], check=True, capture_output=True)
    shim = os.path.join(root, "flagcx_b200", "lib", "libnccl_flagcx_shim.so")
    capi.lib()
    nccl = ctypes.CDLL(shim)
    v = ctypes.c_int()
    assert nccl.ncclGetVersion(ctypes.byref(v)) == 0 and v.value >= 22000
    uid = (ctypes.c_char * 128)()
    assert nccl.ncclGetUniqueId(uid) == 0 and any(bytes(uid))
    assert nccl.ncclCommInitAll(None, 2, None) == 5  # one process per GPU: invalid usage
    res = run_ranks(3, "nccl_shim_program", shim, 30000, timeout=120)
    for rank, out in res.items():
        assert all(v < 1e-5 for v in out.values()), (rank, out)


def test_c_api_example_program_forks_its_ranks_and_checks_results():
    """csrc/examples/allreduce_perf.cc uses only flagcx.h (device handle table, streams,
    events, collectives); role of test/perf/host_api/test_allreduce.cpp in the FlagCX project."""
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    subprocess.run(["make", "-C", os.path.join(root, "csrc"), "examples"], check=True, capture_output=True)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    exe = os.path.join(root, "csrc", "build", "examples", "allreduce_perf")
    env = {k: v for k, v in os.environ.items() if k != "FLAGCX_COMM_ID"}
    for op in ("allreduce", "allgather", "reducescatter", "alltoall", "broadcast"):
        res = subprocess.run([exe, "-n", "3", "--host", "-o", op, "-b", "1K", "-e", "256K", "-f", "4", "-w", "1", "-i", "2",
                              "-p", str(port)], capture_output=True, text=True, timeout=120, env=env)
        assert res.returncode == 0, op + res.stdout + res.stderr
        assert res.stdout.count(" ok") == 5 and "WRONG" not in res.stdout, op + res.stdout


@pytest.mark.parametrize("n,seed", [(2, 1), (4, 2), (5, 3)])
def test_random_schedule_with_per_rank_delays(n, seed):
    """Back-to-back collectives of random kind and size while the ranks drift apart by
    random sleeps: connections, tags and buffers must never get mixed up.  Odd seeds run
    over sockets, even ones over shared memory."""
    res = run_ranks(n, "host_random_stress", 40, seed, env={"FLAGCX_HOST_SHM": int(seed % 2 == 0)}, timeout=180)
    assert all(v < 1e-5 for v in res.values()), res


def test_one_sided_calls_say_not_supported_without_an_nvlink_domain():
    comm = capi.Comm.init_rank(1, capi.get_unique_id(), 0)
    buf = np.zeros(1024, np.uint8)
    lib = capi.lib()
    p = capi.C.c_void_p(buf.ctypes.data)
    assert lib.flagcxOneSideRegister(comm.h, p, capi.C.c_size_t(buf.nbytes)) == capi.flagcxNotSupported
    assert lib.flagcxOneSideDeregister(comm.h) == capi.flagcxNotSupported
    assert lib.flagcxOneSideSignalDeregister(comm.h) == capi.flagcxNotSupported
    comm.destroy()
