"""The point-to-point transfer engine between two processes without a communicator, on host
memory (requests travel over the connection's sockets and the owner's service thread copies)."""
from tests._mp import run_ranks


def test_one_sided_reads_writes_and_notifications_between_two_processes(tmp_path):
    res = run_ranks(2, "p2p_engine_pair", str(tmp_path / "owner.json"), False, timeout=120)
    for rank, worst in res.items():
        bad = {k: v for k, v in worst.items() if v > 0.5}
        assert not bad, (rank, bad)


def test_owner_that_exits_turns_into_error_codes_not_a_hang(tmp_path):
    from flagcx_b200 import capi
    res = run_ranks(2, "p2p_engine_owner_dies", str(tmp_path / "owner.json"), env={"FLAGCX_SOCKET_TIMEOUT_MS": 2000},
                    expect_dead=(0,), timeout=60)
    r = res[1]
    assert all(r[k] in (capi.flagcxRemoteError, capi.flagcxSystemError) for k in ("write", "notify", "read")), r
    assert r["seconds"] < 8, r


def test_c_example_of_the_transfer_engine():
    """csrc/examples/p2p_transfer.cc: the engine's C API from a program that forks its owner."""
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    subprocess.run(["make", "-C", os.path.join(root, "csrc"), "examples"], check=True, capture_output=True)
    exe = os.path.join(root, "csrc", "build", "examples", "p2p_transfer")
    res = subprocess.run([exe, str(5 * (1 << 20) + 17)], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "0 wrong" in res.stdout and res.stdout.strip().endswith("ok"), res.stdout
