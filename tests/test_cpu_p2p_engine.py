"""The point-to-point transfer engine between two processes without a communicator, on host
memory (requests travel over the connection's sockets and the owner's service thread copies)."""
from tests._mp import run_ranks


def test_one_sided_reads_writes_and_notifications_between_two_processes(tmp_path):
    res = run_ranks(2, "p2p_engine_pair", str(tmp_path / "owner.json"), False, timeout=120)
    for rank, worst in res.items():
        bad = {k: v for k, v in worst.items() if v > 0.5}
        assert not bad, (rank, bad)
