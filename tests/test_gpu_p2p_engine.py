"""The point-to-point transfer engine on device memory: the peer's allocation is mapped through
its CUDA IPC handle and every transfer is a copy-engine copy (two processes; on a machine with
one GPU both use it)."""
import pytest

from tests._mp import run_ranks

pytestmark = pytest.mark.gpu


def test_one_sided_transfers_of_device_memory_between_two_processes(tmp_path):
    res = run_ranks(2, "p2p_engine_pair", str(tmp_path / "owner.json"), True, timeout=180)
    for rank, worst in res.items():
        bad = {k: v for k, v in worst.items() if v > 0.5}
        assert not bad, (rank, bad)
