"""torch.distributed backend "flagcx" on CPU tensors (socket path), world_size 2-3:
every ProcessGroup operation, and loss parity of a DDP model against gloo."""
import socket

import pytest

from tests._mp import run_ranks


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("n", [2, 3])
def test_process_group_ops_cpu(n):
    res = run_ranks(n, "torch_backend_ops", free_port(), False, timeout=300)
    assert all(v == "ok" for v in res.values())


def test_backend_options_record_tune_objects_and_bool_reductions():
    res = run_ranks(2, "torch_backend_options", free_port(), timeout=300)
    assert all(v == "ok" for v in res.values())


def test_ddp_loss_parity_with_gloo():
    ours = run_ranks(2, "torch_ddp_parity", free_port(), "flagcx", False, timeout=300)
    gloo = run_ranks(2, "torch_ddp_parity", free_port(), "gloo", False, timeout=300)
    for a, b in zip(ours[0], gloo[0]):
        assert abs(a - b) <= 1e-5 * max(1.0, abs(b)), (ours[0], gloo[0])


def test_example_script_runs_under_torchrun():
    """flagcx_b200/torch_backend/example.py is what a new user runs first."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), "-m", "flagcx_b200.torch_backend.example", "--cpu"]
    res = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "MISMATCH" not in res.stdout and "batch_isend_irecv" in res.stdout
