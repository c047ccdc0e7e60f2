"""Multi-GPU tier: one process per GPU over real NVLink peers.  Skipped on boxes
with a single GPU (the emulated-world tests cover the kernels there)."""
import pytest
import torch

from flagcx_b200 import capi
from tests._mp import run_ranks

pytestmark = pytest.mark.gpu


def ngpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


needs2 = pytest.mark.skipif(ngpus() < 2, reason="needs at least 2 GPUs")


@needs2
@pytest.mark.parametrize("registered", [True, False])
def test_device_collectives_on_real_peers(registered):
    n = min(ngpus(), 8)
    n = 8 if n >= 8 else 4 if n >= 4 else 2
    res = run_ranks(n, "gpu_collectives", 70003, registered, timeout=300)
    for rank, worst in res.items():
        bad = {k: v for k, v in worst.items() if v > 1.0}
        assert not bad, (rank, bad)


@needs2
def test_missing_peer_becomes_an_error_code():
    n = 2
    env = {"NCCL_NVLS_ENABLE": "0", "FLAGCX_NVLS_ENABLE": "0"}
    res = run_ranks(n, "gpu_peer_never_launches", env=env, timeout=120)
    assert res[0] == capi.flagcxRemoteError
