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
@pytest.mark.parametrize("count", [70003, 1 << 19])
def test_device_collectives_on_real_peers(registered, count):
    """The odd count takes the per-thread paths with ragged tails; the power of two has
    16-byte aligned blocks of at least 1 MiB, which the push kinds move by bulk copies."""
    n = min(ngpus(), 8)
    n = 8 if n >= 8 else 4 if n >= 4 else 2
    env = {"FLAGCX_BULK_COPY_MIN_BYTES": "65536"} if count % 4 == 0 else None  # default: tens of MB
    res = run_ranks(n, "gpu_collectives", count, registered, env=env, timeout=300)
    for rank, worst in res.items():
        bad = {k: v for k, v in worst.items() if v > 1.0}
        assert not bad, (rank, bad)


@needs2
@pytest.mark.parametrize("export", [True, False])
def test_plain_tensors_with_a_straggler(export):
    """No buffer is registered by the caller.  With export on, allocations are mapped into
    the peers on first use (no staging copies); with it off, everything goes through the
    staging window, small and large collectives back to back."""
    n = 4 if ngpus() >= 4 else 2
    env = {} if export else {"FLAGCX_USER_BUFFER_EXPORT": "0"}
    res = run_ranks(n, "gpu_user_buffers_under_skew", 9, env=env, timeout=300)
    for rank, out in res.items():
        assert not out["bad"], (rank, out)
        assert out["exporting"] == export
        if export:
            assert out["exports"] > 0 and out["hits"] > 0 and out["refused"] == 0, (rank, out)


@needs2
def test_nvls_multimem_kernels():
    """FLAGCX_NVLS_ENABLE=1: the switch reduces (multimem.ld_reduce) and replicates
    (multimem.st).  Skipped where the GPUs expose no multicast."""
    n = 8 if ngpus() >= 8 else 4 if ngpus() >= 4 else 2
    res = run_ranks(n, "gpu_nvls_collectives", 1 << 16, env={"FLAGCX_NVLS_ENABLE": "1"}, timeout=300)
    if all("skipped" in v for v in res.values()):
        pytest.skip("no NVLink multicast on this machine")
    for rank, worst in res.items():
        bad = {k: v for k, v in worst.items() if v > 1.0}
        assert not bad, (rank, bad)


@needs2
def test_copy_engine_allgather_and_reduce_scatter_with_a_straggler():
    n = 8 if ngpus() >= 8 else 4 if ngpus() >= 4 else 2
    # a 4 MiB staging area makes the 3 M-element reduce-scatter take several chunks
    res = run_ranks(n, "gpu_copy_engine_collectives", 1 << 20, 12, env={"FLAGCX_STAGING_BYTES": str(4 << 20)}, timeout=300)
    for rank, worst in res.items():
        bad = {k: v for k, v in worst.items() if v > 1.0}
        assert not bad, (rank, bad)


@needs2
def test_two_level_route_when_one_machine_poses_as_several_nodes():
    """FLAGCX_HOSTID splits the machine: 2 nodes x 2 GPUs where there are four, else 2 x 1."""
    per_node = 2 if ngpus() >= 4 else 1
    n = 2 * per_node
    env = {r: {"FLAGCX_HOSTID": f"node{r // per_node}"} for r in range(n)}
    res = run_ranks(n, "gpu_two_level", per_node, per_rank_env=env, timeout=300)
    for rank, worst in res.items():
        bad = {k: v for k, v in worst.items() if v > 1.0}
        assert not bad, (rank, bad)


@needs2
def test_pipeline_1f1b_with_one_gpu_per_stage():
    n = 4 if ngpus() >= 4 else 2
    res = run_ranks(n, "pp_1f1b", 6, 64, True, timeout=300)
    for rank, out in res.items():
        assert all(v < 1e-4 for v in out.values()), (rank, out)


@needs2
def test_ulysses_and_ring_attention_on_gpus():
    """Sequence parallelism over NVLink: the all-to-all re-sharding is exact, ring attention
    (next block in flight on a side stream during the block's attention) matches full
    attention computed on one GPU."""
    n = 4 if ngpus() >= 4 else 2
    res = run_ranks(n, "sp_ulysses_and_ring", 64 * n, 8, 32, True, timeout=300)
    for rank, out in res.items():
        assert out["seq_to_heads"] == 0.0 and out["roundtrip"] == 0.0, (rank, out)
        assert out["ring_causal0"] < 1e-4 and out["ring_causal1"] < 1e-4, (rank, out)


@needs2
def test_missing_peer_becomes_an_error_code():
    n = 2
    env = {"NCCL_NVLS_ENABLE": "0", "FLAGCX_NVLS_ENABLE": "0"}
    res = run_ranks(n, "gpu_peer_never_launches", env=env, timeout=120)
    assert res[0] == capi.flagcxRemoteError


@pytest.mark.skipif(ngpus() < 1, reason="needs a GPU")
def test_device_buffers_without_peer_access_go_over_the_host_path():
    """What two machines, or FLAGCX_HOSTID-split ranks of one machine, fall back to."""
    res = run_ranks(2, "gpu_buffers_over_sockets", env={"FLAGCX_FORCE_HOST": "1"}, timeout=120)
    for rank, worst in res.items():
        assert all(v < 1e-5 for v in worst.values()), (rank, worst)
