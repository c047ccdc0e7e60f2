"""Trace ring on the device route: CUDA-event times per call."""
import json

import pytest
import torch

from flagcx_b200 import capi

pytestmark = pytest.mark.gpu


def test_device_calls_are_timed_by_cuda_events(tmp_path):
    torch.cuda.set_device(0)
    comm = capi.Comm.init_rank(1, capi.get_unique_id(), 0)
    assert comm.device_path
    comm.trace_enable(8)
    x = torch.randn(1 << 22, device="cuda")
    y = torch.empty_like(x)
    for _ in range(3):
        comm.all_reduce(x, y, x.numel(), capi.FLOAT, capi.SUM)
    torch.cuda.synchronize()
    assert torch.equal(x, y)
    path = str(tmp_path / "trace.json")
    comm.trace_dump(path)
    recs = json.load(open(path))["records"]
    assert len(recs) == 3 and all(r["route"] == "device" and r["device_ms"] > 0 for r in recs)
    assert comm.stats(capi.OP_ALLREDUCE).lastMs > 0
    comm.destroy()
