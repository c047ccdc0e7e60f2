"""MoE dispatch (all-to-all + permute) and combine (all-to-all + weighted sum) kernels,
run as an emulated world on one GPU and checked against a PyTorch fp32 reference."""
import pytest
import torch

from flagcx_b200 import capi
from flagcx_b200.parallel.moe import MoeDispatcher, route

pytestmark = pytest.mark.gpu


def _sorted_rows(rows: torch.Tensor) -> torch.Tensor:
    """Rows in lexicographic order of their exact bit patterns, so that two tensors hold the
    same multiset of rows exactly when the results are equal element for element."""
    bits = rows.contiguous().view(torch.int16).to(torch.int64).cpu()
    order = list(range(bits.shape[0]))
    order.sort(key=lambda i: bits[i].tolist())
    return bits[order]


# dedup: a token crosses NVLink once per destination rank (1) or once per expert (0);
# reduce: the expert rank adds up a token's weighted outputs (1) or the owner pulls every row (0)
@pytest.mark.parametrize("dedup,reduce", [(1, 1), (1, 0), (0, 1), (0, 0)])
@pytest.mark.parametrize("n,T,H,E,K", [(2, 33, 128, 8, 2), (4, 64, 256, 16, 4), (8, 96, 512, 64, 8), (2, 70, 128, 4, 4)])
def test_dispatch_groups_rows_by_expert_and_combine_weights_them(n, T, H, E, K, dedup, reduce, monkeypatch):
    monkeypatch.setenv("FLAGCX_MOE_DEDUP", str(dedup))
    monkeypatch.setenv("FLAGCX_MOE_COMBINE_REDUCE", str(reduce))
    comms = capi.Comm.emu_world(n, 0)
    try:
        epr = E // n
        cap = T * K * n  # worst case: everything lands on one rank
        moes = [MoeDispatcher(comms[r], T, H, K, E, cap) for r in range(n)]
        g = torch.Generator().manual_seed(0)
        xs = [torch.randn(T, H, generator=g).to(torch.bfloat16).cuda() for _ in range(n)]
        routed = [route(torch.randn(T, E, generator=g).cuda(), K) for _ in range(n)]
        for r in range(n):
            moes[r].dispatch(xs[r], routed[r][0])
        torch.cuda.synchronize()
        for c in comms:
            assert c.async_error() == 0, c.last_error()
        # rows of local expert le on rank d: tokens of rank 0 first, then rank 1, ...
        for d in range(n):
            offs = moes[d].expert_offsets.cpu().tolist()
            for le in range(epr):
                e = d * epr + le
                want_rows = []
                for s in range(n):
                    sel = (routed[s][0] == e).any(dim=1).cpu()
                    rows = xs[s].cpu()[sel]
                    got = moes[d].recv_rows[offs[le] + len(want_rows): offs[le] + len(want_rows) + rows.shape[0]].cpu()
                    # order inside one (source, expert) group is arbitrary: compare whole rows as
                    # multisets (rows sorted lexicographically, then element for element)
                    assert torch.equal(_sorted_rows(got), _sorted_rows(rows)), (d, e, s)
                    want_rows.extend([None] * rows.shape[0])
                assert offs[le + 1] - offs[le] == len(want_rows)
            # the "expert": scale every row of expert e by (e + 1)
            for le in range(epr):
                e = d * epr + le
                moes[d].expert_out[offs[le]:offs[le + 1]] = (moes[d].recv_rows[offs[le]:offs[le + 1]].float() * (e + 1)).to(torch.bfloat16)
        outs = [torch.empty(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(n)]
        for r in range(n):
            moes[r].combine(routed[r][1], outs[r])
        torch.cuda.synchronize()
        for c in comms:
            assert c.async_error() == 0, c.last_error()
        for r in range(n):
            idx, w = routed[r]
            scale = (w * (idx.float() + 1)).sum(1, keepdim=True)  # sum_k w_k (e_k + 1)
            ref = xs[r].float() * scale
            err = ((outs[r].float() - ref).abs() / ref.abs().clamp(min=1.0)).max().item()
            assert err < 0.03, (r, err)
        for m in moes:
            m.close()
    finally:
        capi.Comm.emu_world_destroy(comms)


def test_capacity_overflow_is_reported_not_written():
    n, T, H, E, K = 2, 32, 64, 4, 2
    comms = capi.Comm.emu_world(n, 0)
    try:
        moes = [MoeDispatcher(comms[r], T, H, K, E, 8) for r in range(n)]  # far too small
        xs = [torch.randn(T, H).to(torch.bfloat16).cuda() for _ in range(n)]
        idx = torch.zeros(T, K, dtype=torch.int32, device="cuda")
        idx[:, 1] = 1  # everything to rank 0
        for r in range(n):
            moes[r].dispatch(xs[r], idx)
        torch.cuda.synchronize()
        assert comms[0].async_error() == capi.flagcxInvalidArgument
    finally:
        capi.Comm.emu_world_destroy(comms)
