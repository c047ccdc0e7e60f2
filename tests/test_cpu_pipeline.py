"""Pipeline-parallel schedule over flagcx send/recv, CPU ranks."""
import pytest

from tests._mp import run_ranks


@pytest.mark.parametrize("n,n_micro", [(2, 1), (3, 5), (4, 3), (4, 8)])
def test_1f1b_matches_single_process_gradients(n, n_micro):
    res = run_ranks(n, "pp_1f1b", n_micro, 16, timeout=120)
    for rank, out in res.items():
        assert all(v < 1e-5 for v in out.values()), (rank, out)
    assert "loss" in res[n - 1]
