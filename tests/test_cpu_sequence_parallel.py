"""Ulysses all-to-all re-sharding and ring attention over the host path."""
import pytest

from tests._mp import run_ranks


@pytest.mark.parametrize("n", [2, 4])
def test_ulysses_and_ring_attention_match_full_attention(n):
    res = run_ranks(n, "sp_ulysses_and_ring", 32, 8, 16, timeout=120)
    for rank, out in res.items():
        assert all(v < 1e-5 for v in out.values()), (rank, out)
