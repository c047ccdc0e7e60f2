"""tcgen05 GEMM and the fused tensor-parallel kernels against PyTorch references."""
import pytest
import torch

from tests._mp import run_ranks

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (256, 512, 128), (1024, 3584, 1024),
                                   (2048, 1024, 8192)])
@pytest.mark.parametrize("pair", [1, 0])
def test_tcgen05_gemm_matches_fp32_reference(M, N, K, pair, monkeypatch):
    """pair=1: CTA pairs (cta_group::2, 256-row tiles) where M allows; pair=0: single CTAs."""
    from flagcx_b200.parallel.tp import gemm_bf16
    monkeypatch.setenv("FLAGCX_GEMM_PAIR", str(pair))
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = (torch.randn(M, K, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    b = (torch.randn(N, K, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    out = gemm_bf16(a, b)
    torch.cuda.synchronize()
    ref = a.float() @ b.float().T
    # bf16 output of an fp32 accumulation: half an ulp of the result, relative to its scale
    err = ((out.float() - ref).abs() / (ref.abs().mean() + ref.abs())).max().item()
    assert err < 2 ** -7, err


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_fused_tensor_parallel_kernels_on_real_peers():
    n = 8 if torch.cuda.device_count() >= 8 else 4 if torch.cuda.device_count() >= 4 else 2
    res = run_ranks(n, "tp_fused", 128 * n * 2, 512, 1024, timeout=300)
    for rank, errs in res.items():
        assert errs["ag_gemm"] < 2 ** -6 and errs["gemm_rs"] < 2 ** -5, (rank, errs)
