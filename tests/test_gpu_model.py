"""Fused model kernels and the sharding engine against plain PyTorch fp32 references."""
import pytest
import torch
import torch.nn.functional as F

from tests._mp import run_ranks

pytestmark = pytest.mark.gpu


def _ops():
    from flagcx_b200 import ops
    ops.ext()  # must be the compiled extension
    return ops


def test_rmsnorm_forward_backward():
    ops = _ops()
    torch.manual_seed(0)
    # widths: each forward variant (4 / 8 / 16 packs per lane, then one CTA per row) and each
    # backward variant; 2500 rows make every persistent CTA of the backward wrap its ring of
    # shared-memory slots, 37 rows leave most of the grid without work
    for rows, H in ((2500, 256), (37, 1000), (37, 2048), (2500, 4096), (37, 4096), (700, 8192), (37, 16384)):
        x = torch.randn(rows, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16).requires_grad_()
        y = ops.rmsnorm(x, w, 1e-5)
        g = torch.randn_like(y)
        y.backward(g)
        xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
        yr = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
        yr.backward(g.float())
        assert (y.float() - yr).abs().max() < 0.05
        assert (x.grad.float() - xf.grad).abs().max() < 0.05
        assert ((w.grad.float() - wf.grad).abs() / wf.grad.abs().clamp(min=1)).max() < 0.05, (rows, H)


def test_rope_matches_reference_and_backward_is_inverse():
    ops = _ops()
    T, Hn, D = 64, 4, 128
    x = torch.randn(T, Hn, D, device="cuda", dtype=torch.bfloat16)
    y = ops.rope(x, 500000.0)
    half = D // 2
    inv = 500000.0 ** (-torch.arange(0, half, device="cuda", dtype=torch.float32) * 2 / D)
    ang = torch.arange(T, device="cuda", dtype=torch.float32)[:, None] * inv[None]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    x1, x2 = x[..., :half].float(), x[..., half:].float()
    ref = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)
    assert (y.float() - ref).abs().max() < 0.03
    xg = x.clone().requires_grad_()
    ops.rope(xg, 500000.0).backward(y)  # rotating back a rotated vector gives the original
    assert (xg.grad.float() - x.float()).abs().max() < 0.06


def test_rope_on_the_fused_projection_rotates_q_and_k_and_copies_v():
    ops = _ops()
    T, nh, nkv, D = 70, 8, 2, 128
    qkv = torch.randn(T, (nh + 2 * nkv) * D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    out = ops.rope_fused_qkv(qkv, nh, nkv, D, 500000.0)
    q, k, v = out.split([nh * D, nkv * D, nkv * D], dim=-1)
    q0, k0, v0 = qkv.detach().split([nh * D, nkv * D, nkv * D], dim=-1)
    assert torch.equal(v, v0)
    half = D // 2
    inv = 500000.0 ** (-torch.arange(0, half, device="cuda", dtype=torch.float32) * 2 / D)
    ang = torch.arange(T, device="cuda", dtype=torch.float32)[:, None] * inv[None]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]

    def rot(x, heads):
        x = x.reshape(T, heads, D).float()
        x1, x2 = x[..., :half], x[..., half:]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1).reshape(T, heads * D)

    assert (q.float() - rot(q0, nh)).abs().max() < 0.03
    assert (k.float() - rot(k0, nkv)).abs().max() < 0.03
    # backward: the rotation's transpose on q and k (rotating back what was rotated), identity on v
    out.backward(out.detach())
    gq, gk, gv = qkv.grad.split([nh * D, nkv * D, nkv * D], dim=-1)
    assert (gq.float() - q0.float()).abs().max() < 0.06
    assert (gk.float() - k0.float()).abs().max() < 0.06
    assert torch.equal(gv, v0)


def test_norm_branch_and_residual_linear_match_the_unfused_graph():
    """y = linear(f(norm(x)), w) + x, written with rmsnorm_branch / linear(residual=...),
    against the same expression in fp32: output, dx (skip gradient added inside the norm's
    backward), dw of the norm and of the linear."""
    ops = _ops()
    torch.manual_seed(1)
    T, H = 333, 1024
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    wn = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16).requires_grad_()
    w = (0.03 * torch.randn(H, H, device="cuda")).to(torch.bfloat16).requires_grad_()
    h, skip = ops.rmsnorm_branch(x, wn, 1e-5)
    y = ops.linear(h, w, residual=skip)
    g = torch.randn_like(y)
    y.backward(g)
    xf, wnf, wf = (t.detach().float().requires_grad_() for t in (x, wn, w))
    hf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wnf
    yf = hf @ wf.T + xf
    yf.backward(g.float())
    assert (y.float() - yf).abs().max() < 0.06
    assert (x.grad.float() - xf.grad).abs().max() < 0.06
    # the weight gradients are sums over 333 rows of bf16 products: compare in the L2 norm
    assert (wn.grad.float() - wnf.grad).norm() / wnf.grad.norm() < 0.01
    assert (w.grad.float() - wf.grad).norm() / wf.grad.norm() < 0.01
    # only the skip connection used: the gradient passes through untouched
    x2 = x.detach().clone().requires_grad_()
    _, skip2 = ops.rmsnorm_branch(x2, wn.detach(), 1e-5)
    skip2.backward(g)
    assert torch.equal(x2.grad, g)


def test_swiglu_forward_backward():
    ops = _ops()
    ab = torch.randn(50, 2 * 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    out = ops.swiglu(ab)
    g = torch.randn_like(out)
    out.backward(g)
    abf = ab.detach().float().requires_grad_()
    ref = F.silu(abf[:, :512]) * abf[:, 512:]
    ref.backward(g.float())
    assert (out.float() - ref).abs().max() < 0.05
    assert (ab.grad.float() - abf.grad).abs().max() < 0.06


# vocabulary sizes: one CTA per row; the Llama-3 vocabulary (a cluster of 4 CTAs per row);
# a row that does not divide evenly over its cluster; parts above 72 KiB (one CTA per SM);
# a row too long for shared memory (the kernel that streams it three times)
@pytest.mark.parametrize("T,V", [(33, 1024), (9, 128256), (5, 50264), (3, 300000), (2, 2000000)])
def test_cross_entropy_loss_and_gradient(T, V):
    ops = _ops()
    logits = (3 * torch.randn(T, V, device="cuda")).to(torch.bfloat16)
    tgt = torch.randint(0, V, (T,), device="cuda")
    lf = logits.float().requires_grad_()
    ref = F.cross_entropy(lf, tgt)
    ref.backward()
    work = logits.clone().requires_grad_()
    w2 = work * 1.0  # non-leaf, as in the model (the kernel overwrites it)
    loss = ops.cross_entropy_(w2, tgt)
    loss.backward()
    assert abs(float(loss) - float(ref)) < 2e-3
    assert (work.grad.float() - lf.grad).abs().max() < 2e-3
    # relative check where the gradient is not tiny: two bf16 roundings at most
    big = lf.grad.abs() > 1e-4
    if big.any():
        rel = ((work.grad.float() - lf.grad).abs() / lf.grad.abs())[big].max()
        assert rel < 1.2e-2


def test_adamw_matches_torch():
    ops = _ops()
    torch.manual_seed(5)
    n = 10007
    p = torch.randn(n, device="cuda").to(torch.bfloat16)
    g = torch.randn(n, device="cuda").to(torch.bfloat16)
    m = torch.zeros_like(p)
    v = torch.zeros_like(p)
    pr = torch.nn.Parameter(p.float().clone())
    opt = torch.optim.AdamW([pr], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in (1, 2, 3):
        pr.grad = g.float()
        opt.step()
        ops.adamw_flat_(p, g, m, v, 1e-2, 0.9, 0.95, 1e-8, 0.1, step)
    # parameters and both moments are rounded to bf16 after every step: half an ulp each time,
    # i.e. 2^-9 relative for |p| >= 1 and 2^-9 absolute below
    assert ((p.float() - pr.detach()).abs() / pr.detach().abs().clamp(min=1)).max() < 0.02


def test_sharded_engine_world1_matches_fp32_reference():
    from flagcx_b200 import ops
    from flagcx_b200.models.llama import LlamaConfig, build_units, reference_forward
    from flagcx_b200.parallel.fsdp import ShardedModel
    cfg = LlamaConfig.tiny()
    ops.assume_unit_loss_grad = True
    model = ShardedModel(build_units(cfg), None, 0, 1, torch.device("cuda", 0), lr=1e-3)
    tok = torch.randint(0, cfg.vocab, (129,), device="cuda")
    params = model.full_parameters()
    ref = reference_forward(cfg, params, tok[:-1], tok[1:])
    loss0 = model.train_step(tok[:-1], tok[1:])
    assert abs(float(loss0) - float(ref)) < 0.05, (float(loss0), float(ref))
    losses = [float(model.train_step(tok[:-1], tok[1:])) for _ in range(8)]
    assert losses[-1] < float(loss0) - 0.5, (float(loss0), losses)  # it learns the batch
    model.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_sharded_engine_world2_matches_world1():
    """Same seed, same batch on every rank: the sharded run must reproduce the
    single-GPU losses (gradients are averaged over identical replicas)."""
    from tests.test_cpu_torch_backend import free_port
    one = run_ranks(1, "fsdp_losses", free_port(), 4, timeout=300)[0]
    two = run_ranks(2, "fsdp_losses", free_port(), 4, timeout=300)
    for a, b in zip(one, two[0]):
        assert abs(a - b) < 0.05, (one, two[0])
    assert two[0] == two[1]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_torch_fsdp_over_flagcx_matches_nccl():
    """torch.distributed.fsdp.fully_shard with backend='flagcx' trains like backend='nccl'."""
    from tests.test_cpu_torch_backend import free_port
    ours = run_ranks(2, "torch_fsdp2_losses", free_port(), "flagcx", timeout=300)
    nccl = run_ranks(2, "torch_fsdp2_losses", free_port(), "nccl", timeout=300)
    for a, b in zip(ours[0], nccl[0]):
        assert abs(a - b) <= 0.02 * max(1.0, abs(b)), (ours[0], nccl[0])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_torch_backend_ops_on_gpus():
    from tests.test_cpu_torch_backend import free_port
    n = 2
    res = run_ranks(n, "torch_backend_ops", free_port(), True, timeout=300)
    assert all(v == "ok" for v in res.values())


def test_optimizer_under_backward_gives_the_same_model():
    """AdamW of a unit queued right behind that unit's gradients (on its own stream, under
    the rest of the backward pass) against AdamW after the whole backward pass: same
    losses, same parameters."""
    from flagcx_b200 import ops
    from flagcx_b200.models.llama import LlamaConfig, build_units
    from flagcx_b200.parallel.fsdp import ShardedModel
    cfg = LlamaConfig.tiny()
    ops.assume_unit_loss_grad = True
    g = torch.Generator().manual_seed(3)
    batches = [torch.randint(0, cfg.vocab, (129,), generator=g).cuda() for _ in range(4)]
    runs = []
    for overlap in (False, True):
        m = ShardedModel(build_units(cfg), None, 0, 1, torch.device("cuda", 0), overlap_optimizer=overlap)
        losses = [float(m.train_step(b[:-1], b[1:])) for b in batches]
        torch.cuda.synchronize()
        runs.append((losses, [s.clone() for s in m.shard]))
        m.close()
    (la, pa), (lb, pb) = runs
    assert max(abs(x - y) for x, y in zip(la, lb)) < 2e-2, (la, lb)
    for x, y in zip(pa, pb):
        assert (x.float() - y.float()).abs().max().item() < 2e-2


def test_checkpoint_round_trip_resumes_with_the_same_loss():
    """state_dict -> load_state_dict into a fresh engine: the next step's loss is the one
    the original engine computes (parameters, both AdamW moments and the step counter)."""
    from flagcx_b200 import ops
    from flagcx_b200.models.llama import LlamaConfig, build_units
    from flagcx_b200.parallel.fsdp import ShardedModel
    cfg = LlamaConfig.tiny()
    ops.assume_unit_loss_grad = True
    g = torch.Generator().manual_seed(11)
    batches = [torch.randint(0, cfg.vocab, (129,), generator=g).cuda() for _ in range(4)]
    a = ShardedModel(build_units(cfg), None, 0, 1, torch.device("cuda", 0), lr=1e-3)
    for b in batches[:2]:
        a.train_step(b[:-1], b[1:])
    sd = a.state_dict()
    want = [float(a.train_step(b[:-1], b[1:])) for b in batches[2:]]
    fresh = ShardedModel(build_units(cfg), None, 0, 1, torch.device("cuda", 0), lr=1e-3, seed=999)  # other weights
    fresh.load_state_dict(sd)
    got = [float(fresh.train_step(b[:-1], b[1:])) for b in batches[2:]]
    assert fresh.step_count == a.step_count
    assert max(abs(x - y) for x, y in zip(want, got)) < 2e-2, (want, got)
    a.close()
    fresh.close()
