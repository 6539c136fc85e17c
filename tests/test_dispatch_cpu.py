"""all_to_all dispatcher on CPU ranks: round trip and gradients against a dense single-process computation."""
import pytest
import torch

from tests.distutil import run_ranks


def _moe_dense(x, idx, w, scale):
    """y[t] = sum_k w[t,k] * scale[e(t,k)] * x[t] computed without any dispatch."""
    return (x[:, None, :] * (w * scale[idx])[..., None]).sum(1)


def _worker(rank, world, pad):
    import torch.distributed as dist
    from system_lab_b200.moe.dispatch import AllToAllDispatcher
    from system_lab_b200.parallel.mesh import build_mesh, init_distributed
    init_distributed("cpu")
    mesh = build_mesh(1, world, 1)
    torch.manual_seed(10 + rank)
    T, K, E, H = 37, 2, 8, 16
    x = torch.randn(T, H, requires_grad=True)
    w = torch.rand(T, K, requires_grad=True)
    idx = torch.stack([torch.randperm(E)[:K] for _ in range(T)])
    scale = torch.arange(1, E + 1, dtype=torch.float32)           # expert e multiplies by e+1
    d = AllToAllDispatcher(mesh.ep_group, E, pad)
    plan = d.plan(idx)
    assert int(plan.expert_offsets[0]) == 0 and all(int(o) % pad == 0 for o in plan.expert_offsets)
    xe = d.dispatch_rows(plan, x)
    pe = d.dispatch_scalars(plan, w)
    e_local = E // world
    ye = torch.zeros_like(xe)
    for j in range(e_local):
        o, c = int(plan.expert_offsets[j]), int(plan.expert_counts[j])
        ye[o:o + c] = xe[o:o + c] * pe[o:o + c, None] * scale[rank * e_local + j]
    y = d.combine_rows(plan, ye)
    ref = _moe_dense(x, idx, w, scale)
    g = torch.randn(T, H)
    gx, gw = torch.autograd.grad(y, [x, w], g)
    rx, rw = torch.autograd.grad(ref, [x, w], g)
    ok = torch.allclose(y, ref, atol=1e-5) and torch.allclose(gx, rx, atol=1e-5) and torch.allclose(gw, rw, atol=1e-4)
    # weighted combine (gate applied at combine time) is equivalent
    ye2 = torch.zeros_like(xe)
    for j in range(e_local):
        o, c = int(plan.expert_offsets[j]), int(plan.expert_counts[j])
        ye2[o:o + c] = xe[o:o + c] * scale[rank * e_local + j]
    y2 = d.combine_rows(plan, ye2, w)
    g2 = torch.autograd.grad(y2, [x, w], g)
    ok = ok and torch.allclose(y2, ref, atol=1e-5) and torch.allclose(g2[0], rx, atol=1e-5) and torch.allclose(g2[1], rw, atol=1e-4)
    s = d.combine_scalars(plan, pe)
    ok = ok and torch.allclose(s, w)
    if dist.is_initialized():
        dist.barrier()
    return bool(ok)


@pytest.mark.parametrize("world,pad", [(1, 1), (2, 1), (2, 8), (4, 4)])
def test_alltoall_dispatch_combine(world, pad):
    assert all(run_ranks(_worker, world, pad))
