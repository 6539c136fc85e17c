"""The hand-written attention forward against a plain fp32 reference.  The kernel is an opt-in path
(``SLAB_ATTENTION_KERNEL=1``); its tests run when it is switched on."""
import math
import os

import pytest
import torch

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(os.environ.get("SLAB_ATTENTION_KERNEL") != "1",
                                 reason="attention kernel is opt-in: set SLAB_ATTENTION_KERNEL=1")]


def _reference(q, k, v, scale, window):
    b, s, hq, d = q.shape
    hkv = k.shape[2]
    qf = q.float().transpose(1, 2)                                   # [b, hq, s, d]
    kf = k.float().transpose(1, 2).repeat_interleave(hq // hkv, 1)
    vf = v.float().transpose(1, 2).repeat_interleave(hq // hkv, 1)
    sc = qf @ kf.transpose(-1, -2) * scale
    i = torch.arange(s, device=q.device)
    vis = i[None, :] <= i[:, None]
    if window > 0:
        vis &= i[None, :] > i[:, None] - window
    sc = sc.masked_fill(~vis, float("-inf"))
    lse = torch.logsumexp(sc, -1)
    return (torch.softmax(sc, -1) @ vf).transpose(1, 2), lse


@pytest.mark.parametrize("b,s,hq,hkv,d,window", [(1, 256, 4, 2, 64, 0), (2, 512, 4, 1, 128, 0), (1, 512, 8, 8, 64, 128),
                                                 (1, 1024, 2, 1, 128, 200)])
def test_forward_matches_fp32_reference(b, s, hq, hkv, d, window):
    from system_lab_b200.ops import attention_kernel as ak, cuda
    torch.manual_seed(0)
    dev = torch.device("cuda")
    # q, k, v as column slices of one packed projection, the layout the model hands over
    qkv = torch.randn(b, s, (hq + 2 * hkv) * d, device=dev, dtype=torch.bfloat16)
    q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)
    q, k, v = q.unflatten(-1, (hq, d)), k.unflatten(-1, (hkv, d)), v.unflatten(-1, (hkv, d))
    assert ak.shape_ok(q, k, v, window)
    scale = 1.0 / math.sqrt(d)
    out, lse = ak.forward(q, k, v, scale, window)
    torch.cuda.synchronize()
    cuda.check_status()
    ref, ref_lse = _reference(q, k, v, scale, window)
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(lse, ref_lse, rtol=1e-3, atol=1e-3)


def test_autograd_wrapper_gives_library_gradients():
    from system_lab_b200.ops import attention_kernel as ak
    from system_lab_b200.ops.attention import _library
    torch.manual_seed(1)
    dev = torch.device("cuda")
    q = torch.randn(1, 256, 4, 64, device=dev, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(1, 256, 2, 64, device=dev, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(1, 256, 2, 64, device=dev, dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(1, 256, 4, 64, device=dev, dtype=torch.bfloat16)
    ak.attention(q, k, v, 0.125, 0).backward(g)
    got = [t.grad.clone() for t in (q, k, v)]
    for t in (q, k, v):
        t.grad = None
    _library(q, k, v, 0.125, 0).backward(g)
    for a, e in zip(got, (q.grad, k.grad, v.grad)):
        torch.testing.assert_close(a.float(), e.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("b,s,hq,hkv,d,window", [(1, 256, 4, 2, 64, 0), (2, 384, 4, 1, 128, 0), (1, 512, 4, 4, 64, 128)])
def test_backward_kernel_matches_fp32_autograd(b, s, hq, hkv, d, window):
    from system_lab_b200.ops import attention_kernel as ak, cuda
    torch.manual_seed(2)
    dev = torch.device("cuda")
    qkv = torch.randn(b, s, (hq + 2 * hkv) * d, device=dev, dtype=torch.bfloat16)
    q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)
    q, k, v = q.unflatten(-1, (hq, d)), k.unflatten(-1, (hkv, d)), v.unflatten(-1, (hkv, d))
    g = torch.randn(b, s, hq, d, device=dev, dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    out, lse = ak.forward(q, k, v, scale, window)
    dq, dk, dv = ak.backward(q, k, v, out, lse, g, scale, window)
    torch.cuda.synchronize()
    cuda.check_status()
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref, _ = _reference(qf, kf, vf, scale, window)
    ref.backward(g.float())
    for got, want, name in ((dq, qf.grad, "dq"), (dk, kf.grad, "dk"), (dv, vf.grad, "dv")):
        err = (got.float() - want).abs().max().item()
        assert err < 3e-2 * (want.abs().max().item() + 1e-6), (name, err)
