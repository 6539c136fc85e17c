"""The PyTorch oracles themselves, against independent formulations."""
import math

import pytest
import torch
import torch.nn.functional as F

from system_lab_b200.ops import reference as ref


def test_rmsnorm_matches_torch():
    x, w = torch.randn(7, 64), torch.rand(64) + 0.5
    assert torch.allclose(ref.rmsnorm(x, w, 1e-6), F.rms_norm(x, (64,), w, 1e-6), atol=1e-6)
    y, xpr = ref.rmsnorm_residual(x, x * 0.5, w, 1e-6)
    assert torch.allclose(xpr, 1.5 * x) and torch.allclose(y, F.rms_norm(1.5 * x, (64,), w, 1e-6), atol=1e-6)


def test_rope_is_a_rotation_and_relative():
    cos, sin = ref.rope_tables(16, 32, 10000.0, "cpu")
    q, k = torch.randn(1, 16, 2, 32), torch.randn(1, 16, 2, 32)
    qr, kr = ref.rope(q, cos, sin), ref.rope(k, cos, sin)
    assert torch.allclose(qr.norm(dim=-1), q.norm(dim=-1), atol=1e-5)
    # score between positions depends only on their distance
    q1 = q[:, :1].expand(1, 16, 2, 32).contiguous()
    k1 = k[:, :1].expand(1, 16, 2, 32).contiguous()
    s = (ref.rope(q1, cos, sin)[0, 5, 0] * ref.rope(k1, cos, sin)[0, 3, 0]).sum()
    s2 = (ref.rope(q1, cos, sin)[0, 9, 0] * ref.rope(k1, cos, sin)[0, 7, 0]).sum()
    assert torch.allclose(s, s2, atol=1e-4)


def test_swiglu_probs_gradients():
    gu = torch.randn(5, 16, requires_grad=True)
    p = torch.rand(5, requires_grad=True)
    g = torch.randn(5, 8)
    dgu, dp = torch.autograd.grad(ref.swiglu_probs(gu, p), [gu, p], g)
    gate, up = gu[:, :8].double().detach(), gu[:, 8:].double().detach()
    s = torch.sigmoid(gate)
    act = gate * s
    gd, pd = g.double(), p.double().detach()[:, None]
    assert torch.allclose(dp.double(), (gd * act * up).sum(-1), atol=1e-5)
    assert torch.allclose(dgu[:, 8:].double(), gd * pd * act, atol=1e-5)
    assert torch.allclose(dgu[:, :8].double(), gd * pd * up * s * (1 + gate * (1 - s)), atol=1e-5)


@pytest.mark.parametrize("score", ["softmax", "sigmoid"])
def test_router_topk_properties(score):
    logits = torch.randn(50, 16)
    bias = torch.zeros(16)
    bias[3] = 100.0
    w, idx, scores = ref.router_topk(logits, 4, score, bias, True, 2.0)
    assert (idx == 3).any(dim=1).all()                       # bias steers the selection ...
    assert torch.allclose(w.sum(-1), torch.full((50,), 2.0), atol=1e-5)
    w3 = w[idx == 3]
    assert (w3 < 2.0).all()                                  # ... but not the gate weight
    assert ref.aux_loss(scores, idx, 16, 0.01) > 0


def test_block_quantisation_roundtrip():
    x = torch.randn(9, 256) * 5
    q, s = ref.quant_1x128(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (9, 2)
    assert ((ref.dequant_1x128(q, s) - x).abs() <= 0.07 * x.abs() + 1e-2).all()
    w = torch.randn(2, 128, 256) * 0.02
    qw, sw = ref.quant_128x128(w)
    assert sw.shape == (2, 1, 2)
    assert ((ref.dequant_128x128(qw, sw) - w).abs() <= 0.07 * w.abs() + 1e-4).all()


def test_grouped_gemm_matches_loop_and_grads():
    torch.manual_seed(0)
    counts = torch.tensor([3, 0, 5])
    offsets = torch.tensor([0, 4, 4])
    a = torch.randn(12, 8)
    b = torch.randn(3, 6, 8)
    out = ref.grouped_gemm(a, b, offsets, counts)
    assert torch.allclose(out[0:3], a[0:3] @ b[0].t(), atol=1e-5) and torch.allclose(out[4:9], a[4:9] @ b[2].t(), atol=1e-5)
    assert not out[3].any() and not out[9:].any()
    dy = torch.randn(12, 6)
    assert torch.allclose(ref.grouped_gemm_dgrad(dy, b, offsets, counts)[4:9], dy[4:9] @ b[2], atol=1e-5)
    dw = ref.grouped_gemm_wgrad(dy, a, offsets, counts)
    assert torch.allclose(dw[2], dy[4:9].t() @ a[4:9], atol=1e-5) and not dw[1].any()


def test_causal_attention_matches_sdpa_gqa_and_window():
    torch.manual_seed(1)
    q, k, v = torch.randn(2, 12, 4, 8), torch.randn(2, 12, 2, 8), torch.randn(2, 12, 2, 8)
    out = ref.causal_attention(q, k, v)
    exp = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                         enable_gqa=True).transpose(1, 2)
    assert torch.allclose(out, exp, atol=1e-5)
    win = ref.causal_attention(q, k, v, window=3)
    i = torch.arange(12)
    mask = (i[None, :] <= i[:, None]) & (i[None, :] > i[:, None] - 3)
    exp_w = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask,
                                           enable_gqa=True).transpose(1, 2)
    assert torch.allclose(win, exp_w, atol=1e-5)


def test_adamw_step_matches_torch_optimizer():
    torch.manual_seed(2)
    p0 = torch.randn(100)
    p = torch.nn.Parameter(p0.clone())
    opt = torch.optim.AdamW([p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    mine, m, v = p0.clone(), torch.zeros(100), torch.zeros(100)
    for step in range(1, 5):
        g = torch.randn(100)
        p.grad = g.clone()
        opt.step()
        ref.adamw_step(mine, g, m, v, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
    assert torch.allclose(mine, p.detach(), atol=1e-6)


def test_linear_cross_entropy():
    h, w, t = torch.randn(10, 8), torch.randn(20, 8), torch.randint(0, 20, (10,))
    assert torch.allclose(ref.linear_cross_entropy(h, w, t), F.cross_entropy(h @ w.t(), t))
    assert abs(ref.cross_entropy(torch.zeros(4, 1024), torch.zeros(4, dtype=torch.long)).item() - math.log(1024)) < 1e-5
