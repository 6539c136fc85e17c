"""CUDA kernels vs the plain PyTorch fp32 oracle of the same op (forward and backward)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cops():
    from system_lab_b200.ops import cuda
    cuda.lib()
    return cuda


def _close(a, b, rtol, atol):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    assert bool((err <= tol).all()), f"max err {err.max().item():.4e} (tol rtol={rtol} atol={atol})"


@pytest.mark.parametrize("rows,h", [(37, 256), (512, 2048), (64, 2880), (33, 7168)])
def test_rmsnorm_fwd_bwd(cops, rows, h):
    from system_lab_b200.ops import reference as ref
    torch.manual_seed(0)
    x = torch.randn(rows, h, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(h, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    g = torch.randn(rows, h, device="cuda", dtype=torch.bfloat16)
    y = cops.rmsnorm(x, w, 1e-6)
    y.backward(g)
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = ref.rmsnorm(xf, wf, 1e-6)
    yr.backward(g.float())
    _close(y, yr, 1e-2, 1e-2)
    _close(x.grad, xf.grad, 2e-2, 2e-2)
    _close(w.grad, wf.grad, 2e-2, 0.05 * rows ** 0.5)


@pytest.mark.parametrize("rows,h", [(129, 2048), (40, 2880)])
def test_rmsnorm_residual_fwd_bwd(cops, rows, h):
    from system_lab_b200.ops import reference as ref
    torch.manual_seed(1)
    x = torch.randn(rows, h, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(rows, h, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(h, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    gy = torch.randn(rows, h, device="cuda", dtype=torch.bfloat16)
    gx = torch.randn(rows, h, device="cuda", dtype=torch.bfloat16)
    y, xpr = cops.rmsnorm_residual(x, r, w, 1e-6)
    torch.autograd.backward([y, xpr], [gy, gx])
    xf, rf, wf = (t.detach().float().requires_grad_(True) for t in (x, r, w))
    yr, xr = ref.rmsnorm_residual(xf, rf, wf, 1e-6)
    torch.autograd.backward([yr, xr], [gy.float(), gx.float()])
    _close(y, yr, 1e-2, 1e-2)
    _close(xpr, xr, 1e-2, 1e-2)
    _close(x.grad, xf.grad, 2e-2, 3e-2)
    _close(r.grad, rf.grad, 2e-2, 3e-2)
    _close(w.grad, wf.grad, 2e-2, 0.05 * rows ** 0.5)


@pytest.mark.parametrize("rows,f,with_probs", [(100, 768, True), (257, 2048, True), (64, 512, False)])
def test_swiglu_fwd_bwd(cops, rows, f, with_probs):
    from system_lab_b200.ops import reference as ref
    torch.manual_seed(2)
    gu = torch.randn(rows, 2 * f, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    p = torch.rand(rows, device="cuda", requires_grad=True) if with_probs else None
    g = torch.randn(rows, f, device="cuda", dtype=torch.bfloat16)
    out = cops.swiglu_probs(gu, p) if with_probs else cops.swiglu(gu)
    out.backward(g)
    guf = gu.detach().float().requires_grad_(True)
    pf = p.detach().clone().requires_grad_(True) if with_probs else None
    outr = ref.swiglu_probs(guf, pf) if with_probs else ref.swiglu(guf)
    outr.backward(g.float())
    _close(out, outr, 1e-2, 1e-2)
    _close(gu.grad, guf.grad, 2e-2, 2e-2)
    if with_probs:
        _close(p.grad, pf.grad, 2e-2, 0.05 * f ** 0.5)


@pytest.mark.parametrize("d", [64, 128])
def test_rope_fwd_bwd(cops, d):
    from system_lab_b200.ops import reference as ref
    torch.manual_seed(3)
    b, s, hh = 2, 96, 5
    x = torch.randn(b, s, hh, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    cos, sin = ref.rope_tables(s, d, 1e6, "cuda")
    g = torch.randn_like(x)
    y = cops.rope(x, cos, sin)
    y.backward(g)
    xf = x.detach().float().requires_grad_(True)
    yr = ref.rope(xf, cos, sin)
    yr.backward(g.float())
    _close(y, yr, 1e-2, 1e-2)
    _close(x.grad, xf.grad, 1e-2, 1e-2)


@pytest.mark.parametrize("score,e,k,bias", [("softmax", 128, 8, False), ("sigmoid", 256, 8, True), ("softmax", 8, 2, False)])
def test_router_topk(cops, score, e, k, bias):
    from system_lab_b200.ops import reference as ref
    torch.manual_seed(4)
    t = 333
    logits = torch.randn(t, e, device="cuda", requires_grad=True)
    b = 0.1 * torch.randn(e, device="cuda") if bias else None
    w, idx, _ = cops.router_topk(logits, k, score, b, True, 2.5)
    gw = torch.randn_like(w)
    w.backward(gw)
    lr = logits.detach().clone().requires_grad_(True)
    wr, idxr, _ = ref.router_topk(lr, k, score, b, True, 2.5)
    wr.backward(gw)
    assert torch.equal(idx.long().sort(-1).values, idxr.sort(-1).values)
    order, order_r = idx.long().argsort(-1), idxr.argsort(-1)
    _close(torch.gather(w, 1, order), torch.gather(wr, 1, order_r), 1e-4, 1e-5)
    _close(logits.grad, lr.grad, 1e-3, 1e-5)


@pytest.mark.parametrize("score,e,k,bias,norm,coeff", [("softmax", 128, 8, False, True, 0.01),
                                                        ("sigmoid", 256, 8, True, True, 0.05),
                                                        ("softmax", 8, 2, False, False, 0.0),
                                                        ("softmax", 33, 4, False, True, 0.3)])
def test_router_fused_forward_stats_aux_and_backward(cops, score, e, k, bias, norm, coeff):
    """One launch gives selection, gate weights, per-expert counts and the load-balancing loss; one more gives the
    logit gradient of the gate weights and of the loss together.  Against the fp32 PyTorch formulas."""
    from system_lab_b200.ops import reference as ref
    torch.manual_seed(5)
    t = 517
    logits = torch.randn(t, e, device="cuda", requires_grad=True)
    b = 0.1 * torch.randn(e, device="cuda") if bias else None
    w, idx, aux, counts = cops.router_fused(logits, k, score, b, norm, 2.5, coeff)
    gw = torch.randn_like(w)
    (w * gw).sum().add(aux * 3.0).backward()
    lr = logits.detach().clone().requires_grad_(True)
    wr, idxr, scores = ref.router_topk(lr, k, score, b, norm, 2.5)
    auxr = ref.aux_loss(scores, idxr, e, coeff)
    gw_r = torch.gather(gw, 1, _match(idx.long(), idxr))     # the same upstream gradient, expert by expert
    ((wr * gw_r).sum() + auxr * 3.0).backward()
    assert torch.equal(idx.long().sort(-1).values, idxr.sort(-1).values)
    assert torch.equal(counts.long(), torch.bincount(idxr.reshape(-1), minlength=e))
    _close(aux, auxr, 1e-4, 1e-6)
    _close(logits.grad, lr.grad, 2e-3, 1e-5)
    # the statistics are integer sums: a second run gives the same bits whatever the block order
    _, _, aux2, _ = cops.router_fused(logits.detach(), k, score, b, norm, 2.5, coeff)
    assert torch.equal(aux.detach(), aux2)


def _match(idx, idxr):
    """For every reference selection (row-wise), the column of the same expert in the kernel's selection."""
    return (idxr.unsqueeze(-1) == idx.unsqueeze(1)).float().argmax(-1)


def test_quant_roundtrip(cops):
    from system_lab_b200.ops import reference as ref
    torch.manual_seed(5)
    x = torch.randn(300, 1024, device="cuda", dtype=torch.bfloat16) * 3
    q, s = cops.quant_1x128(x)
    qr, sr = ref.quant_1x128(x)
    _close(s, sr, 1e-6, 0)
    _close(ref.dequant_1x128(q, s), ref.dequant_1x128(qr, sr), 0.13, 1e-6)   # at most one e4m3 step apart
    _close(ref.dequant_1x128(q, s), x, 0.07, 1e-3)
    w = torch.randn(3, 256, 384, device="cuda", dtype=torch.bfloat16) * 0.02
    qw, sw = cops.quant_128x128(w)
    qwr, swr = ref.quant_128x128(w)
    _close(sw, swr, 1e-6, 0)
    _close(ref.dequant_128x128(qw, sw), w, 0.07, 1e-5)


def test_ce_matches_reference(cops):
    from system_lab_b200.ops import reference as ref
    torch.manual_seed(6)
    n, hd, v = 700, 256, 1024
    h = torch.randn(n, hd, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (0.05 * torch.randn(v, hd, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    tgt = torch.randint(0, v, (n,), device="cuda")
    loss = cops.linear_cross_entropy(h, w, tgt, chunk_rows=256)
    (loss * 3.0).backward()
    hf, wf = h.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    lr = ref.linear_cross_entropy(hf, wf, tgt)
    (lr * 3.0).backward()
    assert abs(loss.item() - lr.item()) < 2e-2
    _close(h.grad, hf.grad, 5e-2, 2e-4)
    _close(w.grad, wf.grad, 5e-2, 2e-4)


@pytest.mark.parametrize("kind", ["fp32", "bf16", "fp8"])
@pytest.mark.parametrize("p_dtype", [torch.float32, torch.bfloat16])
def test_adamw_flat(cops, kind, p_dtype):
    from system_lab_b200.ops import reference as ref
    from system_lab_b200.trainer.optim import _Moment
    torch.manual_seed(7)
    n = 128 * 37

    class G:
        pass
    g = G()
    g.shard = (0.02 * torch.randn(n, device="cuda")).to(p_dtype)
    g.full = g.shard
    g.sharded = True
    de = 128 * 30                                   # the tail of the shard holds 1-D parameters: no weight decay there
    g.shard_decay_end = lambda: de
    p_ref = g.shard.float().clone()
    m_ref, v_ref = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    m, v = _Moment(n, kind, "cuda"), _Moment(n, kind, "cuda", sqrt_domain=(kind != "fp32"))
    coef = torch.tensor(0.5, device="cuda")
    for step in range(1, 4):
        grad = torch.randn(n, device="cuda") * 1e-2
        g.grad_shard = grad.clone()
        cops.adamw_flat(g, m, v, coef, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
        for lo, hi, wd in ((0, de, 0.1), (de, n, 0.0)):
            ref.adamw_step(p_ref[lo:hi], grad[lo:hi] * 0.5, m_ref[lo:hi], v_ref[lo:hi], lr=1e-2, beta1=0.9, beta2=0.95,
                           eps=1e-8, weight_decay=wd, step=step)
    tol = {"fp32": 1e-5, "bf16": 3e-2, "fp8": 0.3}[kind]
    if p_dtype == torch.bfloat16:
        tol = max(tol, 2e-2)
    # compare the *update* (p - p0 is O(lr)); relative tolerance on the parameter itself
    _close(g.shard, p_ref, tol, 1e-2 * tol + (1e-3 if p_dtype == torch.bfloat16 else 0))
    if kind == "fp32" and p_dtype == torch.float32:
        # the boundary is exact: with decay everywhere the tail would differ by lr * wd * p per step
        assert torch.allclose(g.shard[de:], p_ref[de:], atol=1e-7)


@pytest.mark.parametrize("kind", ["fp32", "fp8"])
def test_background_adamw_in_pieces_equals_one_launch(cops, kind):
    """An update that runs beside other streams' kernels (``ctas_per_sm`` > 0) is cut into launches of a set number of elements (2^23 here);
    two and a bit pieces give bit for bit what the single full-width launch gives, sum of squares included."""
    from system_lab_b200.trainer.optim import _Moment
    torch.manual_seed(11)
    n = 2 * (1 << 23) + 128 * 4101
    de = (1 << 23) + 128 * 77                      # the decay boundary falls inside the second piece

    def run(ctas):
        class G:
            pass
        g = G()
        gen = torch.Generator(device="cuda").manual_seed(5)
        g.shard = 0.02 * torch.randn(n, device="cuda", generator=gen)
        g.full, g.sharded = g.shard, True
        g.shard_decay_end = lambda: de
        g.shard_lp = torch.empty(n, device="cuda", dtype=torch.bfloat16)
        m, v = _Moment(n, kind, "cuda"), _Moment(n, kind, "cuda", sqrt_domain=(kind != "fp32"))
        sq = torch.zeros(1, device="cuda")
        before = cops.LAUNCHES[0]
        for step in (1, 2):
            g.grad_shard = 1e-2 * torch.randn(n, device="cuda", generator=gen)
            cops.adamw_flat(g, m, v, None, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step,
                            sq_out=sq, ctas_per_sm=ctas)
        return g.shard, m.data, v.data, sq, cops.LAUNCHES[0] - before

    p0, m0, v0, sq0, l0 = run(0)
    cops.set_adamw_background_piece(1 << 23)
    try:
        p1, m1, v1, sq1, l1 = run(2)
    finally:
        cops.set_adamw_background_piece(1 << 25)
    raw = lambda t: t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t
    assert torch.equal(p0, p1) and torch.equal(raw(m0), raw(m1)) and torch.equal(raw(v0), raw(v1))
    assert abs(sq0.item() - sq1.item()) <= 1e-5 * sq0.item()
    assert l0 == 2 and l1 == 6                     # three launches per background update


def test_sumsq(cops):
    x = torch.randn(1_000_003, device="cuda")
    out = torch.zeros(1, device="cuda")
    cops.sumsq(x, 0.5, out)
    assert abs(out.item() - 0.5 * x.double().pow(2).sum().item()) / out.item() < 1e-4
