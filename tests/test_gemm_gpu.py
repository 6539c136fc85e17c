"""tcgen05 grouped GEMM (forward, dgrad, wgrad) vs fp32 PyTorch on the same bf16 inputs."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _segments(counts, pad=128, device="cuda"):
    counts = torch.tensor(counts, dtype=torch.int32)
    padded = (counts + pad - 1) // pad * pad
    offsets = torch.cumsum(padded, 0) - padded
    return offsets.to(device).int(), counts.to(device).int(), int(padded.sum())


def _inputs(counts, n, k, seed=0):
    torch.manual_seed(seed)
    offsets, cnts, rows = _segments(counts)
    e = len(counts)
    a = torch.zeros(rows, k, device="cuda", dtype=torch.bfloat16)
    dy = torch.zeros(rows, n, device="cuda", dtype=torch.bfloat16)
    for o, c in zip(offsets.tolist(), cnts.tolist()):
        a[o:o + c] = torch.randn(c, k, device="cuda")
        dy[o:o + c] = torch.randn(c, n, device="cuda")
    w = (0.05 * torch.randn(e, n, k, device="cuda")).to(torch.bfloat16)
    return a, dy, w, offsets, cnts


def _check(out, ref, what):
    from system_lab_b200.ops import cuda
    cuda.check_status()
    err = (out.float() - ref.float()).abs().max().item()
    scale = ref.float().abs().max().item() + 1e-6
    assert err / scale < 2e-2, f"{what}: max abs err {err:.4e} vs scale {scale:.3e}"


CASES = [([128], 256, 128), ([100, 0, 300, 129], 512, 256), ([5, 700, 64, 1], 768, 2048), ([130, 250], 2880, 192)]


@pytest.mark.parametrize("counts,n,k", CASES)
@pytest.mark.parametrize("bn", [128, 256])
def test_forward(counts, n, k, bn):
    from system_lab_b200.ops import cuda, reference as ref
    a, dy, w, off, cnt = _inputs(counts, n, k)
    out = cuda.grouped_gemm_raw(0, a, w, off, cnt, n, k, block_n=bn)
    _check(out, ref.grouped_gemm(a, w, off, cnt), "fwd")


@pytest.mark.parametrize("counts,n,k", CASES)
@pytest.mark.parametrize("bn", [128, 256])
def test_dgrad(counts, n, k, bn):
    from system_lab_b200.ops import cuda, reference as ref
    a, dy, w, off, cnt = _inputs(counts, n, k, 1)
    out = cuda.grouped_gemm_raw(1, dy, w, off, cnt, n, k, block_n=bn)
    _check(out, ref.grouped_gemm_dgrad(dy, w, off, cnt), "dgrad")


@pytest.mark.parametrize("counts,n,k", CASES[:3])
@pytest.mark.parametrize("bn", [128, 256])
def test_wgrad(counts, n, k, bn):
    from system_lab_b200.ops import cuda, reference as ref
    a, dy, w, off, cnt = _inputs(counts, n, k, 2)
    out = cuda.grouped_gemm_raw(2, dy, a, off, cnt, n, k, block_n=bn)
    _check(out, ref.grouped_gemm_wgrad(dy, a, off, cnt), "wgrad")
    acc = out.clone()
    cuda.grouped_gemm_raw(2, dy, a, off, cnt, n, k, out=acc, accumulate=True, block_n=bn)
    _check(acc, 2 * ref.grouped_gemm_wgrad(dy, a, off, cnt).float(), "wgrad accumulate")


@pytest.mark.parametrize("counts,n,k", [([130, 250], 2880, 192), ([64, 0, 300], 192, 320)])
@pytest.mark.parametrize("bn", [128, 256])
def test_wgrad_partial_row_tile(counts, n, k, bn):
    """N % 128 == 64 (hidden 2880): the last 64 rows of every expert's gradient come from a tile that hangs over
    the expert boundary; it must be written in full and must not touch the next expert's rows."""
    from system_lab_b200.ops import cuda, reference as ref
    a, dy, w, off, cnt = _inputs(counts, n, k, 2)
    out = cuda.grouped_gemm_raw(2, dy, a, off, cnt, n, k, block_n=bn)
    _check(out, ref.grouped_gemm_wgrad(dy, a, off, cnt), "wgrad partial")
    acc = out.clone()
    cuda.grouped_gemm_raw(2, dy, a, off, cnt, n, k, out=acc, accumulate=True, block_n=bn)
    _check(acc, 2 * ref.grouped_gemm_wgrad(dy, a, off, cnt).float(), "wgrad partial accumulate")


def test_autograd_grouped_linear():
    from system_lab_b200 import ops
    from system_lab_b200.ops import reference as ref
    a, dy, w, off, cnt = _inputs([200, 56, 0, 384], 512, 256, 3)
    a.requires_grad_(True)
    w.requires_grad_(True)
    out = ops.grouped_linear(a, w, off, cnt)
    out.backward(dy)
    _check(out, ref.grouped_gemm(a.detach(), w.detach(), off, cnt), "fwd")
    _check(a.grad, ref.grouped_gemm_dgrad(dy, w.detach(), off, cnt), "dgrad")
    _check(w.grad, ref.grouped_gemm_wgrad(dy, a.detach(), off, cnt), "wgrad")


@pytest.mark.parametrize("counts,n,k", [([128], 128, 128), ([100, 0, 300, 129], 512, 256), ([5, 700, 64, 1], 768, 2048)])
def test_fp8_block_scaled_forward(counts, n, k):
    from system_lab_b200.ops import cuda, reference as ref
    a, dy, w, off, cnt = _inputs(counts, n, k, 5)
    aq, sa = cuda.quant_1x128(a)
    wq, sw = cuda.quant_128x128(w)
    out = cuda.grouped_gemm_fp8_raw(aq, sa.contiguous(), wq, sw.contiguous(), off, cnt)
    # oracle on the *dequantised* operands: isolates the kernel from the quantisation error
    exp = ref.grouped_gemm(ref.dequant_1x128(aq, sa), ref.dequant_128x128(wq, sw), off, cnt)
    _check(out, exp, "fp8 fwd")
    # and the end-to-end error against the bf16 operands stays at the fp8 level
    full = ref.grouped_gemm(a, w, off, cnt)
    rel = (out.float() - full.float()).norm() / full.float().norm()
    assert rel < 0.06, rel


@pytest.mark.parametrize("counts,n,k", [([128], 256, 128), ([100, 0, 300, 129], 512, 256), ([5, 700, 64, 1], 768, 2048),
                                        ([130, 250], 2880, 384), ([77], 64, 128)])
def test_fp8_row_scaled_forward(counts, n, k):
    from system_lab_b200.ops import cuda, reference as ref
    a, dy, w, off, cnt = _inputs(counts, n, k, 6)
    aq, sa = cuda.quant_rowwise(a)
    wq, sw = cuda.quant_rowwise(w)
    aq_ref, sa_ref = ref.quant_rowwise(a)
    torch.testing.assert_close(sa, sa_ref, rtol=1e-5, atol=0)
    assert (aq.float() - aq_ref.float()).abs().max() <= 0.13 * aq_ref.float().abs().max()
    out = cuda.grouped_gemm_fp8_rowwise_raw(aq, sa, wq, sw.contiguous(), off, cnt)
    exp = ref.grouped_gemm(aq.float() * sa[:, None], wq.float() * sw[..., None], off, cnt)
    _check(out, exp, "fp8 rowwise fwd")
    full = ref.grouped_gemm(a, w, off, cnt)
    rel = (out.float() - full.float()).norm() / full.float().norm()
    assert rel < 0.06, rel


@pytest.mark.parametrize("recipe", ["rowwise", "tensorwise", "blockwise"])
def test_autograd_grouped_linear_fp8_forward_bf16_backward(recipe):
    from system_lab_b200 import ops
    from system_lab_b200.ops import reference as ref
    a, dy, w, off, cnt = _inputs([200, 56, 0, 384], 512, 256, 7)
    a.requires_grad_(True)
    w.requires_grad_(True)
    out = ops.grouped_linear(a, w, off, cnt, fp8=recipe)
    out.backward(dy)
    full = ref.grouped_gemm(a.detach(), w.detach(), off, cnt)
    rel = (out.float() - full.float()).norm() / full.float().norm()
    assert 1e-4 < rel < 0.06, rel                 # quantised, but within e4m3 noise of the bf16 product
    _check(a.grad, ref.grouped_gemm_dgrad(dy, w.detach(), off, cnt), "dgrad")
    _check(w.grad, ref.grouped_gemm_wgrad(dy, a.detach(), off, cnt), "wgrad")


@pytest.mark.parametrize("lead,n,k", [((300,), 5120, 2048), ((2, 130), 1024, 512), ((4096,), 576, 7168), ((77,), 128, 64)])
def test_dense_linear_forward_and_both_gradients(lead, n, k):
    """``ops.linear`` = the grouped kernel with one segment: forward, input gradient and weight gradient against fp32
    PyTorch; the result is a fresh tensor (callers modify it in place)."""
    from system_lab_b200 import ops
    torch.manual_seed(7)
    x = torch.randn(*lead, k, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (0.05 * torch.randn(n, k, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    g = torch.randn(*lead, n, device="cuda", dtype=torch.bfloat16)
    y = ops.linear(x, w)
    assert y._base is None and y.shape == (*lead, n)
    y.mul_(1.0)                                    # in-place use of the result must be legal
    y.backward(g)
    xf, wf, gf = x.detach().float(), w.detach().float(), g.float()
    _check(y, xf @ wf.t(), "linear fwd")
    _check(x.grad, gf @ wf, "linear dgrad")
    _check(w.grad, gf.reshape(-1, n).t() @ xf.reshape(-1, k), "linear wgrad")


def test_dense_linear_writes_and_accumulates_into_main_grad():
    from system_lab_b200 import ops
    torch.manual_seed(8)
    n, k = 512, 256
    x = torch.randn(200, k, device="cuda", dtype=torch.bfloat16)
    w = torch.nn.Parameter((0.05 * torch.randn(n, k, device="cuda")).to(torch.bfloat16))
    w.main_grad = torch.full((n, k), 123.0, device="cuda", dtype=torch.bfloat16)     # garbage: the first write overwrites
    w.main_grad_written = False
    g = torch.randn(200, n, device="cuda", dtype=torch.bfloat16)
    for _ in range(2):                                                              # the weight is used twice
        ops.linear(x, w).backward(g)
    assert w.grad is None and w.main_grad_written
    _check(w.main_grad, 2 * (g.float().t() @ x.float()), "linear wgrad into main_grad, twice")


def test_linear_cross_entropy_on_own_gemms_matches_reference():
    from system_lab_b200 import ops
    from system_lab_b200.ops import reference as ref
    torch.manual_seed(9)
    rows, hd, v = 700, 256, 1024
    h = torch.randn(rows, hd, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (0.05 * torch.randn(v, hd, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    t = torch.randint(0, v, (rows,), device="cuda")
    from system_lab_b200.ops import cuda
    loss = cuda._LinearCE.apply(h, w, t, 256)          # three chunks: the weight gradient overwrites, then accumulates
    (loss * 2.0).backward()
    hr = h.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    lr = ref.linear_cross_entropy(hr, wr, t)
    (lr * 2.0).backward()
    assert abs(float(loss) - float(lr)) < 2e-2
    _check(h.grad, hr.grad, "ce dh")
    _check(w.grad, wr.grad, "ce dw")


@pytest.mark.parametrize("counts,n,k", [([100, 0, 300, 129], 512, 256), ([5, 700, 64, 1], 768, 2048)])
def test_fp8_row_scaled_input_gradient(counts, n, k):
    """dgrad on the fp8 path: dY quantised per row, the weight from its transposed e4m3 copy (one scale per expert and
    k), against the fp32 product of the same bf16 operands; the cached copy is rebuilt when the weight changes."""
    from system_lab_b200.ops import cuda, reference as ref
    a, dy, w, off, cnt = _inputs(counts, n, k, 5)
    out = cuda.grouped_gemm_fp8_dgrad_rowwise(dy, w, off, cnt)
    want = ref.grouped_gemm_dgrad(dy, w, off, cnt)
    cuda.check_status()
    err = (out.float() - want.float()).abs().max().item()
    assert err < 8e-2 * (want.float().abs().max().item() + 1e-6), err          # e4m3 operands: ~6 % relative noise
    w.mul_(2.0)                                                                 # version bump: the cache must notice
    out2 = cuda.grouped_gemm_fp8_dgrad_rowwise(dy, w, off, cnt)
    err2 = (out2.float() - 2 * want.float()).abs().max().item()
    assert err2 < 8e-2 * (2 * want.float().abs().max().item() + 1e-6), err2
