"""The allocation-free RMSNorm backward (``slab_rmsnorm_bwd_noalloc``), called through its exported C
symbol exactly as a host program without an allocator would call it.

Such a caller owns a fixed set of device buffers and may not ask for more, so the entry point keeps its
scratch inside the library.  The check: for the same inputs it must produce what the regular entry point
(``slab_rmsnorm_bwd``, scratch supplied by the caller) produces, and what the formula gives in fp32 PyTorch, on
two calls in a row with different inputs -- the second call finds the first call's leftovers in the shared
scratch and must not be disturbed by them.  Neither PyTorch's allocator nor the driver's free-memory figure may
move across the warm call.  This file sorts last so a run that stops at the first failure has already exercised
everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from system_lab_b200.ops import cuda as cops
    lib = cops.lib()
    fn = lib.slab_rmsnorm_bwd_noalloc
    fn.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return cops, fn


def _case(rows, h, seed, with_res):
    torch.manual_seed(seed)
    dev = "cuda"
    x = torch.randn(rows, h, device=dev, dtype=torch.bfloat16)
    g = torch.randn(rows, h, device=dev, dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(h, device=dev)).to(torch.bfloat16)
    gres = torch.randn(rows, h, device=dev, dtype=torch.bfloat16) if with_res else None
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
    return x, g, w, gres, rstd


@pytest.mark.parametrize("h", [2048, 2880, 7168])
def test_noalloc_matches_regular_entry_point_twice(h):
    cops, fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (rows, seed, with_res) in enumerate([(517, 11, False), (96, 12, True)]):
        x, g, w, gres, rstd = _case(rows, h, seed, with_res)
        # regular entry point: the caller brings the scratch
        nb = cops.lib().slab_rmsnorm_bwd_blocks(rows)
        part = torch.empty(nb, h, dtype=torch.float32, device="cuda")
        counters = torch.zeros(cops.lib().slab_rmsnorm_bwd_counters(), dtype=torch.int32, device="cuda")
        dx_ref, dw_ref = torch.empty_like(x), torch.empty_like(w)
        cops.call("slab_rmsnorm_bwd", g, x, w, rstd, gres, dx_ref, part, counters, dw_ref, rows, h, stream)
        assert int(counters.abs().sum()) == 0, "the regular entry point must leave its counters at zero"
        # allocation-free entry point: outputs only
        dx, dw = torch.empty_like(x), torch.empty_like(w)
        args = (g.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                gres.data_ptr() if gres is not None else None, dx.data_ptr(), dw.data_ptr(), rows, h, stream)
        # unmeasured call first: the first call on a device resolves the scratch address, and the first use of a
        # kernel variant makes the driver load its code (which moves the free-memory figure by itself)
        assert fn(*args) == 0
        torch.cuda.synchronize()
        before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        rc = fn(*args)
        torch.cuda.synchronize()
        assert rc == 0, f"call {call}: rc={rc}"
        assert torch.cuda.memory_allocated() == before
        assert torch.cuda.mem_get_info()[0] == free_before, "the driver's free memory moved: something allocated"
        assert torch.allclose(dx.float(), dx_ref.float(), rtol=2e-2, atol=2e-2), f"call {call}: dx differs"
        assert torch.allclose(dw.float(), dw_ref.float(), rtol=2e-2, atol=2e-2), f"call {call}: dw differs"
        # the formula itself, in fp32
        xf, gf, wf = x.float(), g.float(), w.float()
        gw = gf * wf
        dx_f = rstd[:, None] * gw - xf * (rstd ** 3)[:, None] * (gw * xf).mean(-1, keepdim=True)
        if gres is not None:
            dx_f = dx_f + gres.float()
        dw_f = (gf * xf * rstd[:, None]).sum(0)
        assert torch.allclose(dx.float(), dx_f, rtol=2e-2, atol=2e-2), f"call {call}: dx differs from fp32 PyTorch"
        assert torch.allclose(dw.float(), dw_f, rtol=2e-2, atol=2e-2 * max(1.0, float(dw_f.abs().max()) / 16)), \
            f"call {call}: dw differs from fp32 PyTorch"


def test_noalloc_rejects_oversized_hidden():
    cops, fn = _lib()
    h = 8192 + 8
    x, g, w, gres, rstd = _case(4, h, 0, False)
    dx, dw = torch.empty_like(x), torch.empty_like(w)
    rc = fn(g.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), None, dx.data_ptr(), dw.data_ptr(), 4, h,
            torch.cuda.current_stream().cuda_stream)
    assert rc == -101


def test_noalloc_zero_rows_writes_zero_gain_gradient():
    cops, fn = _lib()
    h = 2048
    x, g, w, gres, rstd = _case(4, h, 0, False)
    dx = torch.empty_like(x)
    dw = torch.full_like(w, 7.0)
    rc = fn(g.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), None, dx.data_ptr(), dw.data_ptr(), 0, h,
            torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0
    assert float(dw.float().abs().max()) == 0.0
