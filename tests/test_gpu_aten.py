"""The drop-in boundary: after b200norm.enable_aten_overrides() the stock PyTorch entry points
(torch.nn.functional.*, torch.ops.aten.*, autograd) run on these kernels for CUDA tensors.  The
cases mirror what the reference's re-hosted suites exercise: functional + .out overloads, autograd
through the backward operators, non-contiguous inputs, every softmax dim, the OpInfo sample inputs."""
import math

import pytest
import torch
import torch.nn.functional as F

import b200norm
from b200norm import capi
from oracle import aten_oracle as ao

from gpu_util import DEV, forced_path, wgrad_gate

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _overrides():
    b200norm.enable_aten_overrides()
    yield


def test_the_dispatcher_really_lands_in_this_library():
    # forcing the ring family makes a ring-ineligible shape fail inside OUR wrapper: proof that the
    # CUDA dispatch key now points here and not at PyTorch's own kernels
    x = torch.randn(4, 33, device=DEV)
    with forced_path(b200norm.PATH_RING):
        with pytest.raises(RuntimeError, match="b200norm"):
            F.softmax(x, -1)
        with pytest.raises(RuntimeError, match="b200norm"):
            F.layer_norm(x, [33])
    F.softmax(x, -1)
    assert capi.last_path() == "generic"
    F.layer_norm(torch.randn(8, 1024, device=DEV), [1024])
    assert capi.last_path() == "ring"


@pytest.mark.parametrize("dt,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.float32),
                                    (torch.bfloat16, torch.bfloat16), (torch.float16, torch.float16)])
@pytest.mark.parametrize("shape,ns", [((6, 128), [128]), ((2, 5, 1024), [1024]), ((3, 4, 6), [4, 6]), ((5, 7), [7])])
def test_layer_norm_autograd(shape, ns, dt, wdt):
    x = ao.randn(shape, 600, dt)
    g, b = ao.randn(ns, 601, wdt, 1.0, 0.1), ao.randn(ns, 602, wdt)
    dy = ao.randn(shape, 603, dt)
    xd, gd, bd = (t.to(DEV).requires_grad_(True) for t in (x, g, b))
    y = F.layer_norm(xd, ns, gd, bd, 1e-5)
    y.backward(dy.to(DEV))
    ry, rmean, rrstd = ao.layer_norm_fwd(x, ns, g, b, 1e-5)
    rdx, rdg, rdb = ao.layer_norm_bwd(dy, x, ns, rmean, rrstd, g, b)
    if dt == torch.float32:
        assert ao.fp32_err(y, ry) <= 1 and ao.fp32_err(xd.grad, rdx) <= 2
    else:
        assert ao.lowp_mismatch(y.detach(), ry)[0] == 0 and ao.lowp_mismatch(xd.grad, rdx)[0] == 0
    assert gd.grad.dtype == wdt and bd.grad.dtype == wdt
    rows = x.reshape(-1, math.prod(ns)).double()
    dyr = dy.reshape(-1, math.prod(ns)).double()
    xh = (rows - rmean.double().reshape(-1, 1)) * rrstd.double().reshape(-1, 1)
    wgrad_gate(gd.grad, dyr * xh, "dgamma")
    wgrad_gate(bd.grad, dyr, "dbeta")


def test_layer_norm_non_contiguous_input_and_stats():
    x = ao.randn((16, 6, 64), 610).transpose(0, 1)  # non-contiguous
    g = ao.randn((64,), 611)
    y, mean, rstd = torch.ops.aten.native_layer_norm(x.to(DEV), [64], g.to(DEV), None, 1e-5)
    ry, rmean, rrstd = torch.ops.aten.native_layer_norm(x, [64], g, None, 1e-5)
    assert y.shape == ry.shape and mean.shape == rmean.shape == (6, 16, 1)
    assert ao.fp32_err(y, ry) <= 1 and ao.fp32_err(rstd, rrstd) <= 1


def test_rms_norm_ops_directly():
    x, w, dy = ao.randn((32, 4096), 620, torch.bfloat16), ao.randn((4096,), 621, torch.float32, 1.0, 0.02), ao.randn((32, 4096), 622, torch.bfloat16)
    y, rstd = torch.ops.aten._fused_rms_norm(x.to(DEV), [4096], w.to(DEV), 1e-6)
    dx, dw = torch.ops.aten._fused_rms_norm_backward(dy.to(DEV), x.to(DEV), [4096], rstd, w.to(DEV), [True, True])
    ry, rrstd = ao.rms_norm_fwd(x, [4096], w, 1e-6)
    rdx, rdw = ao.rms_norm_bwd(dy, x, [4096], w, 1e-6)
    assert rstd.shape == (32, 1) and dw.dtype == torch.float32
    assert ao.lowp_mismatch(y, ry)[0] == 0 and ao.lowp_mismatch(dx, rdx)[0] == 0
    wgrad_gate(dw, dy.double() * x.double() * rstd.cpu().double().reshape(-1, 1), "dweight")
    # same-dtype weights go through F.rms_norm's fused dispatch and autograd
    xd = ao.randn((8, 256), 623).to(DEV).requires_grad_(True)
    wd = ao.randn((256,), 624, mean=1.0, std=0.1).to(DEV).requires_grad_(True)
    F.rms_norm(xd, [256], wd, 1e-6).sum().backward()
    xc = xd.detach().cpu().requires_grad_(True)
    wc = wd.detach().cpu().requires_grad_(True)
    F.rms_norm(xc, [256], wc, 1e-6).sum().backward()
    assert ao.fp32_err(xd.grad, xc.grad) <= 4 and torch.allclose(wd.grad.cpu(), wc.grad, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(7, 50), (2, 3, 129), (4, 5, 6, 7)])
def test_softmax_autograd_every_dim(shape, dt):
    x = ao.randn(shape, 630, dt, 0.0, 2.0)
    dy = ao.randn(shape, 631, dt)
    for dim in range(len(shape)):
        for fn, is_log in ((F.softmax, False), (F.log_softmax, True)):
            xd = x.to(DEV).requires_grad_(True)
            y = fn(xd, dim)
            y.backward(dy.to(DEV))
            ry = ao.softmax_fwd(x, dim, is_log)
            rdx = ao.softmax_bwd(dy, y.detach().cpu(), dim, is_log, dt)
            if dt == torch.float32:
                assert ao.fp32_err(y, ry) <= 1 and ao.fp32_err(xd.grad, rdx) <= 2
            else:
                assert ao.lowp_mismatch(y.detach(), ry)[0] == 0 and ao.lowp_mismatch(xd.grad, rdx)[0] == 0


def test_softmax_out_variants_and_dtype_argument():
    x = ao.randn((9, 70), 640)
    xd = x.to(DEV)
    out = torch.empty(1, device=DEV)
    torch.ops.aten._softmax.out(xd, 1, False, out=out)  # resized
    assert out.shape == (9, 70) and ao.fp32_err(out, ao.softmax_fwd(x, 1, False)) <= 1
    out2 = torch.empty(9, 70, device=DEV)
    torch.ops.aten._log_softmax.out(xd, 0, False, out=out2)
    assert ao.fp32_err(out2, ao.softmax_fwd(x, 0, True)) <= 1
    gi = torch.empty(9, 70, device=DEV)
    dy = ao.randn((9, 70), 641)
    torch.ops.aten._softmax_backward_data.out(dy.to(DEV), out, 1, torch.float32, grad_input=gi)
    assert ao.fp32_err(gi, ao.softmax_bwd(dy, out.cpu(), 1, False, torch.float32)) <= 2
    # softmax(half, dtype=float) is the half_to_float path
    h = ao.randn((5, 300), 642, torch.float16)
    y = F.softmax(h.to(DEV), -1, dtype=torch.float32)
    assert y.dtype == torch.float32 and ao.fp32_err(y, ao.softmax_fwd(h, -1, False, out_dtype=torch.float32)) <= 1
    with pytest.raises(RuntimeError):
        torch.ops.aten._softmax.out(xd, 1, False, out=torch.empty(9, 70, device=DEV, dtype=torch.float16))


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_cross_entropy_end_to_end(dt):
    M, V = 256, 3001
    logits = ao.randn((M, V), 650, dt, 0.0, 2.0)
    t = ao.randint(V, (M,), 651)
    t[10] = -100
    ld = logits.to(DEV).requires_grad_(True)
    loss = F.cross_entropy(ld, t.to(DEV), ignore_index=-100)
    loss.backward()
    lc = logits.float().requires_grad_(True)
    rloss = F.cross_entropy(lc, t, ignore_index=-100)
    rloss.backward()
    if dt == torch.float32:
        assert abs(float(loss) - float(rloss)) <= 1e-5 * abs(float(rloss)) + 1e-6
        assert ao.fp32_err(ld.grad, lc.grad) <= 2
    else:
        assert abs(float(loss) - float(rloss)) <= 2e-2 * abs(float(rloss))
        assert torch.allclose(ld.grad.float().cpu(), lc.grad, rtol=2e-2, atol=1e-5)
    w = ao.randn((V,), 652).abs() + 0.1
    for red in ("none", "sum", "mean"):
        a = F.nll_loss(torch.log_softmax(logits.float(), -1).to(DEV), t.to(DEV), w.to(DEV), reduction=red)
        b = F.nll_loss(torch.log_softmax(logits.float(), -1), t, w, reduction=red)
        assert torch.allclose(a.cpu(), b, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("shape,ns,has_w,has_b", [((1, 2, 3), [1, 2, 3], True, True), ((2, 2, 3), [2, 3], True, False),
                                                  ((1,), [1], False, False), ((1, 2), [2], True, True),
                                                  ((0, 1), [1], True, True), ((2, 0, 4), [4], True, True),
                                                  ((3, 5, 7), [5, 7], False, True)])
def test_layer_norm_sample_matrix(shape, ns, has_w, has_b):
    # the shape / optional-argument matrix of upstream's sample_inputs_native_layer_norm, compared with CPU
    x = ao.randn(shape, 660)
    g = ao.randn(ns, 661) if has_w else None
    b = ao.randn(ns, 662) if has_b else None
    dev = lambda t: None if t is None else t.to(DEV)
    got = torch.ops.aten.native_layer_norm(dev(x), ns, dev(g), dev(b), 0.5)
    exp = torch.ops.aten.native_layer_norm(x, ns, g, b, 0.5)
    for a, e in zip(got, exp):
        assert a.shape == e.shape
        torch.testing.assert_close(a.cpu(), e, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("shape", [(5, 3), (3,), (0, 4), (2, 3, 4, 5)])
@pytest.mark.parametrize("red", ["none", "mean", "sum"])
def test_nll_loss_sample_matrix(shape, red):
    # batch / no-batch / empty-batch / spatial inputs through F.nll_loss, weights and ignore_index included
    c = shape[1] if len(shape) > 1 else shape[0]
    logp = torch.log_softmax(ao.randn(shape, 670), 1 if len(shape) > 1 else 0)
    tshape = (shape[0],) + tuple(shape[2:]) if len(shape) > 1 else ()
    t = ao.randint(c, tshape, 671)
    w = ao.randn((c,), 672).abs() + 0.1
    for weight in (None, w):
        for ign in (-100, 1):
            a = F.nll_loss(logp.to(DEV), t.to(DEV), None if weight is None else weight.to(DEV), ignore_index=ign, reduction=red)
            e = F.nll_loss(logp, t, weight, ignore_index=ign, reduction=red)
            assert a.shape == e.shape
            torch.testing.assert_close(a.cpu(), e, rtol=1e-5, atol=1e-6, equal_nan=True)


def test_safe_softmax_through_the_dispatcher_with_autograd():
    x = torch.randn(6, 2048)
    x[2] = float("-inf")
    x[x > 1.5] = float("-inf")
    xd = x.to(DEV).requires_grad_(True)
    with forced_path(b200norm.PATH_RING):  # a kernel of PyTorch's own would not fail here for a ring-ineligible shape
        with pytest.raises(RuntimeError, match="b200norm"):
            torch._safe_softmax(torch.randn(4, 33, device=DEV), -1)
    y = torch._safe_softmax(xd, -1)
    assert capi.last_path() == "ring"
    g = torch.randn(6, 2048)
    y.backward(g.to(DEV))
    xr = x.clone().requires_grad_(True)
    yr = torch._safe_softmax(xr, -1)
    yr.backward(g)
    assert float(y[2].abs().max()) == 0.0 and not bool(torch.isnan(y).any())
    assert torch.allclose(y.detach().cpu(), yr.detach(), rtol=1e-5, atol=1e-7)
    assert torch.allclose(xd.grad.cpu(), xr.grad, rtol=1e-4, atol=1e-6)
    y16 = torch._safe_softmax(x.to(DEV).half(), -1, torch.float32)
    assert y16.dtype == torch.float32 and float(y16[2].abs().max()) == 0.0


def test_out_of_range_target_surfaces_as_an_error_one_call_late():
    # The reference asserts inside the kernel (LossNLLKernel.cpp:30-35).  Here nothing traps: the row contributes
    # nothing, the kernel records the failure, and the binding raises on the next operator call that finds the
    # record — without any synchronisation of its own.
    logp = torch.log_softmax(ao.randn((8, 10), 690), -1).to(DEV)
    bad = ao.randint(10, (8,), 691)
    bad[3] = 10  # == n_classes
    assert capi.device_status() == 0
    loss = F.nll_loss(logp, bad.to(DEV))
    torch.cuda.synchronize()  # the test's: lets the status copy land so that the NEXT call must see it
    assert torch.isfinite(loss)
    with pytest.raises(RuntimeError, match="target"):
        torch.softmax(logp, -1)
    # reported once; the device word is clear again and the operators carry on
    torch.cuda.synchronize()
    y = torch.softmax(logp, -1)
    assert float((y.sum(-1) - 1).abs().max()) < 1e-5
    assert capi.device_status() == 0
    # ignore_index outside the class range stays legal (test_nn: nll_loss with an out-of-range ignore_index)
    ok = bad.clone()
    F.nll_loss(logp, ok.to(DEV), ignore_index=10)
    torch.cuda.synchronize()
    torch.softmax(logp, -1)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_cross_entropy_autograd_takes_the_fused_backward(dt, reduction):
    # F.cross_entropy with class-index targets: same forward operators, but the backward is ONE pass over the
    # log-probabilities (no dense nll_loss_backward gradient in between) — for every user of the dispatcher
    M, C = 37, 1000
    logits = ao.randn((M, C), 695, dt, 0.0, 2.0)
    t = ao.randint(C, (M,), 696)
    t[3] = -100
    w = ao.randn((C,), 697).abs() + 0.1
    for weight in (None, w):
        ld = logits.detach().clone().to(DEV).requires_grad_(True)
        loss = F.cross_entropy(ld, t.to(DEV), None if weight is None else weight.to(DEV).to(dt), reduction=reduction)
        assert "FusedCrossEntropy" in loss.grad_fn.name()
        gout = ao.randn(tuple(loss.shape), 698, dt).to(DEV) if reduction == "none" else torch.ones((), device=DEV, dtype=dt)
        loss.backward(gout)
        lc = logits.detach().float().clone().requires_grad_(True)
        rloss = F.cross_entropy(lc, t, weight, reduction=reduction)
        rloss.backward(gout.cpu().float())
        if dt == torch.float32:
            assert ao.fp32_err(loss.detach(), rloss.detach()) <= 2 and ao.fp32_err(ld.grad, lc.grad) <= 4
        else:
            assert torch.allclose(loss.detach().float().cpu(), rloss.detach(), rtol=2e-2, atol=1e-2)
            # bf16: the backward works from the bf16-rounded log-probabilities the forward stored, as the stock path does
            assert torch.allclose(ld.grad.float().cpu(), lc.grad, rtol=5e-2, atol=2e-3)
    # what the fused kernel does not cover goes to the composite: label smoothing, probability targets, class dim not last
    ld = logits.detach().clone().to(DEV).requires_grad_(True)
    ls = F.cross_entropy(ld, t.to(DEV), label_smoothing=0.1)
    assert "FusedCrossEntropy" not in ls.grad_fn.name()
    ls.backward()
    lc = logits.detach().float().clone().requires_grad_(True)
    F.cross_entropy(lc, t, label_smoothing=0.1).backward()
    assert torch.allclose(ld.grad.float().cpu(), lc.grad, rtol=5e-2, atol=2e-3)
    probs = torch.softmax(ao.randn((M, C), 699), -1)
    lp = F.cross_entropy(logits.to(DEV).float(), probs.to(DEV))
    assert torch.allclose(lp.cpu(), F.cross_entropy(logits.float(), probs), rtol=1e-4)
    x4 = ao.randn((2, 5, 3, 3), 700).to(DEV).requires_grad_(True)
    l4 = F.cross_entropy(x4, ao.randint(5, (2, 3, 3), 701).to(DEV))
    assert "FusedCrossEntropy" not in l4.grad_fn.name()
    torch.cuda.synchronize()
    assert capi.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_softmax_results_matrix_of_the_reference(dtype):
    # test/xpu/test_nn_xpu.py:14056-14108 (test_softmax_results): non-even sizes, empty tensors and one-element shifts
    # (sliced, non-contiguous, misaligned views) for softmax and log_softmax with dtype=float over dim 0 AND dim 1,
    # forward, backward and double backward, against CPU
    sizes = [(0, 10), (32, 20), (10, 0), (31, 20), (32, 21), (31, 23), (32, 1536), (31, 2048), (33, 2049), (16, 30576)]
    shifts = [(0, 0), (1, 0), (0, 1), (1, 1)]
    gen = torch.Generator().manual_seed(720)
    for fn in (F.softmax, F.log_softmax):
        for size in sizes:
            for shift in shifts:
                base = torch.rand(size, generator=gen).to(dtype)
                if dtype == torch.float16:
                    base = base / 100.0
                gbase = torch.rand(size, generator=gen).to(dtype)
                inp = base.to(DEV)[shift[0]:, shift[1]:].detach().requires_grad_(True)
                ref_inp = base[shift[0]:, shift[1]:].clone().detach().requires_grad_(True)
                for dim in (0, 1):
                    out = fn(inp, dtype=torch.float, dim=dim)
                    ref_out = fn(ref_inp, dtype=torch.float, dim=dim)
                    go = gbase.to(DEV)[shift[0]:, shift[1]:]
                    ref_go = gbase[shift[0]:, shift[1]:].clone()
                    (gi,) = torch.autograd.grad(out, inp, grad_outputs=go, create_graph=True)
                    (ref_gi,) = torch.autograd.grad(ref_out, ref_inp, grad_outputs=ref_go, create_graph=True)
                    gi.sum().backward()
                    ref_gi.sum().backward()
                    # the reference compares with assertEqual's defaults (float32: rtol 1.3e-6, atol 1e-5); the stated
                    # fp32 tolerance of this build is 1e-5 relative, with that same absolute floor
                    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-3, atol=1e-4)
                    torch.testing.assert_close(out.detach().cpu(), ref_out.detach(), **tol)
                    torch.testing.assert_close(gi.detach().cpu(), ref_gi.detach(), **tol)
                    torch.testing.assert_close(inp.grad.cpu(), ref_inp.grad, **tol)
    torch.cuda.synchronize()
    assert capi.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_softmax_backward_with_only_one_unaligned_operand(dtype):
    # test_nn_xpu.py:17922-17999: 2048 elements (the shared-memory path), 2049 (not a whole number of vectors), and
    # each operand alone off the 16-byte boundary: the vector kernels must step aside for exactly those
    gen = torch.Generator().manual_seed(721)

    def unaligned(t):
        buf = torch.ones(t.numel() + 1, dtype=t.dtype, device=DEV)
        view = buf[1:]
        view.copy_(t)
        assert view.data_ptr() % 16 != 0
        return view

    for numel in (2048, 2049):
        out = torch.rand(numel, generator=gen).to(dtype)
        go = (torch.rand(numel, generator=gen) / numel).to(dtype)
        expect = torch._softmax_backward_data(go, out, 0, dtype)
        cases = [(go.to(DEV), out.to(DEV)), (go.to(DEV), unaligned(out)), (unaligned(go), out.to(DEV))]
        for g, o in cases:
            got = torch._softmax_backward_data(g, o, 0, dtype)
            if dtype == torch.float32:
                assert ao.fp32_err(got, expect) <= 2.0
            else:
                assert ao.lowp_mismatch(got, expect)[0] == 0 or torch.allclose(got.float().cpu(), expect.float(), rtol=2e-3, atol=1e-7)
