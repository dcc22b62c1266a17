"""GroupNorm forward and backward, BatchNorm statistics: CUDA kernels through the C ABI and the dispatcher vs CPU ATen.

Tolerances as for layer norm: fp32 outputs |a-b| <= 1e-5*|b| + 1e-6*max(1, rms(b)); 16-bit outputs within 1 ulp of
the fp32-accumulated reference (CPU ATen on fp32 upcasts, rounded once) or the same absolute floor; statistics
relative 1e-5 (+1e-6 absolute).  Shapes: the (N, C, HxW, G) grid the reference's kernel driver distinguishes
(src/ATen/native/xpu/sycl/GroupNormKernels.cpp:365-499: vectorisable or not, one channel per group, one group) and
scaled-down versions of test/microbench/group_norm.py's."""
import pytest
import torch
import torch.nn.functional as F

import b200norm
from b200norm import capi
from oracle import aten_oracle as ao

from gpu_util import DEV, forced_path, wgrad_gate

pytestmark = pytest.mark.gpu

# (N, C, spatial, groups)
GN_SHAPES = [((2, 6, 5), 3), ((1, 4, 1), 2), ((3, 8, 7, 9), 4), ((4, 32, 16, 16), 32), ((2, 32, 8, 8), 1),
             ((8, 128, 32, 32), 16), ((3, 33, 31), 11), ((2, 64, 4, 8, 8), 8), ((1, 16, 128, 128), 4), ((5, 12, 1000), 3)]


def _stat_err(a, ref):
    a, ref = a.detach().cpu().double().reshape(-1), ref.detach().cpu().double().reshape(-1)
    return float(((a - ref).abs() / (1e-5 * ref.abs() + 1e-6)).max()) if a.numel() else 0.0


@pytest.mark.parametrize("affine", [True, False])
@pytest.mark.parametrize("dt,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                    (torch.bfloat16, torch.float32), (torch.float16, torch.float16)])
@pytest.mark.parametrize("shape,G", GN_SHAPES)
def test_group_norm_forward(shape, G, dt, wdt, affine):
    N, C = shape[0], shape[1]
    HxW = 1
    for d in shape[2:]:
        HxW *= d
    x = ao.randn(shape, 1100 + C, dt, 0.5, 2.0)
    g = ao.randn((C,), 1101, wdt, 1.0, 0.2) if affine else None
    b = ao.randn((C,), 1102, wdt, 0.0, 0.2) if affine else None
    dev = lambda t: None if t is None else t.to(DEV)
    y, mean, rstd = capi.native_group_norm(dev(x), dev(g), dev(b), N, C, HxW, G, 1e-5)
    f32 = lambda t: None if t is None else t.float()
    ry, rmean, rrstd = torch.ops.aten.native_group_norm(x.float(), f32(g), f32(b), N, C, HxW, G, 1e-5)
    assert y.shape == x.shape and mean.shape == (N, G) and rstd.shape == (N, G)
    want_stat = torch.float32 if (affine and wdt == torch.float32) else dt
    assert mean.dtype == want_stat and rstd.dtype == want_stat
    if dt == torch.float32:
        assert ao.fp32_err(y, ry) <= 1.0
        assert _stat_err(mean, rmean) <= 1.0 and _stat_err(rstd, rrstd) <= 1.0
    else:
        assert ao.lowp_mismatch(y, ry.to(dt))[0] == 0
        if want_stat == torch.float32:
            assert _stat_err(mean, rmean) <= 1.0 and _stat_err(rstd, rrstd) <= 1.0
        else:
            assert ao.ulp_distance(mean.cpu(), rmean.to(dt)) <= 1 and ao.ulp_distance(rstd.cpu(), rrstd.to(dt)) <= 1
    assert capi.device_status() == 0


@pytest.mark.parametrize("affine", [True, False])
@pytest.mark.parametrize("dt,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                    (torch.bfloat16, torch.float32), (torch.float16, torch.float16)])
@pytest.mark.parametrize("shape,G", GN_SHAPES)
def test_group_norm_backward(shape, G, dt, wdt, affine):
    # dX against CPU ATen on fp32 upcasts (rounded once); dgamma / dbeta element by element against an fp64 sum of
    # their terms (1e-6 of the L1 norm; 16-bit: one ulp of that sum); the statistics are the forward's own
    N, C = shape[0], shape[1]
    HxW = 1
    for d in shape[2:]:
        HxW *= d
    x = ao.randn(shape, 1400 + C, dt, 0.5, 2.0)
    dy = ao.randn(shape, 1401 + C, dt)
    g = ao.randn((C,), 1402, wdt, 1.0, 0.2) if affine else None
    dev = lambda t: None if t is None else t.to(DEV)
    _, mean, rstd = capi.native_group_norm(dev(x), dev(g), None, N, C, HxW, G, 1e-5)
    dx, dg, db = capi.native_group_norm_backward(dev(dy), dev(x), mean, rstd, dev(g), N, C, HxW, G, (True, True, True))
    vec = 16 // x.element_size()
    assert capi.last_path() == ("ring" if HxW % vec == 0 and (C // G) * HxW <= 8192 else "generic")
    f32 = lambda t: None if t is None else t.float()
    m32, r32 = mean.float().cpu(), rstd.float().cpu()
    rdx, _, _ = torch.ops.aten.native_group_norm_backward(dy.float(), x.float(), m32, r32, f32(g), N, C, HxW, G,
                                                          [True, affine, affine])
    assert dx.shape == x.shape and dx.dtype == dt
    if dt == torch.float32:
        assert ao.fp32_err(dx, rdx) <= 1.0
    else:
        assert ao.lowp_mismatch(dx, rdx.to(dt))[0] == 0
    if affine:
        assert dg.shape == (C,) and db.shape == (C,) and dg.dtype == wdt and db.dtype == wdt
        D = C // G
        x64 = x.double().reshape(N, C, HxW)
        xh = (x64 - m32.double().repeat_interleave(D, 1).view(N, C, 1)) * r32.double().repeat_interleave(D, 1).view(N, C, 1)
        d64 = dy.double().reshape(N, C, HxW)
        wgrad_gate(dg, (d64 * xh).permute(0, 2, 1).reshape(-1, C), "dgamma")
        wgrad_gate(db, d64.permute(0, 2, 1).reshape(-1, C), "dbeta")
    else:
        assert dg is None and db is None
    # masked-off outputs are not computed
    only_dx = capi.native_group_norm_backward(dev(dy), dev(x), mean, rstd, dev(g), N, C, HxW, G, (True, False, False))
    assert only_dx[1] is None and only_dx[2] is None and torch.equal(only_dx[0], dx)
    # the plain kernels (what shapes the ring cannot take run) pass the same gate on every shape
    with forced_path(b200norm.PATH_GENERIC):
        gdx = capi.native_group_norm_backward(dev(dy), dev(x), mean, rstd, dev(g), N, C, HxW, G, (True, False, False))[0]
        assert capi.last_path() == "generic"
    if dt == torch.float32:
        assert ao.fp32_err(gdx, rdx) <= 1.0
    else:
        assert ao.lowp_mismatch(gdx, rdx.to(dt))[0] == 0
    assert capi.device_status() == 0


def test_group_norm_large_offset_and_argument_checks():
    x = (torch.randn(2, 8, 64) + 3.0e4).to(DEV)  # mean far from the first element's neighbourhood in relative terms
    y, mean, rstd = capi.native_group_norm(x, None, None, 2, 8, 64, 2, 1e-5)
    ry, rmean, rrstd = torch.ops.aten.native_group_norm(x.cpu().double(), None, None, 2, 8, 64, 2, 1e-5)
    assert torch.allclose(y.cpu().double(), ry, atol=2e-2)  # fp32 input at 3e4: one ulp of x is 2e-3 before the 1/std scaling
    assert _stat_err(mean, rmean) <= 1.0
    with pytest.raises(RuntimeError):
        capi.native_group_norm(x, None, None, 2, 8, 64, 3, 1e-5)
    with pytest.raises(RuntimeError):
        capi.native_group_norm(x, torch.ones(7, device=DEV), None, 2, 8, 64, 2, 1e-5)


def test_group_norm_through_the_dispatcher_with_autograd():
    b200norm.enable_aten_overrides()
    x = ao.randn((4, 32, 16, 16), 1110)
    m = torch.nn.GroupNorm(8, 32)
    with torch.no_grad():
        m.weight.copy_(ao.randn((32,), 1111, mean=1.0, std=0.2))
        m.bias.copy_(ao.randn((32,), 1112, std=0.2))
    xr = x.clone().requires_grad_(True)
    yr = m(xr)
    yr.backward(torch.ones_like(yr) * 0.5)
    md = torch.nn.GroupNorm(8, 32).to(DEV)
    md.load_state_dict(m.state_dict())
    xd = x.to(DEV).requires_grad_(True)
    capi.native_group_norm(xd.detach(), md.weight.detach(), md.bias.detach(), 4, 32, 256, 8, 1e-5)
    launches = capi.launch_count()
    yd = md(xd)
    assert capi.launch_count() == launches + 1  # the dispatcher reached this library's forward kernel
    yd.backward(torch.ones_like(yd) * 0.5)
    # ... and autograd's native_group_norm_backward reached this library's kernels too (it runs on the autograd engine's
    # own thread, whose launch counter this thread cannot see: the gradients are bit-identical to a direct call)
    _, mean, rstd = capi.native_group_norm(xd.detach(), md.weight.detach(), md.bias.detach(), 4, 32, 256, 8, 1e-5)
    ddx, ddg, ddb = capi.native_group_norm_backward(torch.full_like(yd, 0.5), xd.detach(), mean, rstd, md.weight.detach(), 4, 32,
                                                    256, 8)
    assert torch.equal(xd.grad, ddx) and torch.equal(md.weight.grad, ddg) and torch.equal(md.bias.grad, ddb)
    assert ao.fp32_err(yd, yr) <= 1.0
    assert ao.fp32_err(xd.grad, xr.grad) <= 1.0
    assert torch.allclose(md.weight.grad.cpu(), m.weight.grad, rtol=1e-5, atol=1e-4)
    assert torch.allclose(md.bias.grad.cpu(), m.bias.grad, rtol=1e-5, atol=1e-4)
    # channels-last input: made contiguous by the composite, same result
    yc = md(x.to(DEV).contiguous(memory_format=torch.channels_last))
    assert ao.fp32_err(yc.contiguous(), yr) <= 1.0


# the last four take several CTAs per channel (few channels with much data each): the reference microbenchmark's
# (4, 8, 640, 1024) and (24, 512, 28, 28), and two with ragged splits
BN_SHAPES = [(8, 16), (64, 33), (4, 8, 5), (16, 32, 16, 16), (3, 7, 33, 9), (2, 64, 4, 8, 8), (128, 256), (2, 3, 100000),
             (4, 8, 640, 1024), (24, 512, 28, 28), (7, 5, 3000, 8), (129, 2, 72, 56)]


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", BN_SHAPES)
def test_batch_norm_stats(shape, dt):
    x = ao.randn(shape, 1200 + shape[1], dt, 1.5, 3.0)
    mean, invstd = capi.batch_norm_stats(x.to(DEV), 1e-5)
    dims = [0] + list(range(2, len(shape)))
    x64 = x.double()
    rmean = x64.mean(dims)
    rvar = x64.var(dims, unbiased=False)
    assert mean.dtype == torch.float32 and mean.shape == (shape[1],)
    assert _stat_err(mean, rmean) <= 1.0 and _stat_err(invstd, 1.0 / torch.sqrt(rvar + 1e-5)) <= 1.0

    # update_stats: the biased variance out, the running statistics blended with the unbiased one
    for rdt in (torch.float32, dt):
        rm0, rv0 = ao.randn((shape[1],), 1201, rdt), ao.randn((shape[1],), 1202, rdt).abs() + 0.5
        rm, rv = rm0.to(DEV), rv0.to(DEV)
        m2, v2 = capi.batch_norm_update_stats(x.to(DEV), rm, rv, 0.1)
        n = x.numel() // shape[1]
        assert _stat_err(m2, rmean) <= 1.0 and _stat_err(v2, rvar) <= 1.0
        want_rm = 0.9 * rm0.double() + 0.1 * rmean
        want_rv = 0.9 * rv0.double() + 0.1 * rvar * n / max(n - 1, 1)
        tol = 1e-5 if rdt == torch.float32 else 1e-2
        assert torch.allclose(rm.cpu().double(), want_rm, rtol=tol, atol=tol)
        assert torch.allclose(rv.cpu().double(), want_rv, rtol=tol, atol=tol)
    m3, v3 = capi.batch_norm_update_stats(x.to(DEV), None, None, 0.1)
    assert _stat_err(m3, rmean) <= 1.0 and _stat_err(v3, rvar) <= 1.0
    assert capi.device_status() == 0


def test_batch_norm_ops_through_the_dispatcher():
    b200norm.enable_aten_overrides()
    x = ao.randn((8, 24, 10, 10), 1210).to(DEV)
    launches = capi.launch_count()
    mean, invstd = torch.batch_norm_stats(x, 1e-5)
    rm, rv = torch.zeros(24, device=DEV), torch.ones(24, device=DEV)
    m2, v2 = torch.batch_norm_update_stats(x, rm, rv, 0.1)
    assert capi.launch_count() == launches + 2, capi.launch_count() - launches
    xr = x.cpu().double()
    assert _stat_err(mean, xr.mean((0, 2, 3))) <= 1.0
    assert _stat_err(invstd, 1 / torch.sqrt(xr.var((0, 2, 3), unbiased=False) + 1e-5)) <= 1.0
    crm, crv = torch.zeros(24), torch.ones(24)
    cm, cv = torch.batch_norm_update_stats(x.cpu(), crm, crv, 0.1)
    assert _stat_err(m2, cm) <= 1.0 and _stat_err(v2, cv) <= 1.0
    assert torch.allclose(rm.cpu(), crm, rtol=1e-5, atol=1e-6) and torch.allclose(rv.cpu(), crv, rtol=1e-5, atol=1e-6)


def test_batch_norm_stats_split_over_several_ctas_is_reproducible_and_survives_a_large_offset():
    # [6, 4, 200, 1000] bf16: four channels, so every channel is shared by dozens of CTAs whose partial sums are added
    # in a fixed order — two runs give the same bits, and the one-CTA-per-channel path (no scratch) agrees to fp32
    # rounding.  Then a mean 300 standard deviations away from zero: the sums about a few sampled elements stay
    # well conditioned; and a channel whose sampled elements are outliers takes the second pass about its mean.
    lib = b200norm.load_library()
    x = ao.randn((6, 4, 200, 1000), 1300, torch.bfloat16, 0.5, 2.0)
    N, C, HxW = 6, 4, 200 * 1000
    assert lib.b2n_batch_norm_stats_workspace_bytes(N, C, HxW, b200norm.BF16) > 0
    xd = x.to(DEV)
    m1, i1 = capi.batch_norm_stats(xd, 1e-5)
    m2, i2 = capi.batch_norm_stats(xd, 1e-5)
    assert torch.equal(m1, m2) and torch.equal(i1, i2)
    m0, i0 = torch.empty_like(m1), torch.empty_like(i1)
    rc = lib.b2n_batch_norm_stats(xd.data_ptr(), m0.data_ptr(), i0.data_ptr(), None, None, N, C, HxW, 1e-5, 0.0, 0,
                                  b200norm.BF16, b200norm.F32, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    x64 = x.double()
    rmean, rvar = x64.mean((0, 2, 3)), x64.var((0, 2, 3), unbiased=False)
    for m, i in ((m1, i1), (m0, i0)):
        assert _stat_err(m, rmean) <= 1.0 and _stat_err(i, 1.0 / torch.sqrt(rvar + 1e-5)) <= 1.0
    y = ao.randn((6, 4, 200, 1000), 1301, torch.float32, 300.0, 1.0)
    y[:, 1, 0, 0] = -5000.0  # channel 1: the sampled elements are outliers, the first pass cancels, the second repairs it
    m, i = capi.batch_norm_stats(y.to(DEV), 1e-5)
    y64 = y.double()
    assert _stat_err(m, y64.mean((0, 2, 3))) <= 1.0
    assert _stat_err(i, 1.0 / torch.sqrt(y64.var((0, 2, 3), unbiased=False) + 1e-5)) <= 2.0
    assert capi.device_status() == 0
