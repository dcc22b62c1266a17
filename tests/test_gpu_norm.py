"""Layer norm / RMS norm parity: CUDA kernels through the C ABI vs the CPU oracle.

Tolerances (stated by the task): fp32 outputs |a-b| <= 1e-5*|b| + 1e-6*max(1, rms(b)); 16-bit outputs
within 1 ulp of the fp32-accumulated reference (CPU ATen on fp32 upcasts, rounded once) or, for outputs
near zero, within the same absolute floor 1e-6*max(1, rms) (oracle.aten_oracle.lowp_mismatch); mean/rstd
relative 1e-5; fp32 weight-gradient sums within 1e-6 of the L1 norm of their terms from an fp64 sum.
"""
import math

import pytest
import torch

import b200norm
from b200norm import capi
from oracle import aten_oracle as ao
from oracle import restate

from gpu_util import DEV, forced_path, guarded_empty, misaligned, ring_eligible, wgrad_gate

pytestmark = pytest.mark.gpu

SHAPES = [(1, 1), (3, 5), (7, 128), (33, 130), (257, 1024), (64, 4096), (19, 8192), (5, 16384), (3, 40000)]
DTYPES = [(torch.float32, torch.float32), (torch.bfloat16, torch.float32), (torch.bfloat16, torch.bfloat16),
          (torch.float16, torch.float16), (torch.float16, torch.float32)]
PATHS = [b200norm.PATH_AUTO, b200norm.PATH_GENERIC]


def check_out(a, ref, what):
    if ref.dtype in (torch.bfloat16, torch.float16):
        n_bad, worst = ao.lowp_mismatch(a, ref)
        assert n_bad == 0, f"{what}: {n_bad} elements beyond 1 ulp and the absolute floor (worst {worst} ulp)"
    else:
        e = ao.fp32_err(a, ref)
        assert e <= 1.0, f"{what}: error {e:.3f} x tolerance"


def check_stat(a, ref, what):
    a, ref = a.cpu().double().reshape(-1), ref.double().reshape(-1)
    err = ((a - ref).abs() / (1e-5 * ref.abs() + 1e-6)).max()
    assert err <= 1.0, f"{what}: {float(err):.3f} x tolerance"


def check_wgrad(a, terms, what):
    """a: kernel result [N]; terms: fp64 [M, N] summands (see gpu_util.wgrad_gate for the bound)."""
    wgrad_gate(a, terms, what)


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("dt,wdt", DTYPES)
@pytest.mark.parametrize("M,N", SHAPES)
def test_layer_norm_fwd_bwd(M, N, dt, wdt, path):
    x = ao.randn((M, N), 100 + N, dt)
    g = ao.randn((N,), 101, wdt, 1.0, 0.02)
    b = ao.randn((N,), 102, wdt, 0.0, 0.02)
    dy = ao.randn((M, N), 103, dt)
    with forced_path(path):
        y_buf, y_chk = guarded_empty((M, N), dt)
        mean_buf, mean_chk = guarded_empty((M,), torch.float32)
        rstd_buf, rstd_chk = guarded_empty((M,), torch.float32)
        y, mean, rstd = capi.native_layer_norm(x.to(DEV), [N], g.to(DEV), b.to(DEV), 1e-5, out=(y_buf, mean_buf, rstd_buf))
        used = capi.last_path()
        dx_buf, dx_chk = guarded_empty((M, N), dt)
        dg_buf, dg_chk = guarded_empty((N,), wdt)
        db_buf, db_chk = guarded_empty((N,), wdt)
        dx, dg, db = capi.native_layer_norm_backward(dy.to(DEV), x.to(DEV), [N], mean, rstd, g.to(DEV), b.to(DEV),
                                                     out=(dx_buf, dg_buf, db_buf))
    torch.cuda.synchronize()
    for chk in (y_chk, mean_chk, rstd_chk, dx_chk, dg_chk, db_chk):
        chk()
    if path == b200norm.PATH_AUTO and ring_eligible(N, dt, 16):
        assert used == "ring"
    if path == b200norm.PATH_GENERIC:
        assert used == "generic"
    ry, rmean, rrstd = ao.layer_norm_fwd(x, [N], g, b, 1e-5)
    check_out(y, ry, "y")
    check_stat(mean, rmean, "mean")
    check_stat(rstd, rrstd, "rstd")
    # the backward is a function of its inputs: the oracle gets the same mean/rstd the kernel got
    kmean, krstd = mean.cpu(), rstd.cpu()
    if N == 1:
        # a one-element row has dx == 0 exactly, as the difference of two terms of size rstd*|dy*gamma|
        # (rstd = 1/sqrt(eps) ~ 316): fp32 evaluations (CPU ATen's as well) leave a few ulps of THOSE
        # terms, so the gate is a few fp32 ulps of rstd*|dy*gamma| instead of the unit-scale floor
        scale = (krstd.double().reshape(-1, 1) * (dy.double() * g.double())).abs()
        assert bool((dx.cpu().double().abs() <= 4e-7 * scale + 1e-30).all()), "dx of a one-element row"
    else:
        rdx, _, _ = ao.layer_norm_bwd(dy, x, [N], kmean, krstd, g, b)
        check_out(dx, rdx, "dx")
    xh = (x.double() - kmean.double().reshape(-1, 1)) * krstd.double().reshape(-1, 1)
    check_wgrad(dg, dy.double() * xh, "dgamma")
    check_wgrad(db, dy.double(), "dbeta")
    assert capi.device_status() == 0


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("dt,wdt", DTYPES)
@pytest.mark.parametrize("M,N", SHAPES)
def test_rms_norm_fwd_bwd(M, N, dt, wdt, path):
    x = ao.randn((M, N), 200 + N, dt)
    w = ao.randn((N,), 201, wdt, 1.0, 0.02)
    dy = ao.randn((M, N), 202, dt)
    with forced_path(path):
        y, rstd = capi._fused_rms_norm(x.to(DEV), [N], w.to(DEV), 1e-6)
        dx_buf, dx_chk = guarded_empty((M, N), dt)
        dw_buf, dw_chk = guarded_empty((N,), wdt)
        dx, dw = capi._fused_rms_norm_backward(dy.to(DEV), x.to(DEV), [N], rstd, w.to(DEV), out=(dx_buf, dw_buf))
    torch.cuda.synchronize()
    dx_chk(); dw_chk()
    ry, rrstd = ao.rms_norm_fwd(x, [N], w, 1e-6)
    check_out(y, ry, "y")
    check_stat(rstd, rrstd, "rstd")
    rdx, rdw = ao.rms_norm_bwd(dy, x, [N], w, 1e-6)
    check_out(dx, rdx, "dx")
    check_wgrad(dw, dy.double() * x.double() * rstd.cpu().double().reshape(-1, 1), "dweight")
    # the restated closed form of the reference's rms backward agrees too (no CPU ATen kernel exists)
    cdx, cdw, _ = restate.norm_bwd(dy, x, None, rrstd, w, rms=True)
    if dt == torch.float32:
        assert ao.fp32_err(dx, cdx) <= 4.0
    else:
        assert ao.lowp_mismatch(dx, cdx.to(dt), floor_scale=4e-6)[0] == 0


@pytest.mark.parametrize("has_w,has_b", [(False, False), (True, False), (False, True)])
@pytest.mark.parametrize("N", [5, 128, 2048])
def test_layer_norm_optional_affine(N, has_w, has_b):
    M = 21
    x = ao.randn((M, N), 300, torch.float32)
    g = ao.randn((N,), 301, torch.float32, 1.0, 0.1) if has_w else None
    b = ao.randn((N,), 302, torch.float32) if has_b else None
    dy = ao.randn((M, N), 303, torch.float32)
    dev = lambda t: None if t is None else t.to(DEV)
    y, mean, rstd = capi.native_layer_norm(dev(x), [N], dev(g), dev(b), 1e-5)
    dx, dg, db = capi.native_layer_norm_backward(dev(dy), dev(x), [N], mean, rstd, dev(g), dev(b))
    ry, rmean, rrstd = ao.layer_norm_fwd(x, [N], g, b, 1e-5)
    rdx, rdg, rdb = ao.layer_norm_bwd(dy, x, [N], rmean, rrstd, g, b, mask=(True, g is not None, b is not None))
    check_out(y, ry, "y"); check_out(dx, rdx, "dx")
    assert (dg is None) == (g is None) and (db is None) == (b is None)
    xh = (x.double() - mean.cpu().double().reshape(-1, 1)) * rstd.cpu().double().reshape(-1, 1)
    if g is not None:
        check_wgrad(dg, dy.double() * xh, "dgamma")
    if b is not None:
        check_wgrad(db, dy.double(), "dbeta")


@pytest.mark.parametrize("mask", [(True, False, False), (False, True, True), (True, True, False), (False, False, True)])
def test_layer_norm_backward_masks(mask):
    M, N = 40, 1024
    x, dy = ao.randn((M, N), 310, torch.bfloat16), ao.randn((M, N), 311, torch.bfloat16)
    g, b = ao.randn((N,), 312, torch.float32, 1.0, 0.02), ao.randn((N,), 313, torch.float32)
    y, mean, rstd = capi.native_layer_norm(x.to(DEV), [N], g.to(DEV), b.to(DEV), 1e-5)
    dx, dg, db = capi.native_layer_norm_backward(dy.to(DEV), x.to(DEV), [N], mean, rstd, g.to(DEV), b.to(DEV), mask)
    rdx, rdg, rdb = ao.layer_norm_bwd(dy, x, [N], mean.cpu(), rstd.cpu(), g, b)
    assert (dx is not None) == mask[0] and (dg is not None) == mask[1] and (db is not None) == mask[2]
    if dx is not None:
        assert ao.lowp_mismatch(dx, rdx)[0] == 0
    xh = (x.double() - mean.cpu().double().reshape(-1, 1)) * rstd.cpu().double().reshape(-1, 1)
    if dg is not None:
        check_wgrad(dg, dy.double() * xh, "dgamma")
    if db is not None:
        check_wgrad(db, dy.double(), "dbeta")


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("N", [128, 1000])
def test_unaligned_pointers_take_the_generic_kernels(N, dt):
    M = 17
    x, dy = ao.randn((M, N), 320, dt), ao.randn((M, N), 321, dt)
    g, b = ao.randn((N,), 322, dt, 1.0, 0.02), ao.randn((N,), 323, dt)
    xd, dyd = misaligned(x.to(DEV)), misaligned(dy.to(DEV))
    assert xd.data_ptr() % 16 != 0
    y, mean, rstd = capi.native_layer_norm(xd, [N], g.to(DEV), b.to(DEV), 1e-5)
    assert capi.last_path() == "generic"
    dx, dg, db = capi.native_layer_norm_backward(dyd, xd, [N], mean, rstd, g.to(DEV), b.to(DEV))
    ry, rmean, rrstd = ao.layer_norm_fwd(x, [N], g, b, 1e-5)
    rdx, _, _ = ao.layer_norm_bwd(dy, x, [N], rmean, rrstd, g, b)
    check_out(y, ry, "y"); check_out(dx, rdx, "dx")


def test_float64_goes_through_the_generic_kernels():
    M, N = 9, 77
    x, dy = ao.randn((M, N), 330).double(), ao.randn((M, N), 331).double()
    g, b = ao.randn((N,), 332).double(), ao.randn((N,), 333).double()
    y, mean, rstd = capi.native_layer_norm(x.to(DEV), [N], g.to(DEV), b.to(DEV), 1e-5)
    assert mean.dtype == torch.float64
    dx, dg, db = capi.native_layer_norm_backward(dy.to(DEV), x.to(DEV), [N], mean, rstd, g.to(DEV), b.to(DEV))
    ry, rmean, rrstd = ao.layer_norm_fwd(x, [N], g, b, 1e-5)
    rdx, rdg, rdb = ao.layer_norm_bwd(dy, x, [N], rmean, rrstd, g, b)
    for a, r in ((y, ry), (dx, rdx), (dg, rdg), (db, rdb)):
        assert torch.allclose(a.cpu(), r, rtol=1e-10, atol=1e-10)


def test_large_offset_row_is_finite_and_matches():
    # the reference's regression case: 1e15 + {0..4} must not turn into NaN
    x = torch.tensor([[1e15 + i for i in range(5)]] * 3, dtype=torch.float32)
    y, mean, rstd = capi.native_layer_norm(x.to(DEV), [5], None, None, 1e-5)
    ry, _, _ = ao.layer_norm_fwd(x, [5], None, None, 1e-5)
    assert torch.isfinite(y).all()
    assert torch.allclose(y.cpu(), ry, atol=1e-5)
    # the vector / ring path too: a constant huge row must come out as exactly zero
    x = torch.full((4, 64), 1e15)
    y, mean, _ = capi.native_layer_norm(x.to(DEV), [64], None, None, 1e-5)
    assert capi.last_path() == "ring"
    assert float(y.abs().max()) == 0.0 and torch.equal(mean.cpu().reshape(-1), x[:, 0])


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("N", [256, 4096, 8192])
def test_rows_whose_first_element_is_far_from_the_mean(N, dt):
    # The ring forward shifts a row by its first element and takes both moments in one reduction unless that
    # element lies far from the row mean, in which case it recomputes the variance about the mean.  Rows of
    # every kind, interleaved so that both kinds meet in one tile: ordinary, first element an outlier by
    # 3..1000 standard deviations, large common offset with small spread, constant.
    M = 64
    x = ao.randn((M, N), 350 + N, torch.float32)
    for r in range(M):
        kind = r % 8
        if kind in (1, 2, 3):
            x[r, 0] += (3.0, 30.0, 1000.0)[kind - 1]
        elif kind == 4:
            x[r] = 300.0 + 0.25 * x[r]
        elif kind == 5:
            x[r] = -7.5
        elif kind == 6:
            x[r] = 1e4 + x[r]
            x[r, 0] = 0.0
    x = x.to(dt)
    g = ao.randn((N,), 351, torch.float32, 1.0, 0.02)
    b = ao.randn((N,), 352, torch.float32, 0.0, 0.02)
    y, mean, rstd = capi.native_layer_norm(x.to(DEV), [N], g.to(DEV), b.to(DEV), 1e-5)
    assert capi.last_path() == "ring"
    ry, rmean, rrstd = ao.layer_norm_fwd(x, [N], g, b, 1e-5)
    # statistics against fp64
    xd = x.double()
    mu = xd.mean(1)
    rs = 1.0 / torch.sqrt(xd.var(1, unbiased=False) + 1e-5)
    check_stat(mean, mu, "mean")
    check_stat(rstd, rs, "rstd")
    if dt == torch.float32:
        # CPU ATen's own fp32 statistics carry a few 1e-6 of error on the offset rows; judge y by fp64
        ref = ((xd - mu[:, None]) * rs[:, None] * g.double() + b.double())
        err = ((y.cpu().double() - ref).abs() / (1e-5 * ref.abs() + 1e-6 * max(1.0, float(ref.pow(2).mean().sqrt())))).max()
        assert float(err) <= 1.0, f"y: {float(err):.3f} x tolerance"
    else:
        check_out(y, ry, "y")
    assert capi.device_status() == 0


def test_rms_default_eps_is_accumulate_type_epsilon():
    x = ao.randn((8, 256), 340, torch.bfloat16)
    w = ao.randn((256,), 341, torch.bfloat16, 1.0, 0.02)
    y, rstd = capi._fused_rms_norm(x.to(DEV), [256], w.to(DEV), None)
    ry, rrstd = ao.rms_norm_fwd(x, [256], w, torch.finfo(torch.float32).eps)
    check_out(y, ry, "y"); check_stat(rstd, rrstd, "rstd")


def test_rms_dweight_equals_row_count_terms():
    # reference regression: with dy == 1 and x == 1, dweight_j = M * rstd (rstd ~ 1)
    M, N = 3000, 512
    x = torch.ones(M, N, dtype=torch.bfloat16)
    w = torch.ones(N, dtype=torch.float32)
    y, rstd = capi._fused_rms_norm(x.to(DEV), [N], w.to(DEV), 1e-6)
    dx, dw = capi._fused_rms_norm_backward(x.to(DEV), x.to(DEV), [N], rstd, w.to(DEV))
    assert torch.allclose(dw.cpu(), torch.full((N,), float(M)), rtol=1e-5)


def test_multi_dim_normalized_shape_and_stat_shapes():
    x = ao.randn((2, 3, 4, 8), 350, torch.float32)
    g, b = ao.randn((4, 8), 351), ao.randn((4, 8), 352)
    y, mean, rstd = capi.native_layer_norm(x.to(DEV), [4, 8], g.to(DEV), b.to(DEV), 1e-5)
    ry, rmean, rrstd = ao.layer_norm_fwd(x, [4, 8], g, b, 1e-5)
    assert list(mean.shape) == [2, 3, 1, 1] == list(rmean.shape)
    check_out(y, ry, "y")


def test_empty_batch_and_bad_shapes():
    x = torch.empty(0, 16, device=DEV)
    g = torch.ones(16, device=DEV)
    y, mean, rstd = capi.native_layer_norm(x, [16], g, g, 1e-5)
    assert y.shape == (0, 16) and mean.shape == (0, 1)
    dx, dg, db = capi.native_layer_norm_backward(x, x, [16], mean, rstd, g, g)
    assert float(dg.abs().sum()) == 0 and float(db.abs().sum()) == 0
    with pytest.raises(RuntimeError):
        capi.native_layer_norm(torch.ones(4, 8, device=DEV), [16], None, None, 1e-5)
    with pytest.raises(RuntimeError):
        capi.native_layer_norm(torch.ones(4, 16, device=DEV), [16], torch.ones(8, device=DEV), None, 1e-5)
    with pytest.raises(ValueError):
        capi.native_layer_norm(torch.ones(4, 16), [16], None, None, 1e-5)  # CPU tensor: no CPU path


def test_weight_gradients_are_bit_reproducible():
    M, N = 5000, 4096
    x, dy = ao.randn((M, N), 360, torch.bfloat16).to(DEV), ao.randn((M, N), 361, torch.bfloat16).to(DEV)
    g, b = ao.randn((N,), 362).to(DEV), ao.randn((N,), 363).to(DEV)
    y, mean, rstd = capi.native_layer_norm(x, [N], g, b, 1e-5)
    runs = [capi.native_layer_norm_backward(dy, x, [N], mean, rstd, g, b) for _ in range(3)]
    for dx, dg, db in runs[1:]:
        assert torch.equal(dg, runs[0][1]) and torch.equal(db, runs[0][2]) and torch.equal(dx, runs[0][0])


def test_workspace_too_small_is_rejected():
    lib = b200norm.load_library()
    M, N = 64, 1024
    x = torch.zeros(M, N, device=DEV)
    st = torch.zeros(M, device=DEV)
    g = torch.ones(N, device=DEV)
    need = lib.b2n_norm_bwd_workspace_bytes(M, N, b200norm.F32, b200norm.F32, 1)
    assert need > 0
    ws = torch.empty(need // 2, dtype=torch.uint8, device=DEV)
    rc = lib.b2n_layer_norm_bwd(x.data_ptr(), x.data_ptr(), st.data_ptr(), st.data_ptr(), g.data_ptr(), x.data_ptr(),
                                g.data_ptr(), g.data_ptr(), ws.data_ptr(), need // 2, M, N, 0, 0, None)
    assert rc == b200norm.ERR_WORKSPACE
    rc = lib.b2n_layer_norm_fwd(x.data_ptr(), None, None, x.data_ptr(), st.data_ptr(), st.data_ptr(), M, N, 1e-5,
                                b200norm.F32, b200norm.F16, None)
    assert rc == b200norm.OK  # weight dtype is irrelevant when there are no weights
    rc = lib.b2n_layer_norm_fwd(x.data_ptr(), g.data_ptr(), None, x.data_ptr(), st.data_ptr(), st.data_ptr(), M, N, 1e-5,
                                b200norm.F32, b200norm.F16, None)
    assert rc == b200norm.ERR_UNSUPPORTED_DTYPE
    torch.cuda.synchronize()


def test_sm_margin_changes_the_grid_not_the_results():
    # persistent kernels leave SMs free when asked to (for a collective running beside them): fewer CTAs, same rows
    M, N = 5000, 2048
    x = ao.randn((M, N), 360, torch.bfloat16).to(DEV)
    dy = ao.randn((M, N), 361, torch.bfloat16).to(DEV)
    g = ao.randn((N,), 362, torch.float32, 1.0, 0.02).to(DEV)
    b = ao.randn((N,), 363, torch.float32, 0.0, 0.02).to(DEV)

    def run():
        y, mean, rstd = capi.native_layer_norm(x, [N], g, b, 1e-5)
        dx, dg, db = capi.native_layer_norm_backward(dy, x, [N], mean, rstd, g, b)
        p = capi._softmax(x, -1, False)
        return y, mean, rstd, dx, dg, db, p

    base = run()
    try:
        for margin in (1, 8, 140):
            capi.set_tuning(b200norm.TUNE_SM_MARGIN, margin)
            got = run()
            assert capi.last_path() == "ring"
            for a, r in zip(got[:4] + got[6:], base[:4] + base[6:]):
                assert torch.equal(a, r)           # per-row results do not depend on which CTA took the row
            for a, r in zip(got[4:6], base[4:6]):  # the weight gradients are summed over a different set of partial rows
                assert torch.allclose(a, r, rtol=1e-4, atol=1e-3)
    finally:
        capi.set_tuning(b200norm.TUNE_SM_MARGIN, 0)
    assert capi.device_status() == 0


@pytest.mark.parametrize("rms", [False, True])
@pytest.mark.parametrize("M,N,dt,wdt", [(4096, 8192, torch.bfloat16, torch.float32), (300, 1000, torch.float32, torch.float32),
                                        (64, 33, torch.float32, torch.float32), (777, 4096, torch.float16, torch.float16)])
def test_backward_in_two_steps_equals_the_one_call_backward(M, N, dt, wdt, rms):
    # b2n_norm_bwd_partials + b2n_norm_wgrad_fold are the one-call entry point's own two kernels: same bits
    x, dy = ao.randn((M, N), 900, dt).to(DEV), ao.randn((M, N), 901, dt).to(DEV)
    g = ao.randn((N,), 902, wdt, 1.0, 0.02).to(DEV)
    if rms:
        _, rstd = capi._fused_rms_norm(x, [N], g, 1e-6)
        mean = None
        dx1, dg1 = capi._fused_rms_norm_backward(dy, x, [N], rstd, g)
        db1 = None
    else:
        _, mean, rstd = capi.native_layer_norm(x, [N], g, g, 1e-5)
        dx1, dg1, db1 = capi.native_layer_norm_backward(dy, x, [N], mean, rstd, g, g)
    dx2, ws, rows = capi.native_layer_norm_backward_partials(dy, x, [N], mean, rstd, g, rms=rms)
    assert rows > 0
    dg2 = torch.empty_like(g)
    db2 = None if rms else torch.empty_like(g)
    side = torch.cuda.Stream(DEV)  # the fold on a second stream, behind an event: the use the split exists for
    ev = torch.cuda.Event()
    ev.record()
    side.wait_event(ev)
    with torch.cuda.stream(side):
        capi.norm_wgrad_fold(ws, rows, dt, dg2, db2)
    torch.cuda.synchronize()
    assert torch.equal(dx1, dx2) and torch.equal(dg1, dg2) and (rms or torch.equal(db1, db2))
    assert capi.device_status() == 0


@pytest.mark.parametrize("ctas", [1, 8, 128, 256])
@pytest.mark.parametrize("rms", [False, True])
def test_fused_fold_allreduce_on_one_rank_is_the_fold(ctas, rms):
    # world = 1: the peer-memory kernel reduces to the fold (another fixed summation order: gated like any weight
    # gradient, not bit-compared); several calls in a row walk through its two buffer generations
    from b200norm.peer import WgradExchange
    M, N = 2500, 4096
    dt = torch.bfloat16
    ex = WgradExchange(N, DEV, ctas=ctas)
    for it in range(3):
        x, dy = ao.randn((M, N), 910 + it, dt), ao.randn((M, N), 920 + it, dt)
        g = ao.randn((N,), 930, torch.float32, 1.0, 0.02).to(DEV)
        if rms:
            _, rstd = capi._fused_rms_norm(x.to(DEV), [N], g, 1e-6)
            mean = None
            mu = torch.zeros(M, 1, dtype=torch.float64)
        else:
            _, mean, rstd = capi.native_layer_norm(x.to(DEV), [N], g, g, 1e-5)
            mu = mean.cpu().double().reshape(-1, 1)
        _, ws, rows = capi.native_layer_norm_backward_partials(dy.to(DEV), x.to(DEV), [N], mean, rstd, g, rms=rms)
        dg = torch.full((N,), float("nan"), device=DEV)
        db = None if rms else torch.full((N,), float("nan"), device=DEV)
        ex.fold_allreduce(ws, rows, dg, db)
        torch.cuda.synchronize()
        xh = (x.double() - mu) * rstd.cpu().double().reshape(-1, 1)
        check_wgrad(dg, dy.double() * xh, "dgamma")
        if not rms:
            check_wgrad(db, dy.double(), "dbeta")
    ex.close()
    assert capi.device_status() == 0


LONG_SHAPES = [(1, 16384), (5, 12288), (37, 16384), (300, 16384), (700, 12288), (9, 32768), (160, 32768), (6, 65536),
               (40, 65536), (11, 12296), (7, 40000)]


@pytest.mark.parametrize("rms", [False, True])
@pytest.mark.parametrize("dt,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.float32), (torch.float16, torch.float16)])
@pytest.mark.parametrize("M,N", LONG_SHAPES)
def test_long_rows_take_the_two_walk_ring_and_the_slab_kernels(M, N, dt, wdt, rms):
    # rows beyond one CTA's threads (the reference's few-long-rows regime, sycl/Norm.h:620-696): column slabs over a
    # thread-block cluster, statistics exchanged through distributed shared memory, weight gradients still fused;
    # 12296 and 40000 leave a ragged last slab, 300 x 16384 and 700 x 12288 give every cluster several tiles
    x = ao.randn((M, N), 940 + N % 89, dt)
    x[0] += 3.0  # a row whose slabs' first elements lie far from the slab means: the exact second pass
    dy = ao.randn((M, N), 941, dt)
    g = ao.randn((N,), 942, wdt, 1.0, 0.02)
    b = ao.randn((N,), 943, wdt, 0.0, 0.02)
    y_buf, y_chk = guarded_empty((M, N), dt)
    dx_buf, dx_chk = guarded_empty((M, N), dt)
    dg_buf, dg_chk = guarded_empty((N,), wdt)
    # forward: rows up to 16384 stay inside one CTA (weights in registers, the row walked twice in shared memory)
    fwd_path = "ring2w" if N <= 16384 else "slab"
    if rms:
        y, rstd = capi._fused_rms_norm(x.to(DEV), [N], g.to(DEV), 1e-6, out=(y_buf, torch.empty(M, device=DEV)))
        assert capi.last_path() == fwd_path
        dx, dw = capi._fused_rms_norm_backward(dy.to(DEV), x.to(DEV), [N], rstd, g.to(DEV), out=(dx_buf, dg_buf))
        # RMS backward: 16-bit rows up to 16384 stay inside one CTA too (gamma and dgamma in registers); fp32 rows
        # of that length leave fewer than three stages in shared memory and take the slabs
        assert capi.last_path() == ("ring2w" if N <= 16384 and dt != torch.float32 else "slab")
        torch.cuda.synchronize()
        y_chk(); dx_chk(); dg_chk()
        ry, rrstd = ao.rms_norm_fwd(x, [N], g, 1e-6)
        check_out(y, ry, "y"); check_stat(rstd, rrstd, "rstd")
        rdx, _ = ao.rms_norm_bwd(dy, x, [N], g, 1e-6)
        check_out(dx, rdx, "dx")
        check_wgrad(dw, dy.double() * x.double() * rstd.cpu().double().reshape(-1, 1), "dweight")
    else:
        db_buf, db_chk = guarded_empty((N,), wdt)
        y, mean, rstd = capi.native_layer_norm(x.to(DEV), [N], g.to(DEV), b.to(DEV), 1e-5,
                                               out=(y_buf, torch.empty(M, device=DEV), torch.empty(M, device=DEV)))
        assert capi.last_path() == fwd_path
        dx, dg, db = capi.native_layer_norm_backward(dy.to(DEV), x.to(DEV), [N], mean, rstd, g.to(DEV), b.to(DEV),
                                                     out=(dx_buf, dg_buf, db_buf))
        assert capi.last_path() == "slab"
        torch.cuda.synchronize()
        y_chk(); dx_chk(); dg_chk(); db_chk()
        ry, rmean, rrstd = ao.layer_norm_fwd(x, [N], g, b, 1e-5)
        check_out(y, ry, "y"); check_stat(mean, rmean, "mean"); check_stat(rstd, rrstd, "rstd")
        kmean, krstd = mean.cpu(), rstd.cpu()
        rdx, _, _ = ao.layer_norm_bwd(dy, x, [N], kmean, krstd, g, b)
        check_out(dx, rdx, "dx")
        xh = (x.double() - kmean.double().reshape(-1, 1)) * krstd.double().reshape(-1, 1)
        check_wgrad(dg, dy.double() * xh, "dgamma")
        check_wgrad(db, dy.double(), "dbeta")
    assert capi.device_status() == 0


@pytest.mark.parametrize("cluster", [2, 4, 8])
@pytest.mark.parametrize("M,N,dt", [(33, 2048, torch.bfloat16), (130, 1000, torch.float32), (64, 8192, torch.float16)])
def test_pinned_slab_kernels_on_rows_the_ring_would_take(M, N, dt, cluster):
    # every cluster size on shapes small enough to compare whole, bit for bit, with the ring kernels' results for
    # the per-row outputs' gates
    x, dy = ao.randn((M, N), 950, dt), ao.randn((M, N), 951, dt)
    g, b = ao.randn((N,), 952, torch.float32, 1.0, 0.02), ao.randn((N,), 953, torch.float32, 0.0, 0.02)
    if dt == torch.float16:
        g, b = g.half(), b.half()
    capi.set_tuning(b200norm.TUNE_CLUSTER_SIZE, cluster)
    try:
        with forced_path(b200norm.PATH_CLUSTER):
            y, mean, rstd = capi.native_layer_norm(x.to(DEV), [N], g.to(DEV), b.to(DEV), 1e-5)
            assert capi.last_path() == "slab"
            dx, dg, db = capi.native_layer_norm_backward(dy.to(DEV), x.to(DEV), [N], mean, rstd, g.to(DEV), b.to(DEV))
            assert capi.last_path() == "slab"
            dxo, _, _ = capi.native_layer_norm_backward(dy.to(DEV), x.to(DEV), [N], mean, rstd, g.to(DEV), b.to(DEV),
                                                        (True, False, False))
    finally:
        capi.set_tuning(b200norm.TUNE_CLUSTER_SIZE, 0)
    ry, rmean, rrstd = ao.layer_norm_fwd(x, [N], g, b, 1e-5)
    check_out(y, ry, "y"); check_stat(mean, rmean, "mean"); check_stat(rstd, rrstd, "rstd")
    rdx, _, _ = ao.layer_norm_bwd(dy, x, [N], mean.cpu(), rstd.cpu(), g, b)
    check_out(dx, rdx, "dx")
    assert torch.equal(dx, dxo)  # with and without the weight gradients: the same dx
    xh = (x.double() - mean.cpu().double().reshape(-1, 1)) * rstd.cpu().double().reshape(-1, 1)
    check_wgrad(dg, dy.double() * xh, "dgamma")
    check_wgrad(db, dy.double(), "dbeta")
    assert capi.device_status() == 0
