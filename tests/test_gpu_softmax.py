"""softmax / log-softmax parity: CUDA kernels through the C ABI vs the CPU oracle (tolerances as in
test_gpu_norm.py: fp32 1e-5 relative with an absolute floor, 16-bit within 1 ulp of the
fp32-accumulated reference)."""
import math

import ctypes

import pytest
import torch

import b200norm
from b200norm import capi
from oracle import aten_oracle as ao

from gpu_util import DEV, forced_path, guarded_empty, misaligned

pytestmark = pytest.mark.gpu

ROW_SHAPES = [(1, 1), (3, 5), (7, 128), (33, 130), (129, 1000), (64, 2048), (40, 4096), (9, 8192), (4, 16384),
              (3, 40000), (2, 128256),
              # long rows that are NOT a whole number of 16-byte vectors (GPT-2's vocabulary among them): the
              # two-pass kernels cannot take them, the generic ones must
              (3, 40001), (2, 50257)]
DTYPES = [torch.float32, torch.bfloat16, torch.float16]
PATHS = [b200norm.PATH_AUTO, b200norm.PATH_GENERIC]


def check_out(a, ref, what, tol=1.0):
    if ref.dtype in (torch.bfloat16, torch.float16):
        n_bad, worst = ao.lowp_mismatch(a, ref)
        assert n_bad == 0, f"{what}: {n_bad} elements beyond 1 ulp and the absolute floor (worst {worst} ulp)"
    else:
        e = ao.fp32_err(a, ref)
        assert e <= tol, f"{what}: error {e:.3f} x tolerance"


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("is_log", [False, True])
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("M,N", ROW_SHAPES)
def test_last_dim_fwd_bwd(M, N, dt, is_log, path):
    x = ao.randn((M, N), 400 + N, dt, 0.0, 2.0)
    dy = ao.randn((M, N), 401, dt)
    fwd = capi._log_softmax if is_log else capi._softmax
    bwd = capi._log_softmax_backward_data if is_log else capi._softmax_backward_data
    with forced_path(path):
        y_buf, y_chk = guarded_empty((M, N), dt)
        y = fwd(x.to(DEV), -1, False, out=y_buf)
        used = capi.last_path()
        dx_buf, dx_chk = guarded_empty((M, N), dt)
        dx = bwd(dy.to(DEV), y, -1, dt, out=dx_buf)
    torch.cuda.synchronize()
    y_chk(); dx_chk()
    if path == b200norm.PATH_GENERIC:
        assert used == "generic"
    ry = ao.softmax_fwd(x, -1, is_log)
    check_out(y, ry, "y")
    # backward on the kernel's own forward output, as autograd would
    rdx = ao.softmax_bwd(dy, y.cpu(), -1, is_log, dt)
    check_out(dx, rdx, "dx", tol=2.0)
    assert capi.device_status() == 0


@pytest.mark.parametrize("is_log", [False, True])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape,dim", [((6, 5, 3), 0), ((2, 7, 4), 1), ((4, 33, 65), 1), ((128, 16), 0), ((3, 4, 5, 6), 2),
                                       ((5, 8, 64), 1), ((3, 16, 34), 1), ((2, 64, 130), 1), ((2, 65, 128), 1), ((9, 40, 7), 1),
                                       ((4, 19, 32, 32), 1),
                                       ((2, 3, 4), -1), ((5,), 0)])
def test_any_dim(shape, dim, dt, is_log):
    x = ao.randn(shape, 410, dt, 0.0, 2.0)
    dy = ao.randn(shape, 411, dt)
    fwd = capi._log_softmax if is_log else capi._softmax
    bwd = capi._log_softmax_backward_data if is_log else capi._softmax_backward_data
    y = fwd(x.to(DEV), dim, False)
    dx = bwd(dy.to(DEV), y, dim, dt)
    check_out(y, ao.softmax_fwd(x, dim, is_log), "y")
    check_out(dx, ao.softmax_bwd(dy, y.cpu(), dim, is_log, dt), "dx", tol=2.0)


def test_zero_dim_tensor():
    x = torch.tensor(3.0, device=DEV)
    assert float(capi._softmax(x, 0, False)) == 1.0
    assert float(capi._log_softmax(x, -1, False)) == 0.0
    with pytest.raises(IndexError):
        capi._softmax(x, 1, False)


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("N", [64, 2048, 5000])
def test_masked_and_degenerate_rows(N, dt, path):
    # row 0: causal-style -inf tail; row 1: all -inf (NaN on CPU ATen and in the reference); row 2: one +inf;
    # row 3: one NaN; row 4: ordinary
    x = ao.randn((5, N), 420, torch.float32)
    x[0, N // 3:] = float("-inf")
    x[1, :] = float("-inf")
    x[2, 7] = float("inf")
    x[3, 9] = float("nan")
    x = x.to(dt)
    with forced_path(path):
        for is_log in (False, True):
            fwd = capi._log_softmax if is_log else capi._softmax
            y = fwd(x.to(DEV), -1, False).cpu()
            ry = ao.softmax_fwd(x, -1, is_log)
            assert torch.equal(torch.isnan(y), torch.isnan(ry)), "NaN pattern"
            assert torch.isnan(y[1]).all() and torch.isnan(y[2]).all() and torch.isnan(y[3]).all()
            if is_log:
                assert (y[0, N // 3:] == float("-inf")).all()
            else:
                assert (y[0, N // 3:] == 0).all()
            check_out(y[0:1], ry[0:1], "masked row")
            check_out(y[4:5], ry[4:5], "plain row")


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape,dim", [((9, 64), -1), ((3, 1000), 1), ((4, 6, 10), 1), ((2, 2048), -1)])
def test_half_to_float(shape, dim, dt):
    # the reference's regression (fp16 -> fp32 output for every dim); CPU has no such kernel: oracle = op(x.float())
    x = ao.randn(shape, 430, dt, 0.0, 2.0)
    dy = ao.randn(shape, 431, torch.float32)
    for is_log in (False, True):
        fwd = capi._log_softmax if is_log else capi._softmax
        bwd = capi._log_softmax_backward_data if is_log else capi._softmax_backward_data
        y = fwd(x.to(DEV), dim, True)
        assert y.dtype == torch.float32
        ry = ao.softmax_fwd(x, dim, is_log, out_dtype=torch.float32)
        assert ao.fp32_err(y, ry) <= 1.0
        dx = bwd(dy.to(DEV), y, dim, dt)
        assert dx.dtype == dt
        rdx = ao.softmax_bwd(dy, y.cpu(), dim, is_log, dt)
        assert ao.lowp_mismatch(dx, rdx)[0] == 0
    with pytest.raises(RuntimeError):
        capi._softmax(torch.ones(4, 4, device=DEV), -1, True)  # only 16-bit inputs convert


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("N", [33, 128, 1001])
@pytest.mark.parametrize("shift", [1, 3])
def test_alignment_shifts(N, dt, shift):
    # the reference's test_softmax_results matrix: odd sizes and 1-element shifts that break alignment
    x = ao.randn((11, N), 440, dt, 0.0, 2.0)
    dy = ao.randn((11, N), 441, dt)
    xd, dyd = misaligned(x.to(DEV), shift), misaligned(dy.to(DEV), shift)
    for is_log in (False, True):
        fwd = capi._log_softmax if is_log else capi._softmax
        bwd = capi._log_softmax_backward_data if is_log else capi._softmax_backward_data
        y = fwd(xd, -1, False)
        assert capi.last_path() == "generic"
        check_out(y, ao.softmax_fwd(x, -1, is_log), "y")
        dx = bwd(dyd, y, -1, dt)
        check_out(dx, ao.softmax_bwd(dy, y.cpu(), -1, is_log, dt), "dx", tol=2.0)


def test_known_answers():
    # log_softmax is shift invariant; exp(log_softmax) sums to one (reference test_log_softmax_big / _double)
    x = ao.randn((8, 4096), 450).to(DEV)
    a = capi._log_softmax(x, -1, False)
    b = capi._log_softmax(x + 1000.0, -1, False)
    assert torch.allclose(a, b, atol=2e-4)
    assert torch.allclose(a.exp().sum(-1), torch.ones(8, device=DEV), atol=1e-5)
    # _softmax_backward_data(x, x) with x == 1/numel gives out[0] == 1/numel (reference :17914-17920)
    n = 1 << 16
    v = torch.full((1, n), 1.0 / n, device=DEV)
    out = capi._softmax_backward_data(v, v, -1, torch.float32)
    assert math.isclose(float(out[0, 0]), (1.0 / n) * (1.0 / n - 1.0 / n), abs_tol=1e-9)


def test_float64():
    x = ao.randn((5, 333), 460).double()
    dy = ao.randn((5, 333), 461).double()
    for is_log in (False, True):
        fwd = capi._log_softmax if is_log else capi._softmax
        bwd = capi._log_softmax_backward_data if is_log else capi._softmax_backward_data
        y = fwd(x.to(DEV), -1, False)
        assert torch.allclose(y.cpu(), ao.softmax_fwd(x, -1, is_log), rtol=1e-12, atol=1e-12)
        dx = bwd(dy.to(DEV), y, -1, torch.float64)
        assert torch.allclose(dx.cpu(), ao.softmax_bwd(dy, y.cpu(), -1, is_log, torch.float64), rtol=1e-12, atol=1e-12)


def test_ring_is_used_for_aligned_rows_and_refuses_others_when_forced():
    x = ao.randn((64, 2048), 470, torch.bfloat16).to(DEV)
    capi._softmax(x, -1, False)
    assert capi.last_path() == "ring"
    with forced_path(b200norm.PATH_RING):
        with pytest.raises(b200norm.B200NormError):
            capi._softmax(ao.randn((4, 33), 471).to(DEV), -1, False)  # 33 floats: not a multiple of 16 bytes


@pytest.mark.parametrize("dt", DTYPES)
def test_pinned_twopass_refuses_ragged_rows(dt):
    # a row that is not a multiple of 16 bytes: the vector kernels would drop its tail and misplace every later row
    x = ao.randn((3, 40001), 470, dt).to(DEV)
    with forced_path(b200norm.PATH_TWOPASS):
        with pytest.raises(b200norm.B200NormError):
            capi._softmax(x, -1, False)
        with pytest.raises(b200norm.B200NormError):
            capi._log_softmax_backward_data(x, x, -1, dt)
    y = capi._softmax(x, -1, False)
    assert capi.last_path() == "generic"
    check_out(y, ao.softmax_fwd(x.cpu(), -1, False), "y")


@pytest.mark.parametrize("path,name", [(b200norm.PATH_CLUSTER, "cluster"), (b200norm.PATH_TWOPASS, "twopass")])
@pytest.mark.parametrize("is_log", [False, True])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("M,N", [(5, 16384), (3, 40000), (7, 65544), (2, 128256), (300, 20008)])
def test_long_row_kernels(M, N, dt, is_log, path, name):
    # the two kernel families for rows beyond the ring: slices resident in the shared memory of a cluster, and
    # two passes through the ring (ragged last slice / chunk included: 65544 and 20008 elements do not divide
    # evenly); degenerate rows keep the CPU semantics
    x = ao.randn((M, N), 480 + N % 97, torch.float32, 0.0, 2.0)
    x[0, N // 2:] = float("-inf")
    if M > 2:
        x[1, :] = float("-inf")
        x[2, 11] = float("nan")
    x = x.to(dt)
    dy = ao.randn((M, N), 481, dt)
    fwd = capi._log_softmax if is_log else capi._softmax
    bwd = capi._log_softmax_backward_data if is_log else capi._softmax_backward_data
    with forced_path(path):
        y_buf, y_chk = guarded_empty((M, N), dt)
        y = fwd(x.to(DEV), -1, False, out=y_buf)
        assert capi.last_path() == name
        dx_buf, dx_chk = guarded_empty((M, N), dt)
        dx = bwd(dy.to(DEV), y, -1, dt, out=dx_buf)
        assert capi.last_path() == name
    torch.cuda.synchronize()
    y_chk(); dx_chk()
    ry = ao.softmax_fwd(x, -1, is_log)
    assert torch.equal(torch.isnan(y.cpu()), torch.isnan(ry))
    check_out(y, ry, "y")
    if dt == torch.float32:
        # judged against the fp64 evaluation: the fp32 CPU kernel's own sum over a row this long is the
        # larger error (see oracle.aten_oracle.softmax_bwd_fp64)
        check_out(dx, ao.softmax_bwd_fp64(dy, y.cpu(), -1, is_log, dt), "dx", tol=2.0)
    else:
        check_out(dx, ao.softmax_bwd(dy, y.cpu(), -1, is_log, dt), "dx", tol=2.0)
    assert capi.device_status() == 0


# ---- _safe_softmax: rows of all -inf give zeros (SoftMaxKernels.cpp:327-330 of the reference, test/regressions/
# test_safe_softmax.py) ----------------------------------------------------------------------------------------
def _safe_case(M, N, dt, seed=900):
    x = ao.randn((M, N), seed, torch.float32)
    x[x > 1.0] = float("-inf")          # scattered masked entries
    for r in range(0, M, 3):
        x[r] = float("-inf")            # fully masked rows
    if M > 4:
        x[4] = float("-inf")
        x[4, N // 2] = float("nan")     # masked but for a NaN: must stay NaN
        x[1, 0] = float("inf")          # +inf in an ordinary row: NaN as in the plain softmax
    return x.to(dt)


def _safe_ref(x, dim, out_dtype):
    ref = torch.ops.aten._safe_softmax(x.float(), dim)
    return ref.to(out_dtype)


@pytest.mark.parametrize("path,N", [(b200norm.PATH_AUTO, 64), (b200norm.PATH_AUTO, 2048), (b200norm.PATH_GENERIC, 2048),
                                    (b200norm.PATH_GENERIC, 333), (b200norm.PATH_AUTO, 20008),
                                    (b200norm.PATH_TWOPASS, 16384), (b200norm.PATH_AUTO, 40000)])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.float16])
def test_safe_softmax_last_dim(N, dt, path):
    M = 11
    x = _safe_case(M, N, dt)
    with forced_path(path):
        y = capi._safe_softmax(x.to(DEV), -1)
    ref = _safe_ref(x, -1, dt)
    got = y.cpu()
    assert torch.equal(torch.isnan(got), torch.isnan(ref)), "NaN pattern"
    for r in range(0, M, 3):
        assert float(got[r].abs().max()) == 0.0, "a fully masked row must be exactly zero"
    assert bool(torch.isnan(got[4]).all()) and bool(torch.isnan(got[1]).all())
    ok = ~torch.isnan(ref)
    if dt == torch.float32:
        assert torch.allclose(got[ok], ref[ok], rtol=1e-5, atol=1e-7)
    else:
        n_bad, worst = ao.lowp_mismatch(got[ok], ref[ok])
        assert n_bad == 0, (n_bad, worst)
    assert capi.device_status() == 0


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_safe_softmax_other_dims_and_half_to_float(dt):
    x = _safe_case(12, 40, dt).reshape(3, 4, 40).clone()
    x[:, 2, 7] = float("-inf")  # a fully masked line along dim 0
    y = capi._safe_softmax(x.to(DEV), 0).cpu()
    ref = _safe_ref(x, 0, dt)
    assert torch.equal(torch.isnan(y), torch.isnan(ref))
    assert float(y[:, 2, 7].abs().max()) == 0.0
    ok = ~torch.isnan(ref)
    assert torch.allclose(y[ok].float(), ref[ok].float(), rtol=1e-2 if dt != torch.float32 else 1e-5, atol=1e-6)
    if dt != torch.float32:
        y32 = capi._safe_softmax(x.to(DEV), -1, torch.float32).cpu()
        assert y32.dtype == torch.float32
        r32 = torch.ops.aten._safe_softmax(x.float(), -1)
        ok = ~torch.isnan(r32)
        assert torch.equal(torch.isnan(y32), torch.isnan(r32)) and torch.allclose(y32[ok], r32[ok], rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("N", [9, 64, 100])
@pytest.mark.parametrize("is_log", [False, True])
def test_degenerate_lines_along_an_inner_dim(N, is_log):
    # the same edge semantics as over the last dim, for lines held in registers (N <= 64) and streamed ones
    x = ao.randn((3, N, 10), 420)
    x[0, :, 2] = float("-inf")           # a line of -inf: NaN
    x[1, 3, 3] = float("inf")            # +inf in a line: NaN
    x[2, N - 1, 4] = float("nan")        # NaN in a line: NaN
    x[0, : N // 2, 5] = float("-inf")    # partly masked: zeros / -inf there, finite elsewhere
    fwd = capi._log_softmax if is_log else capi._softmax
    y = fwd(x.to(DEV), 1, False).cpu()
    ref = ao.softmax_fwd(x, 1, is_log)
    assert torch.equal(torch.isnan(y), torch.isnan(ref))
    ok = ~torch.isnan(ref) & ~torch.isinf(ref)
    assert torch.equal(torch.isinf(y), torch.isinf(ref))
    assert torch.allclose(y[ok], ref[ok], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("is_log", [False, True])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("shape", [(3, 150, 2048), (2, 300, 512), (1, 19, 200), (5, 64, 64), (2, 2, 4096), (1, 700, 136),
                                   (4, 33, 1000)])
def test_middle_dim_tiles(shape, dt, is_log, path):
    # softmax over dim 1 of [outer, N, inner]: under PATH_AUTO the tensor-map TMA tiles (boxes of N x W elements; 300
    # and 700 lines take two and three boxes of 256 rows; inner = 200, 136 and 1000 leave a ragged last tile that the
    # copy fills with zeros on the way in and clips on the way out), under PATH_GENERIC the plain-load tile kernels;
    # lines of -inf, a NaN and a +inf keep the CPU semantics
    x = ao.randn(shape, 490 + shape[1], torch.float32, 0.0, 2.0)
    x[0, :, 3] = float("-inf")
    x[0, 1, 5] = float("nan")
    x[-1, 0, 7] = float("inf")
    x[0, shape[1] // 2:, 9] = float("-inf")
    x = x.to(dt)
    dy = ao.randn(shape, 491, dt)
    fwd = capi._log_softmax if is_log else capi._softmax
    bwd = capi._log_softmax_backward_data if is_log else capi._softmax_backward_data
    with forced_path(path):
        y_buf, y_chk = guarded_empty(shape, dt)
        y = fwd(x.to(DEV), 1, False, out=y_buf)
        dx_buf, dx_chk = guarded_empty(shape, dt)
        dx = bwd(dy.to(DEV), y, 1, dt, out=dx_buf)
    torch.cuda.synchronize()
    y_chk(); dx_chk()
    ry = ao.softmax_fwd(x, 1, is_log)
    assert torch.equal(torch.isnan(y.cpu()), torch.isnan(ry))
    check_out(y, ry, "y")
    ok = ~torch.isnan(ry).any(dim=1, keepdim=True).expand_as(ry)  # lines that are NaN forward give NaN backward on both sides
    rdx = ao.softmax_bwd(dy, y.cpu(), 1, is_log, dt)
    assert torch.equal(torch.isnan(dx.cpu()), torch.isnan(rdx))
    check_out(torch.where(ok, dx.cpu(), torch.zeros_like(rdx)), torch.where(ok, rdx, torch.zeros_like(rdx)), "dx", tol=2.0)
    if not is_log:
        ys = capi._safe_softmax(x.to(DEV), 1)
        assert float(ys[0, :, 3].abs().max()) == 0.0  # the all -inf line: zeros instead of NaN
    assert capi.device_status() == 0


def _random_middle_dim_shapes(count, seed):
    g = torch.Generator().manual_seed(seed)
    shapes = []
    for _ in range(count):
        outer = int(torch.randint(1, 6, (1,), generator=g))
        n = int(torch.randint(2, 600, (1,), generator=g))
        inner = 8 * int(torch.randint(8, 400, (1,), generator=g))
        shapes.append((outer, n, inner))
    return shapes


@pytest.mark.parametrize("shape", _random_middle_dim_shapes(24, 77))
def test_middle_dim_random_shapes_take_the_tma_tiles(shape):
    # seeded random [outer, N, inner] with inner a whole number of 16-byte vectors: whatever tile geometry the planner
    # picks (boxes of 128..512 bytes, one to four per tile, one or several boxes of rows, ragged last tiles), forward and
    # backward agree with the oracle in bf16, and log-softmax in fp32; the path is reported
    outer, n, inner = shape
    x = ao.randn(shape, 7000 + n, torch.float32, 0.0, 3.0)
    dy = ao.randn(shape, 7001 + inner, torch.float32)
    for dt, is_log in ((torch.bfloat16, False), (torch.float32, True), (torch.float16, True)):
        xt, dyt = x.to(dt), dy.to(dt)
        fwd = capi._log_softmax if is_log else capi._softmax
        bwd = capi._log_softmax_backward_data if is_log else capi._softmax_backward_data
        y_buf, y_chk = guarded_empty(shape, dt)
        y = fwd(xt.to(DEV), 1, False, out=y_buf)
        used = capi.last_path()
        dx_buf, dx_chk = guarded_empty(shape, dt)
        dx = bwd(dyt.to(DEV), y, 1, dt, out=dx_buf)
        torch.cuda.synchronize()
        y_chk(); dx_chk()
        plan = (ctypes.c_int * 8)()
        assert b200norm.load_library().b2n_softmax_tile_plan(outer, n, inner, xt.element_size(), 0, 148, 232448, plan) == 0
        assert (used == "tma") == bool(plan[0]), (used, list(plan))
        check_out(y, ao.softmax_fwd(xt, 1, is_log), f"y {dt} {shape}")
        rdx = ao.softmax_bwd(dyt, y.cpu(), 1, is_log, dt)
        if dt == torch.float32:
            # dx = dy - exp(y) * sum(dy): where the two cancel, the error is that of the line's SUM, taken here in
            # another order than on the CPU.  Its a-priori bound for pairwise summation in fp32 is log2(n) * 2^-24 of
            # the L1 norm of the terms (5.5e-7 for n <= 600); the element-wise 1e-5 stays for everything else.
            l1 = dyt.abs().sum(1, keepdim=True)
            tol = 1e-5 * rdx.abs() + 5.5e-7 * l1 + 1e-6
            assert bool(((dx.cpu() - rdx).abs() <= tol).all()), f"dx {dt} {shape}"
        else:
            check_out(dx, rdx, f"dx {dt} {shape}")
    assert capi.device_status() == 0
