"""Fused cross-entropy backward (nll_loss_backward + _log_softmax_backward_data in one pass) through the C ABI
vs the same composition on CPU ATen.

Tolerances: fp32 |a-b| <= 1e-5*|b| + 1e-6*max(1, rms(b)); fp64 1e-12; 16-bit outputs within 1 ulp of the
composition evaluated on fp32 upcasts and rounded once (or the absolute floor of oracle.aten_oracle.lowp_mismatch).
"""
import pytest
import torch

import b200norm
from b200norm import capi
from oracle import aten_oracle as ao

from gpu_util import DEV, forced_path

pytestmark = pytest.mark.gpu

dev = lambda z: None if z is None else z.to(DEV)


def check(a, ref, what):
    if ref.dtype in (torch.bfloat16, torch.float16):
        n_bad, worst = ao.lowp_mismatch(a, ref)
        assert n_bad == 0, f"{what}: {n_bad} elements beyond 1 ulp and the absolute floor (worst {worst} ulp)"
    elif ref.dtype == torch.float64:
        assert torch.allclose(a.cpu(), ref, rtol=1e-12, atol=1e-14), what
    else:
        e = ao.fp32_err(a, ref)
        assert e <= 1.0, f"{what}: error {e:.3f} x tolerance"


def make_case(M, C, dt, weighted, reduction, seed=600):
    logp = torch.log_softmax(ao.randn((M, C), seed, torch.float32, 0.0, 2.0), -1).to(dt)
    t = ao.randint(C, (M,), seed + 1)
    if M > 4:
        t[3] = -100
        t[M - 1] = C - 1
        t[0] = 0
    w = (ao.randn((C,), seed + 2).abs() + 0.1).to(dt) if weighted else None
    _, tw = ao.nll_fwd(logp, t, w, reduction, -100)
    g = ao.randn((M,), seed + 3).to(dt) if reduction == 0 else torch.tensor(0.7, dtype=dt)
    return logp, t, w, tw, g


@pytest.mark.parametrize("reduction", [0, 1, 2])
@pytest.mark.parametrize("weighted", [False, True])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.float16, torch.float64])
@pytest.mark.parametrize("M,C", [(1, 1), (16, 10), (300, 1000), (37, 8192), (9, 40000), (5, 40001)])
def test_matches_the_two_step_composition(M, C, dt, weighted, reduction):
    logp, t, w, tw, g = make_case(M, C, dt, weighted, reduction)
    dx = capi.cross_entropy_backward(dev(g), dev(logp), dev(t), dev(w), reduction, -100, dev(tw))
    used = capi.last_path()
    ref = ao.cross_entropy_bwd(g, logp, t, w, reduction, -100, tw)
    check(dx, ref, "dx")
    if dt != torch.float64 and C * logp.element_size() >= 16384 and C % (16 // logp.element_size()) == 0:
        assert used == "ring"
    else:
        assert used == "generic"
    if M > 4:
        assert float(dx[3].abs().max()) == 0.0  # the ignored row
    assert capi.device_status() == 0


@pytest.mark.parametrize("path", [b200norm.PATH_RING, b200norm.PATH_GENERIC])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,C", [(400, 512), (1000, 2056), (149, 16384 + 8), (3, 128256)])
def test_both_kernel_families(M, C, dt, path):
    logp, t, w, tw, g = make_case(M, C, dt, True, 1, seed=610)
    with forced_path(path):
        dx = capi.cross_entropy_backward(dev(g), dev(logp), dev(t), dev(w), 1, -100, dev(tw))
        assert capi.last_path() == ("ring" if path == b200norm.PATH_RING else "generic")
    check(dx, ao.cross_entropy_bwd(g, logp, t, w, 1, -100, tw), "dx")
    assert capi.device_status() == 0


def test_in_place_and_uint8_targets():
    logp, t, w, tw, g = make_case(64, 200 * 8, torch.bfloat16, False, 1, seed=620)
    t = t % 256
    t[3] = 255  # the ignore index chosen below
    _, tw = ao.nll_fwd(logp, t, None, 1, 255)
    ref = ao.cross_entropy_bwd(g, logp, t, None, 1, 255, tw)
    for path in (b200norm.PATH_RING, b200norm.PATH_GENERIC):
        with forced_path(path):
            buf = logp.to(DEV).clone()
            out = capi.cross_entropy_backward(dev(g), buf, dev(t.to(torch.uint8)), None, 1, 255, dev(tw), out=buf)
        assert out.data_ptr() == buf.data_ptr()
        check(out, ref, "in-place dx with uint8 targets")


def test_out_of_range_target_is_flagged_and_its_row_is_zero():
    logp, t, w, tw, g = make_case(12, 4096, torch.float32, False, 2, seed=630)
    bad = t.clone()
    bad[5] = 4096
    for path in (b200norm.PATH_RING, b200norm.PATH_GENERIC):
        with forced_path(path):
            dx = capi.cross_entropy_backward(dev(g), dev(logp), dev(bad), None, 2, -100, dev(tw))
        assert capi.device_status() == b200norm.ERR_TARGET_RANGE
        assert float(dx[5].abs().max()) == 0.0
        good = ao.cross_entropy_bwd(g, logp, t, None, 2, -100, tw)
        keep = [i for i in range(12) if i != 5]
        check(dx[keep], good[keep], "rows with valid targets")
    assert capi.device_status() == 0


@pytest.mark.parametrize("reduction", ["none", "mean", "sum"])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_autograd_function_matches_torch_cross_entropy(dt, reduction):
    M, C = 48, 32768
    x = ao.randn((M, C), 640, torch.float32, 0.0, 2.0).to(dt)
    t = ao.randint(C, (M,), 641)
    t[7] = -100
    w = (ao.randn((C,), 642).abs() + 0.1).to(dt)
    xg = x.to(DEV).requires_grad_(True)
    loss = capi.cross_entropy(xg, t.to(DEV), w.to(DEV), reduction, -100)
    up = torch.ones_like(loss) if reduction != "none" else ao.randn((M,), 643).to(dt).to(DEV)
    loss.backward(up)
    xr = x.float().requires_grad_(True)
    rloss = torch.nn.functional.cross_entropy(xr, t, w.float(), reduction=reduction, ignore_index=-100)
    rloss.backward(up.cpu().float())
    if dt == torch.float32:
        assert torch.allclose(loss.detach().cpu(), rloss.detach(), rtol=1e-5, atol=1e-6)
        assert ao.fp32_err(xg.grad, xr.grad) <= 1.0
    else:
        assert ao.ulp_distance(loss.detach().cpu().reshape(-1), rloss.detach().to(dt).reshape(-1)) <= 1
        # the saved log-probabilities are bf16 here, torch's are fp32: compare with the composition on what was saved
        logp = capi._log_softmax(x.to(DEV), -1, False).cpu()
        _, tw = ao.nll_fwd(logp, t, w, {"none": 0, "mean": 1, "sum": 2}[reduction], -100)
        ref = ao.cross_entropy_bwd(up.cpu(), logp, t, w, {"none": 0, "mean": 1, "sum": 2}[reduction], -100, tw)
        n_bad, worst = ao.lowp_mismatch(xg.grad, ref)
        assert n_bad == 0, (n_bad, worst)
