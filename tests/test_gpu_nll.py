"""nll_loss forward / backward parity through the C ABI vs CPU ATen."""
import math

import pytest
import torch

import b200norm
from b200norm import capi
from oracle import aten_oracle as ao

from gpu_util import DEV

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("reduction", [0, 1, 2])
@pytest.mark.parametrize("weighted", [False, True])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.float16, torch.float64])
@pytest.mark.parametrize("M,C", [(1, 1), (16, 10), (1000, 257), (20000, 33)])
def test_forward_backward(M, C, dt, weighted, reduction):
    logp = torch.log_softmax(ao.randn((M, C), 500, torch.float32, 0.0, 2.0), -1).to(dt)
    t = ao.randint(C, (M,), 501)
    if M > 4:
        t[3] = -100
    w = (ao.randn((C,), 502).abs() + 0.1).to(dt) if weighted else None
    dev = lambda z: None if z is None else z.to(DEV)
    out, tw = capi.nll_loss_forward(dev(logp), dev(t), dev(w), reduction, -100)
    rout, rtw = ao.nll_fwd(logp, t, w, reduction, -100)
    assert out.shape == rout.shape and tw.shape == rtw.shape
    if dt == torch.float64:
        assert torch.allclose(out.cpu(), rout, rtol=1e-12, equal_nan=True) and torch.allclose(tw.cpu(), rtw, rtol=1e-12)
    elif dt == torch.float32:
        assert torch.allclose(out.cpu(), rout, rtol=1e-5, atol=1e-6, equal_nan=True)
        assert torch.allclose(tw.cpu(), rtw, rtol=1e-5)
    else:
        assert ao.ulp_distance(out.cpu().reshape(-1), rout.reshape(-1)) <= 1
        assert ao.ulp_distance(tw.cpu().reshape(-1), rtw.reshape(-1)) <= 1
    g = ao.randn((M,), 503).to(dt) if reduction == 0 else torch.tensor(0.7, dtype=dt)
    gi = capi.nll_loss_backward(dev(g), dev(logp), dev(t), dev(w), reduction, -100, tw)
    rgi = ao.nll_bwd(g, logp, t, w, reduction, -100, tw.cpu())
    if dt in (torch.float32, torch.float64):
        assert torch.allclose(gi.cpu(), rgi, rtol=1e-5, atol=1e-7)
    else:
        assert ao.ulp_distance(gi.cpu(), rgi) <= 1
    assert capi.device_status() == 0


def test_uint8_targets_match_int64():
    # reference: test/xpu/test_nn_xpu.py:16047-16069
    logp = torch.log_softmax(ao.randn((64, 20), 510), -1).to(DEV)
    t = ao.randint(20, (64,), 511)
    a = capi.nll_loss_forward(logp, t.to(DEV), None, 1, -100)
    b = capi.nll_loss_forward(logp, t.to(torch.uint8).to(DEV), None, 1, -100)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_all_ignored_and_ignore_index_out_of_range():
    # :16003-16045 — all rows ignored: sum 0, mean NaN; :15868-15872 — an ignore_index beyond C is legal
    logp = torch.log_softmax(ao.randn((8, 6), 520), -1).to(DEV)
    t = torch.full((8,), 255, dtype=torch.int64, device=DEV)
    out, tw = capi.nll_loss_forward(logp, t, None, 1, 255)
    assert math.isnan(float(out)) and float(tw) == 0.0
    out, _ = capi.nll_loss_forward(logp, t, None, 2, 255)
    assert float(out) == 0.0
    out, _ = capi.nll_loss_forward(logp, t, None, 0, 255)
    assert float(out.abs().sum()) == 0.0
    assert capi.device_status() == 0


def test_out_of_range_target_sets_the_status_word_without_trapping():
    logp = torch.log_softmax(ao.randn((8, 6), 530), -1).to(DEV)
    t = torch.tensor([0, 1, 2, 99, 3, 4, 5, 0], device=DEV)
    out, tw = capi.nll_loss_forward(logp, t, None, 2, -100)
    assert capi.device_status() == b200norm.ERR_TARGET_RANGE
    assert capi.device_status() == 0  # read-and-clear
    assert float(tw) == 7.0  # the bad row contributes nothing
    torch.cuda.synchronize()


def test_one_dimensional_input():
    logp = torch.log_softmax(ao.randn((12,), 540), -1)
    t = torch.tensor(5)
    for red in (0, 1, 2):
        out, tw = capi.nll_loss_forward(logp.to(DEV), t.to(DEV), None, red, -100)
        rout, rtw = ao.nll_fwd(logp, t, None, red, -100)
        assert out.shape == rout.shape and torch.allclose(out.cpu(), rout)


def test_log_softmax_of_ones_gives_log_vocab():
    V = 50000
    logp = capi._log_softmax(torch.ones(4, V, device=DEV), -1, False)
    out, tw = capi.nll_loss_forward(logp, torch.tensor([0, 1, V - 1, 17], device=DEV), None, 1, -100)
    assert math.isclose(float(out), math.log(V), rel_tol=1e-5)


def test_sums_for_row_sharding():
    logp = torch.log_softmax(ao.randn((300, 40), 550), -1).to(DEV)
    t = ao.randint(40, (300,), 551).to(DEV)
    out, tw, sums = capi.nll_loss_forward(logp, t, None, 1, -100, return_sums=True)
    parts = [capi.nll_loss_forward(logp[a:b], t[a:b], None, 2, -100, return_sums=True)[2] for a, b in ((0, 100), (100, 300))]
    total = parts[0] + parts[1]
    assert torch.allclose(total, sums, rtol=1e-6)
    assert math.isclose(float(total[0] / total[1]), float(out), rel_tol=1e-6)
