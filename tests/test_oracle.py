"""Pins the oracle: the C restatement of the reference's algorithms against PyTorch CPU ATen, both
against the committed golden vectors, and the known-answer properties the reference's own tests
assert for this path."""
import math
from pathlib import Path

import pytest
import torch

from oracle import aten_oracle as ao
from oracle import restate

GOLDEN = torch.load(Path(__file__).parent / "golden" / "golden_v1.pt")


def close32(a, b, tol=1.0):
    return ao.fp32_err(a, b) <= tol


@pytest.mark.parametrize("name", ["ln_f32", "ln_bf16_w32", "ln_f16", "ln_f32_n5"])
def test_golden_layer_norm_matches_aten_and_restatement(name):
    c = GOLDEN[name]
    n = c["x"].shape[-1]
    y, mean, rstd = ao.layer_norm_fwd(c["x"], [n], c["gamma"], c["beta"], c["eps"])
    assert torch.equal(y, c["y"]) and torch.equal(mean, c["mean"]) and torch.equal(rstd, c["rstd"])
    # restatement (Welford, 1 lane and a 32-lane split as the reference's work-group does)
    for lanes in (1, 32):
        ry, rmean, rrstd = restate.norm_fwd(c["x"], c["gamma"], c["beta"], c["eps"], rms=False, lanes=lanes)
        assert close32(rmean, c["mean"].reshape(-1)) and close32(rrstd, c["rstd"].reshape(-1))
        if c["x"].dtype == torch.float32:
            assert close32(ry, c["y"])
        else:
            assert ao.ulp_distance(ry.to(c["x"].dtype), c["y"]) <= 1
    rdx, rdg, rdb = restate.norm_bwd(c["dy"], c["x"], c["mean"], c["rstd"], c["gamma"], rms=False)
    if c["x"].dtype == torch.float32:
        assert close32(rdx, c["dx"], tol=4.0)
    else:
        assert ao.ulp_distance(rdx.to(c["x"].dtype), c["dx"]) <= 1
    assert torch.allclose(rdg.float(), c["dgamma"].float(), rtol=1e-4, atol=1e-4)
    assert torch.allclose(rdb.float(), c["dbeta"].float(), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("name", ["rms_f32", "rms_bf16_w32"])
def test_golden_rms_norm(name):
    c = GOLDEN[name]
    n = c["x"].shape[-1]
    y, rstd = ao.rms_norm_fwd(c["x"], [n], c["weight"], c["eps"])
    assert torch.equal(y, c["y"]) and torch.equal(rstd, c["rstd"])
    ry, _, rrstd = restate.norm_fwd(c["x"], c["weight"], None, c["eps"], rms=True)
    assert close32(rrstd, c["rstd"].reshape(-1))
    # the backward has no CPU ATen kernel: autograd through the composite (golden) vs the restated
    # closed form of the reference (rms branch of its backward functor)
    rdx, rdw, _ = restate.norm_bwd(c["dy"], c["x"], None, c["rstd"], c["weight"], rms=True)
    if c["x"].dtype == torch.float32:
        assert close32(ry, c["y"]) and close32(rdx, c["dx"], tol=4.0)
    else:
        assert ao.ulp_distance(ry.to(c["x"].dtype), c["y"]) <= 1
        assert ao.ulp_distance(rdx.to(c["x"].dtype), c["dx"]) <= 1
    assert torch.allclose(rdw.float(), c["dweight"].float(), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("name", ["sm_f32_last", "sm_bf16_last", "sm_f32_dim0", "sm_f32_dim1"])
def test_golden_softmax(name):
    c = GOLDEN[name]
    dt = c["x"].dtype
    for is_log, tag in ((False, "softmax"), (True, "log_softmax")):
        y = ao.softmax_fwd(c["x"], c["dim"], is_log)
        assert torch.equal(y, c[tag])
        ry = restate.softmax_fwd(c["x"], c["dim"], is_log)
        rdx = restate.softmax_bwd(c["dy"], c[tag], c["dim"], is_log)
        if dt == torch.float32:
            assert close32(ry, c[tag], tol=2.0) and close32(rdx, c[tag + "_bwd"], tol=4.0)
        else:
            assert ao.ulp_distance(ry.to(dt), c[tag]) <= 1
            assert ao.ulp_distance(rdx.to(dt), c[tag + "_bwd"]) <= 1


def test_golden_nll():
    c = GOLDEN["nll_f32"]
    for red in (0, 1, 2):
        for w, tag in ((None, "now"), (c["weight"], "w")):
            out, tw = ao.nll_fwd(c["logp"], c["target"], w, red, c["ignore_index"])
            assert torch.equal(out, c[f"out_{red}_{tag}"]) and torch.equal(tw, c[f"tw_{red}_{tag}"])
            if red:
                rout, rtw = restate.nll_fwd(c["logp"], c["target"], w, red == 1, c["ignore_index"])
                assert math.isclose(float(rout), float(out), rel_tol=1e-5) and math.isclose(float(rtw), float(tw), rel_tol=1e-6)


# ---- known-answer properties taken from the reference's tests --------------------------------------
def test_layer_norm_large_offset_stays_finite():
    # test/regressions/test_layer_norm.py:19-28 — a row of 1e15 + {0..4} must not produce NaN
    x = torch.tensor([[1e15 + i for i in range(5)]], dtype=torch.float32)
    y, mean, rstd = restate.norm_fwd(x, None, None, 1e-5, rms=False)
    ry, _, _ = ao.layer_norm_fwd(x, [5], None, None, 1e-5)
    assert torch.isfinite(y).all() and torch.isfinite(ry).all()


def test_rms_dbeta_free_and_dgamma_formula():
    # test/regressions/test_rms_norm.py:76-79 — dgamma == sum_i dy * x * rstd
    x = ao.randn((33, 48), 5)
    dy = ao.randn((33, 48), 6)
    w = ao.randn((48,), 7, mean=1.0, std=0.02)
    _, rstd = ao.rms_norm_fwd(x, [48], w, 1e-6)
    _, dw = ao.rms_norm_bwd(dy, x, [48], w, 1e-6)
    expect = (dy.double() * x.double() * rstd.double()).sum(0)
    assert torch.allclose(dw.double(), expect, rtol=1e-5, atol=1e-5)
    _, rdw, _ = restate.norm_bwd(dy, x, None, rstd, w, rms=True)
    assert torch.allclose(rdw, expect, rtol=1e-6, atol=1e-6)


def test_log_softmax_shift_invariance_and_unit_mass():
    # test/xpu/test_nn_xpu.py:14177-14190, :14141-14147
    x = ao.randn((5, 300), 8)
    a = restate.softmax_fwd(x, -1, True)
    b = restate.softmax_fwd(x + 100.0, -1, True)
    assert torch.allclose(a, b, atol=1e-4)
    assert torch.allclose(a.exp().sum(-1), torch.ones(5), atol=1e-5)


def test_log_softmax_of_ones_gives_log_vocab():
    # test/xpu/test_nn_xpu.py:17902-17911 — nll of a constant row over V classes is log V
    V = 5000
    logp = restate.softmax_fwd(torch.ones(3, V), -1, True)
    out, tw = restate.nll_fwd(logp, torch.tensor([0, 7, V - 1]), None, True, -100)
    assert math.isclose(float(out), math.log(V), rel_tol=1e-5) and float(tw) == 3.0


def test_nll_all_ignored_is_nan_for_mean_and_zero_for_sum():
    # test/xpu/test_nn_xpu.py:16003-16045
    logp = torch.log_softmax(ao.randn((4, 6), 9), -1)
    t = torch.full((4,), -100)
    out, tw = ao.nll_fwd(logp, t, None, 1, -100)
    assert math.isnan(float(out)) and float(tw) == 0.0
    out, _ = ao.nll_fwd(logp, t, None, 2, -100)
    assert float(out) == 0.0
    rout, rtw = restate.nll_fwd(logp, t, None, True, -100)
    assert math.isnan(float(rout)) and float(rtw) == 0.0


def test_all_masked_row_is_nan_on_cpu_aten():
    # the semantics the kernels must reproduce: an all -inf row gives NaN, single -inf entries 0 / -inf
    x = torch.tensor([[float("-inf")] * 4, [0.0, float("-inf"), 1.0, 2.0]])
    y = ao.softmax_fwd(x, -1, False)
    assert torch.isnan(y[0]).all() and y[1, 1] == 0
    ly = ao.softmax_fwd(x, -1, True)
    assert torch.isnan(ly[0]).all() and ly[1, 1] == float("-inf")


def test_comparators():
    a = torch.tensor([1.0, 2.0, -3.0], dtype=torch.bfloat16)
    b = a.clone()
    assert ao.ulp_distance(a, b) == 0
    b[0] = torch.nextafter(torch.tensor(1.0), torch.tensor(2.0)).to(torch.bfloat16)  # rounds back to 1.0
    assert ao.ulp_distance(a, b) == 0
    c = (a.view(torch.int16) + 1).view(torch.bfloat16)
    assert ao.ulp_distance(a, c) == 1
    assert ao.fp32_err(torch.tensor([1.0, 0.0]), torch.tensor([1.0 + 5e-6, 1e-7])) <= 1.0
    assert ao.fp32_err(torch.tensor([1.0]), torch.tensor([1.001])) > 1.0


# ---- golden_v2: the operators around the core path -------------------------------------------------
GOLDEN2 = torch.load(Path(__file__).parent / "golden" / "golden_v2.pt")


def _wide(t):
    return t.double() if t.dtype == torch.float64 else t.float()


@pytest.mark.parametrize("name", ["safe_f32", "safe_bf16", "safe_f32_dim0"])
def test_golden_safe_softmax(name):
    c = GOLDEN2[name]
    y = torch.ops.aten._safe_softmax(_wide(c["x"]), c["dim"]).to(c["x"].dtype)
    assert torch.equal(y, c["y"]) and not bool(torch.isnan(y).any())
    # the definition: softmax with the all -inf lines replaced by zeros
    plain = torch.softmax(_wide(c["x"]), c["dim"])
    dead = (c["x"] == float("-inf")).all(c["dim"], keepdim=True)
    assert bool(dead.any())
    assert torch.equal(torch.where(dead, torch.zeros_like(plain), plain).to(c["x"].dtype), c["y"])


@pytest.mark.parametrize("name", ["masked_f32", "masked_bf16"])
def test_golden_masked_softmax(name):
    c = GOLDEN2[name]
    dt = c["x"].dtype
    x = _wide(c["x"])
    B, H, T, _ = x.shape
    for tag, mtype in (("full", 2), ("txt", 0), ("bxt", 1)):
        m = c["mask_" + tag]
        y = torch._masked_softmax(x, m, -1, mtype).to(dt)
        assert torch.equal(torch.isnan(y), torch.isnan(c["y_" + tag]))
        ok = ~torch.isnan(y)
        assert torch.equal(y[ok], c["y_" + tag][ok])
        # the definition: softmax of the scores with the masked ones at -inf
        full = m if tag == "full" else (m.view(B, 1, 1, T) if tag == "bxt" else m).expand(B, H, T, T)
        ref = torch.softmax(x.masked_fill(full, float("-inf")), -1).to(dt)
        if dt == torch.float32:  # two CPU kernels: the same values up to the last bits of their row sums
            assert torch.allclose(ref[ok], c["y_" + tag][ok], rtol=1e-6, atol=1e-8)
        else:
            assert ao.ulp_distance(ref[ok], c["y_" + tag][ok]) <= 1
    dx = torch.ops.aten._masked_softmax_backward(_wide(c["grad"]), _wide(c["y_full"]), c["mask_full"], -1).to(dt)
    assert torch.equal(dx, c["dx_full"]) and not bool(torch.isnan(dx).any())
    assert float(dx[c["mask_full"]].abs().max()) == 0.0


@pytest.mark.parametrize("name", ["ce_f32", "ce_bf16"])
def test_golden_cross_entropy_backward(name):
    c = GOLDEN2[name]
    logp, t = c["logp"], c["target"]
    for red in (0, 1, 2):
        for w, tag in ((None, "now"), (c["weight"], "w")):
            dx = ao.cross_entropy_bwd(c[f"grad_{red}"], logp, t, w, red, c["ignore_index"], c[f"tw_{red}_{tag}"])
            assert torch.equal(dx, c[f"dx_{red}_{tag}"])
            # closed form the fused kernel evaluates: s_i * (exp(logp) - onehot)
            lp = _wide(logp)
            wt = torch.ones(lp.shape[1]) if w is None else _wide(w)
            valid = t != c["ignore_index"]
            tt = torch.where(valid, t, torch.zeros_like(t))
            s = wt[tt] * _wide(c[f"grad_{red}"]) * valid
            if red == 1:
                s = s / _wide(c[f"tw_{red}_{tag}"])
            onehot = torch.nn.functional.one_hot(tt, lp.shape[1]).to(lp.dtype)
            closed = (s.reshape(-1, 1) * (lp.exp() - onehot)).to(logp.dtype)
            if logp.dtype == torch.float32:
                assert torch.allclose(closed, dx, rtol=1e-5, atol=1e-7)
            else:
                assert ao.ulp_distance(closed, dx) <= 1


# ---- golden_v3: group norm, batch norm statistics, softmax over a middle dim, layer norm on long rows -------------
GOLDEN3 = torch.load(Path(__file__).parent / "golden" / "golden_v3.pt")


@pytest.mark.parametrize("name", ["smd1_bf16", "smd1_f32", "smd1_f16"])
def test_golden_softmax_over_dim_1(name):
    # the oracle the GPU tests use reproduces the fixture bit for bit, and the fixture has the properties of the op
    c = GOLDEN3[name]
    x, dt = c["x"], c["x"].dtype
    for is_log, key in ((False, "softmax"), (True, "log_softmax")):
        y = ao.softmax_fwd(x, 1, is_log)
        assert torch.equal(torch.isnan(y), torch.isnan(c[key]))
        ok = ~torch.isnan(y)
        assert torch.equal(y[ok], c[key][ok])
        dx = ao.softmax_bwd(c["dy"], c[key], 1, is_log, dt)
        okb = ~torch.isnan(dx)
        assert torch.equal(torch.isnan(dx), torch.isnan(c[key + "_bwd"])) and torch.equal(dx[okb], c[key + "_bwd"][okb])
    live = ~torch.isnan(c["softmax"]).any(1)
    assert bool(live.any()) and not bool(live.all())          # the all -inf line is there, and it is the only dead one
    sums = _wide(c["softmax"]).sum(1)[live]
    assert float((sums - 1).abs().max()) <= (1e-5 if dt == torch.float32 else 3e-2)


def test_golden_layer_norm_long_rows():
    c = GOLDEN3["ln_long_bf16_w32"]
    n = c["x"].shape[-1]
    assert n > 8192                                             # longer than one CTA's threads hold
    y, mean, rstd = ao.layer_norm_fwd(c["x"], [n], c["gamma"], c["beta"], c["eps"])
    assert torch.equal(y, c["y"]) and torch.equal(mean.reshape(-1), c["mean"].reshape(-1))
    dx, dg, db = ao.layer_norm_bwd(c["dy"], c["x"], [n], c["mean"], c["rstd"], c["gamma"], c["beta"])
    assert torch.equal(dx, c["dx"]) and torch.equal(dg, c["dgamma"]) and torch.equal(db, c["dbeta"])
    # known answer: normalised rows have zero mean and unit variance before the affine map
    xh = (_wide(c["x"]) - c["mean"].reshape(-1, 1)) * c["rstd"].reshape(-1, 1)
    assert float(xh.mean(1).abs().max()) <= 1e-5 and float((xh.var(1, unbiased=False) - 1).abs().max()) <= 1e-4


@pytest.mark.parametrize("name", ["gn_f32", "gn_bf16", "gn_f32_odd"])
def test_golden_group_norm(name):
    c = GOLDEN3[name]
    x, dt = c["x"], c["x"].dtype
    N, C = x.shape[0], x.shape[1]
    hw = x.numel() // (N * C)
    y, mean, rstd = torch.ops.aten.native_group_norm(_wide(x), _wide(c["weight"]), _wide(c["bias"]), N, C, hw, c["G"], c["eps"])
    assert torch.equal(y.to(dt), c["y"]) and torch.equal(mean.float(), c["mean"]) and torch.equal(rstd.float(), c["rstd"])
    # the definition: a layer norm of each (sample, group) row with per-channel weights
    rows = _wide(x).reshape(N, c["G"], -1)
    ref = (rows - rows.mean(2, keepdim=True)) / torch.sqrt(rows.var(2, unbiased=False, keepdim=True) + c["eps"])
    ref = ref.reshape(N, C, hw) * _wide(c["weight"]).view(1, C, 1) + _wide(c["bias"]).view(1, C, 1)
    assert torch.allclose(ref.reshape(x.shape), _wide(c["y"]), rtol=2e-2 if dt != torch.float32 else 1e-4, atol=2e-2 if dt != torch.float32 else 1e-5)


@pytest.mark.parametrize("name", ["bn_f32", "bn_bf16", "bn_f32_small"])
def test_golden_batch_norm_statistics(name):
    c = GOLDEN3[name]
    x = c["x"]
    cm, cinv = None, None
    crm, crv = c["running_mean"].clone(), c["running_var"].clone()
    m, v = torch.batch_norm_update_stats(_wide(x), crm, crv, c["momentum"])     # CPU ATen against the float64 fixture
    assert torch.allclose(m, c["mean"], rtol=1e-5, atol=1e-6) and torch.allclose(v, c["var"], rtol=1e-4, atol=1e-6)
    assert torch.allclose(crm, c["running_mean_out"], rtol=1e-5, atol=1e-6)
    assert torch.allclose(crv, c["running_var_out"], rtol=1e-4, atol=1e-6)
    assert torch.allclose(c["invstd"], 1.0 / torch.sqrt(c["var"] + c["eps"]), rtol=1e-5)
