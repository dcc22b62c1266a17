"""The five workloads at their full sizes.  A CPU oracle over gigabytes would take minutes, so each
case checks (a) sampled rows (<= 1 ulp / 1e-5) against the oracle and (b) properties that
hold for every row: softmax rows sum to one and masked entries are exactly zero, log-softmax rows have
zero log-sum-exp, weight gradients are additive over row blocks (what row sharding relies on), the
loss equals the mean of the gathered log-probabilities.

Inputs come from the seeded CPU generator, seed = 1000 * config + tensor index, drawn in row blocks
(gpu_util.seeded_rows_to_device), so the oracle and the kernels see the same bits.  Each 16-bit comparison
goes through gpu_util.gate_16bit, which also counts the elements that pass only through the absolute
floor and compares against the float64 evaluation without any floor."""
import math

import pytest
import torch

import b200norm
from b200norm import capi
from oracle import aten_oracle as ao

from gpu_util import DEV, gate_16bit, seeded_rows_to_device

pytestmark = pytest.mark.gpu


def sample_rows(m, k=48, seed=0):
    g = torch.Generator().manual_seed(seed)
    idx = torch.randperm(m, generator=g)[:k].sort().values
    idx[0], idx[-1] = 0, m - 1
    return idx


def test_config1_layer_norm_fp32_4096x1024_full_compare():
    M, N = 4096, 1024
    x = ao.randn((M, N), 1001)
    g, b = ao.randn((N,), 1002, mean=1.0, std=0.02), ao.randn((N,), 1003, std=0.02)
    y, mean, rstd = capi.native_layer_norm(x.to(DEV), [N], g.to(DEV), b.to(DEV), 1e-5)
    assert capi.last_path() == "ring"
    ry, rmean, rrstd = ao.layer_norm_fwd(x, [N], g, b, 1e-5)
    assert ao.fp32_err(y, ry) <= 1.0
    assert float((mean.cpu() - rmean).abs().max()) <= 1e-6
    assert float(((rstd.cpu() - rrstd) / rrstd).abs().max()) <= 1e-5


def test_config2_rms_norm_bf16_8192x4096_full_compare():
    M, N = 8192, 4096
    x, dy = ao.randn((M, N), 2001, torch.bfloat16), ao.randn((M, N), 2004, torch.bfloat16)
    w = ao.randn((N,), 2002, mean=1.0, std=0.02)
    y, rstd = capi._fused_rms_norm(x.to(DEV), [N], w.to(DEV), 1e-6)
    assert capi.last_path() == "ring"
    dx, dw = capi._fused_rms_norm_backward(dy.to(DEV), x.to(DEV), [N], rstd, w.to(DEV))
    assert capi.last_path() == "ring"
    ry, rrstd = ao.rms_norm_fwd(x, [N], w, 1e-6)
    rdx, rdw = ao.rms_norm_bwd(dy, x, [N], w, 1e-6)
    gate_16bit("config 2 y", y, ry, ao.rms_norm_fwd64(x, [N], w, 1e-6))
    dx64, dw64 = ao.rms_norm_bwd64(dy, x, [N], w, 1e-6)
    gate_16bit("config 2 dx", dx, rdx, dx64)
    terms = dy.double() * x.double() * rrstd.double()
    err = ((dw.cpu().double() - terms.sum(0)).abs() / terms.abs().sum(0)).max()
    assert float(err) <= 1e-6, float(err)
    # ... and against the autograd result of the fp64 composite, on the same L1 scale
    err64 = ((dw.cpu().double() - dw64).abs() / terms.abs().sum(0)).max()
    assert float(err64) <= 1e-6, float(err64)


def test_config3_causal_softmax_bf16_8x32x2048x2048():
    B, H, T = 8, 32, 2048
    cols = torch.arange(T).view(1, -1)

    def causal(block, first_row):  # strict upper triangle of every [T, T] slice at -inf, before the rounding
        rows = (torch.arange(first_row, first_row + block.shape[0]) % T).view(-1, 1)
        return block.masked_fill_(cols > rows, float("-inf"))

    s = seeded_rows_to_device(3001, B * H * T, T, torch.bfloat16, std=1.0 / math.sqrt(128), post=causal).view(B, H, T, T)
    mask = torch.ones(T, T, dtype=torch.bool, device=DEV).triu(1)
    p = capi._softmax(s, -1, False)
    assert capi.last_path() == "ring"
    flat_s, flat_p = s.view(-1, T), p.view(-1, T)
    # every row: masked entries exactly zero, the rest sums to one within the bf16 rounding of T terms
    assert float(p.masked_select(mask.expand_as(p)).abs().max()) == 0.0
    sums = flat_p.float().sum(-1)
    assert float((sums - 1).abs().max()) <= 4e-3
    idx = sample_rows(flat_s.shape[0])
    xs = flat_s[idx.to(DEV)].cpu()
    gate_16bit("config 3 softmax", flat_p[idx.to(DEV)], ao.softmax_fwd(xs, -1, False), ao.softmax_fwd64(xs, -1, False))
    g = seeded_rows_to_device(3002, B * H * T, T, torch.bfloat16).view(B, H, T, T)
    dx = capi._softmax_backward_data(g, p, -1, torch.bfloat16)
    assert capi.last_path() == "ring"
    flat_g, flat_dx = g.view(-1, T), dx.view(-1, T)
    gs, ps = flat_g[idx.to(DEV)].cpu(), flat_p[idx.to(DEV)].cpu()
    gate_16bit("config 3 softmax backward", flat_dx[idx.to(DEV)], ao.softmax_bwd(gs, ps, -1, False, torch.bfloat16),
               ao.softmax_bwd64(gs, ps, -1, False))
    # softmax gradients sum to ~0 along the row, and are exactly zero where p is zero
    assert float(dx.masked_select(mask.expand_as(dx)).abs().max()) == 0.0
    assert float(flat_dx.float().sum(-1).abs().max()) <= 5e-2
    assert capi.device_status() == 0


def test_config4_layer_norm_bf16_65536x8192():
    M, N = 65536, 8192
    x = seeded_rows_to_device(4001, M, N, torch.bfloat16)
    dy = seeded_rows_to_device(4004, M, N, torch.bfloat16)
    g, b = ao.randn((N,), 4002, mean=1.0, std=0.02).to(DEV), ao.randn((N,), 4003, std=0.02).to(DEV)
    y, mean, rstd = capi.native_layer_norm(x, [N], g, b, 1e-5)
    assert capi.last_path() == "ring"
    dx, dg, db = capi.native_layer_norm_backward(dy, x, [N], mean, rstd, g, b)
    assert capi.last_path() == "ring"
    idx = sample_rows(M).to(DEV)
    ry, rmean, rrstd = ao.layer_norm_fwd(x[idx].cpu(), [N], g.cpu(), b.cpu(), 1e-5)
    y64, mean64, rstd64 = ao.layer_norm_fwd64(x[idx].cpu(), [N], g.cpu(), b.cpu(), 1e-5)
    gate_16bit("config 4 y", y[idx], ry, y64)
    assert float((mean[idx].cpu() - rmean).abs().max()) <= 1e-6
    assert float(((rstd[idx].cpu() - rrstd) / rrstd).abs().max()) <= 1e-5
    rdx, _, _ = ao.layer_norm_bwd(dy[idx].cpu(), x[idx].cpu(), [N], rmean, rrstd, g.cpu(), b.cpu())
    dx64, _, _ = ao.layer_norm_bwd64(dy[idx].cpu(), x[idx].cpu(), [N], mean64, rstd64, g.cpu(), b.cpu())
    gate_16bit("config 4 dx", dx[idx], rdx, dx64)
    # every row: the normalised output before the affine map has zero mean and unit variance
    z = (y[:4096].float() - b) / g
    assert float(z.mean(-1).abs().max()) <= 2e-3 and float((z.var(-1, unbiased=False) - 1).abs().max()) <= 1e-2
    # weight gradients: additive over row blocks (what row sharding relies on) ...
    parts = []
    for k in range(4):
        sl = slice(k * M // 4, (k + 1) * M // 4)
        _, pg, pb = capi.native_layer_norm_backward(dy[sl], x[sl], [N], mean[sl], rstd[sl], g, b, (False, True, True))
        parts.append(torch.stack([pg, pb]).double())
    total = sum(parts)
    l1 = (dy[:, :64].double().abs()).sum(0)  # L1 scale of the dbeta terms on a column sample
    assert float(((total[1, :64] - db[:64].double()).abs() / l1).max()) <= 1e-6
    xh64 = (x[:, :64].double() - mean.double().view(-1, 1)) * rstd.double().view(-1, 1)
    l1g = (dy[:, :64].double() * xh64).abs().sum(0)  # L1 scale of the dgamma terms on the same column sample
    assert float(((total[0, :64] - dg[:64].double()).abs() / l1g).max()) <= 1e-6
    # ... and dbeta equals an fp64 column sum of dy on a column sample
    ref_db = dy[:, :64].double().sum(0)
    assert float(((db[:64].double() - ref_db).abs() / l1).max()) <= 1e-6
    terms = dy[:, :64].double() * xh64
    assert float(((dg[:64].double() - terms.sum(0)).abs() / terms.abs().sum(0)).max()) <= 1e-6
    assert capi.device_status() == 0


def test_config5_log_softmax_nll_bf16_16384x128256():
    M, V = 16384, 128256
    logits = seeded_rows_to_device(5001, M, V, torch.bfloat16, std=2.0, block=1024)
    t = ao.randint(V, (M,), 5002).to(DEV)
    logp = capi._log_softmax(logits, -1, False)
    assert capi.last_path() in ("cluster", "twopass")
    idx = sample_rows(M, 24).to(DEV)
    ls = logits[idx].cpu()
    gate_16bit("config 5 log-softmax", logp[idx], ao.softmax_fwd(ls, -1, True), ao.softmax_fwd64(ls, -1, True))
    # every row: log-sum-exp of the output is zero up to the bf16 rounding of the entries
    lse = torch.cat([torch.logsumexp(logp[k:k + 1024].float(), -1) for k in range(0, M, 1024)])
    assert float(lse.abs().max()) <= 2e-2
    out, tw, sums = capi.nll_loss_forward(logp, t, None, 1, -100, return_sums=True)
    picked = logp.gather(1, t.view(-1, 1)).double().cpu()
    assert float(tw) == M
    assert math.isclose(float(sums[0]), float(-picked.sum()), rel_tol=1e-6)
    assert ao.ulp_distance(out.cpu().reshape(1), torch.tensor([-picked.mean()]).to(torch.bfloat16)) <= 1
    del logits
    grad_logp = capi.nll_loss_backward(torch.ones((), device=DEV, dtype=torch.bfloat16), logp, t, None, 1, -100, tw)
    assert float(grad_logp.gather(1, t.view(-1, 1)).float().mean()) == pytest.approx(-1.0 / M, rel=1e-2)
    dlogits = capi._log_softmax_backward_data(grad_logp, logp, -1, torch.bfloat16)
    assert capi.last_path() in ("cluster", "twopass")
    gl, lp = grad_logp[idx].cpu(), logp[idx].cpu()
    gate_16bit("config 5 log-softmax backward", dlogits[idx], ao.softmax_bwd(gl, lp, -1, True, torch.bfloat16),
               ao.softmax_bwd64(gl, lp, -1, True))
    # rows of the cross-entropy gradient sum to ~0
    rs = torch.cat([dlogits[k:k + 1024].float().sum(-1) for k in range(0, M, 1024)])
    assert float(rs.abs().max()) <= 1e-5
    assert capi.device_status() == 0


def test_softmax_over_a_middle_dim_beyond_2_to_the_31_elements():
    # [2, 33000, 33000] bf16 (2.2e9 elements, 4.4 GB per tensor), softmax over dim 1: element offsets need 64 bits
    # with inner > 1.  Sampled lines against the oracle (first and last line of each outer slice included).
    O, N, I = 2, 33000, 33000
    x = torch.empty((O, N, I), dtype=torch.bfloat16, device=DEV)
    gen = torch.Generator(device=DEV).manual_seed(9001)
    for o in range(O):
        for r in range(0, N, 3000):
            k = min(3000, N - r)
            x[o, r:r + k] = (torch.randn((k, I), generator=gen, device=DEV) * 2.0).to(torch.bfloat16)
    y = capi._softmax(x, 1, False)
    lines = [(0, 0), (0, I - 1), (1, 0), (1, I - 1), (0, 12345), (1, 31999), (1, 7), (0, 16384)]
    xs = torch.stack([x[o, :, i] for o, i in lines]).cpu()   # [lines, N]
    ys = torch.stack([y[o, :, i] for o, i in lines])
    assert ao.lowp_mismatch(ys, ao.softmax_fwd(xs, -1, False))[0] == 0
    # every line sums to one (checked on a slab of lines per outer slice, and on the very last elements)
    assert float((y[:, :, :512].float().sum(1) - 1).abs().max()) <= 2e-2
    assert float((y[:, :, -512:].float().sum(1) - 1).abs().max()) <= 2e-2
    dy = x  # any tensor of the shape will do as the upstream gradient: reuse the input
    dx = capi._softmax_backward_data(dy, y, 1, torch.bfloat16)
    dxs = torch.stack([dx[o, :, i] for o, i in lines])
    ref = ao.softmax_bwd(xs, ys.cpu(), -1, False, torch.bfloat16)
    assert ao.lowp_mismatch(dxs, ref)[0] == 0
    assert capi.device_status() == 0


@pytest.mark.parametrize("C", [19, 64, 150])
def test_softmax_over_dim_1_of_16xCx512x512_bf16(C):
    # the shapes of the bench's sm_c19 / sm_c64 / sm_c150 lines (tensor-map TMA tiles): sampled lines against the
    # oracle, and for EVERY line: the softmax sums to one, the backward sums to zero (sum_j y_j (dy_j - s) = 0)
    O, HW = 16, 512 * 512
    x = seeded_rows_to_device(11000 + C, O * C, HW, torch.bfloat16, std=2.0, block=64).view(O, C, HW)
    dy = seeded_rows_to_device(12000 + C, O * C, HW, torch.bfloat16, block=64).view(O, C, HW)
    y = capi._softmax(x, 1, False)
    assert capi.last_path() == "tma"
    dx = capi._softmax_backward_data(dy, y, 1, torch.bfloat16)
    assert capi.last_path() == "tma"
    g = torch.Generator().manual_seed(C)
    lines = [(0, 0), (O - 1, HW - 1)] + [(int(torch.randint(0, O, (1,), generator=g)), int(torch.randint(0, HW, (1,), generator=g)))
                                        for _ in range(62)]
    xs = torch.stack([x[o, :, i] for o, i in lines]).cpu()
    ys = torch.stack([y[o, :, i] for o, i in lines])
    gate_16bit(f"dim-1 softmax C={C} y", ys, ao.softmax_fwd(xs, -1, False), ao.softmax_fwd64(xs, -1, False))
    dys = torch.stack([dy[o, :, i] for o, i in lines]).cpu()
    dxs = torch.stack([dx[o, :, i] for o, i in lines])
    gate_16bit(f"dim-1 softmax C={C} dx", dxs, ao.softmax_bwd(dys, ys.cpu(), -1, False, torch.bfloat16),
               ao.softmax_bwd64(dys, ys.cpu(), -1, False))
    assert float((y.float().sum(1) - 1).abs().max()) <= C * 2e-3          # bf16 rounding of C terms
    scale = float((y.float() * dy.float().abs()).sum(1).max())
    assert float(dx.float().sum(1).abs().max()) <= 8e-3 * max(1.0, scale)
    assert capi.device_status() == 0
