"""CPU ATen oracle, comparators and seeded inputs.  Test infrastructure: see oracle/__init__.py."""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch
import torch.nn.functional as F

aten = torch.ops.aten


# ---------------------------------------------------------------------------------------------------
# seeded inputs (CPU generator, so CPU oracle and GPU kernels see bit-identical data)
# ---------------------------------------------------------------------------------------------------
def randn(shape, seed: int, dtype=torch.float32, mean: float = 0.0, std: float = 1.0) -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(int(seed))
    t = torch.randn(shape, generator=g, dtype=torch.float32) * std + mean
    return t.to(dtype)


def randint(high: int, shape, seed: int) -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(int(seed))
    return torch.randint(0, high, shape, generator=g, dtype=torch.int64)


def causal_scores(shape, seed: int, dtype, head_dim: int = 128) -> torch.Tensor:
    """N(0,1)/sqrt(head_dim) scores with the strict upper triangle of the last two dims at -inf."""
    s = randn(shape, seed, torch.float32) / math.sqrt(head_dim)
    t = shape[-1]
    mask = torch.ones(shape[-2], t, dtype=torch.bool).triu(1)
    s = s.masked_fill(mask, float("-inf"))
    return s.to(dtype)


# ---------------------------------------------------------------------------------------------------
# comparators
# ---------------------------------------------------------------------------------------------------
def _ordered_int(t: torch.Tensor) -> torch.Tensor:
    """Map 16-bit floats to integers whose order matches the floats' (sign-magnitude -> two's complement)."""
    i = t.contiguous().view(torch.int16).to(torch.int32)
    return torch.where(i < 0, -(i & 0x7FFF), i)


def ulp_distance(a: torch.Tensor, b: torch.Tensor) -> int:
    """Largest distance in units in the last place between two bf16/fp16 tensors; NaNs must coincide."""
    assert a.dtype == b.dtype and a.dtype in (torch.bfloat16, torch.float16), (a.dtype, b.dtype)
    assert a.shape == b.shape, (a.shape, b.shape)
    if a.numel() == 0:
        return 0
    a, b = a.cpu(), b.cpu()
    na, nb = torch.isnan(a), torch.isnan(b)
    if not torch.equal(na, nb):
        return 1 << 30
    d = (_ordered_int(a) - _ordered_int(b)).abs()
    d = torch.where(na, torch.zeros_like(d), d)
    return int(d.max())


def lowp_report(a: torch.Tensor, ref: torch.Tensor, floor_scale: float = 1e-6) -> dict:
    """Gate for bf16/fp16 outputs, with its accounting.  An element passes when it is within 1 ulp of the
    reference OR within the absolute floor floor_scale * max(1, rms(ref)) — the same floor the fp32 gate uses.
    An element can need the floor only where one 16-bit ulp of the reference is SMALLER than the floor (a
    difference below one ulp is at most one ulp apart), i.e. for outputs near zero, where the fp32 rounding of
    terms of size ~1 already exceeds that ulp.  Returned: 'bad' elements failing both tests and the 'worst' ulp
    distance among them; 'floor_only' elements more than 1 ulp apart that passed through the floor; 'numel'."""
    assert a.dtype == ref.dtype and a.dtype in (torch.bfloat16, torch.float16), (a.dtype, ref.dtype)
    assert a.shape == ref.shape, (a.shape, ref.shape)
    if a.numel() == 0:
        return {"bad": 0, "worst": 0, "floor_only": 0, "numel": 0}
    a, ref = a.detach().cpu(), ref.detach().cpu()
    na, nb = torch.isnan(a), torch.isnan(ref)
    if not torch.equal(na, nb):
        return {"bad": int((na != nb).sum()), "worst": 1 << 30, "floor_only": 0, "numel": a.numel()}
    d = (_ordered_int(a) - _ordered_int(ref)).abs()
    d = torch.where(na, torch.zeros_like(d), d)
    af, rf = a.double(), ref.double()
    finite = torch.isfinite(rf)
    rms = float(rf[finite].pow(2).mean().sqrt()) if finite.any() else 0.0
    floor = floor_scale * max(1.0, rms)
    absdiff = torch.where(finite & torch.isfinite(af), (af - rf).abs(), torch.full_like(rf, float("inf")))
    absdiff = torch.where(af == rf, torch.zeros_like(absdiff), absdiff)  # equal infinities
    bad = (d > 1) & (absdiff > floor)
    n_bad = int(bad.sum())
    return {"bad": n_bad, "worst": int(d[bad].max()) if n_bad else 0,
            "floor_only": int(((d > 1) & (absdiff <= floor)).sum()), "numel": a.numel()}


def lowp_mismatch(a: torch.Tensor, ref: torch.Tensor, floor_scale: float = 1e-6):
    """(number of failing elements, worst ulp distance among them) of lowp_report."""
    r = lowp_report(a, ref, floor_scale)
    return r["bad"], r["worst"]


def strict_ulp_failures(a: torch.Tensor, ref64: torch.Tensor) -> int:
    """Elements of the 16-bit tensor `a` more than 1 ulp from the float64 result rounded once to a's dtype — no
    floor of any kind.  NaN patterns must coincide (a mismatch counts every element)."""
    assert a.dtype in (torch.bfloat16, torch.float16) and ref64.dtype == torch.float64
    a, r = a.detach().cpu(), ref64.detach().cpu().to(a.dtype)
    na, nb = torch.isnan(a), torch.isnan(r)
    if not torch.equal(na, nb):
        return a.numel()
    d = (_ordered_int(a) - _ordered_int(r)).abs()
    return int(((d > 1) & ~na).sum())


def fp32_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """max |a-b| / (1e-5*|b| + 1e-6*max(1, rms(b))): <= 1 means "fp32 relative error <= 1e-5" with the
    absolute floor that outputs near zero need (element-wise relative error is unbounded there)."""
    a, b = a.detach().cpu().double(), b.detach().cpu().double()
    assert a.shape == b.shape, (a.shape, b.shape)
    if b.numel() == 0:
        return 0.0
    nan_a, nan_b = torch.isnan(a), torch.isnan(b)
    if not torch.equal(nan_a, nan_b):
        return float("inf")
    inf_b = torch.isinf(b)
    if inf_b.any():
        if not torch.equal(a[inf_b], b[inf_b]):
            return float("inf")
    ok = ~(nan_b | inf_b)
    if not ok.any():
        return 0.0
    a, b = a[ok], b[ok]
    rms = float(b.pow(2).mean().sqrt())
    tol = 1e-5 * b.abs() + 1e-6 * max(1.0, rms)
    return float(((a - b).abs() / tol).max())


def reduction_err(a: torch.Tensor, terms_l1: torch.Tensor, ref64: torch.Tensor) -> float:
    """|a - ref64| / L1 norm of the summed terms: the conditioning-aware error of a long fp32 sum."""
    a = a.detach().cpu().double()
    denom = terms_l1.double().clamp_min(1e-30)
    return float(((a - ref64.double()).abs() / denom).max())


# ---------------------------------------------------------------------------------------------------
# reference ops
# ---------------------------------------------------------------------------------------------------
def _f32(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    return None if t is None else t.detach().cpu().float()


def _cpu(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    return None if t is None else t.detach().cpu()


def layer_norm_fwd(x, normalized_shape, weight, bias, eps, exact: bool = True):
    """(y, mean, rstd).  exact: CPU ATen on fp32 upcasts, y rounded once to x's dtype, stats fp32."""
    if exact and x.dtype != torch.float64:
        y, mean, rstd = aten.native_layer_norm(_f32(x), list(normalized_shape), _f32(weight), _f32(bias), eps)
        return y.to(x.dtype), mean, rstd
    y, mean, rstd = aten.native_layer_norm(_cpu(x), list(normalized_shape), _cpu(weight), _cpu(bias), eps)
    return y, mean, rstd


def layer_norm_bwd(dy, x, normalized_shape, mean, rstd, weight, bias, mask=(True, True, True), exact: bool = True):
    """(dx, dgamma, dbeta).  exact: fp32 upcasts; dx rounded once; dgamma/dbeta left in fp32."""
    if exact and x.dtype != torch.float64:
        dx, dg, db = aten.native_layer_norm_backward(_f32(dy), _f32(x), list(normalized_shape), _f32(mean),
                                                     _f32(rstd), _f32(weight), _f32(bias), list(mask))
        return (None if dx is None else dx.to(x.dtype)), dg, db
    return aten.native_layer_norm_backward(_cpu(dy), _cpu(x), list(normalized_shape), _cpu(mean), _cpu(rstd),
                                           _cpu(weight), _cpu(bias), list(mask))


def rms_norm_fwd(x, normalized_shape, weight, eps):
    """(y, rstd) from the CPU composite on fp32 upcasts (aten::_fused_rms_norm has no CPU kernel)."""
    xf = _f32(x) if x.dtype != torch.float64 else _cpu(x)
    wf = None if weight is None else (_f32(weight) if x.dtype != torch.float64 else _cpu(weight))
    acc = xf.dtype
    if eps is None:
        eps = torch.finfo(acc).eps
    y = F.rms_norm(xf, list(normalized_shape), wf, eps)
    dims = tuple(range(xf.dim() - len(normalized_shape), xf.dim()))
    rstd = torch.rsqrt(xf.pow(2).mean(dim=dims, keepdim=True) + eps)
    return y.to(x.dtype), rstd


def rms_norm_bwd(dy, x, normalized_shape, weight, eps):
    """(dx, dweight) by autograd through the CPU composite in fp32/fp64 (no CPU backward kernel exists)."""
    hi = torch.float64 if x.dtype == torch.float64 else torch.float32
    xf = x.detach().cpu().to(hi).requires_grad_(True)
    wf = None if weight is None else weight.detach().cpu().to(hi).requires_grad_(True)
    if eps is None:
        eps = torch.finfo(hi).eps
    y = F.rms_norm(xf, list(normalized_shape), wf, eps)
    grads = torch.autograd.grad(y, [xf] + ([wf] if wf is not None else []), dy.detach().cpu().to(hi))
    dx = grads[0].to(x.dtype)
    dw = grads[1] if wf is not None else None
    return dx, dw


def softmax_fwd(x, dim, is_log: bool, out_dtype=None, exact: bool = True):
    out_dtype = out_dtype or x.dtype
    op = aten._log_softmax if is_log else aten._softmax
    if exact and x.dtype != torch.float64:
        return op(_f32(x), dim, False).to(out_dtype)
    return op(_cpu(x), dim, False).to(out_dtype)


def softmax_bwd(dy, y, dim, is_log: bool, input_dtype, exact: bool = True):
    op = aten._log_softmax_backward_data if is_log else aten._softmax_backward_data
    if exact and dy.dtype != torch.float64:
        return op(_f32(dy), _f32(y), dim, torch.float32).to(input_dtype)
    return op(_cpu(dy), _cpu(y), dim, input_dtype)


def softmax_bwd_fp64(dy, y, dim, is_log: bool, out_dtype):
    """The backward evaluated in float64 on the same inputs, rounded once.  Over rows of tens of thousands of
    elements the fp32 CPU kernel's own row sum carries ~1e-4 of absolute error, which the kernel under test
    does not share; this is the reference to use where that matters."""
    op = aten._log_softmax_backward_data if is_log else aten._softmax_backward_data
    return op(dy.detach().cpu().double(), y.detach().cpu().double(), dim, torch.float64).to(out_dtype)


def nll_fwd(logp, target, weight, reduction: int, ignore_index: int, exact: bool = True):
    """(output, total_weight); exact: fp32 upcast, rounded once."""
    if exact and logp.dtype != torch.float64:
        out, tw = aten.nll_loss_forward(_f32(logp), _cpu(target), _f32(weight), reduction, ignore_index)
        return out.to(logp.dtype), tw.to(logp.dtype)
    return aten.nll_loss_forward(_cpu(logp), _cpu(target), _cpu(weight), reduction, ignore_index)


def nll_bwd(grad_out, logp, target, weight, reduction: int, ignore_index: int, total_weight):
    return aten.nll_loss_backward(_cpu(grad_out), _cpu(logp), _cpu(target), _cpu(weight), reduction, ignore_index,
                                  _cpu(total_weight))


def cross_entropy_bwd(grad_out, logp, target, weight, reduction: int, ignore_index: int, total_weight):
    """nll_loss_backward followed by _log_softmax_backward_data(dim=-1), both on fp32 upcasts (fp64 stays
    fp64), rounded once to logp's dtype: the composition a fused cross-entropy backward must equal."""
    wide = torch.float64 if logp.dtype == torch.float64 else torch.float32
    up = lambda t: None if t is None else t.detach().cpu().to(wide)
    y = up(logp)
    grad = aten.nll_loss_backward(up(grad_out), y, _cpu(target), up(weight), reduction, ignore_index,
                                  up(total_weight))
    return aten._log_softmax_backward_data(grad, y, -1, wide).to(logp.dtype)


# ---------------------------------------------------------------------------------------------------
# float64 evaluations (for strict_ulp_failures: the op on fp64 upcasts of the same 16-bit inputs)
# ---------------------------------------------------------------------------------------------------
def _f64(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    return None if t is None else t.detach().cpu().double()


def layer_norm_fwd64(x, normalized_shape, weight, bias, eps):
    return aten.native_layer_norm(_f64(x), list(normalized_shape), _f64(weight), _f64(bias), eps)


def layer_norm_bwd64(dy, x, normalized_shape, mean, rstd, weight, bias):
    return aten.native_layer_norm_backward(_f64(dy), _f64(x), list(normalized_shape), _f64(mean), _f64(rstd),
                                           _f64(weight), _f64(bias), [True, True, True])


def rms_norm_fwd64(x, normalized_shape, weight, eps):
    return F.rms_norm(_f64(x), list(normalized_shape), _f64(weight), eps)


def rms_norm_bwd64(dy, x, normalized_shape, weight, eps):
    xf = _f64(x).requires_grad_(True)
    wf = _f64(weight).requires_grad_(True)
    y = F.rms_norm(xf, list(normalized_shape), wf, eps)
    return torch.autograd.grad(y, [xf, wf], _f64(dy))


def softmax_fwd64(x, dim, is_log: bool):
    return (aten._log_softmax if is_log else aten._softmax)(_f64(x), dim, False)


def softmax_bwd64(dy, y, dim, is_log: bool):
    op = aten._log_softmax_backward_data if is_log else aten._softmax_backward_data
    return op(_f64(dy), _f64(y), dim, torch.float64)

