"""ctypes front end of oracle/restate.c on CPU torch tensors.  Test infrastructure."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .build import build_restate

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        l = ctypes.CDLL(str(build_restate()))
        vp, i64, i32, f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
        l.ref_norm_fwd.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, f32, i32, i32]
        l.ref_norm_bwd_dx.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i32]
        l.ref_norm_bwd_wgrad.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i32]
        l.ref_softmax_fwd.argtypes = [vp, vp, i64, i64, i64, i32]
        l.ref_softmax_bwd.argtypes = [vp, vp, vp, i64, i64, i64, i32]
        l.ref_nll_fwd.argtypes = [vp, vp, vp, vp, vp, i64, i64, i32, i64]
        l.ref_nll_fwd.restype = i32
        for name in ("ref_norm_fwd", "ref_norm_bwd_dx", "ref_norm_bwd_wgrad", "ref_softmax_fwd", "ref_softmax_bwd"):
            getattr(l, name).restype = None
        _lib = l
    return _lib


def _f(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    return None if t is None else t.detach().cpu().float().contiguous()


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def norm_fwd(x, gamma, beta, eps: float, rms: bool, lanes: int = 1):
    x2 = _f(x).reshape(-1, x.shape[-1])
    M, N = x2.shape
    g, b = _f(gamma), _f(beta)
    y = torch.empty_like(x2)
    mean = torch.zeros(M)
    rstd = torch.empty(M)
    lib().ref_norm_fwd(_p(x2), _p(g), _p(b), _p(y), _p(mean), _p(rstd), M, N, eps, int(rms), lanes)
    return y.reshape(x.shape), mean, rstd


def norm_bwd(dy, x, mean, rstd, gamma, rms: bool):
    x2 = _f(x).reshape(-1, x.shape[-1])
    dy2 = _f(dy).reshape(x2.shape)
    M, N = x2.shape
    g = _f(gamma)
    m = _f(mean).reshape(-1) if mean is not None else None
    r = _f(rstd).reshape(-1)
    dx = torch.empty_like(x2)
    lib().ref_norm_bwd_dx(_p(dy2), _p(x2), _p(m), _p(r), _p(g), _p(dx), M, N, int(rms))
    dgamma = torch.empty(N, dtype=torch.float64)
    dbeta = torch.zeros(N, dtype=torch.float64)
    lib().ref_norm_bwd_wgrad(_p(dy2), _p(x2), _p(m), _p(r), _p(dgamma), _p(dbeta), M, N, int(rms))
    return dx.reshape(x.shape), dgamma, dbeta


def softmax_fwd(x, dim: int, is_log: bool):
    xf = _f(x)
    dim %= max(xf.dim(), 1)
    outer = int(torch.tensor(xf.shape[:dim]).prod()) if dim > 0 else 1
    n = xf.shape[dim] if xf.dim() else 1
    inner = int(torch.tensor(xf.shape[dim + 1:]).prod()) if dim + 1 < xf.dim() else 1
    y = torch.empty_like(xf)
    lib().ref_softmax_fwd(_p(xf), _p(y), outer, n, inner, int(is_log))
    return y


def softmax_bwd(dy, y, dim: int, is_log: bool):
    dyf, yf = _f(dy), _f(y)
    dim %= max(yf.dim(), 1)
    outer = int(torch.tensor(yf.shape[:dim]).prod()) if dim > 0 else 1
    n = yf.shape[dim] if yf.dim() else 1
    inner = int(torch.tensor(yf.shape[dim + 1:]).prod()) if dim + 1 < yf.dim() else 1
    dx = torch.empty_like(yf)
    lib().ref_softmax_bwd(_p(dyf), _p(yf), _p(dx), outer, n, inner, int(is_log))
    return dx


def nll_fwd(logp, target, weight, mean: bool, ignore_index: int):
    lf, w = _f(logp), _f(weight)
    t = target.detach().cpu().to(torch.int64).contiguous()
    out = torch.empty(1)
    tw = torch.empty(1)
    rc = lib().ref_nll_fwd(_p(lf), _p(t), _p(w), _p(out), _p(tw), lf.shape[0], lf.shape[1], int(mean), ignore_index)
    if rc != 0:
        raise ValueError("target out of range")
    return out[0], tw[0]
