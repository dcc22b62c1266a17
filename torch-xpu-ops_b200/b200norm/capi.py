"""ctypes wrappers over the C ABI, with the reference's operator names and argument meaning.

Each function mirrors the ATen operator that intel/torch-xpu-ops implements for this path
(src/ATen/native/xpu/LayerNorm.cpp, SoftMax.cpp, LossNLL.cpp): same arguments, same outputs, same
error behaviour for bad shapes.  torch is used for device memory and streams only — every result
is produced by a kernel of libb200norm.so, called with raw pointers and sizes.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch

from . import (BF16, F16, F32, F64, OK, REDUCE_MEAN, REDUCE_NONE, REDUCE_SUM, B200NormError,
               load_library)

_DTYPES = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16, torch.float64: F64}


def _dt(t: torch.dtype) -> int:
    try:
        return _DTYPES[t]
    except KeyError:
        raise TypeError(f"b200norm: unsupported dtype {t}") from None


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream(t: torch.Tensor):
    return torch.cuda.current_stream(t.device).cuda_stream


def _check(status: int, what: str) -> None:
    if status != OK:
        raise B200NormError(status, what)


def _require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("b200norm: expected CUDA tensors (there is no CPU path)")


def _norm_dims(x: torch.Tensor, normalized_shape: Sequence[int], weight, bias) -> Tuple[int, int]:
    """M, N with the checks of at::native::_check_layer_norm_inputs."""
    ns = tuple(int(s) for s in normalized_shape)
    if len(ns) < 1:
        raise RuntimeError("Expected normalized_shape to be at least 1-dimensional")
    for name, w in (("weight", weight), ("bias", bias)):
        if w is not None and tuple(w.shape) != ns:
            raise RuntimeError(f"Expected {name} to be of same shape as normalized_shape, but got {name} of shape "
                               f"{tuple(w.shape)} and normalized_shape = {ns}")
    if x.dim() < len(ns) or tuple(x.shape[x.dim() - len(ns):]) != ns:
        raise RuntimeError(f"Given normalized_shape={list(ns)}, expected input with shape [*, "
                           f"{', '.join(map(str, ns))}], but got input of size {list(x.shape)}")
    n = math.prod(ns)
    m = math.prod(x.shape[: x.dim() - len(ns)])
    return m, n


def _stat_shape(x: torch.Tensor, normalized_ndim: int):
    axis = x.dim() - normalized_ndim
    return list(x.shape[:axis]) + [1] * normalized_ndim


def _acc_dtype(t: torch.dtype) -> torch.dtype:
    return torch.float64 if t == torch.float64 else torch.float32


def _weight_dtype(x, weight, bias) -> int:
    w = weight if weight is not None else bias
    if w is None:
        return _dt(x.dtype)
    if weight is not None and bias is not None and weight.dtype != bias.dtype:
        raise RuntimeError("weight and bias must have the same dtype")
    if w.dtype != x.dtype and w.dtype != torch.float32:
        raise RuntimeError(f"weight dtype must equal the input dtype or be float32, got {w.dtype} for {x.dtype}")
    return _dt(w.dtype)


def set_path(path: int) -> int:
    """Force a kernel family (b200norm.PATH_*) for this thread; returns the previous setting."""
    return load_library().b2n_set_path(path)


def set_tuning(knob: int, value: int) -> None:
    """Override a ring-kernel launch parameter for this thread (b200norm.TUNE_*; 0 = automatic)."""
    _check(load_library().b2n_set_tuning(knob, value), "b2n_set_tuning")


def last_path() -> str:
    return load_library().b2n_last_path().decode()


def device_status(device=None) -> int:
    """Read-and-clear the device status word (synchronises the current stream)."""
    with torch.cuda.device(device):
        return load_library().b2n_device_status(torch.cuda.current_stream().cuda_stream)


def launch_count() -> int:
    """Kernels launched through the library by this thread so far."""
    return int(load_library().b2n_launch_count())


def profile_begin() -> None:
    """Start bracketing every main kernel launch of this thread with CUDA events."""
    _check(load_library().b2n_profile_begin(), "b2n_profile_begin")


def profile_end() -> dict:
    """Stop, synchronise, and return {kernel name: (launches, total milliseconds)}."""
    import ctypes
    buf = ctypes.create_string_buffer(8192)
    _check(load_library().b2n_profile_end(buf, len(buf)), "b2n_profile_end")
    out = {}
    for line in buf.value.decode().splitlines():
        name, n, ms = line.split()
        out[name] = (int(n), float(ms))
    return out


def check_status(device=None) -> None:
    """Raise if a kernel on `device` has recorded a failure (an nll_loss target out of range, a bounded wait that
    gave up).  Synchronises the current stream; the ATen overrides do the same check without blocking, one call late."""
    st = device_status(device)
    if st != OK:
        raise B200NormError(st, "device status")


class Prepared:
    """One C-ABI call with every argument converted once: calling the object enqueues the kernels again on the
    stream that was current when it was prepared.  For loops that launch the same operator on the same buffers
    many times (a training step replayed, a benchmark), where the per-call argument checks of the operator
    wrappers above would cost more host time than the kernels take on the device."""
    __slots__ = ("fn", "args", "name", "keep")

    def __init__(self, fn, args, name, keep):
        self.fn, self.args, self.name, self.keep = fn, args, name, keep  # keep: the tensors whose pointers are baked in

    def __call__(self):
        rc = self.fn(*self.args)
        if rc != OK:
            raise B200NormError(rc, self.name)


def prepare_layer_norm(x, gamma, beta, eps, y, mean, rstd) -> Prepared:
    """native_layer_norm on preallocated contiguous tensors, as a Prepared call."""
    _require_cuda(x, gamma, beta, y, mean, rstd)
    lib = load_library()
    M, N = _norm_dims(x, (x.shape[-1],), gamma, beta)
    assert x.is_contiguous() and y.is_contiguous() and mean.numel() == M and rstd.numel() == M
    args = (_ptr(x), _ptr(gamma), _ptr(beta), _ptr(y), _ptr(mean), _ptr(rstd), M, N, float(eps), _dt(x.dtype),
            _weight_dtype(x, gamma, beta), _stream(x))
    return Prepared(lib.b2n_layer_norm_fwd, args, "b2n_layer_norm_fwd", (x, gamma, beta, y, mean, rstd))


def prepare_layer_norm_backward(dy, x, mean, rstd, gamma, dx, dgamma, dbeta, workspace) -> Prepared:
    """native_layer_norm_backward on preallocated contiguous tensors, as a Prepared call."""
    _require_cuda(dy, x, mean, rstd, gamma, dx, dgamma, dbeta, workspace)
    lib = load_library()
    M, N = _norm_dims(x, (x.shape[-1],), gamma, None)
    assert x.is_contiguous() and dy.is_contiguous() and (dx is None or dx.is_contiguous())
    xdt, wdt = _dt(x.dtype), _weight_dtype(x, gamma, None)
    nbytes = lib.b2n_norm_bwd_workspace_bytes(M, N, xdt, wdt, int(dgamma is not None or dbeta is not None))
    if nbytes and (workspace is None or workspace.numel() < nbytes):
        raise ValueError(f"workspace too small: need {nbytes} bytes")
    args = (_ptr(dy), _ptr(x), _ptr(mean), _ptr(rstd), _ptr(gamma), _ptr(dx), _ptr(dgamma), _ptr(dbeta),
            _ptr(workspace) if nbytes else None, nbytes, M, N, xdt, wdt, _stream(x))
    return Prepared(lib.b2n_layer_norm_bwd, args, "b2n_layer_norm_bwd", (dy, x, mean, rstd, gamma, dx, dgamma, dbeta, workspace))


def prepare_rms_norm(x, weight, eps, y, rstd) -> Prepared:
    _require_cuda(x, weight, y, rstd)
    lib = load_library()
    M, N = _norm_dims(x, (x.shape[-1],), weight, weight)
    assert x.is_contiguous() and y.is_contiguous() and rstd.numel() == M
    args = (_ptr(x), _ptr(weight), _ptr(y), _ptr(rstd), M, N, float(eps), _dt(x.dtype), _weight_dtype(x, weight, None),
            _stream(x))
    return Prepared(lib.b2n_rms_norm_fwd, args, "b2n_rms_norm_fwd", (x, weight, y, rstd))


def prepare_rms_norm_backward(dy, x, rstd, weight, dx, dweight, workspace) -> Prepared:
    _require_cuda(dy, x, rstd, weight, dx, dweight, workspace)
    lib = load_library()
    M, N = _norm_dims(x, (x.shape[-1],), weight, weight)
    assert x.is_contiguous() and dy.is_contiguous() and (dx is None or dx.is_contiguous())
    xdt, wdt = _dt(x.dtype), _weight_dtype(x, weight, None)
    nbytes = lib.b2n_norm_bwd_workspace_bytes(M, N, xdt, wdt, int(dweight is not None))
    if nbytes and (workspace is None or workspace.numel() < nbytes):
        raise ValueError(f"workspace too small: need {nbytes} bytes")
    args = (_ptr(dy), _ptr(x), _ptr(rstd), _ptr(weight), _ptr(dx), _ptr(dweight), _ptr(workspace) if nbytes else None,
            nbytes, M, N, xdt, wdt, _stream(x))
    return Prepared(lib.b2n_rms_norm_bwd, args, "b2n_rms_norm_bwd", (dy, x, rstd, weight, dx, dweight, workspace))


def prepare_norm_backward_partials(rms: bool, dy, x, mean, rstd, gamma, dx, workspace):
    """The backward's row kernels only (b2n_norm_bwd_partials) as a Prepared call: dx is written, the weight-gradient
    partial sums stay in `workspace`.  Returns (call, partial_rows): the number of partial rows depends only on the
    shape and the SM margin in force now, so it is taken from one run of the call made here."""
    import ctypes
    _require_cuda(dy, x, mean, rstd, gamma, dx, workspace)
    lib = load_library()
    M, N = _norm_dims(x, (x.shape[-1],), gamma, None)
    assert x.is_contiguous() and dy.is_contiguous() and dx.is_contiguous()
    xdt, wdt = _dt(x.dtype), _weight_dtype(x, gamma, None)
    nbytes = lib.b2n_norm_bwd_workspace_bytes(M, N, xdt, wdt, 1)
    if workspace is None or workspace.numel() < nbytes:
        raise ValueError(f"workspace too small: need {nbytes} bytes")
    rows = ctypes.c_int64(0)
    args = (int(bool(rms)), _ptr(dy), _ptr(x), _ptr(mean), _ptr(rstd), _ptr(gamma), _ptr(dx), _ptr(workspace), nbytes,
            M, N, xdt, wdt, ctypes.byref(rows), _stream(x))
    call = Prepared(lib.b2n_norm_bwd_partials, args, "b2n_norm_bwd_partials", (dy, x, mean, rstd, gamma, dx, workspace, rows))
    call()
    return call, int(rows.value)


def prepare_wgrad_fold(workspace, partial_rows: int, x_dtype, dgamma, dbeta) -> Prepared:
    """b2n_norm_wgrad_fold as a Prepared call on the CURRENT stream (typically a second stream, behind an event
    recorded after the row kernels)."""
    _require_cuda(workspace, dgamma, dbeta)
    lib = load_library()
    w = dgamma if dgamma is not None else dbeta
    args = (_ptr(workspace), int(partial_rows), int(w.numel()), _ptr(dgamma), _ptr(dbeta), _dt(x_dtype), _dt(w.dtype),
            _stream(w))
    return Prepared(lib.b2n_norm_wgrad_fold, args, "b2n_norm_wgrad_fold", (workspace, dgamma, dbeta))


def native_layer_norm_backward_partials(grad_out, input, normalized_shape, mean, rstd, weight=None, workspace=None,
                                        out=None, rms: bool = False):
    """The row kernels of native_layer_norm_backward (or, with rms=True, of _fused_rms_norm_backward): returns
    (dX, workspace, partial_rows); norm_wgrad_fold(workspace, partial_rows, ...) completes dgamma / dbeta."""
    import ctypes
    _require_cuda(grad_out, input, mean, rstd, weight)
    lib = load_library()
    M, N = _norm_dims(input, normalized_shape, weight, None)
    x, dy = input.contiguous(), grad_out.contiguous()
    acc = _acc_dtype(x.dtype)
    mean_c = None if rms else mean.to(acc).contiguous().view(-1)
    rstd_c = rstd.to(acc).contiguous().view(-1)
    g = weight.contiguous() if weight is not None else None
    dx = out if out is not None else torch.empty_like(x)
    xdt, wdt = _dt(x.dtype), _weight_dtype(x, weight, None)
    rows = ctypes.c_int64(0)
    with torch.cuda.device(x.device):
        nbytes = lib.b2n_norm_bwd_workspace_bytes(M, N, xdt, wdt, 1)
        ws = workspace if workspace is not None else torch.empty(max(nbytes, 1), dtype=torch.uint8, device=x.device)
        if ws.numel() < nbytes:
            raise ValueError(f"workspace too small: {ws.numel()} < {nbytes}")
        _check(lib.b2n_norm_bwd_partials(int(bool(rms)), _ptr(dy), _ptr(x), _ptr(mean_c), _ptr(rstd_c), _ptr(g), _ptr(dx),
                                         _ptr(ws), nbytes, M, N, xdt, wdt, ctypes.byref(rows), _stream(x)),
               "b2n_norm_bwd_partials")
    return dx, ws, int(rows.value)


def norm_wgrad_fold(workspace, partial_rows: int, x_dtype, dgamma=None, dbeta=None):
    """Folds the partial sums left by native_layer_norm_backward_partials into dgamma / dbeta (current stream)."""
    w = dgamma if dgamma is not None else dbeta
    if w is None:
        return
    with torch.cuda.device(w.device):
        _check(load_library().b2n_norm_wgrad_fold(_ptr(workspace), int(partial_rows), int(w.numel()), _ptr(dgamma),
                                                  _ptr(dbeta), _dt(x_dtype), _dt(w.dtype), _stream(w)),
               "b2n_norm_wgrad_fold")


# ---- layer norm / RMS norm -------------------------------------------------------------------------
def native_layer_norm(input, normalized_shape, weight=None, bias=None, eps=1e-5, out=None):
    """aten::native_layer_norm -> (Y, mean, rstd); mean/rstd in the accumulate dtype.

    out: optional preallocated (Y, mean[M], rstd[M]) to write into (no allocation on the call path).
    """
    _require_cuda(input, weight, bias)
    lib = load_library()
    M, N = _norm_dims(input, normalized_shape, weight, bias)
    x = input.contiguous()
    g = weight.contiguous() if weight is not None else None
    b = bias.contiguous() if bias is not None else None
    acc = _acc_dtype(x.dtype)
    if out is not None:
        y, mean, rstd = out
        mean, rstd = mean.view(-1), rstd.view(-1)
    else:
        y = torch.empty_like(x, memory_format=torch.contiguous_format)
        mean = torch.empty(M, dtype=acc, device=x.device)
        rstd = torch.empty(M, dtype=acc, device=x.device)
    if M > 0:
        with torch.cuda.device(x.device):
            _check(lib.b2n_layer_norm_fwd(_ptr(x), _ptr(g), _ptr(b), _ptr(y), _ptr(mean), _ptr(rstd), M, N,
                                          float(eps), _dt(x.dtype), _weight_dtype(x, g, b), _stream(x)),
                   "b2n_layer_norm_fwd")
    shape = _stat_shape(input, len(normalized_shape))
    return y, mean.view(shape), rstd.view(shape)


def native_layer_norm_backward(grad_out, input, normalized_shape, mean, rstd, weight=None, bias=None,
                               output_mask=(True, True, True), out=None, workspace=None):
    """aten::native_layer_norm_backward -> (dX?, dgamma?, dbeta?); masked-off outputs are None.

    out: optional preallocated (dX, dgamma, dbeta) (entries may be None to allocate);
    workspace: optional preallocated uint8 scratch of b2n_norm_bwd_workspace_bytes(...) bytes.
    """
    _require_cuda(grad_out, input, mean, rstd, weight, bias)
    lib = load_library()
    M, N = _norm_dims(input, normalized_shape, weight, bias)
    x = input.contiguous()
    dy = grad_out.contiguous()
    if dy.dtype != x.dtype:
        raise RuntimeError(f"grad_out dtype {dy.dtype} does not match input dtype {x.dtype}")
    g = weight.contiguous() if weight is not None else None
    acc = _acc_dtype(x.dtype)
    mean_c = mean.to(acc).contiguous().view(-1)
    rstd_c = rstd.to(acc).contiguous().view(-1)
    o_dx, o_dg, o_db = out if out is not None else (None, None, None)
    mk = (torch.empty_like if M > 0 else torch.zeros_like)
    dx = (o_dx if o_dx is not None else torch.empty_like(x)) if output_mask[0] else None
    dgamma = ((o_dg if o_dg is not None else mk(weight.contiguous()))
              if (output_mask[1] and weight is not None) else None)
    dbeta = ((o_db if o_db is not None else mk(bias.contiguous()))
             if (output_mask[2] and bias is not None) else None)
    if M > 0 and N > 0:
        xdt, wdt = _dt(x.dtype), _weight_dtype(x, weight, bias)
        want_w = dgamma is not None or dbeta is not None
        with torch.cuda.device(x.device):
            nbytes = lib.b2n_norm_bwd_workspace_bytes(M, N, xdt, wdt, int(want_w))
            ws = workspace if workspace is not None else torch.empty(max(nbytes, 1), dtype=torch.uint8, device=x.device)
            if ws.numel() < nbytes:
                raise ValueError(f"workspace too small: {ws.numel()} < {nbytes}")
            _check(lib.b2n_layer_norm_bwd(_ptr(dy), _ptr(x), _ptr(mean_c), _ptr(rstd_c), _ptr(g), _ptr(dx),
                                          _ptr(dgamma), _ptr(dbeta), _ptr(ws) if nbytes else None, nbytes, M, N,
                                          xdt, wdt, _stream(x)),
                   "b2n_layer_norm_bwd")
    return dx, dgamma, dbeta


def _fused_rms_norm(input, normalized_shape, weight=None, eps=None, out=None):
    """aten::_fused_rms_norm -> (Y, rstd).  eps=None means the accumulate type's machine epsilon.

    out: optional preallocated (Y, rstd[M]).
    """
    _require_cuda(input, weight)
    lib = load_library()
    M, N = _norm_dims(input, normalized_shape, weight, weight)
    x = input.contiguous()
    g = weight.contiguous() if weight is not None else None
    acc = _acc_dtype(x.dtype)
    if eps is None:
        eps = torch.finfo(acc).eps
    if out is not None:
        y, rstd = out
        rstd = rstd.view(-1)
    else:
        y = torch.empty_like(x, memory_format=torch.contiguous_format)
        rstd = torch.empty(M, dtype=acc, device=x.device)
    if M > 0:
        with torch.cuda.device(x.device):
            _check(lib.b2n_rms_norm_fwd(_ptr(x), _ptr(g), _ptr(y), _ptr(rstd), M, N, float(eps), _dt(x.dtype),
                                        _weight_dtype(x, g, None), _stream(x)),
                   "b2n_rms_norm_fwd")
    return y, rstd.view(_stat_shape(input, len(normalized_shape)))


def _fused_rms_norm_backward(grad_out, input, normalized_shape, rstd, weight=None, output_mask=(True, True),
                             out=None, workspace=None):
    """aten::_fused_rms_norm_backward -> (dX?, dW?).  out / workspace: optional preallocated buffers."""
    _require_cuda(grad_out, input, rstd, weight)
    lib = load_library()
    M, N = _norm_dims(input, normalized_shape, weight, weight)
    x = input.contiguous()
    dy = grad_out.contiguous()
    if dy.dtype != x.dtype:
        raise RuntimeError(f"grad_out dtype {dy.dtype} does not match input dtype {x.dtype}")
    g = weight.contiguous() if weight is not None else None
    rstd_c = rstd.to(_acc_dtype(x.dtype)).contiguous().view(-1)
    o_dx, o_dg = out if out is not None else (None, None)
    mk = (torch.empty_like if M > 0 else torch.zeros_like)
    dx = (o_dx if o_dx is not None else torch.empty_like(x)) if output_mask[0] else None
    dgamma = (o_dg if o_dg is not None else mk(g)) if (output_mask[1] and g is not None) else None
    if M > 0 and N > 0:
        xdt, wdt = _dt(x.dtype), _weight_dtype(x, weight, None)
        with torch.cuda.device(x.device):
            nbytes = lib.b2n_norm_bwd_workspace_bytes(M, N, xdt, wdt, int(dgamma is not None))
            ws = workspace if workspace is not None else torch.empty(max(nbytes, 1), dtype=torch.uint8, device=x.device)
            if ws.numel() < nbytes:
                raise ValueError(f"workspace too small: {ws.numel()} < {nbytes}")
            _check(lib.b2n_rms_norm_bwd(_ptr(dy), _ptr(x), _ptr(rstd_c), _ptr(g), _ptr(dx), _ptr(dgamma),
                                        _ptr(ws) if nbytes else None, nbytes, M, N, xdt, wdt, _stream(x)),
                   "b2n_rms_norm_bwd")
    return dx, dgamma


# ---- sibling norms: group norm forward, batch norm statistics -------------------------------------------
def native_group_norm(input, weight, bias, N, C, HxW, group, eps, out=None):
    """aten::native_group_norm -> (Y, mean[N, group], rstd[N, group]); the statistics take the weights' dtype when the
    input is 16-bit and the weights are float32 (upstream's mixed-type rule), else the input's.
    out: optional preallocated (Y, mean, rstd)."""
    _require_cuda(input, weight, bias)
    lib = load_library()
    if input.numel() != N * C * HxW:
        raise RuntimeError(f"Expected input of {N}*{C}*{HxW} elements, got {list(input.shape)}")
    if group < 1 or C % group != 0:
        raise RuntimeError(f"Expected number of channels in input to be divisible by num_groups, but got input of "
                           f"shape {list(input.shape)} and num_groups={group}")
    for name, w in (("weight", weight), ("bias", bias)):
        if w is not None and (w.dim() != 1 or w.numel() != C):
            raise RuntimeError(f"Expected {name} to be a vector of size equal to the number of channels in input, but got "
                               f"{name} of shape {list(w.shape)} and input of shape {list(input.shape)}")
    x = input.contiguous()
    g = weight.contiguous() if weight is not None else None
    b = bias.contiguous() if bias is not None else None
    wdt = _weight_dtype(x, g, b)
    stat = torch.float32 if (wdt == F32 and (g is not None or b is not None)) else x.dtype
    if out is not None:
        y, mean, rstd = out
        if mean.dtype != stat or rstd.dtype != stat or y.dtype != x.dtype:
            raise RuntimeError("native_group_norm: out tensors have the wrong dtype")
    else:
        y = torch.empty_like(x)
        mean = torch.empty((N, group), dtype=stat, device=x.device)
        rstd = torch.empty((N, group), dtype=stat, device=x.device)
    if x.numel() > 0:
        with torch.cuda.device(x.device):
            _check(lib.b2n_group_norm_fwd(_ptr(x), _ptr(g), _ptr(b), _ptr(y), _ptr(mean), _ptr(rstd), N, C, HxW, group,
                                          float(eps), _dt(x.dtype), wdt, _dt(stat), _stream(x)), "b2n_group_norm_fwd")
    return y, mean, rstd


def native_group_norm_backward(grad_out, input, mean, rstd, weight, N, C, HxW, group, output_mask=(True, True, True)):
    """aten::native_group_norm_backward -> (dX?, dgamma?, dbeta?); masked-off outputs are None, and so are dgamma /
    dbeta when there is no weight (upstream sizes them after it).  mean / rstd: the forward's saved statistics."""
    _require_cuda(grad_out, input, mean, rstd, weight)
    lib = load_library()
    if input.numel() != N * C * HxW or grad_out.numel() != input.numel():
        raise RuntimeError(f"Expected input and grad_out of {N}*{C}*{HxW} elements, got {list(input.shape)} and "
                           f"{list(grad_out.shape)}")
    if group < 1 or C % group != 0:
        raise RuntimeError(f"Expected number of channels in input to be divisible by num_groups, but got input of "
                           f"shape {list(input.shape)} and num_groups={group}")
    if mean.numel() != N * group or rstd.numel() != N * group or mean.dtype != rstd.dtype:
        raise RuntimeError("native_group_norm_backward: mean and rstd must be [N, group] tensors of one dtype")
    if weight is not None and (weight.dim() != 1 or weight.numel() != C):
        raise RuntimeError(f"Expected weight to be a vector of size equal to the number of channels in input, but got "
                           f"weight of shape {list(weight.shape)} and input of shape {list(input.shape)}")
    x = input.contiguous()
    dy = grad_out.to(x.dtype).contiguous()
    g = weight.contiguous() if weight is not None else None
    wdt = _weight_dtype(x, g, None)
    m, r = mean.contiguous(), rstd.contiguous()
    dx = torch.empty_like(x) if output_mask[0] else None
    dgamma = torch.empty_like(g) if (output_mask[1] and g is not None) else None
    dbeta = torch.empty_like(g) if (output_mask[2] and g is not None) else None
    if C > 0 and (x.numel() > 0 or dgamma is not None or dbeta is not None):
        if x.numel() == 0:  # sums over nothing
            for t in (dgamma, dbeta):
                if t is not None:
                    t.zero_()
        else:
            with torch.cuda.device(x.device):
                nbytes = int(lib.b2n_group_norm_bwd_workspace_bytes(N, C, HxW, _dt(x.dtype))) if (dgamma is not None or
                                                                                                 dbeta is not None) else 0
                ws = torch.empty(nbytes, dtype=torch.uint8, device=x.device) if nbytes else None
                _check(lib.b2n_group_norm_bwd_ws(_ptr(dy), _ptr(x), _ptr(m), _ptr(r), _ptr(g), _ptr(dx), _ptr(dgamma),
                                                 _ptr(dbeta), N, C, HxW, group, _dt(x.dtype), wdt, _dt(m.dtype),
                                                 _ptr(ws) if ws is not None else None, nbytes, _stream(x)),
                       "b2n_group_norm_bwd_ws")
    return dx, dgamma, dbeta


def _bn_dims(input):
    if input.dim() < 2:
        raise RuntimeError("batch norm statistics need an input with at least two dimensions [N, C, ...]")
    return input.shape[0], input.shape[1], math.prod(input.shape[2:])


def batch_norm_stats(input, eps):
    """aten::batch_norm_stats -> (mean[C], invstd[C]) in float32, over every dimension but the channel."""
    _require_cuda(input)
    lib = load_library()
    N, C, HxW = _bn_dims(input)
    x = input.contiguous()
    mean = torch.empty(C, dtype=torch.float32, device=x.device)
    invstd = torch.empty(C, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        ws, nbytes = _bn_workspace(lib, x, N, C, HxW)
        _check(lib.b2n_batch_norm_stats_ws(_ptr(x), _ptr(mean), _ptr(invstd), None, None, N, C, HxW, float(eps), 0.0, 0,
                                           _dt(x.dtype), F32, _ptr(ws) if ws is not None else None, nbytes, _stream(x)),
               "b2n_batch_norm_stats_ws")
    return mean, invstd


def _bn_workspace(lib, x, N, C, HxW):
    """The scratch b2n_batch_norm_stats_ws asks for (None, 0 when the shape needs none)."""
    nbytes = int(lib.b2n_batch_norm_stats_workspace_bytes(N, C, HxW, _dt(x.dtype)))
    if nbytes == 0:
        return None, 0
    return torch.empty(nbytes, dtype=torch.uint8, device=x.device), nbytes


def batch_norm_update_stats(input, running_mean, running_var, momentum):
    """aten::batch_norm_update_stats -> (mean[C], biased var[C]) in float32; running_mean / running_var (either may be
    None) are blended in place, the variance unbiased."""
    _require_cuda(input, running_mean, running_var)
    lib = load_library()
    N, C, HxW = _bn_dims(input)
    x = input.contiguous()
    r = running_mean if running_mean is not None else running_var
    if running_mean is not None and running_var is not None and running_mean.dtype != running_var.dtype:
        raise RuntimeError("running_mean and running_var must have the same dtype")
    for t in (running_mean, running_var):
        if t is not None and not t.is_contiguous():
            raise RuntimeError("running statistics must be contiguous (they are updated in place)")
    mean = torch.empty(C, dtype=torch.float32, device=x.device)
    var = torch.empty(C, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        ws, nbytes = _bn_workspace(lib, x, N, C, HxW)
        _check(lib.b2n_batch_norm_stats_ws(_ptr(x), _ptr(mean), _ptr(var), _ptr(running_mean), _ptr(running_var), N, C, HxW,
                                           0.0, float(momentum), 1, _dt(x.dtype), _dt(r.dtype) if r is not None else F32,
                                           _ptr(ws) if ws is not None else None, nbytes, _stream(x)),
               "b2n_batch_norm_stats_ws")
    return mean, var


# ---- softmax family ----------------------------------------------------------------------------------
def _softmax_dims(t: torch.Tensor, dim: int):
    if t.dim() == 0:
        if dim not in (0, -1):
            raise IndexError(f"Dimension out of range (expected to be in range of [-1, 0], but got {dim})")
        return 1, 1, 1
    if not -t.dim() <= dim < t.dim():
        raise IndexError(f"Dimension out of range (expected to be in range of [{-t.dim()}, {t.dim() - 1}], "
                         f"but got {dim})")
    dim %= t.dim()
    return math.prod(t.shape[:dim]), t.shape[dim], math.prod(t.shape[dim + 1:])


def _softmax_fwd(input, dim, half_to_float, is_log, name, out=None):
    _require_cuda(input)
    lib = load_library()
    if half_to_float and input.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("conversion is supported for Half and BFloat16 type only")
    outer, n, inner = _softmax_dims(input, dim)
    x = input.contiguous()
    y = out if out is not None else torch.empty_like(x, dtype=torch.float32 if half_to_float else x.dtype)
    if x.numel() > 0:
        with torch.cuda.device(x.device):
            _check(lib.b2n_softmax_fwd(_ptr(x), _ptr(y), outer, n, inner, _dt(x.dtype), _dt(y.dtype), int(is_log),
                                       _stream(x)), name)
    return y


def _softmax(input, dim, half_to_float=False, out=None):
    """aten::_softmax (out: optional preallocated contiguous result)"""
    return _softmax_fwd(input, dim, half_to_float, False, "b2n_softmax_fwd", out)


def _safe_softmax(input, dim, dtype=None, out=None):
    """aten::_safe_softmax: softmax in which a row of all -inf gives zeros instead of NaN."""
    if input.dtype in (torch.float16, torch.bfloat16) and dtype == torch.float32:
        return _softmax_fwd(input, dim, True, 2, "b2n_softmax_fwd(safe)", out)
    x = input.to(dtype) if dtype is not None else input
    return _softmax_fwd(x, dim, False, 2, "b2n_softmax_fwd(safe)", out)


def _log_softmax(input, dim, half_to_float=False, out=None):
    """aten::_log_softmax (out: optional preallocated contiguous result)"""
    return _softmax_fwd(input, dim, half_to_float, True, "b2n_softmax_fwd(log)", out)


def _softmax_bwd(grad_output, output, dim, input_dtype, is_log, name, out=None):
    _require_cuda(grad_output, output)
    lib = load_library()
    if grad_output.dtype != input_dtype and not (
            grad_output.dtype == torch.float32 and input_dtype in (torch.float16, torch.bfloat16)):
        raise RuntimeError("expected input and grad types to match, or input to be at::Half and grad to be at::Float")
    if grad_output.shape != output.shape:
        raise RuntimeError("grad_output and output sizes differ")
    outer, n, inner = _softmax_dims(grad_output, dim)
    g = grad_output.contiguous()
    y = output.to(g.dtype).contiguous()
    dx = out if out is not None else torch.empty_like(g, dtype=input_dtype)
    if g.numel() > 0:
        with torch.cuda.device(g.device):
            _check(lib.b2n_softmax_bwd(_ptr(g), _ptr(y), _ptr(dx), outer, n, inner, _dt(g.dtype), _dt(dx.dtype),
                                       int(is_log), _stream(g)), name)
    return dx


def _softmax_backward_data(grad_output, output, dim, input_dtype, out=None):
    """aten::_softmax_backward_data"""
    return _softmax_bwd(grad_output, output, dim, input_dtype, False, "b2n_softmax_bwd", out)


def _log_softmax_backward_data(grad_output, output, dim, input_dtype, out=None):
    """aten::_log_softmax_backward_data"""
    return _softmax_bwd(grad_output, output, dim, input_dtype, True, "b2n_softmax_bwd(log)", out)


# ---- masked softmax ----------------------------------------------------------------------------------------
def _masked_layout(input, mask, mask_type):
    """(row_div, row_mod) of b2n_masked_softmax_fwd for the three layouts masked_softmax_kernel accepts."""
    if mask.dtype != torch.bool:
        raise RuntimeError("Mask should be a boolean tensor")
    if mask_type is None:
        raise RuntimeError("Mask Type should be defined")
    if mask_type not in (0, 1, 2):
        raise RuntimeError("Mask Type should be 0 (src_mask), 1 (src_key_padding_mask), or 2 (default_mask)")
    rows = input.numel() // max(input.shape[-1], 1) if input.dim() > 0 else 1
    if mask.shape == input.shape:
        return 1, max(rows, 1)
    if (mask_type == 1 and input.dim() == 4 and mask.dim() == 2 and input.shape[0] == mask.shape[0]
            and input.shape[2] == mask.shape[1] and input.shape[3] == mask.shape[1]):
        return input.shape[1] * input.shape[2], input.shape[0]
    if (mask_type == 0 and input.dim() == 4 and mask.dim() == 2 and input.shape[3] == mask.shape[1]
            and input.shape[2] == mask.shape[0] and mask.shape[0] == mask.shape[1]):
        return 1, mask.shape[0]
    raise RuntimeError(f"Mask shape should match input. mask: {list(mask.shape)} input: {list(input.shape)}")


def _masked_softmax(input, mask, dim=None, mask_type=None, out=None):
    """aten::_masked_softmax: softmax with the elements where `mask` is True left out (they give 0)."""
    _require_cuda(input, mask)
    lib = load_library()
    row_div, row_mod = _masked_layout(input, mask, mask_type)
    x = input.reshape(1) if input.dim() == 0 else input
    d = x.dim() - 1 if dim is None else dim % x.dim()
    if d != x.dim() - 1:
        # other dims: the mask applied up front, then the plain kernels (masked elements come out as exp(-inf) = 0)
        full = mask if mask.shape == input.shape else (
            mask.view(mask.shape[0], 1, 1, mask.shape[1]) if mask_type == 1 else mask).expand_as(x)
        return _softmax(x.masked_fill(full, float("-inf")), d, False, out=out).reshape(input.shape)
    xc = x.contiguous()
    m = mask.contiguous()
    y = out if out is not None else torch.empty_like(xc)
    n = xc.shape[-1]
    rows = xc.numel() // n if n > 0 else 0
    if xc.numel() > 0:
        with torch.cuda.device(xc.device):
            _check(lib.b2n_masked_softmax_fwd(_ptr(xc), _ptr(m), _ptr(y), rows, n, row_div, row_mod, _dt(xc.dtype),
                                              _stream(xc)), "b2n_masked_softmax_fwd")
    return y.reshape(input.shape)


def _masked_softmax_backward(grad_output, output, mask, dim=None, out=None):
    """aten::_masked_softmax_backward (mask of grad_output's shape)."""
    _require_cuda(grad_output, output, mask)
    lib = load_library()
    if mask.dtype != torch.bool:
        raise RuntimeError("Mask should be a boolean tensor")
    if grad_output.shape != mask.shape:
        raise RuntimeError("Mask shape should match grad shape")
    g = grad_output.reshape(1) if grad_output.dim() == 0 else grad_output
    d = g.dim() - 1 if dim is None else dim % g.dim()
    if d != g.dim() - 1:
        m = mask.reshape(g.shape)
        gi = _softmax_backward_data(g.masked_fill(m, 0), output.reshape(g.shape).masked_fill(m, 0), d, g.dtype)
        return gi.masked_fill(m, 0).reshape(grad_output.shape)
    gc, yc, mc = g.contiguous(), output.reshape(g.shape).contiguous(), mask.reshape(g.shape).contiguous()
    dx = out if out is not None else torch.empty_like(gc)
    n = gc.shape[-1]
    rows = gc.numel() // n if n > 0 else 0
    if gc.numel() > 0:
        with torch.cuda.device(gc.device):
            _check(lib.b2n_masked_softmax_bwd(_ptr(gc), _ptr(yc), _ptr(mc), _ptr(dx), rows, n, _dt(gc.dtype),
                                              _stream(gc)), "b2n_masked_softmax_bwd")
    return dx.reshape(grad_output.shape)


# ---- nll_loss --------------------------------------------------------------------------------------------
def _nll_check(self, target, weight):
    if not 0 < self.dim() <= 2:
        raise RuntimeError("input tensor should be 1D or 2D")
    if target.dim() > 1:
        raise RuntimeError("0D or 1D target tensor expected, multi-target not supported")
    if not (self.dim() == 1 and target.dim() == 0) and self.shape[0] != target.shape[0]:
        raise RuntimeError(f"size mismatch (got input: {list(self.shape)}, target: {list(target.shape)})")
    if weight is not None and (weight.dim() != 1 or weight.numel() != self.shape[-1]):
        raise RuntimeError("weight tensor should be defined either for all classes or no classes")
    if target.dtype not in (torch.int64, torch.uint8):
        raise RuntimeError(f"expected target dtype Long or Byte but got {target.dtype}")


def nll_loss_forward(self, target, weight=None, reduction=REDUCE_MEAN, ignore_index=-100, return_sums=False):
    """aten::nll_loss_forward -> (output, total_weight).

    return_sums=True additionally returns a float32[2] device tensor {sum -w*x, sum w} taken before
    the mean division: what a row-sharded caller all-reduces.
    """
    _require_cuda(self, target, weight)
    lib = load_library()
    _nll_check(self, target, weight)
    C = self.shape[-1]
    M = 1 if self.dim() == 1 else self.shape[0]
    x = self.contiguous()
    t = target.contiguous()
    w = weight.to(x.dtype).contiguous() if weight is not None else None
    if reduction == REDUCE_NONE and self.dim() == 2:
        out = torch.empty(M, dtype=x.dtype, device=x.device)
    else:
        out = torch.empty((), dtype=x.dtype, device=x.device)
    total_weight = torch.zeros((), dtype=x.dtype, device=x.device)
    sums = torch.zeros(2, dtype=torch.float32, device=x.device) if return_sums else None
    with torch.cuda.device(x.device):
        nbytes = lib.b2n_nll_loss_workspace_bytes(M)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
        _check(lib.b2n_nll_loss_fwd(_ptr(x), _ptr(t), _ptr(w), _ptr(out), _ptr(total_weight), _ptr(sums), _ptr(ws),
                                    nbytes, M, C, int(reduction), int(ignore_index), _dt(x.dtype),
                                    int(t.dtype == torch.uint8), _stream(x)), "b2n_nll_loss_fwd")
    if return_sums:
        return out, total_weight, sums
    return out, total_weight


def nll_loss_backward(grad_output, self, target, weight=None, reduction=REDUCE_MEAN, ignore_index=-100,
                      total_weight=None, out=None):
    """aten::nll_loss_backward -> grad_input (zero-filled, one value scattered per row)."""
    _require_cuda(grad_output, self, target, weight, total_weight)
    lib = load_library()
    _nll_check(self, target, weight)
    C = self.shape[-1]
    M = 1 if self.dim() == 1 else self.shape[0]
    g = grad_output.to(self.dtype).contiguous()
    t = target.contiguous()
    w = weight.to(self.dtype).contiguous() if weight is not None else None
    tw = total_weight.to(self.dtype).contiguous() if total_weight is not None else None
    red = int(reduction)
    if self.dim() == 1 and red == REDUCE_NONE:
        red = REDUCE_SUM  # a single row: the scalar grad_output applies as is
    grad_input = out if out is not None else torch.empty_like(self, memory_format=torch.contiguous_format)
    with torch.cuda.device(self.device):
        _check(lib.b2n_nll_loss_bwd(_ptr(g), _ptr(t), _ptr(w), _ptr(tw), _ptr(grad_input), M, C, red,
                                    int(ignore_index), _dt(self.dtype), int(t.dtype == torch.uint8), _stream(self)),
               "b2n_nll_loss_bwd")
    return grad_input


# ---- fused cross-entropy tail ----------------------------------------------------------------------------
def cross_entropy_backward(grad_output, log_probs, target, weight=None, reduction=REDUCE_MEAN, ignore_index=-100,
                           total_weight=None, out=None):
    """nll_loss_backward followed by _log_softmax_backward_data(dim=-1) as one kernel:
    grad_input[i, j] = s_i * (exp(log_probs[i, j]) - [j == target_i]).  `out` may be `log_probs` itself."""
    _require_cuda(grad_output, log_probs, target, weight, total_weight)
    lib = load_library()
    _nll_check(log_probs, target, weight)
    C = log_probs.shape[-1]
    M = 1 if log_probs.dim() == 1 else log_probs.shape[0]
    y = log_probs.contiguous()
    g = grad_output.to(y.dtype).contiguous()
    t = target.contiguous()
    w = weight.to(y.dtype).contiguous() if weight is not None else None
    tw = total_weight.to(y.dtype).contiguous() if total_weight is not None else None
    red = int(reduction)
    if log_probs.dim() == 1 and red == REDUCE_NONE:
        red = REDUCE_SUM  # a single row: the scalar grad_output applies as is
    dx = out if out is not None else torch.empty_like(y)
    with torch.cuda.device(y.device):
        _check(lib.b2n_cross_entropy_bwd(_ptr(y), _ptr(t), _ptr(w), _ptr(g), _ptr(tw), _ptr(dx), M, C, red,
                                         int(ignore_index), _dt(y.dtype), int(t.dtype == torch.uint8), _stream(y)),
               "b2n_cross_entropy_bwd")
    return dx


class _CrossEntropy(torch.autograd.Function):
    """log_softmax + nll_loss forward on the library's kernels; the fused kernel backward."""

    @staticmethod
    def forward(ctx, logits, target, weight, reduction, ignore_index):
        logp = _log_softmax(logits, -1, False)
        loss, total_weight = nll_loss_forward(logp, target, weight, reduction, ignore_index)
        ctx.save_for_backward(logp, target, weight if weight is not None else logp.new_empty(0), total_weight)
        ctx.has_weight = weight is not None
        ctx.reduction = reduction
        ctx.ignore_index = ignore_index
        return loss

    @staticmethod
    def backward(ctx, grad_loss):
        logp, target, weight, total_weight = ctx.saved_tensors
        dx = cross_entropy_backward(grad_loss, logp, target, weight if ctx.has_weight else None, ctx.reduction,
                                    ctx.ignore_index, total_weight)
        return dx, None, None, None, None


def cross_entropy(logits, target, weight=None, reduction="mean", ignore_index=-100):
    """torch.nn.functional.cross_entropy for class-index targets over the last dim of a 1-D or 2-D input
    (no label smoothing), with the backward fused into one pass over the log-probabilities."""
    red = {"none": REDUCE_NONE, "mean": REDUCE_MEAN, "sum": REDUCE_SUM}[reduction]
    return _CrossEntropy.apply(logits, target, weight, red, ignore_index)
