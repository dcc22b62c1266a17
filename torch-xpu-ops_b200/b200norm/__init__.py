"""b200norm — sm_100a kernels for the row-wise normalization / softmax operator family.

Two ways in, both backed by the same hand-written CUDA kernels (there is no eager or CPU
fallback: if the shared objects are missing, import fails):

* ``b200norm.capi`` — thin ctypes wrappers over the C ABI of ``include/b200norm.h``; they take
  torch CUDA tensors only as (pointer, size) carriers.
* ``b200norm.enable_aten_overrides()`` — loads the ATen registration, after which
  ``torch.nn.functional.layer_norm``, ``softmax``, ``log_softmax``, ``nll_loss`` ... and their
  autograd formulas run on these kernels for CUDA tensors.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

_PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = _PKG_DIR / "libb200norm.so"
ATEN_LIB_PATH = _PKG_DIR / "_b200norm_aten.so"

ABI_VERSION = 1

# b2n_dtype / b2n_status / b2n_path values (include/b200norm.h)
F32, F16, BF16, F64 = 0, 1, 2, 3
OK = 0
ERR_BAD_ARG, ERR_UNSUPPORTED_DTYPE, ERR_WORKSPACE, ERR_CUDA = -1, -2, -3, -4
ERR_TIMEOUT, ERR_TARGET_RANGE, ERR_TOO_LARGE = -5, -6, -7
PATH_AUTO, PATH_GENERIC, PATH_RING, PATH_CLUSTER, PATH_TWOPASS = 0, 1, 2, 3, 4
REDUCE_NONE, REDUCE_MEAN, REDUCE_SUM = 0, 1, 2
TUNE_ROWS_PER_GROUP, TUNE_STAGES, TUNE_STORE_LAG, TUNE_CLUSTER_SIZE, TUNE_SM_MARGIN, TUNE_TILE_KB = 0, 1, 2, 3, 4, 5


class B200NormError(RuntimeError):
    """A C-ABI call returned a non-zero b2n_status."""

    def __init__(self, status: int, what: str):
        self.status = status
        super().__init__(f"{what}: {what_status(status)} (status {status})")


_lib = None
_aten_loaded = False


def load_library() -> ctypes.CDLL:
    """dlopen libb200norm.so (built in-tree by b200norm._build) and declare the C ABI's prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "(b200norm has no fallback implementation)")
    lib = ctypes.CDLL(str(LIB_PATH), mode=ctypes.RTLD_GLOBAL)
    c = ctypes
    vp, i64, i32, dbl, sz = c.c_void_p, c.c_int64, c.c_int, c.c_double, c.c_size_t
    protos = {
        "b2n_abi_version": (i32, []),
        "b2n_strerror": (c.c_char_p, [i32]),
        "b2n_last_cuda_error": (i32, []),
        "b2n_set_path": (i32, [i32]),
        "b2n_last_path": (c.c_char_p, []),
        "b2n_set_tuning": (i32, [i32, i32]),
        "b2n_set_trace_buffer": (i32, [vp, sz]),
        "b2n_device_status": (i32, [vp]),
        "b2n_status_post": (i32, [vp]),
        "b2n_status_poll": (i32, []),
        "b2n_launch_count": (c.c_ulonglong, []),
        "b2n_profile_begin": (i32, []),
        "b2n_profile_end": (i32, [c.c_char_p, sz]),
        "b2n_layer_norm_fwd": (i32, [vp, vp, vp, vp, vp, vp, i64, i64, dbl, i32, i32, vp]),
        "b2n_rms_norm_fwd": (i32, [vp, vp, vp, vp, i64, i64, dbl, i32, i32, vp]),
        "b2n_norm_bwd_workspace_bytes": (sz, [i64, i64, i32, i32, i32]),
        "b2n_layer_norm_bwd": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, vp, sz, i64, i64, i32, i32, vp]),
        "b2n_norm_bwd_partials": (i32, [i32, vp, vp, vp, vp, vp, vp, vp, sz, i64, i64, i32, i32, c.POINTER(i64), vp]),
        "b2n_norm_wgrad_fold": (i32, [vp, i64, i64, vp, vp, i32, i32, vp]),
        "b2n_wgrad_exchange_bytes": (sz, [i64]),
        "b2n_wgrad_exchange_alloc": (i32, [i64, c.POINTER(vp), c.c_char_p]),
        "b2n_wgrad_exchange_open": (i32, [c.c_char_p, c.POINTER(vp)]),
        "b2n_wgrad_exchange_close": (i32, [vp]),
        "b2n_wgrad_exchange_free": (i32, [vp]),
        "b2n_norm_wgrad_fold_allreduce": (i32, [vp, i64, i64, c.POINTER(vp), i64, i32, i32, vp, vp, i32, i32, vp]),
        "b2n_noalloc_scratch_bytes": (sz, []),
        "b2n_layer_norm_bwd_noalloc": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i32, i32, vp]),
        "b2n_rms_norm_bwd": (i32, [vp, vp, vp, vp, vp, vp, vp, sz, i64, i64, i32, i32, vp]),
        "b2n_group_norm_fwd": (i32, [vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, dbl, i32, i32, i32, vp]),
        "b2n_group_norm_bwd": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, i32, i32, i32, vp]),
        "b2n_group_norm_bwd_workspace_bytes": (sz, [i64, i64, i64, i32]),
        "b2n_group_norm_bwd_ws": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, i32, i32, i32, vp, sz, vp]),
        "b2n_batch_norm_stats": (i32, [vp, vp, vp, vp, vp, i64, i64, i64, dbl, dbl, i32, i32, i32, vp]),
        "b2n_batch_norm_stats_workspace_bytes": (sz, [i64, i64, i64, i32]),
        "b2n_batch_norm_stats_ws": (i32, [vp, vp, vp, vp, vp, i64, i64, i64, dbl, dbl, i32, i32, i32, vp, sz, vp]),
        "b2n_softmax_fwd": (i32, [vp, vp, i64, i64, i64, i32, i32, i32, vp]),
        "b2n_softmax_bwd": (i32, [vp, vp, vp, i64, i64, i64, i32, i32, i32, vp]),
        "b2n_softmax_tile_plan": (i32, [i64, i64, i64, i32, i32, i32, i64, vp]),
        "b2n_nll_loss_workspace_bytes": (sz, [i64]),
        "b2n_nll_loss_fwd": (i32, [vp, vp, vp, vp, vp, vp, vp, sz, i64, i64, i32, i64, i32, i32, vp]),
        "b2n_nll_loss_bwd": (i32, [vp, vp, vp, vp, vp, i64, i64, i32, i64, i32, i32, vp]),
        "b2n_masked_softmax_fwd": (i32, [vp, vp, vp, i64, i64, i64, i64, i32, vp]),
        "b2n_masked_softmax_bwd": (i32, [vp, vp, vp, vp, i64, i64, i32, vp]),
        "b2n_cross_entropy_bwd": (i32, [vp, vp, vp, vp, vp, vp, i64, i64, i32, i64, i32, i32, vp]),
    }
    for name, (res, args) in protos.items():
        fn = getattr(lib, name)  # AttributeError here = the library does not export the ABI
        fn.restype = res
        fn.argtypes = args
    if lib.b2n_abi_version() != ABI_VERSION:
        raise ImportError(f"libb200norm.so has ABI {lib.b2n_abi_version()}, expected {ABI_VERSION}")
    _lib = lib
    return lib


def what_status(status: int) -> str:
    return load_library().b2n_strerror(status).decode()


def enable_aten_overrides() -> None:
    """Load the ATen registration: CUDA-key kernels of the operator family become these kernels."""
    global _aten_loaded
    if _aten_loaded:
        return
    import warnings

    import torch

    load_library()
    if not ATEN_LIB_PATH.exists():
        raise ImportError(f"{ATEN_LIB_PATH} is missing: run __graft_entry__.build()")
    with warnings.catch_warnings():
        warnings.filterwarnings("ignore", message=".*Overriding a previously registered kernel.*")
        torch.ops.load_library(str(ATEN_LIB_PATH))
    _aten_loaded = True


from . import capi  # noqa: E402,F401
