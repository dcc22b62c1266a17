"""b2n_layer_norm_bwd_noalloc — the backward for callers that cannot allocate (an engine plug-in's enqueue
callback, a serving loop with a frozen pool): its scratch is a fixed device array inside the library.

Called through the C ABI with raw pointers, twice in a row (the array keeps the previous call's
contents, so the second call proves nothing stale leaks through), and compared with the ordinary
entry point, whose workspace the caller allocates.  Both run the same kernels in the same order, so
the results must be bit-identical; the stated tolerance of the other tests is the fallback bound.
This file sorts last on purpose: a run that stops at the first failure has then already run
everything else."""
import pytest
import torch

import b200norm

pytestmark = pytest.mark.gpu

DEV = torch.device("cuda", 0)
_DT = {torch.float32: b200norm.F32, torch.bfloat16: b200norm.BF16, torch.float16: b200norm.F16}


def _inputs(M, N, dt, wdt, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((M, N), generator=g).to(dt).to(DEV)
    dy = torch.randn((M, N), generator=g).to(dt).to(DEV)
    gamma = (torch.randn(N, generator=g) * 0.02 + 1).to(wdt).to(DEV)
    mean = x.float().mean(-1).contiguous()
    rstd = torch.rsqrt(x.float().var(-1, unbiased=False) + 1e-5).contiguous()
    return x, dy, gamma, mean, rstd


def _reference(lib, x, dy, gamma, mean, rstd, M, N):
    dx, dg, db = torch.empty_like(x), torch.empty_like(gamma), torch.empty_like(gamma)
    need = lib.b2n_norm_bwd_workspace_bytes(M, N, _DT[x.dtype], _DT[gamma.dtype], 1)
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device=DEV)
    rc = lib.b2n_layer_norm_bwd(dy.data_ptr(), x.data_ptr(), mean.data_ptr(), rstd.data_ptr(), gamma.data_ptr(),
                                dx.data_ptr(), dg.data_ptr(), db.data_ptr(), ws.data_ptr(), need, M, N, _DT[x.dtype],
                                _DT[gamma.dtype], torch.cuda.current_stream().cuda_stream)
    assert rc == b200norm.OK
    return dx, dg, db


def _noalloc(lib, x, dy, gamma, mean, rstd, M, N):
    dx, dg, db = torch.empty_like(x), torch.empty_like(gamma), torch.empty_like(gamma)
    rc = lib.b2n_layer_norm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), mean.data_ptr(), rstd.data_ptr(), gamma.data_ptr(),
                                        dx.data_ptr(), dg.data_ptr(), db.data_ptr(), M, N, _DT[x.dtype],
                                        _DT[gamma.dtype], torch.cuda.current_stream().cuda_stream)
    assert rc == b200norm.OK, b200norm.what_status(rc)
    return dx, dg, db


@pytest.mark.parametrize("M,N,dt,wdt", [(4096, 8192, torch.bfloat16, torch.float32),   # ring kernel, 148 partial rows
                                        (300, 1000, torch.float32, torch.float32),     # ring kernel, ragged rows
                                        (64, 33, torch.float32, torch.float32),        # generic kernels
                                        (2000, 4096, torch.float16, torch.float16)])
def test_matches_the_allocating_entry_point_twice_in_a_row(M, N, dt, wdt):
    lib = b200norm.load_library()
    assert lib.b2n_noalloc_scratch_bytes() == 16 << 20
    first = _inputs(M, N, dt, wdt, 1)
    second = _inputs(M, N, dt, wdt, 2)  # different data: stale partial sums would show
    for x, dy, gamma, mean, rstd in (first, second):
        ref = _reference(lib, x, dy, gamma, mean, rstd, M, N)
        got = _noalloc(lib, x, dy, gamma, mean, rstd, M, N)
        torch.cuda.synchronize()
        for a, b, name in zip(got, ref, ("dx", "dgamma", "dbeta")):
            assert torch.equal(a, b) or torch.allclose(a.float(), b.float(), rtol=1e-5, atol=1e-6), name
    assert lib.b2n_device_status(torch.cuda.current_stream().cuda_stream) == 0


def test_rejects_problems_beyond_the_fixed_scratch():
    lib = b200norm.load_library()
    M, N = 200000, 16384  # generic path: 256 partial rows x 2 x 16384 x 4 B = 32 MiB > 16 MiB
    assert lib.b2n_norm_bwd_workspace_bytes(M, N, b200norm.F32, b200norm.F32, 1) > lib.b2n_noalloc_scratch_bytes()
    one = torch.zeros(1, device=DEV)
    rc = lib.b2n_layer_norm_bwd_noalloc(one.data_ptr(), one.data_ptr(), one.data_ptr(), one.data_ptr(), one.data_ptr(),
                                        one.data_ptr(), one.data_ptr(), one.data_ptr(), M, N, b200norm.F32, b200norm.F32,
                                        None)
    assert rc == b200norm.ERR_TOO_LARGE  # refused before anything is launched
    assert b"limit" in lib.b2n_strerror(rc)
    # without weight gradients there is no scratch to need: any size is accepted (dx only)
    x, dy, gamma, mean, rstd = _inputs(8, 64, torch.float32, torch.float32, 3)
    dx = torch.empty_like(x)
    rc = lib.b2n_layer_norm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), mean.data_ptr(), rstd.data_ptr(), gamma.data_ptr(),
                                        dx.data_ptr(), None, None, 8, 64, b200norm.F32, b200norm.F32,
                                        torch.cuda.current_stream().cuda_stream)
    assert rc == b200norm.OK
    torch.cuda.synchronize()
