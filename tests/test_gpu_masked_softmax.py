"""aten::_masked_softmax / _masked_softmax_backward through the C ABI and through the dispatcher vs CPU ATen.

Tolerances: fp32 |a-b| <= 1e-5*|b| + 1e-6; 16-bit outputs within 1 ulp of the CPU op evaluated on fp32 upcasts and
rounded once (or the absolute floor of oracle.aten_oracle.lowp_mismatch).  NaN patterns must agree exactly.
"""
import pytest
import torch

import b200norm
from b200norm import capi
from oracle import aten_oracle as ao

from gpu_util import DEV, forced_path

pytestmark = pytest.mark.gpu


def compare(got, ref, dt, what):
    got = got.cpu()
    assert got.shape == ref.shape and got.dtype == dt, what
    assert torch.equal(torch.isnan(got), torch.isnan(ref)), f"{what}: NaN pattern"
    ok = ~torch.isnan(ref)
    if dt in (torch.float32, torch.float64):
        tol = 1e-5 if dt == torch.float32 else 1e-12
        assert torch.allclose(got[ok], ref[ok].to(dt), rtol=tol, atol=tol * 0.1), what
    else:
        n_bad, worst = ao.lowp_mismatch(got[ok], ref[ok].to(dt))
        assert n_bad == 0, f"{what}: {n_bad} beyond 1 ulp (worst {worst})"


def ref_fwd(x, mask, dim, mask_type):
    wide = torch.float64 if x.dtype == torch.float64 else torch.float32
    return torch._masked_softmax(x.to(wide), mask, dim, mask_type)


def ref_bwd(g, y, mask, dim):
    wide = torch.float64 if g.dtype == torch.float64 else torch.float32
    return torch.ops.aten._masked_softmax_backward(g.to(wide), y.to(wide), mask, dim)


def random_mask(shape, seed, p=0.3):
    gen = torch.Generator().manual_seed(seed)
    return torch.rand(shape, generator=gen) < p


@pytest.mark.parametrize("path", [b200norm.PATH_AUTO, b200norm.PATH_GENERIC])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16, torch.float16, torch.float64])
@pytest.mark.parametrize("shape", [(4, 7), (2, 3, 16, 16), (3, 5, 33), (1, 2, 8, 2048), (6, 1000), (300, 4096), (2, 9000),
                                   (3, 20000)])
def test_same_shape_mask_forward_backward(shape, dt, path):
    x = ao.randn(shape, 700, torch.float32).to(dt)
    mask = random_mask(shape, 701)
    mask.view(-1, shape[-1])[1] = True       # a fully masked row: NaN forward, zero backward
    mask.view(-1, shape[-1])[0] = False      # an unmasked row
    n = shape[-1]
    vec = 16 // x.element_size()
    ring = (path == b200norm.PATH_AUTO and dt != torch.float64 and n % vec == 0 and n <= 512 * 32)
    with forced_path(path):
        y = capi._masked_softmax(x.to(DEV), mask.to(DEV), -1, 2)
        assert capi.last_path() == ("ring" if ring else "generic")
        compare(y, ref_fwd(x, mask, -1, 2), dt, "forward")
        g = ao.randn(shape, 702, torch.float32).to(dt)
        dx = capi._masked_softmax_backward(g.to(DEV), y, mask.to(DEV), -1)
        # the backward stages two tensors per tile: long fp32 rows leave the ring earlier than in the forward
        assert capi.last_path() in (("ring", "generic") if ring else ("generic",))
    compare(dx, ref_bwd(g, y.cpu(), mask, -1), dt, "backward")
    assert capi.device_status() == 0


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,H,T", [(2, 3, 16), (1, 2, 130), (3, 1, 1024), (2, 2, 2048)])
def test_broadcast_masks(B, H, T, dt):
    # T = 130 is not a multiple of the vector width: the plain kernels; the other sizes run on the ring
    x = ao.randn((B, H, T, T), 710, torch.float32).to(dt)
    causal = torch.triu(torch.ones(T, T, dtype=torch.bool), 1)          # mask_type 0: [T, T]
    y0 = capi._masked_softmax(x.to(DEV), causal.to(DEV), -1, 0)
    compare(y0, ref_fwd(x, causal, -1, 0), dt, "src_mask")
    pad = torch.zeros(B, T, dtype=torch.bool)                          # mask_type 1: [B, T]
    pad[:, T - T // 3:] = True
    pad[B - 1, 1:] = True
    y1 = capi._masked_softmax(x.to(DEV), pad.to(DEV), -1, 1)
    compare(y1, ref_fwd(x, pad, -1, 1), dt, "src_key_padding_mask")
    assert float(y1[B - 1, :, :, 0].min()) == 1.0


@pytest.mark.parametrize("dim", [0, 1, 2])
def test_other_dims_and_unaligned(dim):
    x = ao.randn((5, 6, 7), 720)
    mask = random_mask((5, 6, 7), 721)
    y = capi._masked_softmax(x.to(DEV), mask.to(DEV), dim, 2)
    compare(y, ref_fwd(x, mask, dim, 2), torch.float32, f"forward dim {dim}")
    g = ao.randn((5, 6, 7), 722)
    dx = capi._masked_softmax_backward(g.to(DEV), y, mask.to(DEV), dim)
    compare(dx, ref_bwd(g, y.cpu(), mask, dim), torch.float32, f"backward dim {dim}")


def test_argument_checks():
    x = torch.randn(2, 3, 4, 4, device=DEV)
    with pytest.raises(RuntimeError, match="boolean"):
        capi._masked_softmax(x, torch.zeros(2, 3, 4, 4, device=DEV), -1, 2)
    with pytest.raises(RuntimeError, match="Mask Type should be defined"):
        capi._masked_softmax(x, torch.zeros(2, 3, 4, 4, dtype=torch.bool, device=DEV), -1, None)
    with pytest.raises(RuntimeError, match="Mask shape should match input"):
        capi._masked_softmax(x, torch.zeros(3, 4, dtype=torch.bool, device=DEV), -1, 2)
    with pytest.raises(RuntimeError, match="Mask shape should match grad shape"):
        capi._masked_softmax_backward(x, x, torch.zeros(4, 4, dtype=torch.bool, device=DEV), -1)


def test_through_the_dispatcher():
    b200norm.enable_aten_overrides()
    B, H, T = 2, 2, 64
    x = ao.randn((B, H, T, T), 730)
    causal = torch.triu(torch.ones(T, T, dtype=torch.bool), 1)
    n0 = capi.launch_count()
    y = torch._masked_softmax(x.to(DEV), causal.to(DEV), -1, 0)
    assert capi.launch_count() == n0 + 1, "the CUDA dispatch key must land in this library"
    compare(y, ref_fwd(x, causal, -1, 0), torch.float32, "dispatcher forward")
    full = causal.expand(B, H, T, T).contiguous()
    g = ao.randn((B, H, T, T), 731)
    dx = torch.ops.aten._masked_softmax_backward(g.to(DEV), y, full.to(DEV), -1)
    compare(dx, ref_bwd(g, y.cpu(), full, -1), torch.float32, "dispatcher backward")
    y2 = torch._masked_softmax(x.to(DEV), full.to(DEV), 1, 2)
    compare(y2, ref_fwd(x, full, 1, 2), torch.float32, "dispatcher forward, dim 1")
