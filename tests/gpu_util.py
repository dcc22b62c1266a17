"""Helpers shared by the GPU parity tests."""
from __future__ import annotations

import contextlib

import torch

import b200norm
from b200norm import capi

DEV = torch.device("cuda", 0)
POISON = 0x5A


@contextlib.contextmanager
def forced_path(path):
    prev = capi.set_path(path)
    try:
        yield
    finally:
        capi.set_path(prev)


def guarded_empty(shape, dtype, pad_elems: int = 64):
    """A tensor carved out of the middle of a poisoned buffer: (view, check) where check() asserts the
    guard bands before and after the view are untouched.  The view starts 16-byte aligned."""
    numel = 1
    for s in shape:
        numel *= s
    esize = torch.empty((), dtype=dtype).element_size()
    pad = max(pad_elems, 16 // esize)
    pad = (pad * esize + 15) // 16 * 16 // esize
    buf = torch.full(((numel + 2 * pad) * esize,), POISON, dtype=torch.uint8, device=DEV)
    typed = buf.view(dtype)
    view = typed[pad:pad + numel].view(shape)

    def check():
        head = buf[: pad * esize]
        tail = buf[(pad + numel) * esize:]
        assert bool((head == POISON).all()) and bool((tail == POISON).all()), "guard band overwritten"

    return view, check


def misaligned(t: torch.Tensor, elems: int = 1) -> torch.Tensor:
    """A copy of t whose storage starts `elems` elements past a 16-byte boundary (breaks vector alignment)."""
    flat = torch.empty(t.numel() + 64, dtype=t.dtype, device=t.device)
    base_off = 0
    esize = t.element_size()
    while (flat.data_ptr() + (base_off + elems) * esize) % 16 == 0 and elems % (16 // esize) != 0:
        base_off += 1
    out = flat[base_off + elems: base_off + elems + t.numel()].view(t.shape)
    out.copy_(t)
    return out


def ring_eligible(n: int, dtype, ept: int) -> bool:
    esize = torch.empty((), dtype=dtype).element_size()
    if dtype == torch.float64:
        return False
    vec = 16 // esize
    return n % vec == 0 and n <= 512 * ept


def seeded_rows_to_device(seed: int, M: int, N: int, dtype, std: float = 1.0, mean: float = 0.0, block: int = 4096,
                          post=None) -> torch.Tensor:
    """An [M, N] tensor drawn on the CPU from torch.Generator().manual_seed(seed) — fp32 normal draws in blocks of
    `block` rows, scaled, optionally edited by post(block_fp32, first_row), rounded to `dtype` — and copied to the
    device block by block.  The CPU oracle and the kernels then see bit-identical data without the whole fp32
    tensor ever existing on the host."""
    g = torch.Generator(device="cpu").manual_seed(int(seed))
    out = torch.empty((M, N), dtype=dtype, device=DEV)
    for r in range(0, M, block):
        k = min(block, M - r)
        t = torch.randn((k, N), generator=g, dtype=torch.float32)
        if std != 1.0:
            t *= std
        if mean != 0.0:
            t += mean
        if post is not None:
            t = post(t, r)
        out[r:r + k] = t.to(dtype)
    return out


def gate_16bit(name: str, got: torch.Tensor, ref_exact: torch.Tensor, ref64: torch.Tensor, cpu_native=None):
    """The 16-bit gate with its accounting, printed (pytest -s shows it) and asserted:
    * no element beyond 1 ulp of the fp32-accumulated reference and the absolute floor;
    * elements that needed the floor: at most 1 in 10 000 (they sit where one 16-bit ulp is below the floor);
    * against the float64 evaluation rounded once, with NO floor: the kernel's count of elements beyond 1 ulp
      does not exceed what the parity standard itself (CPU ATen on fp32 upcasts) leaves against float64, plus the
      same 1 in 10 000 (both evaluate in fp32; neither can be exact where the output is a small difference)."""
    from oracle import aten_oracle as ao
    rep = ao.lowp_report(got, ref_exact)
    strict = ao.strict_ulp_failures(got, ref64)
    strict_ref = ao.strict_ulp_failures(ref_exact, ref64)
    print(f"[parity] {name}: {rep['numel']} elements, beyond 1 ulp and floor {rep['bad']}, passed only through the floor "
          f"{rep['floor_only']}, beyond 1 ulp of fp64 (no floor) {strict} (CPU ATen fp32 itself: {strict_ref})")
    assert rep["bad"] == 0, f"{name}: {rep['bad']} elements beyond 1 ulp and the floor (worst {rep['worst']} ulp)"
    allowance = max(1, rep["numel"] // 10000)
    assert rep["floor_only"] <= allowance, f"{name}: {rep['floor_only']} elements needed the floor"
    assert strict <= strict_ref + allowance, f"{name}: {strict} elements beyond 1 ulp of fp64 (reference: {strict_ref})"


def wgrad_gate(a: torch.Tensor, terms: torch.Tensor, what: str) -> None:
    """Weight-gradient gate, element by element.  a: kernel result [N]; terms: fp64 [M, N] summands.
    fp32 results: within 1e-6 of the L1 norm of the element's terms of the fp64 sum.  16-bit results (the fp32 sum
    rounded once): within 1 ulp of the fp64 sum rounded once, or — where the sum cancels to something smaller than the
    fp32 rounding of its terms, so that a 16-bit ulp of it means nothing — within that same 1e-6 of L1."""
    from oracle import aten_oracle as ao
    got = a.detach().cpu().reshape(-1)
    ref = terms.sum(0).reshape(-1)
    l1 = terms.abs().sum(0).reshape(-1).clamp_min(1e-30)
    rel = (got.double() - ref).abs() / l1
    if got.dtype in (torch.bfloat16, torch.float16):
        r16 = ref.to(got.dtype)
        assert torch.equal(torch.isnan(got), torch.isnan(r16)), f"{what}: NaN pattern"
        d = (ao._ordered_int(got) - ao._ordered_int(r16)).abs()
        bad = (d > 1) & (rel > 1e-6)
        assert not bool(bad.any()), (f"{what}: {int(bad.sum())} elements beyond 1 ulp and 1e-6 of L1 "
                                     f"(worst {int(d[bad].max())} ulp, {float(rel[bad].max()):.3e} of L1)")
    else:
        assert float(rel.max()) <= 1e-6, f"{what}: {float(rel.max()):.3e} of L1"
