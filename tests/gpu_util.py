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
