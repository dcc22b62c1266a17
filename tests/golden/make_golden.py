"""Generates tests/golden/golden_v1.pt from PyTorch's CPU ATen kernels.

Run from the repository root:  python tests/golden/make_golden.py
The reference project has no golden files for this path (its tests compare with CPU ATen at run
time), so these vectors are CPU ATen outputs on seeded inputs, produced in the build container
(torch 2.11.0) and committed so that every later run — including on the GPU box — checks against
the same bits.  16-bit cases store the CPU op run on fp32 upcasts and rounded once.
"""
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import aten_oracle as ao  # noqa: E402


def main() -> None:
    cases = {}
    # layer norm fp32 [8, 64] and bf16-x / fp32-weights [4, 128]; rows of 5 for the non-vector path
    for name, shape, dt, wdt in (("ln_f32", (8, 64), torch.float32, torch.float32),
                                 ("ln_bf16_w32", (4, 128), torch.bfloat16, torch.float32),
                                 ("ln_f16", (6, 40), torch.float16, torch.float16),
                                 ("ln_f32_n5", (7, 5), torch.float32, torch.float32)):
        n = shape[-1]
        x = ao.randn(shape, 11, dt)
        g = ao.randn((n,), 12, wdt, 1.0, 0.02)
        b = ao.randn((n,), 13, wdt, 0.0, 0.02)
        dy = ao.randn(shape, 14, dt)
        y, mean, rstd = ao.layer_norm_fwd(x, [n], g, b, 1e-5)
        dx, dg, db = ao.layer_norm_bwd(dy, x, [n], mean, rstd, g, b)
        cases[name] = dict(x=x, gamma=g, beta=b, dy=dy, eps=1e-5, y=y, mean=mean, rstd=rstd, dx=dx, dgamma=dg, dbeta=db)
    for name, shape, dt, wdt in (("rms_f32", (8, 64), torch.float32, torch.float32),
                                 ("rms_bf16_w32", (4, 128), torch.bfloat16, torch.float32)):
        n = shape[-1]
        x = ao.randn(shape, 21, dt)
        w = ao.randn((n,), 22, wdt, 1.0, 0.02)
        dy = ao.randn(shape, 23, dt)
        y, rstd = ao.rms_norm_fwd(x, [n], w, 1e-6)
        dx, dw = ao.rms_norm_bwd(dy, x, [n], w, 1e-6)
        cases[name] = dict(x=x, weight=w, dy=dy, eps=1e-6, y=y, rstd=rstd, dx=dx, dweight=dw)
    for name, shape, dim, dt in (("sm_f32_last", (4, 50), -1, torch.float32), ("sm_bf16_last", (3, 64), -1, torch.bfloat16),
                                 ("sm_f32_dim0", (6, 5, 3), 0, torch.float32), ("sm_f32_dim1", (2, 7, 4), 1, torch.float32)):
        x = ao.randn(shape, 31, dt)
        if name == "sm_bf16_last":
            x[0, 5:] = float("-inf")  # masked tail
        dy = ao.randn(shape, 32, dt)
        entry = dict(x=x, dy=dy, dim=dim)
        for is_log, tag in ((False, "softmax"), (True, "log_softmax")):
            y = ao.softmax_fwd(x, dim, is_log)
            entry[tag] = y
            entry[tag + "_bwd"] = ao.softmax_bwd(dy, y, dim, is_log, dt)
        cases[name] = entry
    logp = torch.log_softmax(ao.randn((16, 10), 41, torch.float32), -1)
    t = ao.randint(10, (16,), 42)
    t[3] = -100
    w = ao.randn((10,), 43, torch.float32).abs() + 0.1
    entry = dict(logp=logp, target=t, weight=w, ignore_index=-100)
    for red in (0, 1, 2):
        for wt, tag in ((None, "now"), (w, "w")):
            out, tw = ao.nll_fwd(logp, t, wt, red, -100)
            entry[f"out_{red}_{tag}"] = out
            entry[f"tw_{red}_{tag}"] = tw
    cases["nll_f32"] = entry
    out = Path(__file__).resolve().parent / "golden_v1.pt"
    torch.save(cases, out)
    print(out, out.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
