"""Generates tests/golden/golden_v3.pt: CPU ATen outputs for what was added after golden_v2 —
native_group_norm (forward), batch_norm_stats / batch_norm_update_stats, softmax and log-softmax with their backward
over a dim that is NOT the last at a size the tensor-map TMA tile kernels take, and layer norm forward + backward on
rows longer than 8192 elements (the cluster slab kernels).

Run from the repository root:  python tests/golden/make_golden_v3.py
Same conventions as make_golden.py: seeded inputs, torch 2.11.0 CPU kernels, 16-bit cases store the CPU op run on fp32
upcasts and rounded once.  Shapes are the smallest that reach those kernels, so the file stays small.
"""
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import aten_oracle as ao  # noqa: E402


def wide(t):
    return t.double() if t.dtype == torch.float64 else t.float()


def main() -> None:
    cases = {}
    # ---- group norm forward: a row that fills the ring's threads exactly, one that does not, one with HxW odd
    for name, shape, G, dt in (("gn_f32", (2, 8, 8, 8), 4, torch.float32), ("gn_bf16", (2, 16, 16, 16), 2, torch.bfloat16),
                               ("gn_f32_odd", (3, 6, 5), 3, torch.float32)):
        x = ao.randn(shape, 61, torch.float32, 0.5, 2.0).to(dt)
        C = shape[1]
        w = ao.randn((C,), 62, torch.float32, 1.0, 0.1).to(dt)
        b = ao.randn((C,), 63, torch.float32, 0.0, 0.1).to(dt)
        hw = x.numel() // (shape[0] * C)
        y, mean, rstd = torch.ops.aten.native_group_norm(wide(x), wide(w), wide(b), shape[0], C, hw, G, 1e-5)
        cases[name] = dict(x=x, weight=w, bias=b, G=G, eps=1e-5, y=y.to(dt), mean=mean.float(), rstd=rstd.float())
    # ---- batch norm statistics: two channels with enough data to be shared by several CTAs, and two small ones
    for name, shape, dt in (("bn_f32", (2, 3, 8, 8), torch.float32), ("bn_bf16", (4, 2, 64, 128), torch.bfloat16),
                            ("bn_f32_small", (5, 7, 3, 3), torch.float32)):
        x = ao.randn(shape, 64, torch.float32, 1.5, 3.0).to(dt)
        x64 = x.double()
        dims = (0, 2, 3)
        mean, var = x64.mean(dims), x64.var(dims, unbiased=False)
        rm0, rv0 = ao.randn((shape[1],), 65), ao.randn((shape[1],), 66).abs() + 0.5
        n = x.numel() // shape[1]
        cases[name] = dict(x=x, eps=1e-5, momentum=0.1, mean=mean.float(), invstd=(1.0 / torch.sqrt(var + 1e-5)).float(),
                           var=var.float(), running_mean=rm0, running_var=rv0,
                           running_mean_out=(0.9 * rm0.double() + 0.1 * mean).float(),
                           running_var_out=(0.9 * rv0.double() + 0.1 * var * n / (n - 1)).float())
    # ---- softmax family over dim 1 of [outer, N, inner]: tiles of one box, of several boxes of rows, ragged last tile
    for name, shape, dt in (("smd1_bf16", (2, 19, 256), torch.bfloat16), ("smd1_f32", (1, 260, 64), torch.float32),
                            ("smd1_f16", (1, 64, 72), torch.float16)):
        x = ao.randn(shape, 67, torch.float32, 0.0, 2.0)
        x[0, :, 3] = float("-inf")     # a line of -inf: NaN (softmax), NaN (log-softmax)
        x[0, 1, 5] = float("-inf")
        x = x.to(dt)
        dy = ao.randn(shape, 68, torch.float32).to(dt)
        sm = torch.ops.aten._softmax(wide(x), 1, False)
        lsm = torch.ops.aten._log_softmax(wide(x), 1, False)
        cases[name] = dict(x=x, dy=dy, softmax=sm.to(dt), log_softmax=lsm.to(dt),
                           softmax_bwd=torch.ops.aten._softmax_backward_data(wide(dy), wide(sm.to(dt)), 1, sm.dtype).to(dt),
                           log_softmax_bwd=torch.ops.aten._log_softmax_backward_data(wide(dy), wide(lsm.to(dt)), 1,
                                                                                      lsm.dtype).to(dt))
    # ---- layer norm on rows of 8208 elements (two slabs of a cluster), forward and backward with weight gradients
    for name, dt, wdt in (("ln_long_bf16_w32", torch.bfloat16, torch.float32),):
        M, N = 2, 8208
        x = ao.randn((M, N), 69, torch.float32, 0.3, 1.5).to(dt)
        dy = ao.randn((M, N), 70, torch.float32).to(dt)
        g = ao.randn((N,), 71, torch.float32, 1.0, 0.05).to(wdt)
        b = ao.randn((N,), 72, torch.float32, 0.0, 0.05).to(wdt)
        y, mean, rstd = torch.ops.aten.native_layer_norm(wide(x), [N], wide(g), wide(b), 1e-5)
        dx, dg, db = torch.ops.aten.native_layer_norm_backward(wide(dy), wide(x), [N], mean, rstd, wide(g), wide(b),
                                                               [True, True, True])
        cases[name] = dict(x=x, dy=dy, gamma=g, beta=b, eps=1e-5, y=y.to(dt), mean=mean.float(), rstd=rstd.float(),
                           dx=dx.to(dt), dgamma=dg.to(wdt), dbeta=db.to(wdt))
    out = Path(__file__).parent / "golden_v3.pt"
    torch.save(cases, out)
    print(f"wrote {out} ({out.stat().st_size} bytes, {len(cases)} cases)")


if __name__ == "__main__":
    main()
