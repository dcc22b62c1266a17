"""Generates tests/golden/golden_v2.pt: CPU ATen outputs for the operators added around the core path —
_safe_softmax, _masked_softmax / _masked_softmax_backward (the three mask layouts) and the fused cross-entropy
backward (nll_loss_backward followed by _log_softmax_backward_data).

Run from the repository root:  python tests/golden/make_golden_v2.py
Same conventions as make_golden.py: seeded inputs, torch 2.11.0 CPU kernels, 16-bit cases store the CPU op run on
fp32 upcasts and rounded once.  golden_v1.pt is left untouched.
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
    # ---- safe softmax: fully masked rows give zeros
    for name, shape, dim, dt in (("safe_f32", (6, 40), -1, torch.float32), ("safe_bf16", (5, 64), -1, torch.bfloat16),
                                 ("safe_f32_dim0", (4, 3, 5), 0, torch.float32)):
        x = ao.randn(shape, 51, torch.float32)
        x[x > 1.0] = float("-inf")
        x.view(-1, shape[-1])[1] = float("-inf")
        if dim == 0:
            x[:, 1, 2] = float("-inf")
        x = x.to(dt)
        cases[name] = dict(x=x, dim=dim, y=torch.ops.aten._safe_softmax(wide(x), dim).to(dt))
    # ---- masked softmax, the three layouts of the reference
    gen = torch.Generator().manual_seed(52)
    for name, dt in (("masked_f32", torch.float32), ("masked_bf16", torch.bfloat16)):
        B, H, T = 2, 3, 16
        x = ao.randn((B, H, T, T), 53, torch.float32).to(dt)
        g = ao.randn((B, H, T, T), 54, torch.float32).to(dt)
        full = torch.rand((B, H, T, T), generator=gen) < 0.3
        full[0, 0, 1] = True                                  # a fully masked row
        causal = torch.triu(torch.ones(T, T, dtype=torch.bool), 1)
        pad = torch.zeros(B, T, dtype=torch.bool)
        pad[:, T - 5:] = True
        entry = dict(x=x, grad=g, mask_full=full, mask_txt=causal, mask_bxt=pad)
        for tag, m, mtype in (("full", full, 2), ("txt", causal, 0), ("bxt", pad, 1)):
            y = torch._masked_softmax(wide(x), m, -1, mtype)
            entry["y_" + tag] = y.to(dt)
        y = entry["y_full"]
        entry["dx_full"] = torch.ops.aten._masked_softmax_backward(wide(g), wide(y), full, -1).to(dt)
        cases[name] = entry
    # ---- fused cross-entropy backward
    for name, dt in (("ce_f32", torch.float32), ("ce_bf16", torch.bfloat16)):
        M, C = 12, 40
        logp = torch.log_softmax(ao.randn((M, C), 55, torch.float32, 0.0, 2.0), -1).to(dt)
        t = ao.randint(C, (M,), 56)
        t[3] = -100
        w = (ao.randn((C,), 57).abs() + 0.1).to(dt)
        entry = dict(logp=logp, target=t, weight=w, ignore_index=-100)
        for red in (0, 1, 2):
            for wt, tag in ((None, "now"), (w, "w")):
                _, tw = ao.nll_fwd(logp, t, wt, red, -100)
                g = ao.randn((M,), 58).to(dt) if red == 0 else torch.tensor(0.7, dtype=dt)
                entry[f"grad_{red}"] = g
                entry[f"tw_{red}_{tag}"] = tw
                entry[f"dx_{red}_{tag}"] = ao.cross_entropy_bwd(g, logp, t, wt, red, -100, tw)
        cases[name] = entry
    out = Path(__file__).resolve().parent / "golden_v2.pt"
    torch.save(cases, out)
    print(out, out.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
