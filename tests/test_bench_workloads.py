"""Host-side checks of the bench workloads (no GPU): the algorithmic byte counts the roofline figures rest on, and that
every workload's CPU arm runs on a small sample and returns tensors of the shapes its byte count claims."""
import importlib.util
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
import bench_workloads as bw  # noqa: E402


def _numel_bytes(t):
    return t.numel() * t.element_size()


@pytest.mark.parametrize("name", sorted(bw.EXTRA))
def test_byte_counts_match_the_tensors(name):
    wl = bw.EXTRA[name]()
    rows = {"cfg1": 64, "cfg2": 64, "cfg3": 64, "cfg3m": 64, "cfg5": 8, "cfg5f": 8, "gn": 2, "bn": 2}.get(name, 1)
    per = wl.bytes_per_rows(rows)
    assert per["total"] > 0 and all(v > 0 for v in per.values())
    kernels = {k: v for k, v in per.items() if k != "total"}
    # a workload's total is the sum of its kernels' bytes, except where two names stand for alternative kernels of one
    # operator (group norm, masked softmax: ring or plain) or where small operators between the kernels are counted in the total only
    if name in ("cfg1", "cfg2", "cfg3", "sm_c19", "sm_c64", "sm_c150", "bn"):
        assert per["total"] == sum(kernels.values())
    cpu = wl.make_cpu_state(rows)
    ins = sum(_numel_bytes(cpu[k]) for k in wl.e2e_inputs)
    assert ins == sum(wl._nbytes(rows, k) for k in wl.e2e_inputs)
    out = wl.cpu_step(cpu)
    outs = out if isinstance(out, (tuple, list)) else (out,)
    assert all(torch.is_tensor(o) for o in outs)
    # every input is read at least once, so the total can never be below the inputs' size
    assert per["total"] >= ins


def test_spatial_softmax_bytes_are_five_tensor_passes():
    for cls, c in ((bw.SpatialSoftmax19, 19), (bw.SpatialSoftmax, 64), (bw.SpatialSoftmax150, 150)):
        wl = cls()
        n = 16 * c * 512 * 512 * 2
        per = wl.bytes_per_rows(16)
        assert per == {"total": 5 * n, "softmax_fwd_tma": 2 * n, "softmax_bwd_tma": 3 * n}
        assert wl.name == f"sm_c{c}" and str(c) in wl.describe()
