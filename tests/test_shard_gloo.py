"""The row-shard driver on two CPU ranks (gloo): partitioning, the single all-reduce of the fused
[dgamma|dbeta] buffer and of the {loss sum, weight sum} pair.  The operators are supplied by a
CPU stand-in built on the oracle (the product has no CPU path); what is under test is the
host-side sharding logic, which is identical on GPUs."""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent

from b200norm import shard  # noqa: E402


def test_shard_rows_cover_everything_once():
    for m in (0, 1, 7, 16, 65536, 65537):
        for world in (1, 2, 3, 4, 8):
            spans = [shard.shard_rows(m, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == m
            for a, b in zip(spans, spans[1:]):
                assert a[1] == b[0]
            sizes = [e - s for s, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard.shard_rows(4, 2, 2)


class OracleOps:
    """CPU stand-in with the capi interface, for host-logic tests only."""

    def __init__(self):
        from oracle import aten_oracle as ao
        self.ao = ao

    def native_layer_norm(self, x, shape, g, b, eps):
        return torch.ops.aten.native_layer_norm(x, shape, g, b, eps)

    def native_layer_norm_backward(self, dy, x, shape, mean, rstd, g, b, mask, out=None):
        dx, dg, db = torch.ops.aten.native_layer_norm_backward(dy, x, shape, mean, rstd, g, b, list(mask))
        if out is not None:
            if out[1] is not None:
                out[1].copy_(dg)
            if out[2] is not None:
                out[2].copy_(db)
        return dx, dg, db

    def _fused_rms_norm(self, x, shape, w, eps):
        return self.ao.rms_norm_fwd(x, shape, w, eps)

    def _fused_rms_norm_backward(self, dy, x, shape, rstd, w, mask, out=None):
        dx, dw = self.ao.rms_norm_bwd(dy, x, shape, w, 1e-6)
        if out is not None and out[1] is not None:
            out[1].copy_(dw)
        return dx, dw

    def _log_softmax(self, x, dim, h2f):
        return torch.ops.aten._log_softmax(x, dim, h2f)

    def nll_loss_forward(self, logp, t, w, red, ign, return_sums=False):
        out, tw = torch.ops.aten.nll_loss_forward(logp, t, w, red, ign)
        sums = torch.stack([out.float(), tw.float()])
        return out, tw, sums

    def nll_loss_backward(self, g, logp, t, w, red, ign, tw):
        return torch.ops.aten.nll_loss_backward(g, logp, t, w, red, ign, tw)

    def _log_softmax_backward_data(self, g, y, dim, dt):
        return torch.ops.aten._log_softmax_backward_data(g, y, dim, dt)

    def cross_entropy_backward(self, g, logp, t, w, red, ign, tw):
        from oracle import aten_oracle as ao
        return ao.cross_entropy_bwd(g, logp, t, w, red, ign, tw)


def _worker(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "torch-xpu-ops_b200"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import aten_oracle as ao
        ops = OracleOps()
        M, N = 37, 48  # odd row count: ragged shards
        x, dy = ao.randn((M, N), 1), ao.randn((M, N), 2)
        g, b = ao.randn((N,), 3, mean=1.0, std=0.02), ao.randn((N,), 4, std=0.02)
        s, e = shard.shard_rows(M, world, rank)
        res = shard.layer_norm_step(ops, x[s:e], dy[s:e], g, b, 1e-5)
        y, mean, rstd = torch.ops.aten.native_layer_norm(x, [N], g, b, 1e-5)
        dx, dg, db = torch.ops.aten.native_layer_norm_backward(dy, x, [N], mean, rstd, g, b, [True, True, True])
        assert torch.allclose(res.y, y[s:e]) and torch.allclose(res.dx, dx[s:e], atol=1e-6)
        assert torch.allclose(res.wgrad[0], dg, rtol=1e-5, atol=1e-5) and torch.allclose(res.wgrad[1], db, rtol=1e-5, atol=1e-5)

        res = shard.rms_norm_step(ops, x[s:e], dy[s:e], g, 1e-6)
        _, dw = ao.rms_norm_bwd(dy, x, [N], g, 1e-6)
        assert torch.allclose(res.wgrad[0], dw, rtol=1e-5, atol=1e-5) and float(res.wgrad[1].abs().sum()) == 0.0
        # a caller's reused buffer may hold anything: the dbeta row still comes back as zeros
        dirty = torch.full((2, N), 7.0)
        res = shard.rms_norm_step(ops, x[s:e], dy[s:e], g, 1e-6, wgrad_buf=dirty)
        assert torch.allclose(res.wgrad[0], dw, rtol=1e-5, atol=1e-5) and float(res.wgrad[1].abs().sum()) == 0.0

        V = 29
        logits = ao.randn((M, V), 5, std=2.0)
        t = ao.randint(V, (M,), 6)
        t[5] = -100
        ce = shard.cross_entropy_step(ops, logits[s:e], t[s:e], -100)
        lg = logits.clone().requires_grad_(True)
        loss = torch.nn.functional.cross_entropy(lg, t, ignore_index=-100)
        loss.backward()
        assert abs(float(ce.loss) - float(loss)) < 1e-5
        assert torch.allclose(ce.dlogits, lg.grad[s:e], atol=1e-6)
        assert float(ce.sums[1]) == M - 1
        cef = shard.cross_entropy_step(ops, logits[s:e], t[s:e], -100, fused=True)
        assert abs(float(cef.loss) - float(loss)) < 1e-5 and torch.allclose(cef.dlogits, lg.grad[s:e], atol=1e-6)
        (Path(tmp) / f"ok{rank}").write_text("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_rank_gloo(tmp_path):
    import socket
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
