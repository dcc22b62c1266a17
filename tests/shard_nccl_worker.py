"""One rank of the two-GPU sharding test (launched by tests/test_gpu_shard_nccl.py through torch.distributed.run).

Each rank runs shard.layer_norm_step, shard.rms_norm_step and shard.cross_entropy_step (plain and fused) on its
row block over NCCL; rank 0 then runs the same operators unsharded and compares: per-row results must be
bit-identical (rows are independent), the all-reduced sums within 1e-6 of the L1 norm of their terms."""
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "torch-xpu-ops_b200"):
    sys.path.insert(0, str(p))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from b200norm import capi, shard
    from oracle import aten_oracle as ao

    M, N = 4099, 8192  # odd row count: ragged shards
    x, dy = ao.randn((M, N), 11, torch.bfloat16).to(dev), ao.randn((M, N), 12, torch.bfloat16).to(dev)
    g, b = ao.randn((N,), 13, mean=1.0, std=0.02).to(dev), ao.randn((N,), 14, std=0.02).to(dev)
    s, e = shard.shard_rows(M, world, rank)
    res = shard.layer_norm_step(capi, x[s:e].contiguous(), dy[s:e].contiguous(), g, b, 1e-5)
    rres = shard.rms_norm_step(capi, x[s:e].contiguous(), dy[s:e].contiguous(), g, 1e-6,
                               wgrad_buf=torch.full((2, N), 3.0, device=dev))
    V = 50264
    logits = ao.randn((257, V), 15, torch.bfloat16, std=2.0).to(dev)
    t = ao.randint(V, (257,), 16).to(dev)
    t[5] = -100
    cs, ce_ = shard.shard_rows(257, world, rank)
    ce = shard.cross_entropy_step(capi, logits[cs:ce_].contiguous(), t[cs:ce_].contiguous(), -100)
    cef = shard.cross_entropy_step(capi, logits[cs:ce_].contiguous(), t[cs:ce_].contiguous(), -100, fused=True)
    torch.cuda.synchronize()
    assert capi.device_status() == 0

    # unsharded, on every rank (cheap), compared with this rank's block and the reduced sums
    y, mean, rstd = capi.native_layer_norm(x, [N], g, b, 1e-5)
    dx, dg, db = capi.native_layer_norm_backward(dy, x, [N], mean, rstd, g, b)
    assert torch.equal(res.y, y[s:e]) and torch.equal(res.dx, dx[s:e]), "per-row results depend on the sharding"
    xh = (x.double() - mean.double().view(-1, 1)) * rstd.double().view(-1, 1)
    tg, tb = dy.double() * xh, dy.double()
    for got, terms, what in ((res.wgrad[0], tg, "dgamma"), (res.wgrad[1], tb, "dbeta")):
        err = float(((got.double() - terms.sum(0)).abs() / terms.abs().sum(0)).max())
        assert err <= 1e-6, f"{what}: {err:.2e} of L1 after the all-reduce"
    ry, rr = capi._fused_rms_norm(x, [N], g, 1e-6)
    rdx, rdw = capi._fused_rms_norm_backward(dy, x, [N], rr, g)
    assert torch.equal(rres.y, ry[s:e]) and torch.equal(rres.dx, rdx[s:e])
    tw = dy.double() * x.double() * rr.double().view(-1, 1)
    assert float(((rres.wgrad[0].double() - tw.sum(0)).abs() / tw.abs().sum(0)).max()) <= 1e-6
    assert float(rres.wgrad[1].abs().sum()) == 0.0

    # the library's own fold + all-reduce kernel over peer memory: several generations, against the fp64 sums and
    # bit-identical on every rank (all ranks add the ranks' slices in the same order)
    from b200norm.peer import WgradExchange
    for ctas in (128, 4):
        ex = WgradExchange(N, dev, ctas=ctas)
        for it in range(5):
            xs, dys = x[s:e].contiguous(), (dy[s:e] * float(1 << it)).contiguous()  # powers of two: exact in bf16
            _, m_, r_ = capi.native_layer_norm(xs, [N], g, b, 1e-5)
            _, ws, rows = capi.native_layer_norm_backward_partials(dys, xs, [N], m_, r_, g)
            wg = torch.full((2, N), float("nan"), device=dev)
            ex.fold_allreduce(ws, rows, wg[0], wg[1])
            torch.cuda.synchronize()
            for got, terms, what in ((wg[0], tg * float(1 << it), "dgamma"), (wg[1], tb * float(1 << it), "dbeta")):
                err = float(((got.double() - terms.sum(0)).abs() / terms.abs().sum(0)).max())
                assert err <= 1e-6, f"fused exchange, {ctas} CTAs, call {it}, {what}: {err:.2e} of L1"
            both = [torch.empty_like(wg) for _ in range(world)]
            dist.all_gather(both, wg)
            assert all(torch.equal(both[0], o) for o in both[1:]), "ranks disagree bit-wise after the fused exchange"
        assert capi.device_status() == 0
        ex.close()

    # the whole batch on this GPU alone, straight through the operators (no exchange)
    logp = capi._log_softmax(logits, -1, False)
    _, _, sums = capi.nll_loss_forward(logp, t, None, 2, -100, return_sums=True)
    full_loss = float(sums[0] / sums[1])
    one = torch.ones((), dtype=logp.dtype, device=dev)
    full_dlogits = capi.cross_entropy_backward(one, logp, t, None, 1, -100, sums[1].to(logp.dtype))
    assert abs(float(ce.loss) - full_loss) <= 1e-6 * abs(full_loss), (float(ce.loss), full_loss)
    assert float(ce.sums[1]) == 256.0 and float(sums[1]) == 256.0
    assert torch.equal(cef.dlogits, full_dlogits[cs:ce_])
    ref = ao.cross_entropy_bwd(one, logp[cs:ce_], t[cs:ce_], None, 1, -100, sums[1].to(logp.dtype))
    assert ao.lowp_mismatch(ce.dlogits, ref)[0] == 0
    torch.cuda.synchronize()
    dist.barrier()
    print(f"rank {rank}: shard check ok", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
