"""Row-sharded data-parallel driver for the operator family (one process per GPU).

Every operator on this path is independent per row, so a large workload splits into contiguous,
even row blocks, one per rank, with no data-path collective.  Only two things are sums over ALL
rows and need one exchange step each:

* the weight gradients dgamma/dbeta of layer norm / RMS norm — the ranks' partial sums live in one
  fused fp32 ``[2, N]`` buffer that a single all-reduce(SUM) turns into the global gradient;
* the scalar loss of ``log_softmax + nll_loss`` — a fp32 ``[2]`` buffer {sum of -w*logp, sum of w}
  is all-reduced, and the mean is taken over the GLOBAL weight on every rank.

The collective is ``torch.distributed.all_reduce`` (NCCL over NVLink on GPUs; gloo in the CPU
tests), enqueued on the compute stream right behind the kernel that produced the buffer.  The
reference has no counterpart: there, sharding these ops is left to DDP/FSDP over its c10d backend,
whose all-reduce(SUM) contract (src/xccl/ProcessGroupXCCL.cpp:1327-1344) is the one relied on here.

``ops`` is the module that supplies the operators (``b200norm.capi`` in production).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.distributed as dist


def shard_rows(num_rows: int, world_size: int, rank: int) -> Tuple[int, int]:
    """[start, end) of the contiguous row block of `rank`; the first `num_rows % world_size` ranks get one more."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank/world_size: {rank}/{world_size}")
    base, rem = divmod(num_rows, world_size)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def _world(group) -> int:
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def all_reduce_sum_(buf: torch.Tensor, group=None) -> torch.Tensor:
    """In-place SUM over ranks (no-op for a single process)."""
    if _world(group) > 1:
        dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=group)
    return buf


@dataclass
class NormStepResult:
    y: torch.Tensor
    dx: torch.Tensor
    wgrad: torch.Tensor  # fp32 [2, N]: row 0 = dgamma, row 1 = dbeta (zeros for RMS norm), summed over ranks
    ready: Optional["torch.cuda.Event"] = None  # set when the gradient exchange ran on a side stream: wait for it
                                                # (stream.wait_event) before reading `wgrad`


def layer_norm_step(ops, x_shard, dy_shard, gamma, beta, eps: float, group=None,
                    wgrad_buf: Optional[torch.Tensor] = None, side_stream=None) -> NormStepResult:
    """Forward + backward of native_layer_norm on this rank's rows, then ONE all-reduce of [dgamma|dbeta].

    side_stream: a second CUDA stream.  The weight-gradient fold and the all-reduce are then enqueued there,
    behind an event recorded after the backward's row kernels, so that whatever the caller launches next on its
    own stream follows those row kernels directly; the result carries `ready`, the event to wait for before
    `wgrad` is read (and before the workspace behind it is reused)."""
    n = x_shard.shape[-1]
    y, mean, rstd = ops.native_layer_norm(x_shard, [n], gamma, beta, eps)
    if wgrad_buf is None:
        wgrad_buf = torch.empty(2, n, dtype=torch.float32, device=x_shard.device)
    if side_stream is not None and gamma.dtype == torch.float32:
        dx, ws, rows = ops.native_layer_norm_backward_partials(dy_shard, x_shard, [n], mean, rstd, gamma)
        main = torch.cuda.current_stream(x_shard.device)
        after_rows = torch.cuda.Event()
        after_rows.record(main)
        side_stream.wait_event(after_rows)
        with torch.cuda.stream(side_stream):
            ops.norm_wgrad_fold(ws, rows, x_shard.dtype, wgrad_buf[0], wgrad_buf[1])
            all_reduce_sum_(wgrad_buf, group)
            ready = torch.cuda.Event()
            ready.record(side_stream)
        for t in (ws, wgrad_buf, mean, rstd):
            t.record_stream(side_stream)
        return NormStepResult(y, dx, wgrad_buf, ready)
    if gamma.dtype == torch.float32:
        # the fold kernel writes dgamma | dbeta straight into the buffer the collective sends
        dx, _, _ = ops.native_layer_norm_backward(dy_shard, x_shard, [n], mean, rstd, gamma, beta,
                                                  (True, True, True), out=(None, wgrad_buf[0], wgrad_buf[1]))
    else:
        dx, dgamma, dbeta = ops.native_layer_norm_backward(dy_shard, x_shard, [n], mean, rstd, gamma, beta,
                                                           (True, True, True))
        wgrad_buf[0].copy_(dgamma)
        wgrad_buf[1].copy_(dbeta)
    all_reduce_sum_(wgrad_buf, group)
    return NormStepResult(y, dx, wgrad_buf)


def rms_norm_step(ops, x_shard, dy_shard, weight, eps: float, group=None,
                  wgrad_buf: Optional[torch.Tensor] = None) -> NormStepResult:
    n = x_shard.shape[-1]
    y, rstd = ops._fused_rms_norm(x_shard, [n], weight, eps)
    if wgrad_buf is None:
        wgrad_buf = torch.empty(2, n, dtype=torch.float32, device=x_shard.device)
    wgrad_buf[1].zero_()  # RMS norm has no dbeta: the row is zeros whatever a reused buffer held before
    if weight.dtype == torch.float32:
        dx, _ = ops._fused_rms_norm_backward(dy_shard, x_shard, [n], rstd, weight, (True, True),
                                             out=(None, wgrad_buf[0]))
    else:
        dx, dw = ops._fused_rms_norm_backward(dy_shard, x_shard, [n], rstd, weight, (True, True))
        wgrad_buf[0].copy_(dw)
    all_reduce_sum_(wgrad_buf, group)
    return NormStepResult(y, dx, wgrad_buf)


@dataclass
class CrossEntropyStepResult:
    loss: torch.Tensor       # fp32 scalar: global mean loss (identical on every rank)
    logp: torch.Tensor       # this rank's log-probabilities
    dlogits: torch.Tensor    # this rank's gradient w.r.t. its logits, for d(loss) = 1
    sums: torch.Tensor       # fp32 [2] after the all-reduce: {sum -w*logp, sum w}


def cross_entropy_step(ops, logits_shard, target_shard, ignore_index: int = -100, group=None,
                       fused: bool = False) -> CrossEntropyStepResult:
    """_log_softmax + nll_loss_forward(mean) + both backward ops on this rank's rows.

    The loss is a mean over the GLOBAL weight: the per-rank {loss sum, weight sum} pair is
    all-reduced first, and the backward scatters -1/total_weight with that global total.
    fused=True replaces the two backward operators by the one-pass ``cross_entropy_backward``
    (no dense gradient of the log-probabilities in between); the result is the same.
    """
    logp = ops._log_softmax(logits_shard, -1, False)
    # reduction "sum" locally; the division happens after the exchange
    _, _, sums = ops.nll_loss_forward(logp, target_shard, None, 2, ignore_index, return_sums=True)
    all_reduce_sum_(sums, group)
    loss = sums[0] / sums[1]
    total_weight = sums[1].to(logp.dtype)
    one = torch.ones((), dtype=logp.dtype, device=logp.device)
    if fused:
        dlogits = ops.cross_entropy_backward(one, logp, target_shard, None, 1, ignore_index, total_weight)
    else:
        grad_logp = ops.nll_loss_backward(one, logp, target_shard, None, 1, ignore_index, total_weight)
        dlogits = ops._log_softmax_backward_data(grad_logp, logp, -1, logits_shard.dtype)
    return CrossEntropyStepResult(loss, logp, dlogits, sums)
