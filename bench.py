#!/usr/bin/env python
"""Throughput benchmark of the normalization / softmax path.

    python bench.py --gpus N --steps K --warmup W [--workload cfg4] [--impl reference]

One "step" is one pass of the workload's operators over one batch of seeded synthetic input.  The
default workload is BASELINE config 4: native_layer_norm forward + backward (dx, dgamma, dbeta) on
bf16 [65536, 8192] with fp32 gamma/beta, rows sharded evenly over the N ranks (strong scaling), the
fused fp32 [2, 8192] dgamma|dbeta buffer all-reduced over NCCL each step.  Other workloads
(--workload cfg1|cfg2|cfg3|cfg5) run the other BASELINE configs the same way; cfg5f is config 5 with the fused
cross-entropy backward, cfg3m config 3 with the mask inside the kernels, ln_long layer norm on rows of 16384,
gn a GroupNorm forward, bn batch_norm_stats, sm_c19|sm_c64|sm_c150 softmax over dim 1 of bf16 [16, C, 512, 512].

Prints ONE JSON line (rank 0).  `value` is algorithmic bytes (every tensor of the operators'
signatures read or written once) of all ranks / device time, inputs resident in HBM; `e2e` is the
same metric through the ATen dispatcher with pinned HOST buffers, copies inside the timed region.
`--impl reference` times PyTorch's CPU ATen kernels (the reference path's parity standard, and the
only implementation of it that runs on this box) on the host cores over the same rows.

Timing.  A timed region is EXACTLY --steps steps between two CUDA events on the launching stream, a
barrier and a device synchronisation on both sides, the maximum over ranks.  A region shorter than
50 ms is repeated (9 regions, back to back): `ms_per_step` is then the median region and `spread`
gives the fastest and slowest.  `host_enqueue_us_per_step` is the host time the un-synchronised step
loop took, `collective_us` one in-stream all-reduce of the step's buffer between its own events.

Steps are enqueued through prepared C-ABI calls (arguments converted once) and, with --graph on
(the default wherever a workload supports it), replayed from a CUDA graph holding one cycle of the
workload's rotating buffers — the kernels, their dependent-launch edges and the NCCL all-reduce on
its side stream — so the host's speed does not enter the device-timed number.

With the default workload on one GPU the line also carries `configs`: a short run of every other
BASELINE config (and cfg5f) with its own value and per-kernel roofline.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for _p in (ROOT, ROOT / "torch-xpu-ops_b200"):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
METRIC = "norm/softmax HBM GB/s"


# --------------------------------------------------------------------------------------------------
# workloads: sizes and algorithmic bytes (every tensor of the op signatures read or written once)
# --------------------------------------------------------------------------------------------------
class Workload:
    name = ""
    rows = 0          # global rows that get sharded
    cpu_sample_rows = 0

    def describe(self) -> str:
        raise NotImplementedError

    def bytes_per_rows(self, rows: int) -> dict:
        """{'total': bytes per step over `rows` rows, kernel name: bytes per launch of that kernel}"""
        raise NotImplementedError


class Cfg4LayerNorm(Workload):
    name, rows, N, cpu_sample_rows = "cfg4", 65536, 8192, 65536
    kernel = "layer_norm_bwd_ring"
    l2_note = "inputs larger than L2 (no flush needed)"
    cycle = 2  # steps after which the rotating buffers repeat (the two gradient buffers)

    def describe(self):
        return ("native_layer_norm fwd + native_layer_norm_backward (dx, dgamma, dbeta), bf16 "
                f"[{self.rows}, {self.N}], fp32 gamma/beta, eps 1e-5")

    def bytes_per_rows(self, rows):
        n = self.N
        fwd = 2 * rows * n * 2 + 2 * n * 4 + 2 * rows * 4
        bwd = 3 * rows * n * 2 + 2 * rows * 4 + n * 4 + 2 * n * 4
        return {"total": fwd + bwd, "layer_norm_fwd_ring": fwd, "layer_norm_bwd_ring": bwd,
                "layer_norm_fwd_slab": fwd, "layer_norm_bwd_slab": bwd, "layer_norm_fwd_ring2w": fwd,
                "layer_norm_fwd_generic": fwd, "layer_norm_bwd_dx_generic": bwd}

    def make_device_state(self, rows, dev, seed):
        g = torch.Generator(device=dev).manual_seed(seed)
        n = self.N
        st = {}
        st["x"] = torch.randn((rows, n), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
        st["dy"] = torch.randn((rows, n), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
        cg = torch.Generator().manual_seed(4002)
        st["gamma"] = (torch.randn(n, generator=cg) * 0.02 + 1.0).to(dev)
        st["beta"] = (torch.randn(n, generator=cg) * 0.02).to(dev)
        st["y"] = torch.empty_like(st["x"])
        st["dx"] = torch.empty_like(st["x"])
        st["mean"] = torch.empty(rows, device=dev, dtype=torch.float32)
        st["rstd"] = torch.empty(rows, device=dev, dtype=torch.float32)
        # two gradient buffers: the all-reduce of step i runs on NCCL's stream while step i+1 computes
        st["wgrads"] = [torch.empty((2, n), device=dev, dtype=torch.float32) for _ in range(2)]
        st["works"] = [None, None]
        st["k"] = 0
        from b200norm import F32, BF16, load_library
        nbytes = load_library().b2n_norm_bwd_workspace_bytes(rows, n, BF16, F32, 1)
        st["ws"] = torch.empty(max(nbytes, 1), device=dev, dtype=torch.uint8)
        # "exchange-side": the backward folds into these, the exchange kernel on the second stream reduces them
        # over the ranks into st["wgrads"]
        st["wlocal"] = [torch.empty((2, n), device=dev, dtype=torch.float32) for _ in range(2)] if COLLECTIVE_MODE == "exchange-side" else None
        st["side"] = torch.cuda.Stream(dev)
        st["pending"] = [None, None]
        return st

    def open_exchange(self, st, dev, sm_margin):
        """(collective) the peer-memory exchange buffers of the fused fold + all-reduce kernel."""
        from b200norm.peer import WgradExchange
        ctas = 128 if COLLECTIVE_MODE == "fused" else max(1, sm_margin)
        st["exch"] = WgradExchange(self.N, dev, ctas=ctas)

    def prepare(self, capi, st):
        """Prepared C-ABI calls (pointers and sizes converted once) on the CURRENT stream."""
        st["fwd"] = capi.prepare_layer_norm(st["x"], st["gamma"], st["beta"], 1e-5, st["y"], st["mean"], st["rstd"])
        if COLLECTIVE_MODE == "fused":
            # row kernels, then ONE kernel that folds the partial sums and adds the ranks' results over peer memory
            st["bwd"], st["exc"] = [], []
            for wg in st["wgrads"]:
                call, rows = capi.prepare_norm_backward_partials(False, st["dy"], st["x"], st["mean"], st["rstd"],
                                                                 st["gamma"], st["dx"], st["ws"])
                st["bwd"].append(call)
                st["exc"].append(st["exch"].prepare(st["ws"], rows, wg[0], wg[1]))
            return
        if COLLECTIVE_MODE == "exchange-side":
            # the ordinary backward (row kernels + fold) into a local buffer; the same peer-memory kernel, given that
            # buffer as ONE partial row, adds the ranks' buffers on the second stream
            st["bwd"] = [capi.prepare_layer_norm_backward(st["dy"], st["x"], st["mean"], st["rstd"], st["gamma"], st["dx"],
                                                          wl[0], wl[1], st["ws"]) for wl in st["wlocal"]]
            with torch.cuda.stream(st["side"]):
                st["exc"] = [st["exch"].prepare(wl, 1, wg[0], wg[1]) for wl, wg in zip(st["wlocal"], st["wgrads"])]
            return
        st["bwd"] = [capi.prepare_layer_norm_backward(st["dy"], st["x"], st["mean"], st["rstd"], st["gamma"], st["dx"],
                                                      wg[0], wg[1], st["ws"]) for wg in st["wgrads"]]

    def _fused_step(self, st, k, main, side):
        """Backward on `main`; the peer-memory kernel behind it on `main` ("fused": fold + exchange) or on `side`
        ("exchange-side": exchange only, joined before buffer k is written again)."""
        if st["pending"][k] is not None:
            main.wait_event(st["pending"][k])
            st["pending"][k] = None
        st["fwd"]()
        st["bwd"][k]()
        if COLLECTIVE_MODE == "fused":
            st["exc"][k]()
            return
        ready = torch.cuda.Event()
        ready.record(main)
        side.wait_event(ready)
        with torch.cuda.stream(side):
            st["exc"][k]()
            done = torch.cuda.Event()
            done.record(side)
        st["pending"][k] = done

    def step(self, capi, st, world):
        k = st["k"] = st["k"] ^ 1
        if COLLECTIVE_MODE in ("fused", "exchange-side"):
            self._fused_step(st, k, torch.cuda.current_stream(), st["side"])
            return
        if st["works"][k] is not None:
            st["works"][k].wait()  # stream-level: the buffer's previous all-reduce precedes its reuse
            st["works"][k] = None
        st["fwd"]()
        st["bwd"][k]()
        if world > 1 and COLLECTIVE_MODE != "none":
            # one all-reduce(SUM) of the fused [dgamma | dbeta] buffer the backward just wrote; asynchronous,
            # so it overlaps the next step's forward (nothing reads the reduced gradients inside the step)
            if COLLECTIVE_MODE == "async":
                st["works"][k] = dist.all_reduce(st["wgrads"][k], async_op=True)
            else:
                dist.all_reduce(st["wgrads"][k])

    def capture_cycle(self, capi, st, world, cs, side, cycles=1):
        """Enqueue `cycles` cycles (of two steps) on the capturing stream `cs`; each step's all-reduce goes to `side`
        and is joined where its buffer is next written, or — the last two — at the end.  (A graph is a unit: what is
        still running on `side` when its last step ends cannot overlap the next replay, so the more steps one graph
        holds, the smaller the share of that un-overlapped tail.)"""
        if COLLECTIVE_MODE in ("fused", "exchange-side"):
            # the exchange calls of "exchange-side" were prepared on st["side"]; `side` is not used
            for _ in range(cycles):
                for k in (1, 0):
                    self._fused_step(st, k, cs, st["side"])
            for k in (0, 1):
                if st["pending"][k] is not None:
                    cs.wait_event(st["pending"][k])
                    st["pending"][k] = None
            return
        pending = [None, None]
        for k in [1, 0] * cycles:
            if pending[k] is not None:
                cs.wait_event(pending[k])
                pending[k] = None
            st["fwd"]()
            st["bwd"][k]()
            if world > 1 and COLLECTIVE_MODE != "none":
                if COLLECTIVE_MODE == "async":
                    ready = torch.cuda.Event()
                    ready.record(cs)
                    side.wait_event(ready)
                    with torch.cuda.stream(side):
                        dist.all_reduce(st["wgrads"][k])
                        done = torch.cuda.Event()
                        done.record(side)
                    pending[k] = done
                else:
                    dist.all_reduce(st["wgrads"][k])
        for ev in pending:
            if ev is not None:
                cs.wait_event(ev)

    def collective_buffer(self, st):
        return st["wgrads"][0]

    def finish(self, st):
        for k in (0, 1):
            if st["pending"][k] is not None:
                torch.cuda.current_stream().wait_event(st["pending"][k])
                st["pending"][k] = None
        for i, w in enumerate(st["works"]):
            if w is not None:
                w.wait()
                st["works"][i] = None

    launches_per_step = 3  # forward ring kernel, backward ring kernel, partial-sum fold

    def shard_check(self, capi, st, world, rank, rows_of):
        """After a multi-GPU run: the all-reduced [dgamma | dbeta] against the sum, taken in fp64 on rank 0, of
        the same operators run block by block over every rank's rows (same seeds).  L1-relative error."""
        n = self.N
        self.finish(st)
        got = st["wgrads"][st["k"]].clone()
        torch.cuda.synchronize()
        err = None
        if rank == 0:
            dev = got.device
            total = torch.zeros((2, n), dtype=torch.float64, device=dev)
            for r in range(world):
                rows = rows_of(r)
                blk = st if r == 0 else self.make_device_state(rows, dev, seed=4001 + r)
                wg = torch.empty((2, n), device=dev, dtype=torch.float32)
                _, mean, rstd = capi.native_layer_norm(blk["x"], [n], blk["gamma"], blk["beta"], 1e-5)
                capi.native_layer_norm_backward(blk["dy"], blk["x"], [n], mean, rstd, blk["gamma"], blk["beta"],
                                                (True, True, True), out=(None, wg[0], wg[1]))
                total += wg.double()
                del blk
            err = {"dgamma_l1_err": float((got[0].double() - total[0]).abs().sum() / total[0].abs().sum()),
                   "dbeta_l1_err": float((got[1].double() - total[1]).abs().sum() / total[1].abs().sum()),
                   "what": "all-reduced [dgamma|dbeta] of the last step vs the fp64 sum of every rank's block, "
                           "recomputed on rank 0"}
        return err

    def cpu_step(self, cpu):
        n = self.N
        y, mean, rstd = torch.ops.aten.native_layer_norm(cpu["x"], [n], cpu["gamma"], cpu["beta"], 1e-5)
        return torch.ops.aten.native_layer_norm_backward(cpu["dy"], cpu["x"], [n], mean, rstd, cpu["gamma"],
                                                         cpu["beta"], [True, True, True])

    def make_cpu_state(self, rows):
        g = torch.Generator().manual_seed(4001)
        n = self.N
        cpu = {k: torch.empty((rows, n), dtype=torch.bfloat16) for k in ("x", "dy")}
        blk = 4096
        for k in ("x", "dy"):  # in row blocks: the fp32 draw of the whole tensor would be 2 GiB at a time
            for r in range(0, rows, blk):
                cpu[k][r:r + blk] = torch.randn((min(blk, rows - r), n), generator=g).to(torch.bfloat16)
        cpu["gamma"] = torch.randn(n, generator=g) * 0.02 + 1.0
        cpu["beta"] = torch.randn(n, generator=g) * 0.02
        return cpu

    # ---- end to end through the ATen dispatcher, host buffers, chunked so copies overlap kernels ----
    e2e_chunks = 8  # more chunks change nothing: both PCIe directions are busy for the whole step (measured with 32)

    def make_e2e_state(self, rows, dev):
        n = self.N
        host = {k: torch.empty((rows, n), dtype=torch.bfloat16).pin_memory() for k in ("x", "dy", "y", "dx")}
        g = torch.Generator().manual_seed(4001)
        blk = 4096
        for k in ("x", "dy"):
            for r in range(0, rows, blk):
                host[k][r:r + blk] = torch.randn((min(blk, rows - r), n), generator=g).to(torch.bfloat16)
        host["wgrad"] = torch.empty((2, n), dtype=torch.float32).pin_memory()
        crow = (rows + self.e2e_chunks - 1) // self.e2e_chunks
        devb = {k: [torch.empty((crow, n), device=dev, dtype=torch.bfloat16) for _ in range(2)] for k in ("x", "dy")}
        return {"host": host, "dev": devb, "crow": crow, "rows": rows,
                "streams": [torch.cuda.Stream(dev) for _ in range(3)]}

    def cpu_state_from_e2e(self, e2e):
        """The pinned host inputs of the end-to-end arm double as the CPU arm's inputs (same seed, same rows)."""
        g = torch.Generator().manual_seed(4002)
        n = self.N
        return {"x": e2e["host"]["x"], "dy": e2e["host"]["dy"], "gamma": torch.randn(n, generator=g) * 0.02 + 1.0,
                "beta": torch.randn(n, generator=g) * 0.02}

    def e2e_step(self, st, e2e, world):
        n, rows, crow = self.N, e2e["rows"], e2e["crow"]
        h2d, comp, d2h = e2e["streams"]
        host, devb = e2e["host"], e2e["dev"]
        wgrad = torch.zeros((2, n), device=st["gamma"].device, dtype=torch.float32)
        cur = torch.cuda.current_stream()
        for s in (h2d, comp, d2h):
            s.wait_stream(cur)
        free_evt = [None, None]   # staging slot reusable once its chunk's compute has consumed it
        keep = []
        for c, r0 in enumerate(range(0, rows, crow)):
            r1 = min(rows, r0 + crow)
            slot = c & 1
            with torch.cuda.stream(h2d):
                if free_evt[slot] is not None:
                    h2d.wait_event(free_evt[slot])
                xs, dys = devb["x"][slot][: r1 - r0], devb["dy"][slot][: r1 - r0]
                xs.copy_(host["x"][r0:r1], non_blocking=True)
                dys.copy_(host["dy"][r0:r1], non_blocking=True)
                loaded = torch.cuda.Event()
                loaded.record(h2d)
            with torch.cuda.stream(comp):
                comp.wait_event(loaded)
                y, mean, rstd = torch.ops.aten.native_layer_norm(xs, [n], st["gamma"], st["beta"], 1e-5)
                dx, dg, db = torch.ops.aten.native_layer_norm_backward(dys, xs, [n], mean, rstd, st["gamma"], st["beta"],
                                                                       [True, True, True])
                wgrad[0] += dg
                wgrad[1] += db
                done = torch.cuda.Event()
                done.record(comp)
                free_evt[slot] = done
            with torch.cuda.stream(d2h):
                d2h.wait_event(done)
                host["y"][r0:r1].copy_(y, non_blocking=True)
                host["dx"][r0:r1].copy_(dx, non_blocking=True)
                y.record_stream(d2h)
                dx.record_stream(d2h)
            keep.append((y, dx))
        with torch.cuda.stream(comp):
            if world > 1:
                dist.all_reduce(wgrad)
            host["wgrad"].copy_(wgrad, non_blocking=True)
        cur = torch.cuda.current_stream()
        cur.wait_stream(comp)
        cur.wait_stream(d2h)
        return keep

    def e2e_bytes(self, rows):
        n = self.N
        return 2 * rows * n * 2, 2 * rows * n * 2 + 2 * n * 4


COLLECTIVE_MODE = "async"  # set from --collective in main()
WORKLOADS = {"cfg4": Cfg4LayerNorm}


def _load_more_workloads():
    from bench_workloads import EXTRA, layer_norm_long_rows  # noqa: WPS433  (a sibling module, to keep this file readable)
    WORKLOADS.update(EXTRA)
    WORKLOADS["ln_long"] = layer_norm_long_rows(Cfg4LayerNorm)


# --------------------------------------------------------------------------------------------------
# clocks during the timed region (read-only NVML queries)
# --------------------------------------------------------------------------------------------------
REASON_BITS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
               0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}


class ClockSampler(threading.Thread):
    def __init__(self, device: torch.device, period_s: float = 0.004):
        super().__init__(daemon=True)
        self.period, self.samples, self._stop_evt = period_s, [], threading.Event()
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            props = torch.cuda.get_device_properties(device)
            try:  # the NVML handle of THIS CUDA device, whatever CUDA_VISIBLE_DEVICES says
                self.h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(props.uuid)).encode())
            except Exception:  # noqa: BLE001
                self.h = pynvml.nvmlDeviceGetHandleByIndex(device.index or 0)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        while not self._stop_evt.is_set():
            try:
                mhz = self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM)
                try:
                    reasons = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:  # noqa: BLE001
                    reasons = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((time.perf_counter(), mhz, reasons))
            except Exception:  # noqa: BLE001
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop_evt.set()

    def summary(self, t0: float, t1: float) -> dict:
        inside = [(m, r) for (t, m, r) in self.samples if t0 <= t <= t1]
        scope = "timed_region"
        if not inside:  # region shorter than the sampling period: fall back to everything seen under load
            inside = [(m, r) for (_, m, r) in self.samples if not (r & 0x1)]
            scope = "whole_run_under_load"
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0, "scope": "none"}
        mask = 0
        for _, r in inside:
            mask |= r
        reasons = sorted(name for bit, name in REASON_BITS.items() if mask & bit and name != "gpu_idle")
        return {"sm_mhz": statistics.median(m for m, _ in inside), "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(inside), "scope": scope}


# --------------------------------------------------------------------------------------------------
def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:  # noqa: BLE001
            pass
    return FALLBACK_HBM_GBS, "fallback"


def recorded_traffic(kernel: str, units: int, algorithmic_bytes=None):
    """DRAM bytes per launch from the committed ncu capture (profiles/dram_traffic.json; captured on a smaller
    case of the same row length and scaled by rows).  DRAM READS scale with the rows and are taken from the
    capture; DRAM writes of a small capture under-count (part of the output is still dirty in L2 when the kernel
    ends), so where the file gives the split the write side is the algorithmic figure: every output byte must
    reach DRAM eventually.  None when the kernel was not captured."""
    p = ROOT / "profiles" / "dram_traffic.json"
    if not p.exists():
        return None
    try:
        rec = json.loads(p.read_text()).get(kernel, {})
        if "read" in rec and "write_algorithmic" in rec:
            return round((rec["read"] + rec["write_algorithmic"]) * units)
        per_row = rec.get("dram_bytes_per_row")
        return None if per_row is None else per_row * units
    except Exception:  # noqa: BLE001
        return None


def cpu_measure(wl: Workload, cpu=None, budget_s: float = 12.0):
    rows = wl.cpu_sample_rows
    if cpu is None:
        cpu = wl.make_cpu_state(rows)
    torch.set_num_threads(os.cpu_count() or 1)
    wl.cpu_step(cpu)  # warm-up
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 50):
        t0 = time.perf_counter()
        wl.cpu_step(cpu)
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    gbs = wl.bytes_per_rows(rows)["total"] / med / 1e9
    return {"value": round(gbs, 3), "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"PyTorch CPU ATen, {rows} of {wl.rows} rows, median of {len(times)} passes "
                      f"({med * 1e3:.1f} ms each)"}


def run_reference(args, wl: Workload, rank: int):
    """CPU ATen on the host cores; rank 0 only."""
    if rank != 0:
        return
    rows = wl.cpu_sample_rows
    cpu = wl.make_cpu_state(rows)
    torch.set_num_threads(os.cpu_count() or 1)
    for _ in range(max(args.warmup, 1)):
        wl.cpu_step(cpu)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        wl.cpu_step(cpu)
    dt = time.perf_counter() - t0
    gbs = wl.bytes_per_rows(rows)["total"] * args.steps / dt / 1e9
    sample = f"PyTorch CPU ATen on host cores, {rows} of {wl.rows} rows per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": round(gbs, 3), "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16 storage, f32 accumulate",
        "data": "synthetic", "config": {"workload": f"{wl.name}: {wl.describe()}", "global_rows": wl.rows,
                                        "rows_per_step": rows},
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------------
# device timing of one workload
# --------------------------------------------------------------------------------------------------
SHORT_REGION_MS = 50.0
REPEATS = 9
REGION_PAUSE_S = 0.03


def sustained_ms_per_step(runner, steps, world, dev, barrier, regions=REPEATS):
    """The same steps for `regions` regions' worth back to back, no pause: what the step costs once the power cap
    has been reached."""
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(regions):
        runner.run(steps)
    runner.finish()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    return ms / (regions * steps)


class StepRunner:
    """Runs steps of a workload either call by call (prepared C-ABI calls) or by replaying a CUDA graph that holds
    one cycle of the workload's rotating buffers."""

    def __init__(self, wl, capi, st, world, dev, want_graph, steps):
        self.wl, self.capi, self.st, self.world = wl, capi, st, world
        self.graph = None
        self.graph_note = "off"
        self.cycle = getattr(wl, "cycle", 1)
        self.launches_per_step = wl.launches_per_step
        if hasattr(wl, "prepare"):
            wl.prepare(capi, st)
        self.cycles_per_graph = 1
        if want_graph and hasattr(wl, "capture_cycle"):
            if steps % self.cycle == 0:
                # one graph holds the whole region's steps when that is at most 64 of them, else the largest
                # whole number of cycles that divides the region and stays within 64 steps
                n = steps // self.cycle
                per = max(d for d in range(1, n + 1) if n % d == 0 and d * self.cycle <= max(64, self.cycle))
                self.cycles_per_graph = per
                self._capture(dev)
            else:
                self.graph_note = f"off (--steps {steps} is no whole number of {self.cycle}-step cycles)"

    def _capture(self, dev):
        wl, st, world = self.wl, self.st, self.world
        cs, side = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        try:
            with torch.cuda.stream(cs):
                wl.prepare(self.capi, st)        # the prepared calls carry the stream they are to run on
                for _ in range(2):               # warm-up on the capture stream (lazy attribute set-up, NCCL channels)
                    wl.capture_cycle(self.capi, st, world, cs, side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=cs):
                wl.capture_cycle(self.capi, st, world, cs, side, self.cycles_per_graph)
            self.graph = g
            self.graph_note = f"on: one graph per {self.cycles_per_graph * self.cycle} step(s)"
        except Exception as exc:  # noqa: BLE001
            torch.cuda.synchronize()
            self.graph = None
            self.graph_note = f"off (capture failed: {type(exc).__name__}: {str(exc)[:120]})"
            if hasattr(wl, "prepare"):
                wl.prepare(self.capi, st)        # back onto the current stream

    def run(self, steps):
        if self.graph is not None:
            for _ in range(max(1, steps // (self.cycle * self.cycles_per_graph))):
                self.graph.replay()
            return
        for _ in range(steps):
            self.wl.step(self.capi, self.st, self.world)

    def finish(self):
        if hasattr(self.wl, "finish"):
            self.wl.finish(self.st)


def time_regions(runner: StepRunner, steps: int, world: int, dev, barrier):
    """-> (list of region times in ms, max over ranks each; host seconds per region; wall-clock span)"""
    regions, host = [], []
    t_begin = time.perf_counter()
    while True:
        if regions:
            # Every region is a burst from a rested GPU, like the copy that defines the roofline's peak: under a
            # second of back-to-back HBM-bound kernels the 1 kW power cap starts to bite (sw_power_cap) and the
            # same kernels run 3-5 % slower.  What they sustain is reported separately (sustained_ms_per_step).
            time.sleep(REGION_PAUSE_S)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        h0 = time.perf_counter()
        e0.record()
        runner.run(steps)
        runner.finish()  # outstanding collectives join the timed stream before the closing event
        e1.record()
        host.append(time.perf_counter() - h0)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t[0])
        regions.append(ms)
        # every rank takes the same decision: it is made on the all-reduced time of the first region
        if len(regions) >= (REPEATS if regions[0] < SHORT_REGION_MS else 1):
            break
    return regions, host, (t_begin, time.perf_counter())


def profile_kernels(runner: StepRunner, capi, steps: int, barrier):
    """Per-launch CUDA events around every main kernel, call by call (never from the graph: an event pair between
    two kernels also keeps the second from starting under the first's tail, so these are upper bounds)."""
    g, runner.graph = runner.graph, None
    if g is not None and hasattr(runner.wl, "prepare"):
        runner.wl.prepare(capi, runner.st)
    capi.profile_begin()
    runner.run(steps)
    runner.finish()
    prof = capi.profile_end()
    barrier()
    runner.graph = g
    return prof


def copy_gbs_at_size(nbytes: int, dev, iters: int = 40):
    """torch copy_ between rotating buffers of `nbytes` each (read + write bytes / time): the copy figure at THIS
    problem's size, launch latency included, beside the 2 GiB figure the roofline's peak comes from."""
    nbuf = max(2, min(16, (1 << 30) // max(nbytes, 1)))
    src = [torch.empty(nbytes, dtype=torch.uint8, device=dev).fill_(i) for i in range(nbuf)]
    dst = [torch.empty(nbytes, dtype=torch.uint8, device=dev) for _ in range(nbuf)]
    for i in range(nbuf):
        dst[i].copy_(src[i])
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        dst[i % nbuf].copy_(src[i % nbuf])
    e1.record()
    torch.cuda.synchronize()
    return 2 * nbytes * iters / (e0.elapsed_time(e1) * 1e-3) / 1e9


def measure_workload(wl, capi, st, world, rank, dev, steps, warmup, rows, global_rows, scaling, want_graph, barrier):
    runner = StepRunner(wl, capi, st, world, dev, want_graph, steps)
    runner.run(-(-max(warmup, 1) // (runner.cycle * runner.cycles_per_graph)) * runner.cycle * runner.cycles_per_graph)
    runner.finish()
    barrier()
    regions, host, span = time_regions(runner, steps, world, dev, barrier)
    ms = statistics.median(regions)
    status = capi.device_status()
    assert status == 0, f"device status {status}"
    sustained = sustained_ms_per_step(runner, steps, world, dev, barrier) if len(regions) > 1 else None
    time.sleep(REGION_PAUSE_S * 2)
    prof = profile_kernels(runner, capi, min(steps, 50), barrier)
    peak, peak_kind = measured_peak()
    bytes_local = wl.bytes_per_rows(rows)
    kernels = {}
    for name, (n, total_ms) in prof.items():
        us = total_ms / n * 1e3
        entry = {"us_per_launch": round(us, 2), "launches_timed": n}
        if name in bytes_local:
            gbs = bytes_local[name] / (us * 1e-6) / 1e9
            entry.update({"achieved": round(gbs, 1), "frac": round(gbs / peak, 4),
                          "frac_of_nominal_8TBs": round(gbs / NOMINAL_HBM_GBS, 4)})
        kernels[name] = entry
    top = max(prof, key=lambda k: prof[k][1])
    total_bytes = wl.bytes_per_rows(global_rows)["total"] if scaling == "strong" else bytes_local["total"] * world
    out = {
        "ms_per_step": ms / steps, "value": total_bytes * steps / (ms * 1e-3) / 1e9, "total_bytes": total_bytes,
        "spread": {"regions": len(regions), "min_ms_per_step": round(min(regions) / steps, 5),
                   "max_ms_per_step": round(max(regions) / steps, 5), "pause_between_regions_ms": REGION_PAUSE_S * 1e3},
        "host_enqueue_us_per_step": round(statistics.median(host) / steps * 1e6, 2),
        "sustained_ms_per_step": None if sustained is None else round(sustained, 5),
        "graph": runner.graph_note, "kernels": kernels, "top_kernel": top, "peak": peak, "peak_kind": peak_kind,
        "span": span, "launches": runner.launches_per_step * steps * len(regions), "runner": runner,
    }
    return out


def roofline_of(res, wl, rows):
    k = res["kernels"][res["top_kernel"]]
    return {"bound": "hbm", "kernel": res["top_kernel"], "achieved": k.get("achieved"), "peak": res["peak"], "unit": "GB/s",
            "frac": k.get("frac"), "peak_kind": res["peak_kind"], "frac_of_nominal_8TBs": k.get("frac_of_nominal_8TBs"),
            "us_per_launch": k["us_per_launch"], "launches_timed": k["launches_timed"],
            "traffic": recorded_traffic(res["top_kernel"], rows, wl.bytes_per_rows(rows).get(res["top_kernel"])),
            "all_kernels": res["kernels"],
            "note": "per-launch times come from a separate call-by-call pass with an event pair around each launch; "
                    "the step's ms_per_step is the back-to-back figure"}


def collective_time_us(wl, st, world, iters: int = 20):
    """One in-stream all-reduce of the step's buffer between its own events (median of `iters`)."""
    if world <= 1 or not hasattr(wl, "collective_buffer"):
        return None
    buf = wl.collective_buffer(st).clone()
    for _ in range(3):
        dist.all_reduce(buf)
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        dist.all_reduce(buf)
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)
    return round(statistics.median(times), 2)


def run_other_configs(capi, dev, steps_of, barrier):
    """Short runs of the other BASELINE configs on this GPU: value, step time and per-kernel roofline each."""
    _load_more_workloads()
    out = {}
    for name in ("cfg1", "cfg2", "cfg3", "cfg5", "cfg5f", "ln_long", "gn", "bn", "sm_c19", "sm_c64", "sm_c150"):
        if name not in WORKLOADS:
            continue
        wl = WORKLOADS[name]()
        try:
            st = wl.make_device_state(wl.rows, dev, seed=4001)
            steps = steps_of(name)
            res = measure_workload(wl, capi, st, 1, 0, dev, steps, 3, wl.rows, wl.rows, "strong", True, barrier)
            entry = {"workload": wl.describe(), "value": round(res["value"], 1), "unit": "GB/s", "steps": steps,
                     "ms_per_step": round(res["ms_per_step"], 5), "spread": res["spread"],
                     "sustained_ms_per_step": res["sustained_ms_per_step"],
                     "pct_of_peak_measured": round(100 * res["value"] / res["peak"], 2),
                     "pct_of_peak_nominal": round(100 * res["value"] / NOMINAL_HBM_GBS, 2),
                     "graph": res["graph"], "l2": wl.l2_note, "kernels": res["kernels"],
                     "host_enqueue_us_per_step": res["host_enqueue_us_per_step"]}
            tensor_bytes = getattr(wl, "tensor_bytes", None)
            if tensor_bytes is not None and tensor_bytes < (1 << 29):
                c = copy_gbs_at_size(tensor_bytes, dev)
                entry["copy_same_size_gbs"] = round(c, 1)
                entry["pct_of_copy_same_size"] = round(100 * res["value"] / c, 2)
            out[name] = entry
            res["runner"] = None
            del res, st
        except Exception as exc:  # noqa: BLE001
            out[name] = {"error": f"{type(exc).__name__}: {str(exc)[:200]}"}
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="cfg4")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"])
    ap.add_argument("--collective", default="auto", choices=["auto", "async", "sync", "none", "fused", "exchange-side"],
                    help="cfg4 gradient all-reduce: NCCL overlapped with the next step, NCCL in-stream, (diagnostic) skipped, "
                         "the library's own fold + all-reduce kernel over peer memory in-stream (fused), or its exchange alone "
                         "on a second stream behind an in-stream fold (exchange-side)")
    ap.add_argument("--graph", default="on", choices=["on", "off"],
                    help="replay the steps from a CUDA graph (where the workload supports it) or enqueue them call by call")
    ap.add_argument("--sm-margin", type=int, default=-1,
                    help="SMs the persistent kernels leave free for a collective kernel running beside them (default: 4 from N=4 on, else 0)")
    ap.add_argument("--tune", default="", help="(diagnostic) ring-kernel launch parameters, e.g. rpg=2,stages=4,lag=2")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the short runs of the other BASELINE configs")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--rows", type=int, default=0, help="override the workload's global row count (small cases for ncu)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    global COLLECTIVE_MODE
    # auto: the library's own all-reduce kernel over peer memory on a second stream (2.3 us per step of main-stream
    # time at two GPUs against 12-14 for NCCL's kernel inside the same graph); NCCL if the buffers cannot be opened
    COLLECTIVE_MODE = "exchange-side" if args.collective == "auto" else args.collective

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.workload != "cfg4":
        _load_more_workloads()
    wl = WORKLOADS[args.workload]()
    if args.rows > 0:
        wl.rows = args.rows
        wl.cpu_sample_rows = min(wl.cpu_sample_rows, args.rows)

    if args.impl == "reference":
        run_reference(args, wl, rank)
        return

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    import b200norm
    from b200norm import capi, shard
    # From four GPUs on, the collective's kernel gets four SMs of its own (a ring CTA fills its SM, so without
    # them the all-reduce waits for a kernel boundary and then delays the next kernel's CTAs); at N = 2 the
    # all-reduce is too short for the margin to pay.  Only the config-4 step has a collective that overlaps kernels.
    # NCCL's kernel needs SMs of its own beside the persistent kernels from four GPUs on (a ring CTA fills its SM); the
    # library's one-CTA exchange kernel takes the SM the planner leaves over anyway (no margin)
    overlapped = world >= 4 and args.workload in ("cfg4", "ln_long") and COLLECTIVE_MODE == "async"
    sm_margin = args.sm_margin if args.sm_margin >= 0 else (4 if overlapped else 0)
    capi.set_tuning(b200norm.TUNE_SM_MARGIN, sm_margin)
    for item in filter(None, args.tune.split(",")):
        knob, val = item.split("=")
        capi.set_tuning({"rpg": b200norm.TUNE_ROWS_PER_GROUP, "stages": b200norm.TUNE_STAGES,
                         "lag": b200norm.TUNE_STORE_LAG}[knob], int(val))

    b200norm.load_library()
    if args.scaling == "strong":
        rows_of = lambda r: (lambda a_b: a_b[1] - a_b[0])(shard.shard_rows(wl.rows, world, r))  # noqa: E731
        rows = rows_of(rank)
        global_rows = wl.rows
    else:
        rows_of = lambda r: wl.rows  # noqa: E731
        rows = wl.rows
        global_rows = wl.rows * world
    st = wl.make_device_state(rows, dev, seed=4001 + rank)
    collective_note = None
    if COLLECTIVE_MODE in ("fused", "exchange-side"):
        if not hasattr(wl, "open_exchange") or world == 1:
            if args.collective != "auto" and world > 1:
                raise SystemExit(f"--collective {args.collective}: workload {wl.name} has no weight-gradient exchange")
            COLLECTIVE_MODE = "async"
        else:
            ok = torch.ones(1, device=dev)
            try:
                wl.open_exchange(st, dev, sm_margin)
            except Exception as exc:  # noqa: BLE001
                ok.zero_()
                collective_note = f"peer-memory exchange unavailable ({type(exc).__name__}: {str(exc)[:100]}): NCCL instead"
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)  # every rank takes the same path
            if float(ok) == 0.0:
                if args.collective != "auto":
                    raise SystemExit(collective_note or "a peer could not open the exchange buffers")
                COLLECTIVE_MODE = "async"
                collective_note = collective_note or "peer-memory exchange unavailable on another rank: NCCL instead"
                if args.sm_margin < 0 and world >= 4:
                    sm_margin = 4
                    capi.set_tuning(b200norm.TUNE_SM_MARGIN, sm_margin)
                st = wl.make_device_state(rows, dev, seed=4001 + rank)
    sampler = ClockSampler(dev)
    sampler.start()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if world > 1:  # NCCL's communicator and channels exist before anything is timed or captured
        dist.all_reduce(torch.zeros(1, device=dev))
        barrier()
    res = measure_workload(wl, capi, st, world, rank, dev, args.steps, args.warmup, rows, global_rows, args.scaling,
                           args.graph == "on", barrier)
    clocks = sampler.summary(*res["span"])
    roofline = roofline_of(res, wl, rows)
    coll_us = collective_time_us(wl, st, world)
    shard_check = None
    if world > 1 and hasattr(wl, "shard_check") and COLLECTIVE_MODE != "none":
        shard_check = wl.shard_check(capi, st, world, rank, rows_of)
        barrier()
    value, total_bytes, peak = res["value"], res["total_bytes"], res["peak"]
    res["runner"] = None

    # end to end through the ATen dispatcher with host buffers
    e2e = None
    es = None
    if not args.no_e2e:
        b200norm.enable_aten_overrides()
        es = wl.make_e2e_state(rows, dev)
        for _ in range(2):
            wl.e2e_step(st, es, world)
        barrier()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(args.e2e_steps):
            wl.e2e_step(st, es, world)
        a1.record()
        barrier()
        ems = a0.elapsed_time(a1)
        if world > 1:
            t = torch.tensor([ems], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ems = float(t[0])
        h2d_b, d2h_b = wl.e2e_bytes(rows)
        e2e = {"value": round(total_bytes * args.e2e_steps / (ems * 1e-3) / 1e9, 2), "unit": "GB/s",
               "h2d_bytes_per_step": h2d_b * world, "d2h_bytes_per_step": d2h_b * world,
               "ms_per_step": round(ems / args.e2e_steps, 3), "steps": args.e2e_steps,
               "api": "torch.ops.aten.* on CUDA tensors via the dispatcher override; pinned host buffers, "
                      f"{wl.e2e_chunks} row chunks on 3 streams"}
    sampler.stop()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu_state = wl.cpu_state_from_e2e(es) if (es is not None and hasattr(wl, "cpu_state_from_e2e")
                                                  and wl.cpu_sample_rows == rows) else None
        cpu = cpu_measure(wl, cpu_state)
    del es

    configs = None
    if world == 1 and args.workload == "cfg4" and args.rows == 0 and not args.no_configs:
        del st
        torch.cuda.empty_cache()
        configs = run_other_configs(capi, dev, lambda name: {"cfg1": 64, "cfg2": 40, "cfg3": 10, "cfg5": 4,
                                                              "cfg5f": 4, "ln_long": 10, "gn": 10, "bn": 10, "sm_c19": 20, "sm_c64": 10,
                                                              "sm_c150": 6}[name], barrier)

    if rank == 0:
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(res["ms_per_step"], 5), "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "bf16 storage, f32 accumulate", "data": "synthetic",
            "config": {"workload": f"{wl.name}: {wl.describe()}", "global_rows": global_rows, "rows_per_gpu": rows,
                       "sm_margin": sm_margin, "parallelism": f"row-sharded dp{world}", "l2": wl.l2_note,
                       "graph": res["graph"], "collective_note": collective_note,
                       "collective": (getattr(wl, "collective", "all_reduce(fp32[2,N]) per step, " + {"async": "NCCL, overlapped with the next step", "sync": "NCCL, in stream", "none": "SKIPPED (diagnostic run)", "fused": "own fold + all-reduce kernel over peer memory, in stream", "exchange-side": "fold in stream, own all-reduce kernel over peer memory on a second stream"}[COLLECTIVE_MODE]) if world > 1 else "none")},
            "spread": res["spread"], "sustained_ms_per_step": res["sustained_ms_per_step"],
            "host_enqueue_us_per_step": res["host_enqueue_us_per_step"],
            "collective_us": coll_us, "shard_check": shard_check,
            "pct_of_peak_measured": round(100 * value / world / peak, 2),
            "pct_of_peak_nominal": round(100 * value / world / NOMINAL_HBM_GBS, 2),
            "rows_per_s": round(global_rows / (res["ms_per_step"] * 1e-3), 1),
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(res["launches"]), "clocks": clocks,
        }
        if configs is not None:
            line["configs"] = configs
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
