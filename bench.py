#!/usr/bin/env python
"""Throughput benchmark of the normalization / softmax path.

    python bench.py --gpus N --steps K --warmup W [--workload cfg4] [--impl reference]

One "step" is one pass of the workload's operators over one batch of seeded synthetic input.  The
default workload is BASELINE config 4: native_layer_norm forward + backward (dx, dgamma, dbeta) on
bf16 [65536, 8192] with fp32 gamma/beta, rows sharded evenly over the N ranks (strong scaling), the
fused fp32 [2, 8192] dgamma|dbeta buffer all-reduced over NCCL each step.  Other workloads
(--workload cfg1|cfg2|cfg3|cfg5) run the other BASELINE configs the same way; cfg5f is config 5 with the fused
cross-entropy backward.

Prints ONE JSON line (rank 0).  `value` is algorithmic bytes (every tensor of the operators'
signatures read or written once) of all ranks / device time, inputs resident in HBM; `e2e` is the
same metric through the ATen dispatcher with pinned HOST buffers, copies inside the timed region.
`--impl reference` times PyTorch's CPU ATen kernels (the reference path's parity standard, and the
only implementation of it that runs on this box) on the host cores over a bounded row sample.
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
    name, rows, N, cpu_sample_rows = "cfg4", 65536, 8192, 4096
    kernel = "layer_norm_bwd_ring"

    def describe(self):
        return ("native_layer_norm fwd + native_layer_norm_backward (dx, dgamma, dbeta), bf16 [65536, 8192], "
                "fp32 gamma/beta, eps 1e-5")

    def bytes_per_rows(self, rows):
        n = self.N
        fwd = 2 * rows * n * 2 + 2 * n * 4 + 2 * rows * 4
        bwd = 3 * rows * n * 2 + 2 * rows * 4 + n * 4 + 2 * n * 4
        return {"total": fwd + bwd, "layer_norm_fwd_ring": fwd, "layer_norm_bwd_ring": bwd}

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
        return st

    def step(self, capi, st, world):
        n = self.N
        k = st["k"] = st["k"] ^ 1
        wg = st["wgrads"][k]
        if st["works"][k] is not None:
            st["works"][k].wait()  # stream-level: the buffer's previous all-reduce precedes its reuse
        capi.native_layer_norm(st["x"], [n], st["gamma"], st["beta"], 1e-5, out=(st["y"], st["mean"], st["rstd"]))
        capi.native_layer_norm_backward(st["dy"], st["x"], [n], st["mean"], st["rstd"], st["gamma"], st["beta"],
                                        (True, True, True), out=(st["dx"], wg[0], wg[1]), workspace=st["ws"])
        if world > 1 and COLLECTIVE_MODE != "none":
            # one all-reduce(SUM) of the fused [dgamma | dbeta] buffer the fold kernel just wrote; asynchronous,
            # so it overlaps the next step's forward (nothing reads the reduced gradients inside the step)
            if COLLECTIVE_MODE == "async":
                st["works"][k] = dist.all_reduce(wg, async_op=True)
            else:
                dist.all_reduce(wg)

    def finish(self, st):
        for w in st["works"]:
            if w is not None:
                w.wait()
        st["works"] = [None, None]

    launches_per_step = 3  # forward ring kernel, backward ring kernel, partial-sum fold

    def cpu_step(self, cpu):
        n = self.N
        y, mean, rstd = torch.ops.aten.native_layer_norm(cpu["x"], [n], cpu["gamma"], cpu["beta"], 1e-5)
        return torch.ops.aten.native_layer_norm_backward(cpu["dy"], cpu["x"], [n], mean, rstd, cpu["gamma"],
                                                         cpu["beta"], [True, True, True])

    def make_cpu_state(self, rows):
        g = torch.Generator().manual_seed(4001)
        n = self.N
        return {"x": torch.randn((rows, n), generator=g).to(torch.bfloat16),
                "dy": torch.randn((rows, n), generator=g).to(torch.bfloat16),
                "gamma": torch.randn(n, generator=g) * 0.02 + 1.0, "beta": torch.randn(n, generator=g) * 0.02}

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


COLLECTIVE_MODE = "async"  # --collective: async (default) | sync | none (diagnostic: no gradient exchange)
WORKLOADS = {"cfg4": Cfg4LayerNorm}


def _load_more_workloads():
    from bench_workloads import EXTRA  # noqa: WPS433  (kept in a sibling module to keep this file readable)
    WORKLOADS.update(EXTRA)


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


def recorded_traffic(kernel: str, units: int):
    """DRAM bytes per launch from the committed ncu capture (profiles/dram_traffic.json holds bytes per
    row per kernel, measured on a smaller case of the same row length); None when not captured."""
    p = ROOT / "profiles" / "dram_traffic.json"
    if not p.exists():
        return None
    try:
        per_row = json.loads(p.read_text()).get(kernel, {}).get("dram_bytes_per_row")
        return None if per_row is None else per_row * units
    except Exception:  # noqa: BLE001
        return None


def cpu_measure(wl: Workload, budget_s: float = 12.0):
    rows = wl.cpu_sample_rows
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
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16->f32 accumulate",
        "data": "synthetic", "config": {"workload": f"{wl.name}: {wl.describe()}", "rows_per_step": rows},
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="cfg4")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"])
    ap.add_argument("--collective", default="async", choices=["async", "sync", "none"],
                    help="cfg4 gradient all-reduce: overlapped with the next step, in-stream, or (diagnostic) skipped")
    ap.add_argument("--sm-margin", type=int, default=-1,
                    help="SMs the persistent kernels leave free for a collective kernel running beside them (default: 4 from N=4 on, else 0)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--rows", type=int, default=0, help="override the workload's global row count (small cases for ncu)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    global COLLECTIVE_MODE
    COLLECTIVE_MODE = args.collective

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
    # From four GPUs on, the collective's kernel gets four SMs of its own: measured at N = 8 the step is 132 us with
    # that margin, 163 us without (the all-reduce then waits for a kernel boundary and delays the next kernel's CTAs),
    # 126 us with no collective at all; at N = 2 the all-reduce is too short for the margin to pay.
    # Only the config-4 step has a collective that overlaps kernels; the others keep every SM.
    overlapped = world >= 4 and args.workload == "cfg4" and COLLECTIVE_MODE == "async"
    sm_margin = args.sm_margin if args.sm_margin >= 0 else (4 if overlapped else 0)
    capi.set_tuning(b200norm.TUNE_SM_MARGIN, sm_margin)

    b200norm.load_library()
    if args.scaling == "strong":
        r0, r1 = shard.shard_rows(wl.rows, world, rank)
        rows = r1 - r0
        global_rows = wl.rows
    else:
        rows = wl.rows
        global_rows = wl.rows * world
    st = wl.make_device_state(rows, dev, seed=4001 + rank)
    sampler = ClockSampler(dev)
    sampler.start()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        wl.step(capi, st, world)
    if hasattr(wl, "finish"):
        wl.finish(st)
    barrier()
    n0 = capi.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        wl.step(capi, st, world)
    if hasattr(wl, "finish"):
        wl.finish(st)  # outstanding collectives join the timed stream before the closing event
    e1.record()
    barrier()
    t_end = time.perf_counter()
    launches = capi.launch_count() - n0
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    clocks = sampler.summary(t_begin, t_end)
    status = capi.device_status()
    assert status == 0, f"device status {status}"

    # roofline of the dominant kernel: per-launch CUDA events on the launching stream, same steps again
    prof_steps = min(args.steps, 50)
    capi.profile_begin()
    for _ in range(prof_steps):
        wl.step(capi, st, world)
    if hasattr(wl, "finish"):
        wl.finish(st)
    prof = capi.profile_end()
    barrier()
    kernel = max(prof, key=lambda k: prof[k][1])
    k_launches, k_ms = prof[kernel]
    per_launch_ms = k_ms / k_launches
    bytes_local = wl.bytes_per_rows(rows)
    peak, peak_kind = measured_peak()
    achieved = bytes_local[kernel] / (per_launch_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": kernel, "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                "frac": round(achieved / peak, 4), "peak_kind": peak_kind,
                "frac_of_nominal_8TBs": round(achieved / NOMINAL_HBM_GBS, 4),
                "us_per_launch": round(per_launch_ms * 1e3, 2), "launches_timed": k_launches,
                "traffic": recorded_traffic(kernel, rows),
                "all_kernels_us": {k: round(v[1] / v[0] * 1e3, 2) for k, v in prof.items()}}

    total_bytes = wl.bytes_per_rows(global_rows)["total"] if args.scaling == "strong" else bytes_local["total"] * world
    value = total_bytes * args.steps / (ms * 1e-3) / 1e9

    # end to end through the ATen dispatcher with host buffers
    e2e = None
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
        del es
    sampler.stop()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_measure(wl)

    if rank == 0:
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "bf16 storage, f32 accumulate", "data": "synthetic",
            "config": {"workload": f"{wl.name}: {wl.describe()}", "global_rows": global_rows, "rows_per_gpu": rows,
                       "sm_margin": sm_margin, "parallelism": f"row-sharded dp{world}", "l2": "inputs larger than L2 (no flush needed)",
                       "collective": (getattr(wl, "collective", "all_reduce(fp32[2,N]) per step, " + {"async": "overlapped with the next step", "sync": "in stream", "none": "SKIPPED (diagnostic run)"}[COLLECTIVE_MODE]) if world > 1 else "none")},
            "pct_of_peak_measured": round(100 * value / world / peak, 2),
            "pct_of_peak_nominal": round(100 * value / world / NOMINAL_HBM_GBS, 2),
            "rows_per_s": round(global_rows * args.steps / (ms * 1e-3), 1),
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
