"""The other BASELINE workloads for bench.py (--workload cfg1|cfg2|cfg3|cfg5).  Same conventions as
bench.Cfg4LayerNorm: seeded synthetic inputs, preallocated outputs, algorithmic bytes = every tensor
of the operators' signatures read or written once."""
from __future__ import annotations

import math

import torch
import torch.distributed as dist


class _Simple:
    """Shared plumbing: un-chunked end-to-end step (copy in, ATen ops, copy out)."""
    e2e_chunks = 1
    launches_per_step = 2

    def make_e2e_state(self, rows, dev):
        cpu = self.make_cpu_state(rows)
        host_in = {k: cpu[k].pin_memory() for k in self.e2e_inputs}
        return {"in": host_in, "out": None, "dev": dev}

    def e2e_step(self, st, e2e, world):
        dev_in = {k: v.to(e2e["dev"], non_blocking=True) for k, v in e2e["in"].items()}
        outs = self.aten_step({**st, **dev_in}, world)
        if e2e["out"] is None:
            e2e["out"] = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs]
        for h, o in zip(e2e["out"], outs):
            h.copy_(o, non_blocking=True)
        return outs

    def e2e_bytes(self, rows):
        cpu_in = sum(self._nbytes(rows, k) for k in self.e2e_inputs)
        return cpu_in, self._out_bytes(rows)


class Cfg1LayerNormFwd(_Simple):
    name, rows, N, cpu_sample_rows = "cfg1", 4096, 1024, 4096
    e2e_inputs = ("x",)
    launches_per_step = 1
    cycle = 16
    tensor_bytes = 4096 * 1024 * 4
    l2_note = "tensors (16 MiB) smaller than L2: 16 rotating input/output sets, 0.5 GB, so no launch finds its rows in L2"

    def describe(self):
        return "native_layer_norm fwd, fp32 [4096, 1024], eps 1e-5 (launch-bound: 33.6 MB)"

    def bytes_per_rows(self, rows):
        n = self.N
        fwd = 2 * rows * n * 4 + 2 * n * 4 + 2 * rows * 4
        return {"total": fwd, "layer_norm_fwd_ring": fwd}

    def make_cpu_state(self, rows):
        g = torch.Generator().manual_seed(1001)
        n = self.N
        return {"x": torch.randn((rows, n), generator=g), "gamma": torch.randn(n, generator=g) * 0.02 + 1.0,
                "beta": torch.randn(n, generator=g) * 0.02}

    def make_device_state(self, rows, dev, seed):
        # 16 rotating input/output sets (0.5 GB) so back-to-back launches never find their rows in L2
        st = {k: v.to(dev) for k, v in self.make_cpu_state(rows).items()}
        st["xs"] = [st["x"].clone() for _ in range(16)]
        st["ys"] = [torch.empty_like(st["x"]) for _ in range(16)]
        st["mean"] = torch.empty(rows, device=dev)
        st["rstd"] = torch.empty(rows, device=dev)
        st["i"] = 0
        return st

    def prepare(self, capi, st):
        st["calls"] = [capi.prepare_layer_norm(st["xs"][i], st["gamma"], st["beta"], 1e-5, st["ys"][i], st["mean"], st["rstd"])
                       for i in range(16)]

    def step(self, capi, st, world):
        i = st["i"] = (st["i"] + 1) % 16
        st["calls"][i]()

    def capture_cycle(self, capi, st, world, cs, side, cycles=1):
        for _ in range(cycles):
            for call in st["calls"]:
                call()

    def cpu_step(self, cpu):
        return torch.ops.aten.native_layer_norm(cpu["x"], [self.N], cpu["gamma"], cpu["beta"], 1e-5)

    def aten_step(self, st, world):
        return torch.ops.aten.native_layer_norm(st["x"], [self.N], st["gamma"], st["beta"], 1e-5)

    def _nbytes(self, rows, k):
        return rows * self.N * 4

    def _out_bytes(self, rows):
        return rows * self.N * 4 + 2 * rows * 4


class Cfg2RmsNorm(_Simple):
    name, rows, N, cpu_sample_rows = "cfg2", 8192, 4096, 8192
    collective = "all_reduce(fp32[2,N]) per step"
    e2e_inputs = ("x", "dy")
    launches_per_step = 3
    cycle = 4
    tensor_bytes = 8192 * 4096 * 2
    l2_note = "tensors (64 MiB) smaller than L2: 4 rotating sets of x, dy, y, dx (1 GiB working set)"

    def describe(self):
        return "_fused_rms_norm fwd + _fused_rms_norm_backward (dx, dweight), bf16 [8192, 4096], fp32 weight, eps 1e-6"

    def bytes_per_rows(self, rows):
        n = self.N
        fwd = 2 * rows * n * 2 + n * 4 + rows * 4
        bwd = 3 * rows * n * 2 + rows * 4 + 2 * n * 4
        return {"total": fwd + bwd, "rms_norm_fwd_ring": fwd, "rms_norm_bwd_ring": bwd}

    def make_cpu_state(self, rows):
        g = torch.Generator().manual_seed(2001)
        n = self.N
        return {"x": torch.randn((rows, n), generator=g).to(torch.bfloat16),
                "dy": torch.randn((rows, n), generator=g).to(torch.bfloat16),
                "weight": torch.randn(n, generator=g) * 0.02 + 1.0}

    def make_device_state(self, rows, dev, seed):
        from b200norm import BF16, F32, load_library
        st = {k: v.to(dev) for k, v in self.make_cpu_state(rows).items()}
        # 4 rotating sets: 4 x 4 x 64 MiB = 1 GiB working set, far beyond L2
        st["sets"] = [{"x": st["x"].clone(), "dy": st["dy"].clone(), "y": torch.empty_like(st["x"]),
                       "dx": torch.empty_like(st["x"])} for _ in range(4)]
        st["rstd"] = torch.empty(rows, device=dev)
        st["wgrad"] = torch.zeros((2, self.N), device=dev)
        nbytes = load_library().b2n_norm_bwd_workspace_bytes(rows, self.N, BF16, F32, 1)
        st["ws"] = torch.empty(max(nbytes, 1), device=dev, dtype=torch.uint8)
        st["i"] = 0
        return st

    def prepare(self, capi, st):
        st["calls"] = [(capi.prepare_rms_norm(s["x"], st["weight"], 1e-6, s["y"], st["rstd"]),
                        capi.prepare_rms_norm_backward(s["dy"], s["x"], st["rstd"], st["weight"], s["dx"], st["wgrad"][0],
                                                       st["ws"])) for s in st["sets"]]

    def step(self, capi, st, world):
        i = st["i"] = (st["i"] + 1) % 4
        fwd, bwd = st["calls"][i]
        fwd()
        bwd()
        if world > 1:
            dist.all_reduce(st["wgrad"])

    def capture_cycle(self, capi, st, world, cs, side, cycles=1):
        for _ in range(cycles):
            for fwd, bwd in st["calls"]:
                fwd()
                bwd()
                if world > 1:
                    dist.all_reduce(st["wgrad"])

    def collective_buffer(self, st):
        return st["wgrad"]

    def cpu_step(self, cpu):
        # no CPU kernel exists for _fused_rms_norm(_backward): autograd through the CPU composite
        x = cpu["x"].float().requires_grad_(True)
        w = cpu["weight"].clone().requires_grad_(True)
        y = torch.nn.functional.rms_norm(x, [self.N], w, 1e-6)
        return torch.autograd.grad(y, [x, w], cpu["dy"].float())

    def aten_step(self, st, world):
        n = self.N
        y, rstd = torch.ops.aten._fused_rms_norm(st["x"], [n], st["weight"], 1e-6)
        dx, dw = torch.ops.aten._fused_rms_norm_backward(st["dy"], st["x"], [n], rstd, st["weight"], [True, True])
        if world > 1:
            dist.all_reduce(dw)
        return y, dx, dw

    def _nbytes(self, rows, k):
        return rows * self.N * 2

    def _out_bytes(self, rows):
        return 2 * rows * self.N * 2 + self.N * 4


class Cfg3Softmax(_Simple):
    name, T, cpu_sample_rows = "cfg3", 2048, 8192
    collective = "none (rows are independent)"
    rows = 8 * 32 * 2048
    e2e_inputs = ("s", "g")
    l2_note = "inputs (2 GiB per tensor) larger than L2 (no flush needed)"

    def describe(self):
        return ("_softmax + _softmax_backward_data over the last dim, bf16 [8, 32, 2048, 2048] causal scores "
                "(strict upper triangle -inf, applied before the op)")

    def bytes_per_rows(self, rows):
        t = self.T
        return {"total": 5 * rows * t * 2, "softmax_fwd_ring": 2 * rows * t * 2, "softmax_bwd_ring": 3 * rows * t * 2}

    def _make(self, rows, dev, gen):
        t = self.T
        s = torch.randn((rows, t), generator=gen, device=dev) / math.sqrt(128)
        r = torch.arange(rows, device=dev).remainder(t).view(-1, 1)
        s.masked_fill_(torch.arange(t, device=dev).view(1, -1) > r, float("-inf"))
        g = torch.randn((rows, t), generator=gen, device=dev).to(torch.bfloat16)
        return s.to(torch.bfloat16), g

    def make_cpu_state(self, rows):
        s, g = self._make(rows, torch.device("cpu"), torch.Generator().manual_seed(3001))
        return {"s": s, "g": g}

    def make_device_state(self, rows, dev, seed):
        gen = torch.Generator(device=dev).manual_seed(seed)
        st = {}
        parts = [self._make(min(65536, rows - r), dev, gen) for r in range(0, rows, 65536)]
        st["s"] = torch.cat([p[0] for p in parts])
        st["g"] = torch.cat([p[1] for p in parts])
        del parts
        st["p"] = torch.empty_like(st["s"])
        st["dx"] = torch.empty_like(st["s"])
        return st

    def step(self, capi, st, world):
        capi._softmax(st["s"], -1, False, out=st["p"])
        capi._softmax_backward_data(st["g"], st["p"], -1, torch.bfloat16, out=st["dx"])

    def cpu_step(self, cpu):
        p = torch.ops.aten._softmax(cpu["s"], -1, False)
        return torch.ops.aten._softmax_backward_data(cpu["g"], p, -1, torch.bfloat16)

    def aten_step(self, st, world):
        p = torch.ops.aten._softmax(st["s"], -1, False)
        return p, torch.ops.aten._softmax_backward_data(st["g"], p, -1, torch.bfloat16)

    def _nbytes(self, rows, k):
        return rows * self.T * 2

    def _out_bytes(self, rows):
        return 2 * rows * self.T * 2


class Cfg3Masked(Cfg3Softmax):
    """Config 3 with the causal mask applied INSIDE the kernels (aten::_masked_softmax with a [T, T] source mask,
    aten::_masked_softmax_backward with the mask expanded to the gradient's shape) instead of being written into the
    scores beforehand.  Not a BASELINE config.  Bytes: forward 2 tensors (the 4 MB mask stays in L2); backward 3
    tensors + 1 mask byte per element."""
    name = "cfg3m"

    def describe(self):
        return ("_masked_softmax (mask_type 0: [2048, 2048] causal source mask) + _masked_softmax_backward (mask of "
                "the gradient's shape) over the last dim, bf16 [8, 32, 2048, 2048] unmasked scores")

    def bytes_per_rows(self, rows):
        t = self.T
        fwd, bwd = 2 * rows * t * 2, 3 * rows * t * 2 + rows * t
        return {"total": fwd + bwd, "masked_softmax_fwd_ring": fwd, "masked_softmax_bwd_ring": bwd,
                "masked_softmax_fwd": fwd, "masked_softmax_bwd": bwd}

    def _make(self, rows, dev, gen):
        t = self.T
        s = torch.randn((rows, t), generator=gen, device=dev) / math.sqrt(128)
        g = torch.randn((rows, t), generator=gen, device=dev).to(torch.bfloat16)
        return s.to(torch.bfloat16), g

    def _masks(self, rows, dev):
        t = self.T
        causal = torch.triu(torch.ones(t, t, dtype=torch.bool, device=dev), 1)
        full = causal.repeat((rows + t - 1) // t, 1)[:rows].contiguous()
        return causal, full

    def make_cpu_state(self, rows):
        st = super().make_cpu_state(rows)
        st["causal"], st["full"] = self._masks(rows, torch.device("cpu"))
        return st

    def make_device_state(self, rows, dev, seed):
        st = super().make_device_state(rows, dev, seed)
        st["causal"], st["full"] = self._masks(rows, dev)
        # the [T, T] layout of the reference needs a 4-D input: view the rows as [1, rows / T, T, T]
        st["shape4"] = (1, rows // self.T, self.T, self.T) if rows % self.T == 0 else None
        return st

    def step(self, capi, st, world):
        if st["shape4"] is not None:
            capi._masked_softmax(st["s"].view(st["shape4"]), st["causal"], -1, 0, out=st["p"])
        else:
            capi._masked_softmax(st["s"], st["full"], -1, 2, out=st["p"])
        capi._masked_softmax_backward(st["g"], st["p"], st["full"], -1, out=st["dx"])

    def cpu_step(self, cpu):
        p = torch._masked_softmax(cpu["s"], cpu["full"], -1, 2)
        return torch.ops.aten._masked_softmax_backward(cpu["g"], p, cpu["full"], -1)

    def aten_step(self, st, world):
        p = torch._masked_softmax(st["s"], st["full"], -1, 2)
        return p, torch.ops.aten._masked_softmax_backward(st["g"], p, st["full"], -1)


class Cfg5CrossEntropy(_Simple):
    name, rows, V, cpu_sample_rows = "cfg5", 16384, 128256, 1024
    collective = "all_reduce(fp32[2]: loss sum, weight sum) per step"
    e2e_inputs = ("logits", "target")
    launches_per_step = 6
    l2_note = "inputs (3.9 GiB per tensor) larger than L2 (no flush needed)"

    def describe(self):
        return ("_log_softmax + nll_loss_forward(mean) + nll_loss_backward + _log_softmax_backward_data, "
                "bf16 logits [16384, 128256] ~N(0,2), int64 targets; loss sum/count all-reduced")

    def bytes_per_rows(self, rows):
        v = self.V
        fwd, bwd = 2 * rows * v * 2, 3 * rows * v * 2
        return {"total": fwd + bwd + rows * 40, "log_softmax_fwd_ring": fwd, "log_softmax_bwd_ring": bwd,
                "log_softmax_fwd_generic": fwd, "log_softmax_bwd_generic": bwd,
                "log_softmax_fwd_cluster": fwd, "log_softmax_bwd_cluster": bwd,
                "log_softmax_fwd_twopass": fwd, "log_softmax_bwd_twopass": bwd}

    def make_cpu_state(self, rows):
        g = torch.Generator().manual_seed(5001)
        return {"logits": (torch.randn((rows, self.V), generator=g) * 2.0).to(torch.bfloat16),
                "target": torch.randint(0, self.V, (rows,), generator=g)}

    def make_device_state(self, rows, dev, seed):
        gen = torch.Generator(device=dev).manual_seed(seed)
        st = {"logits": torch.empty((rows, self.V), device=dev, dtype=torch.bfloat16)}
        for r in range(0, rows, 2048):
            k = min(2048, rows - r)
            st["logits"][r:r + k] = (torch.randn((k, self.V), generator=gen, device=dev) * 2.0).to(torch.bfloat16)
        st["target"] = torch.randint(0, self.V, (rows,), generator=gen, device=dev)
        st["logp"] = torch.empty_like(st["logits"])
        st["grad_logp"] = torch.empty_like(st["logits"])
        st["dlogits"] = torch.empty_like(st["logits"])
        st["one"] = torch.ones((), device=dev, dtype=torch.bfloat16)
        return st

    def step(self, capi, st, world):
        logp = capi._log_softmax(st["logits"], -1, False, out=st["logp"])
        _, _, sums = capi.nll_loss_forward(logp, st["target"], None, 2, -100, return_sums=True)
        if world > 1:
            dist.all_reduce(sums)
        st["loss"] = sums[0] / sums[1]
        tw = sums[1].to(torch.bfloat16)
        capi.nll_loss_backward(st["one"], logp, st["target"], None, 1, -100, tw, out=st["grad_logp"])
        capi._log_softmax_backward_data(st["grad_logp"], logp, -1, torch.bfloat16, out=st["dlogits"])

    def cpu_step(self, cpu):
        logp = torch.ops.aten._log_softmax(cpu["logits"], -1, False)
        out, tw = torch.ops.aten.nll_loss_forward(logp, cpu["target"], None, 1, -100)
        g = torch.ops.aten.nll_loss_backward(torch.ones((), dtype=torch.bfloat16), logp, cpu["target"], None, 1, -100, tw)
        return torch.ops.aten._log_softmax_backward_data(g, logp, -1, torch.bfloat16)

    def aten_step(self, st, world):
        logp = torch.ops.aten._log_softmax(st["logits"], -1, False)
        out, tw = torch.ops.aten.nll_loss_forward(logp, st["target"], None, 1, -100)
        g = torch.ops.aten.nll_loss_backward(torch.ones_like(out), logp, st["target"], None, 1, -100, tw)
        return out, torch.ops.aten._log_softmax_backward_data(g, logp, -1, torch.bfloat16)

    def _nbytes(self, rows, k):
        return rows * self.V * 2 if k == "logits" else rows * 8

    def _out_bytes(self, rows):
        return rows * self.V * 2 + 2


class Cfg5FusedTail(Cfg5CrossEntropy):
    """Config 5 with the two backward operators replaced by the fused kernel (b2n_cross_entropy_bwd): the same
    inputs and the same dlogits, without the dense gradient of the log-probabilities.  Not a BASELINE config:
    its bytes are those the fused formulation needs (log-softmax 2 passes + backward 2 passes over the logits)."""
    name = "cfg5f"
    launches_per_step = 4

    def describe(self):
        return ("_log_softmax + nll_loss_forward(mean) + fused cross-entropy backward (nll_loss_backward and "
                "_log_softmax_backward_data in one pass), bf16 logits [16384, 128256] ~N(0,2), int64 targets")

    def bytes_per_rows(self, rows):
        v = self.V
        fwd, bwd = 2 * rows * v * 2, 2 * rows * v * 2
        return {"total": fwd + bwd + rows * 40, "log_softmax_fwd_twopass": fwd, "log_softmax_fwd_generic": fwd,
                "cross_entropy_bwd_ring": bwd, "cross_entropy_bwd_generic": bwd}

    def make_device_state(self, rows, dev, seed):
        st = super().make_device_state(rows, dev, seed)
        del st["grad_logp"]
        return st

    def step(self, capi, st, world):
        logp = capi._log_softmax(st["logits"], -1, False, out=st["logp"])
        _, _, sums = capi.nll_loss_forward(logp, st["target"], None, 2, -100, return_sums=True)
        if world > 1:
            dist.all_reduce(sums)
        st["loss"] = sums[0] / sums[1]
        tw = sums[1].to(torch.bfloat16)
        capi.cross_entropy_backward(st["one"], logp, st["target"], None, 1, -100, tw, out=st["dlogits"])

    def aten_step(self, st, world):
        from b200norm import capi
        x = st["logits"].detach().requires_grad_(True)
        loss = capi.cross_entropy(x, st["target"])
        loss.backward()
        return loss.detach(), x.grad


class GroupNormFwd(_Simple):
    """Not a BASELINE config: native_group_norm forward on the reference microbenchmark's large shape
    (test/microbench/group_norm.py: 16 groups, [1024, 128, 32, 32]), bf16 with bf16 weights.  `rows` are samples."""
    name, rows, C, HW, G, cpu_sample_rows = "gn", 1024, 128, 32 * 32, 16, 64
    e2e_inputs = ("x",)
    launches_per_step = 1
    l2_note = "input (256 MiB) larger than L2 (no flush needed)"

    def describe(self):
        return f"native_group_norm fwd, bf16 [{self.rows}, {self.C}, 32, 32], {self.G} groups, bf16 weight/bias, eps 1e-5"

    def bytes_per_rows(self, rows):
        n = rows * self.C * self.HW
        fwd = 2 * n * 2 + 2 * self.C * 2 + 2 * rows * self.G * 2
        return {"total": fwd, "group_norm_fwd": fwd, "group_norm_fwd_ring": fwd}

    def make_cpu_state(self, rows):
        g = torch.Generator().manual_seed(6001)
        return {"x": torch.randn((rows, self.C, 32, 32), generator=g).to(torch.bfloat16),
                "weight": (torch.randn(self.C, generator=g) * 0.02 + 1.0).to(torch.bfloat16),
                "bias": (torch.randn(self.C, generator=g) * 0.02).to(torch.bfloat16)}

    def make_device_state(self, rows, dev, seed):
        gen = torch.Generator(device=dev).manual_seed(seed)
        st = {"x": torch.randn((rows, self.C, 32, 32), generator=gen, device=dev).to(torch.bfloat16)}
        cg = torch.Generator().manual_seed(6002)
        st["weight"] = (torch.randn(self.C, generator=cg) * 0.02 + 1.0).to(torch.bfloat16).to(dev)
        st["bias"] = (torch.randn(self.C, generator=cg) * 0.02).to(torch.bfloat16).to(dev)
        st["y"] = torch.empty_like(st["x"])
        st["mean"] = torch.empty((rows, self.G), device=dev, dtype=torch.bfloat16)
        st["rstd"] = torch.empty((rows, self.G), device=dev, dtype=torch.bfloat16)
        return st

    def step(self, capi, st, world):
        capi.native_group_norm(st["x"], st["weight"], st["bias"], st["x"].shape[0], self.C, self.HW, self.G, 1e-5,
                               out=(st["y"], st["mean"], st["rstd"]))

    def cpu_step(self, cpu):
        return torch.ops.aten.native_group_norm(cpu["x"], cpu["weight"], cpu["bias"], cpu["x"].shape[0], self.C, self.HW,
                                                self.G, 1e-5)

    def aten_step(self, st, world):
        return torch.ops.aten.native_group_norm(st["x"], st["weight"], st["bias"], st["x"].shape[0], self.C, self.HW,
                                                self.G, 1e-5)

    def _nbytes(self, rows, k):
        return rows * self.C * self.HW * 2

    def _out_bytes(self, rows):
        return rows * self.C * self.HW * 2 + 2 * rows * self.G * 2


class BatchNormStats(_Simple):
    """Not a BASELINE config: batch_norm_stats (per-channel mean and 1/sqrt(var + eps)) on the first shape of the
    reference microbenchmark (test/microbench/batch_norm_2d.py: [256, 256, 56, 56]), bf16.  `rows` are samples.
    A read-only kernel: the roofline compares it with the measured COPY bandwidth, which counts a read and a write."""
    name, rows, C, HW, cpu_sample_rows = "bn", 256, 256, 56 * 56, 32
    e2e_inputs = ("x",)
    launches_per_step = 1
    l2_note = "input (392 MiB) larger than L2 (no flush needed)"

    def describe(self):
        return f"batch_norm_stats, bf16 [{self.rows}, {self.C}, 56, 56], eps 1e-5"

    def bytes_per_rows(self, rows):
        t = rows * self.C * self.HW * 2 + 2 * self.C * 4
        return {"total": t, "batch_norm_stats": t}

    def make_cpu_state(self, rows):
        g = torch.Generator().manual_seed(8001)
        return {"x": torch.randn((rows, self.C, 56, 56), generator=g).to(torch.bfloat16)}

    def make_device_state(self, rows, dev, seed):
        gen = torch.Generator(device=dev).manual_seed(seed)
        return {"x": (torch.randn((rows, self.C, 56, 56), generator=gen, device=dev) * 1.5 + 0.5).to(torch.bfloat16)}

    def step(self, capi, st, world):
        st["out"] = capi.batch_norm_stats(st["x"], 1e-5)

    def cpu_step(self, cpu):
        x = cpu["x"].float()
        var, mean = torch.var_mean(x, (0, 2, 3), unbiased=False)
        return mean, torch.rsqrt(var + 1e-5)

    def aten_step(self, st, world):
        return torch.batch_norm_stats(st["x"], 1e-5)

    def _nbytes(self, rows, k):
        return rows * self.C * self.HW * 2

    def _out_bytes(self, rows):
        return 2 * self.C * 4


class SpatialSoftmax(_Simple):
    """Not a BASELINE config: _softmax + _softmax_backward_data over dim 1 of bf16 [16, C, 512, 512] (the reference's
    spatial kernels, sycl/SoftMaxKernels.cpp:735-950 and :1395-1564; the shape of a segmentation head with C classes).
    `rows` are samples."""
    name, rows, C, HW, cpu_sample_rows = "sm_c64", 16, 64, 512 * 512, 1
    e2e_inputs = ("s", "g")
    collective = "none (samples are independent)"
    l2_note = "inputs (512 MiB per tensor) larger than L2 (no flush needed)"

    def describe(self):
        return f"_softmax + _softmax_backward_data over dim 1, bf16 [{self.rows}, {self.C}, 512, 512]"

    def bytes_per_rows(self, rows):
        n = rows * self.C * self.HW * 2
        return {"total": 5 * n, "softmax_fwd_tma": 2 * n, "softmax_bwd_tma": 3 * n}

    def make_cpu_state(self, rows):
        g = torch.Generator().manual_seed(7001)
        return {"s": torch.randn((rows, self.C, 512, 512), generator=g).to(torch.bfloat16),
                "g": torch.randn((rows, self.C, 512, 512), generator=g).to(torch.bfloat16)}

    def make_device_state(self, rows, dev, seed):
        gen = torch.Generator(device=dev).manual_seed(seed)
        st = {"s": torch.randn((rows, self.C, 512, 512), generator=gen, device=dev).to(torch.bfloat16),
              "g": torch.randn((rows, self.C, 512, 512), generator=gen, device=dev).to(torch.bfloat16)}
        st["p"] = torch.empty_like(st["s"])
        st["dx"] = torch.empty_like(st["s"])
        return st

    def step(self, capi, st, world):
        capi._softmax(st["s"], 1, False, out=st["p"])
        capi._softmax_backward_data(st["g"], st["p"], 1, torch.bfloat16, out=st["dx"])

    def cpu_step(self, cpu):
        p = torch.ops.aten._softmax(cpu["s"], 1, False)
        return torch.ops.aten._softmax_backward_data(cpu["g"], p, 1, torch.bfloat16)

    def aten_step(self, st, world):
        p = torch.ops.aten._softmax(st["s"], 1, False)
        return p, torch.ops.aten._softmax_backward_data(st["g"], p, 1, torch.bfloat16)

    def _nbytes(self, rows, k):
        return rows * self.C * self.HW * 2

    def _out_bytes(self, rows):
        return 2 * rows * self.C * self.HW * 2


class SpatialSoftmax19(SpatialSoftmax):
    name, C = "sm_c19", 19
    l2_note = "inputs (152 MiB per tensor) larger than L2 (no flush needed)"


class SpatialSoftmax150(SpatialSoftmax):
    name, C = "sm_c150", 150
    l2_note = "inputs (1200 MiB per tensor) larger than L2 (no flush needed)"


def layer_norm_long_rows(base):
    """`base` is bench.Cfg4LayerNorm (handed in, so that this module never imports the script that imports it)."""

    class LayerNormLongRows(base):
        """Not a BASELINE config: layer norm on rows twice the length one CTA's threads hold (the reference's
        few-long-rows regime, sycl/Norm.h:620-696), forward + backward with the weight gradients."""
        name, rows, N, cpu_sample_rows = "ln_long", 16384, 16384, 2048
        l2_note = "inputs (512 MiB per tensor) larger than L2 (no flush needed)"

    return LayerNormLongRows


EXTRA = {"bn": BatchNormStats, "sm_c19": SpatialSoftmax19, "sm_c64": SpatialSoftmax, "sm_c150": SpatialSoftmax150, "gn": GroupNormFwd, "cfg1": Cfg1LayerNormFwd, "cfg2": Cfg2RmsNorm, "cfg3": Cfg3Softmax, "cfg3m": Cfg3Masked,
         "cfg5": Cfg5CrossEntropy, "cfg5f": Cfg5FusedTail}
