"""CPU oracle for the normalization / softmax path.  TEST INFRASTRUCTURE ONLY.

Nothing under this package is part of the product: only tests/, __graft_entry__.smoke() and
bench.py's CPU-baseline / reference legs may import it, and only as the checker.  The product
(b200norm) never imports it and has no CPU path.

Two oracles live here:

* aten_oracle — PyTorch's own CPU ATen kernels for the operator family.  This is the parity
  standard the reference itself tests against (its device-vs-CPU suites), and the one the task
  names.  `ref_exact` runs the CPU op on fp32 upcasts and rounds once: the "fp32-accumulated
  reference" for the 1-ulp rule on 16-bit outputs.
* restate (restate.c, built by oracle/build.py) — a plain-C restatement of the reference's own
  algorithms (Welford row moments, the backward row sums, three-pass softmax, single-pass NLL),
  each function citing the SYCL source it follows.  It closes the one hole in the CPU ATen oracle
  (_fused_rms_norm_backward has no CPU kernel) and is pinned against CPU ATen and the committed
  golden vectors in tests/test_oracle.py.

Parity pin: the reference ships no golden files for this path (its tests compare device results
with CPU ATen at run time), and its SYCL sources cannot be compiled here (they need icpx, a SYCL
runtime and a PyTorch source tree).  The pin is therefore CPU ATen itself plus the known-answer
properties the reference's tests assert, restated in tests/; tests/golden/ holds vectors generated
by CPU ATen in the build container with the generating script beside them.
"""
