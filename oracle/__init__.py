"""CPU oracle for the W8A8 linear hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this directory.  Only the test-suite,
the smoke check and the CPU-baseline leg of the benchmark may call it, and only
as the checker / the timed CPU arm -- never as a fallback for a CUDA kernel.

Two layers:

* ``bitspec``   -- NumPy, bit-level definitions (bf16 rounding, the canonical
  Walsh-Hadamard butterfly, Philox4x32-10, quantisation, the exact integer
  matmul, both dequant epilogues, stochastic rounding, the LoRA merge).
* ``torch_path`` -- the same path expressed with multi-threaded CPU PyTorch
  ops; this is what the reference would execute on a machine without a GPU and
  is what gets timed as the CPU baseline.

Parity pin: the reference has no tests or golden vectors of its own, so the
oracle is pinned against outputs of the reference's own functions executed on
seeded inputs (``tests/golden/make_golden.py`` generated the committed
fixtures by importing the reference).
"""
