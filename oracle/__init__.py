"""CPU oracle for the numba-mlir data-parallel offload path.

TEST INFRASTRUCTURE ONLY.  Nothing under this package is part of the product:
only the tests, the smoke check and the CPU-baseline / reference legs of the
benchmark may import it, and only as the checker or the timed CPU baseline.

What the oracle is.  The reference's `njit` *is* upstream `numba.njit` whenever
its MLIR pipeline is switched off (numba_mlir/numba_mlir/decorators.py:89-98),
and its `@kernel` tests compare every device result with a pure-Python
simulator (numba_mlir/numba_mlir/mlir/kernel_sim_impl.py:193-234).  The
reference's own compiler cannot be built here (it needs LLVM/MLIR at the commit
of llvm-sha.txt, TBB and a SYCL toolchain), so this oracle restates each
workload in the form upstream Numba compiles, following the reference file and
lines cited on every function, plus a float64 NumPy ground truth.

Pinning.  tests/test_oracle_pins.py checks the oracle against the known-answer
cases of the reference's own tests (inputs re-derived from the cited lines) and
against golden vectors generated in this container by running the reference's
kernel_sim_impl.py (tests/golden/make_golden.py).  `np.argmin` has no passing
test in the reference (numba_mlir/mlir/tests/test_numba_parfor.py:60,65 mark
it xfail): parity unpinned for argmin beyond NumPy's first-minimum rule.
"""
