"""CPU restatement of the reference's KMeans path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory.  It exists so that the CUDA kernels can be checked against the
arithmetic of soda-inria/sklearn-numba-dpex (whose own device stack, numba_dpex
on a SYCL device, cannot run without the Intel toolchain).  Only the test
suite, the smoke check and the benchmark's CPU-baseline leg may use it.

Parity status: PINNED against the known answers held by the reference's own
tests (RNG raw streams and floats, the k-means++ golden score, the two
empty-cluster relocation cases, the predict-on-centres case, the top-k tie
cases, the argmin cases) and against scikit-learn's Lloyd on the reference's
`make_blobs(random_state=42)` parity case.  See tests/test_oracle_golden.py.
"""
