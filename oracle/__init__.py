"""CPU oracle for the CorrMM convolution path: test infrastructure only.

Nothing in the product package imports this; tests, the smoke check and the
CPU-baseline leg of the benchmark use it as the checker.
"""
