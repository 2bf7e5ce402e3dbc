"""CPU oracle for the INT8 quantized-linear path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this directory; only the tests, the
smoke check and the CPU-baseline leg of the benchmark do.
"""
