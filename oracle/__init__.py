"""CPU checker for the quantized-matmul path (test infrastructure, not product).

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg import
this package; the product library never does.
"""
