"""CPU oracle for the advantage hot path -- test infrastructure, not product.

Only the test-suite, the smoke check and the benchmark's CPU-baseline /
reference arms may import this package.
"""
