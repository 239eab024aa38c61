"""CPU oracle for the PE-attention hot path.  TEST INFRASTRUCTURE ONLY.

Nothing under this package is part of the shipped product: it is imported by
the tests, by the smoke check and by the CPU-baseline leg of the benchmark,
and only as the checker.  The product path (``pe_ablations_b200``) never
imports it and has no CPU fallback.
"""
