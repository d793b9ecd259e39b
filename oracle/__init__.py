"""CPU oracle for the BC4 weight-linear path.

TEST INFRASTRUCTURE ONLY.  Nothing under ``oracle/`` is part of the product:
only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import it, and only as the checker.  The product path (``texelator_b200``)
never imports this package and has no CPU fallback.
"""
