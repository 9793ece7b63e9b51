"""CPU oracle for the RL-step path.  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this package; the product (``gonano_b200``) never does.
"""
