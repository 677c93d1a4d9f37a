"""CPU oracle for the nestedtensor hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this directory.  Only the test-suite,
the smoke check and the benchmark's CPU-baseline / reference arm may.
"""
