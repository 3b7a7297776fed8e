"""CPU oracle for the ChebyKAN layer hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory.  The only permitted importers are the test-suite, the smoke check
and the CPU-baseline / reference arm of the benchmark, where it acts as the
checker or the timed CPU stand-in, never as the thing shipped.
"""
