"""Test infrastructure only: a CPU restatement of the reference's MoE hot path.

Nothing in the shipped package imports this directory.  It is the checker used
by the test-suite, by the smoke entry point and by the CPU-baseline leg of the
benchmark; it is never the thing being measured or shipped.
"""
