"""CPU oracle for the sparse-attention selection path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory; only the tests, the smoke check and the benchmark's CPU-baseline
leg do, and there only as the checker or the timed CPU arm.
"""
