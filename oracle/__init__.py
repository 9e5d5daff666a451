"""CPU oracle for the CRB calibration-time binarization path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory; it is the checker used by the tests, by the smoke entry and by the
CPU-baseline leg of the benchmark.
"""
