"""CPU oracle for the SSPA packed-KV decode path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this
directory; it is the checker used by the tests, by the smoke run and by the
CPU-baseline leg of the benchmark.
"""
