"""CPU oracle for the padding-free BERT encoder path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may import this
directory: it is used by the tests, by the GPU smoke check and by the CPU
baseline leg of the benchmark as the checker, never as the product path.
"""
