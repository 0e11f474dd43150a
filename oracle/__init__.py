"""CPU oracle for the matmul / FlashAttention-2 path.  TEST INFRASTRUCTURE ONLY.

Nothing under this directory is part of the product: only tests/, the smoke
check and the benchmark's CPU-baseline leg may import it, and only as the
checker.  libtmcuda never calls into it and has no CPU fallback.
"""
