"""CPU restatement of the PBS-Attn prefill path. TEST INFRASTRUCTURE ONLY.

Nothing under this package is part of the product: only the test-suite, the
smoke check and the benchmark's CPU-baseline leg may import it, and only as the
checker.  The CUDA path never routes through it.
"""
