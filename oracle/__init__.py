"""CPU oracle for the KV-cache hot path.  TEST INFRASTRUCTURE ONLY.

Everything in this package is a CPU restatement of what the reference
(rahulm520/AMD-PACE) computes on its KV-cache path: cache append / rollback /
beam gather bookkeeping, and scaled-dot-product attention over the cache.  It
exists so the CUDA kernels can be checked against it.  Only the test-suite,
the smoke entry and the benchmark's CPU-baseline leg may import it; the
product package never does and has no CPU fallback.

Pinning: the restatements are checked (tests/test_oracle_*.py) against golden
vectors produced by importing and running the reference's own Python code
(tests/golden/make_golden.py, vectors committed under tests/golden/), and
against the known-answer values of the reference's tests
(tests/llm_infra/test_cache.py:53-64,76-80).
"""
