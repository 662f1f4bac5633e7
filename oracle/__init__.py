"""CPU oracle for the FP8 W8A8 block-scaled linear path.

TEST INFRASTRUCTURE ONLY.  Nothing under this package is part of the product:
only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import it, and only as the checker or as the timed CPU baseline.  The
product (``nano_qwen_b200``) never imports it and has no CPU fallback.

Parity status: "parity unpinned" by the reference — nano_qwen ships no tests,
golden vectors or known-answer values for its linear layers and contains no
FP8 arithmetic at all.  The pins used instead are (1) outputs of the
reference's own ``nano_qwen.layers.linear`` modules run on CPU and committed as
fixtures under ``tests/golden`` (with the generating script), and (2) the
hand-checkable known-answer cases in the tests.
"""
