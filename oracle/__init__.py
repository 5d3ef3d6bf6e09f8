"""CPU restatement of the reference arithmetic for the INT8 chunk-prefill path.

TEST INFRASTRUCTURE ONLY. Nothing in the product package imports this directory; it is
used by the test-suite, by the smoke check and by the CPU-baseline leg of the benchmark,
always as the checker or as the timed CPU baseline, never as a compute fallback.
"""
