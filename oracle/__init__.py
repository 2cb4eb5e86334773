"""TEST INFRASTRUCTURE: CPU oracle for the recurrent-scan hot path (see scan_oracle.c).

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may import this
package; the product (``tsfast_b200``) never does.
"""
