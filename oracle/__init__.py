"""CPU oracle for libstrix_b200 - TEST INFRASTRUCTURE, not product code.

Each function restates, in plain torch on the CPU, the torch reference that the
asf0/libstrix test-suite uses to judge the corresponding kernel (file:line cited
per function). Only tests/, the smoke check and the benchmark's CPU-baseline
leg import this package; nothing under libstrix_b200/ does.

Pinning: the restatements are checked against golden vectors produced by
running the reference's own in-test reference functions
(tests/golden/make_golden.py loads them from the reference tree), see
tests/test_oracle_golden.py.
"""
