"""Test-only checkers for the quantised-linear hot path (see quant_linear.py, quant_linear.c,
test_formula.py).  The shipped package does not import this."""
