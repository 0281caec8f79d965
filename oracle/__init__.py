"""CPU restatement of the reference's FP4 MLA decode arithmetic.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this
directory; it is the checker used by the tests, by the smoke entry and by the
benchmark's CPU-baseline leg.
"""
