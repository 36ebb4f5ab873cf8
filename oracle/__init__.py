"""CPU oracle for the block-scaled quantized product path: test infrastructure only.

Nothing in the ``qiyas_b200`` package imports this; the tests, the smoke check and the
bench's CPU-baseline legs do.
"""
