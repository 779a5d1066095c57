"""Counterpart of the reference's ``constants.py``."""
dimension_numbers = (((1,), (1,)), ((), ()))
MIN_BLOCK_SIZE = 128
