"""CPU oracle for the attention hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this; only tests/, the smoke check and
the CPU-baseline leg of bench.py do.
"""
