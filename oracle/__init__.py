"""CPU oracle for the NVFP4 routed-expert path: test infrastructure only.

Nothing in the product package may import this; it is used by tests/, by the
smoke check and by the CPU-baseline leg of bench.py as the checker.
"""
