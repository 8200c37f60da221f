"""CPU checker for the dequantize-and-multiply path.  TEST INFRASTRUCTURE ONLY.

Nothing under gguf_jax_b200/ imports this package; it is used by tests/, by the smoke
test and by the CPU-baseline leg of bench.py.
"""
