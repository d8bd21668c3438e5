"""CPU oracle for the GPTQ / QEP layer-quantization path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this
directory; it is used by the tests, by the smoke check and by the CPU-baseline
/ reference legs of the benchmark as the checker or the timed CPU arm.

The oracle restates, in plain torch-on-CPU (fp32 math exactly as the reference
performs it) and numpy (integer packing), what OneComp v1.4.0 computes on this
path.  Parity is pinned: ``tests/golden`` holds outputs of the reference
itself (imported from its source tree when the fixtures were generated) and
``tests/test_oracle_golden.py`` checks the oracle against them bit for bit.
"""
