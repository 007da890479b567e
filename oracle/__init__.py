"""CPU restatement of the reference's numpy decode path.

TEST INFRASTRUCTURE ONLY. Nothing in the product package imports this; it is
the checker for the CUDA path (tests, the smoke check and the CPU-baseline leg
of the benchmark), never the thing that is shipped or measured as the product.

Parity status: PINNED.  Every function here is checked against the reference's
own numpy code (models/gpt2.py, models/llama.py), imported unmodified in the
build container by tests/golden/make_golden.py, and against the fixtures that
script commits under tests/golden/.
"""
