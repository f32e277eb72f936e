"""CPU oracle for the block-sparse encoder path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package may import this
package; it is the checker used by the tests, by the smoke entry point and by
the CPU-baseline leg of the benchmark.  It restates, in numpy / torch-fp32, the
algorithm of the reference's own validation model (python/modeling_big_bird.py,
attention_type="block_sparse") and of its host metadata builder
(python/util.py).  Parity status: PINNED - tests/golden/ holds outputs of the
reference module itself (tables and hidden states) that this oracle is checked
against on every CPU test run.
"""
from .bigbird import *  # noqa: F401,F403
