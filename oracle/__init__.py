"""CPU oracle for the grouped-GEMM / per-block-quantiser path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this
directory; it is used by ``tests/``, by ``__graft_entry__.smoke()`` and by the
CPU-baseline legs of ``bench.py`` as the checker that the CUDA kernels are
compared against (and as the timed CPU baseline).  It never stands in for a
missing CUDA extension.
"""

from .torch_oracle import *  # noqa: F401,F403
