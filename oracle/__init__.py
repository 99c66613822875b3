"""CPU oracle for the quantised-projection and MoE hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may import this
directory: it is the checker that the CUDA path is compared against (tests,
the smoke check and the CPU-baseline leg of the benchmark), never the thing
that is measured or shipped.

Every function restates, in NumPy, arithmetic that the reference defines
(file:line cites are relative to the reference project root).  Parity of the
restatement is pinned against the reference's own golden vectors and against
outputs of the reference's importable Python packers (see tests/golden/).
"""

from . import codecs, nvfp4, fp8, moe  # noqa: F401
