"""CPU oracle for the quantized-inference path of qwix (TEST INFRASTRUCTURE ONLY).

This package restates, in NumPy + ml_dtypes, the arithmetic that the reference
performs through JAX for

  * QArray quantize / dequantize           (qwix/_src/core/qarray.py, numerics.py)
  * quantized dot_general / einsum / dot   (qwix/_src/core/dot_general.py, einsum.py,
                                            einsum_info.py, dot.py)
  * Hadamard rotation + tile quantizer     (qwix/contrib/hadamard_rot.py,
                                            qwix/contrib/kernels/fused_hadamard_quantized_matmul.py)

It is the checker for the CUDA path and the timed CPU baseline.  Nothing in the
shipped package imports it: only tests, the smoke entry and the benchmark's
cpu_baseline / reference arm do.

Parity pins.  The reference is Python-on-JAX and JAX is not installable where
this was built, so the oracle is pinned against every known-answer vector that
the reference's own tests hold and that does not depend on JAX's PRNG stream
(see tests/golden/reference_known_answers.json and the test that replays it).
For bfloat16 inputs no reference test asserts qvalues bit-for-bit, so that part
is "parity unpinned"; the oracle offers both roundings that JAX can produce:

  mode="strict"  every primitive rounds to the array dtype (JAX eager semantics;
                 the normative mode here)
  mode="fused"   intermediates of the divide/add/round chain stay in float32
                 (what XLA does under jit with excess precision allowed)
"""

from oracle import numerics  # noqa: F401
from oracle import qarray  # noqa: F401
from oracle import dot_general  # noqa: F401
from oracle import einsum  # noqa: F401
from oracle import hadamard  # noqa: F401
