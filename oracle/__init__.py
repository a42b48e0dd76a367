"""CPU oracle for the quantized-linear path.  TEST INFRASTRUCTURE ONLY.

This package restates, on the CPU, the arithmetic of the reference's weight-only
int4 / int8 quantized linear layers and of the quantizer that produces their
weights.  It exists so that the CUDA kernels can be checked against it; it is
never the thing that is shipped or measured.  Only the test-suite, the smoke
check and the CPU-baseline leg of the benchmark import it.  The product package
(`linnet_b200`) never does, and raises when its CUDA library is missing.

Pinning: every function here is checked against fixtures produced by running
the reference's own Python (`linnet.quant`, `linnet.torch.quantized`,
`linnet.torch.native`, and `linnet.torch.load` of small cards) in the build
container; the fixtures and the script that made them live in `tests/golden/`.
"""

from . import linear_oracle, quant_oracle  # noqa: F401
