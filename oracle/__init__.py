"""CPU oracle for the EPTQ quantized-linear path.

TEST INFRASTRUCTURE ONLY.  This package restates, in numpy, the arithmetic of
the reference's reconstruct path (codebook generation, `dequantize_layer`,
fp32 matmul of the reconstructed weights).  It is the checker the CUDA path is
compared against; nothing in the product package imports it.  Importers are
limited to the test-suite, the smoke check and the CPU-baseline leg of the
benchmark.

Parity status: PINNED.  Every function here is checked against outputs of the
reference's own Python (imported and run on CPU when the fixtures were made)
stored under ``tests/golden/`` together with the script that produced them.
"""
from .codebooks import e8_raw_points, d4_raw_codes, e8_table, d4_table  # noqa: F401
from .reconstruct import (  # noqa: F401
    LayerArrays, dequantize_layer, linear_reference, gemv_formula_reference,
    csr_from_q,
)
