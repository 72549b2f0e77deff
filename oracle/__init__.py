"""CPU oracle for the quantized-linear path (TEST INFRASTRUCTURE, not product code).

This package restates, in plain torch/numpy on the host, the arithmetic of
lyraDiff's quantized-linear hot path: activation quantizers (int8 / e4m3 /
int4-group-64), weight quantizers, the INT8, FP8 and W4A4 GEMMs with their
dequant/bias/GELU/residual epilogues, and the LayerNorm / AdaLN / GEGLU
producers that feed the quantizers.  Every function cites the reference file
and lines it follows.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this
package, and only as the checker or as the timed host baseline.  The shipped
library never routes through it: the CUDA path fails loudly when its shared
library is missing.

PARITY UNPINNED: the reference ships no tests, golden vectors or known-answer
fixtures for this path, its CUDA/CUTLASS/cuBLASLt sources cannot be built or
run without a GPU and without the un-vendored CUTLASS submodule, so this oracle
is pinned only against (a) independent known-answer facts of the number formats
(e4m3 code table, round-half-even ties, saturation bounds) and (b) its own
committed golden vectors, which guard against regressions rather than prove
agreement with the reference binary.
"""

from . import e4m3, quant, gemm, norms, workloads  # noqa: F401
