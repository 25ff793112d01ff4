"""CPU oracle for the block-scaled grouped-GEMM / MoE hot path.

TEST INFRASTRUCTURE ONLY. Nothing in the product package imports this directory:
it exists so that tests, the smoke entry and the benchmark's CPU-baseline leg can
check the CUDA path against an independent restatement of the reference's
arithmetic. Every function cites the reference file:line it follows.
"""
