"""Parallelism building blocks that sit next to the EP core: the single-GPU emulation of a
multi-rank job, all-gather / reduce-scatter sessions, pipeline send / recv, Engram, and the
fused tensor-parallel GEMM + collective operators."""
