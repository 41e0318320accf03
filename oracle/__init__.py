"""CPU oracle for the decode / speculative-verify hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this directory: it is the
checker that the parity tests, the smoke entry and the CPU-baseline leg of the benchmark
compare the CUDA kernels against.  It restates, in numpy, the arithmetic of the reference
bundle's `qwen36_layer` / `qwen36_lmhead8` nodes (snapshot `qwen36_nodes_kb34`) at the target
shapes (512 experts, top-10, fp8 block scales / int8 W8A8, explicit GDN state); every function
cites the reference file:line whose rounding points and summation order it follows.

Pinning status.  The reference ships no golden vectors or tests.  The pieces of the reference
that run on a CPU (its torch quantisers and its Triton router / SwiGLU / combine kernels under
the Triton interpreter, at the reference's own 256-expert / top-8 shapes) were run once and
their outputs are committed under `tests/golden/` together with the generating script; the
oracle functions that have such a counterpart are checked against them.  The GDN recurrence,
the fp8 128x128 block-scaled GEMMs, the fused attention front at GEMM level, the attention-verify
core and the LM-head argmax have no CPU-runnable counterpart in the reference: for those rows PARITY IS UNPINNED by
the reference and rests on this restatement alone.
"""
