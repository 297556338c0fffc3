"""CPU oracle for the quantized Pi0.5 inference hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory; only the test-suite, the smoke check and the benchmark's CPU
baseline leg do, and only as the checker.

Every function restates, in numpy, the arithmetic of one reference routine and
cites it (paths are relative to the reference project root).  The restatements
are pinned two ways:

* against the reference's only deterministic known-answer test
  (openpi/src/openpi/tests/debug_packer.py:41-117), and
* against golden vectors produced by importing the reference's own Python
  modules on seeded inputs (tests/golden/, with the generating script).

Parity status per routine:
  INT4 packers / dequant / GEMV math ........ pinned (known-answer + golden)
  NVFP4 quantise / pack / dequant-GEMV ...... pinned (golden)
  NVFP4 sim quantise / dequant (E4M3 scales)  pinned (golden)
  kv_fuse quantise + fallback projection .... pinned (golden)
  RoPE + KV-cache append .................... pinned (golden; the reference
      has no test of its own for this, so the pin is the output of its
      stand-alone RoPE restatement run on seeded inputs)
  plugin CUDA quantisers (INT4 / NVFP4-E4M3 / FP8 activation): parity
      unpinned -- the reference holds no vectors for them and its CUDA cannot
      run in the container that generates fixtures; they follow the kernel
      source line by line.
"""
