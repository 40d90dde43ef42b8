"""CPU oracle package: TEST INFRASTRUCTURE ONLY.

Restates the reference's algorithms for the two hot paths on the CPU so that the CUDA library can be
checked against them.  Only tests/, the smoke check and bench.py's cpu_baseline / reference legs may import
anything from here; the product package (tmq_b200) never does and fails loudly without its CUDA library.

  oracle.softstep        numpy fp32 restatement of the soft-staircase formulas (tmq/tmq.py:353-493)
  oracle.softstep_torch  the same op sequence as PyTorch CPU eager ops (what the reference executes on CPU);
                         used for the timed CPU baseline
  oracle.ternary         ctypes front end of oracle.c: pack / unpack / decode-then-matmul / range coder
  oracle.build_ref       compiles the reference's own extension sources into oracle/_ref/
"""
