"""CPU oracle for the FP8 fine-grained-scaled GEMM path -- TEST INFRASTRUCTURE ONLY.

Parity unpinned: the reference holds no golden vectors for this path.  `ref` is the
torch-CPU restatement (also the timed CPU baseline), `cref` loads the independent C
restatement (oracle/fp8_oracle.c).  Only tests, the smoke check and the benchmark's
CPU-baseline leg may import this package.
"""
