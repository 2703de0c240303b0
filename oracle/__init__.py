"""CPU oracle for the GEMQ real-quantized MoE inference path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory; only the test-suite, the smoke check and the CPU-baseline leg of the
benchmark may.  Every function restates, in numpy/torch on the CPU, what one
reference routine computes and cites the reference file:line it follows.
"""
