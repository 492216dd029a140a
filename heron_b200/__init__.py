"""heron_b200 — sm_100a kernels for the tensor programs Heron tunes (GEMM, batched GEMM, NHWC
conv2d; fp16 -> fp32 and u8/s8 -> s32), behind Heron's own operator / Task interface.

Importing the package does not load the CUDA library; the first kernel call does, and fails
loudly if ``libheron_b200.so`` has not been built (``python -m heron_b200.build``).
"""
__version__ = "0.1.0"
