"""neuralrs_b200 — Blackwell (sm_100a) backend for the NeuralRs resident-GPU training path.

The product is ``libnrs_b200.so`` (C ABI: ``include/nrs.h``, ``include/nrs_graph.h``).
This package holds the CUDA/C++ sources (``csrc/``), the build step
(``python -m neuralrs_b200.build``) and a thin ctypes mirror of the reference's
operator API (``neuralrs_b200.cuda``) used by the tests and the benchmark.
"""
from ._lib import (ACT_GELU, ACT_NONE, ACT_RELU, LIB_PATH, MATH_3XTF32, MATH_FP32, MATH_TF32, NrsError, lib)

__all__ = ["lib", "NrsError", "LIB_PATH", "MATH_3XTF32", "MATH_TF32", "MATH_FP32", "ACT_NONE", "ACT_RELU",
           "ACT_GELU"]
