"""alto_b200 -- B200 (sm_100a) implementation of ALTO's low-precision linear hot path.

Host code is thin PyTorch glue over a C-ABI CUDA library (``libaltob200.so``): block
quantizers (MXFP4 / NVFP4 / MXFP8, randomised Hadamard transform, round-to-nearest and
stochastic rounding) and tcgen05 block-scaled GEMMs, behind the reference's Python
surface (``convert_to_*``, ``_to_*_then_scaled_mm``, ``TrainingOpConfig``,
``LowPrecisionTrainingModifier``).  There is no Triton, no CPU path and no fallback.
"""
__version__ = "0.1.0"
