"""flashbias_b200: the FlashBias attention path (low-rank additive bias, never materialised) for
NVIDIA B200, behind the reference's ``flash_bias_func`` signature.

The compute path is a C-ABI CUDA library (``libflashbias_b200.so``, built in-tree with
``python -m flashbias_b200.build``); importing the package does not need a GPU, calling the operator does.
"""
from .flash_bias import (FlashBiasAlibiFunc, FlashBiasFunc, check_device_status, flash_bias_alibi_func,
                         flash_bias_backward, flash_bias_forward, flash_bias_func)

__all__ = ["FlashBiasFunc", "flash_bias_func", "flash_bias_forward", "flash_bias_backward",
           "FlashBiasAlibiFunc", "flash_bias_alibi_func", "check_device_status"]
