"""B200-native implementation of FLASHNN's quantized-GEMM operators
(DynamicQuantize, GemmA8W8, GemmWeightOnly) and of the fused norm + quantise
producers of their int8 operand (RMSNormDquant, LayernormDquant) behind the
reference's module API."""
from .kernel_backend import (get_autotune_triton_kernels, get_use_triton,
                             set_autotune_triton_kernels, set_use_triton)
from .fused_moe import fused_moe_a16w4_forward, fused_moe_a8w8_forward
from .norm import LayernormDquant, RMSNormDquant
from .quant_gemm import DynamicQuantize, GemmA8W8, GemmWeightOnly

__all__ = ["DynamicQuantize", "GemmA8W8", "GemmWeightOnly", "RMSNormDquant", "LayernormDquant", "fused_moe_a8w8_forward", "fused_moe_a16w4_forward", "set_use_triton",
           "set_autotune_triton_kernels", "get_use_triton", "get_autotune_triton_kernels"]
