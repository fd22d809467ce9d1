"""Drop-in alias: `import flashnn` resolves to the B200-native operators, so code
written against the reference's quantized-GEMM API (flashnn/__init__.py:7,10)
runs unchanged."""
from flashnn_b200 import (DynamicQuantize, GemmA8W8, GemmWeightOnly,  # noqa: F401
                          LayernormDquant, RMSNormDquant, fused_moe_a16w4_forward, fused_moe_a8w8_forward,
                          set_autotune_triton_kernels, set_use_triton)
