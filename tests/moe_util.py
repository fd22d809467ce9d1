"""Fused-MoE test cases: the generators live with the other seeded workloads."""
from flashnn_b200.workloads import make_moe_case, make_moe_w4_case, moe_align_block_size  # noqa: F401
