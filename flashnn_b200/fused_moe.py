"""fused_moe_a8w8_forward with the reference's signature
(flashnn/triton_kernels/fused_moe_a8w8.py:176-190): int8 tokens x the int8 weights of the expert each
expert-sorted slot belongs to, scaled per token and per (expert, channel), optionally by the routing weight,
written to the caller's output rows."""
import torch

from . import _lib
from .quant_gemm import _DT, _require_cuda, _stream, _workspace


def _i32(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.int32 else t.to(torch.int32)


def fused_moe_a8w8_forward(A, B, C, alpha_row_ptr, alpha_col_ptr, topk_weights, topk_ids, sorted_token_ids,
                           expert_ids, num_tokens_post_padded, mul_routed_weight, top_k, BM):
    """A [M, K] int8; B [E, N, K] int8; C [M, top_k, N] fp16/bf16 (written in place, rows named by no slot are left
    alone); alpha_row_ptr [M]; alpha_col_ptr [E, N]; topk_weights, topk_ids [M, top_k]; sorted_token_ids [EM],
    expert_ids [EM / BM] and num_tokens_post_padded [1] as produced by the block-aligned expert sort."""
    _require_cuda(A, B, C, alpha_row_ptr, alpha_col_ptr, topk_weights, sorted_token_ids, expert_ids, num_tokens_post_padded)
    assert topk_weights.stride(1) == 1
    assert sorted_token_ids.stride(0) == 1
    assert B.shape[1] % 16 == 0 and B.shape[2] % 16 == 0
    assert A.dtype == torch.int8 and B.dtype == torch.int8, "A and B must be int8"
    assert C.dtype in (torch.float16, torch.bfloat16) and C.dim() == 3 and C.stride(2) == 1
    assert C.stride(0) == C.shape[1] * C.stride(1), "C must be viewable as [M * top_k, N]"
    E, N, K = B.shape
    a2 = A.reshape(-1, K)
    if a2.stride(1) != 1:
        a2 = a2.contiguous()
    b = B if B.is_contiguous() else B.contiguous()
    col = alpha_col_ptr if alpha_col_ptr.is_contiguous() else alpha_col_ptr.contiguous()
    row = alpha_row_ptr.reshape(-1)
    row = row if row.is_contiguous() else row.contiguous()
    tw = topk_weights if topk_weights.is_contiguous() else topk_weights.contiguous()
    if tw.dtype not in _DT:
        tw = tw.float()
    sid, eid, npp = _i32(sorted_token_ids), _i32(expert_ids), _i32(num_tokens_post_padded)
    em = sid.shape[0]
    with torch.cuda.device(A.device):
        need = _lib.lib().fnn_fused_moe_a8w8_workspace_bytes(em, K)
        ws = _workspace(A.device, need)
        _lib.check(_lib.lib().fnn_fused_moe_a8w8(
            a2.data_ptr(), a2.stride(0), b.data_ptr(), E, N, K, row.data_ptr(), _DT[row.dtype], col.data_ptr(),
            _DT[col.dtype], tw.data_ptr(), _DT[tw.dtype], sid.data_ptr(), em, eid.data_ptr(), npp.data_ptr(),
            topk_ids.numel(), int(top_k), int(BM), int(bool(mul_routed_weight)), C.data_ptr(), _DT[C.dtype], C.stride(1),
            ws.data_ptr(), ws.numel(), _stream(A)))
    return C
