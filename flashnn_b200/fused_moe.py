"""fused_moe_a8w8_forward and fused_moe_a16w4_forward with the reference's signatures
(flashnn/triton_kernels/fused_moe_a8w8.py:176-190, fused_moe_a16w4.py:326-340): tokens x the weights of the expert
each expert-sorted slot belongs to (int8 x int8 with per-token and per-channel scales, or fp16/bf16 x packed int4
with per-channel or per-group scales), optionally scaled by the routing weight, written to the caller's output rows."""
import torch

from . import _lib
from .quant_gemm import _DT, _on_device, _require_cuda, _stream, _workspace


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
    with _on_device(A):
        need = _lib.lib().fnn_fused_moe_a8w8_workspace_bytes(em, K)
        ws = _workspace(A.device, need)
        _lib.check(_lib.lib().fnn_fused_moe_a8w8(
            a2.data_ptr(), a2.stride(0), b.data_ptr(), E, N, K, row.data_ptr(), _DT[row.dtype], col.data_ptr(),
            _DT[col.dtype], tw.data_ptr(), _DT[tw.dtype], sid.data_ptr(), em, eid.data_ptr(), npp.data_ptr(),
            topk_ids.numel(), int(top_k), int(BM), int(bool(mul_routed_weight)), C.data_ptr(), _DT[C.dtype], C.stride(1),
            ws.data_ptr(), ws.numel(), _stream(A)))
    return C


def fused_moe_a16w4_forward(A, B, C, scale_b, zero_points, topk_weights, topk_ids, sorted_token_ids, expert_ids,
                            num_tokens_post_padded, mul_routed_weight, top_k, BM):
    """A [M, K] fp16/bf16; B [E, N/2, K] packed int4 (int8 or uint8 bytes: channel 2j in the low nibble of byte (j, k),
    2j+1 in the high one); C [M, top_k, N] in A's dtype (written in place, rows named by no slot are left alone);
    scale_b / zero_points [E, N] per channel or [E, N, K / group] per K group (zero_points may be None);
    the routing tensors as for fused_moe_a8w8_forward."""
    _require_cuda(A, B, C, scale_b, zero_points, topk_weights, sorted_token_ids, expert_ids, num_tokens_post_padded)
    assert topk_weights.stride(1) == 1
    assert sorted_token_ids.stride(0) == 1
    assert B.shape[1] % 16 == 0 and B.shape[2] % 16 == 0
    assert B.dtype in (torch.int8, torch.uint8), "B must hold packed int4 bytes"
    assert A.dtype in (torch.float16, torch.bfloat16) and C.dtype == A.dtype and C.dim() == 3 and C.stride(2) == 1
    assert C.stride(0) == C.shape[1] * C.stride(1), "C must be viewable as [M * top_k, N]"
    E, NP, K = B.shape
    N = 2 * NP
    assert C.shape[2] == N, "C's last dimension must be twice B's packed dimension"
    a2 = A.reshape(-1, K)
    if a2.stride(1) != 1:
        a2 = a2.contiguous()
    b = B if B.is_contiguous() else B.contiguous()
    assert scale_b.dim() in (2, 3) and scale_b.shape[0] == E and scale_b.shape[1] == N and scale_b.dtype in _DT
    if scale_b.dim() == 3:
        assert K % scale_b.shape[2] == 0, "scale_b's last dimension must divide K"
        group = K // scale_b.shape[2]
    else:
        group = 0
    scale = scale_b if scale_b.is_contiguous() else scale_b.contiguous()
    zp = None
    if zero_points is not None:
        assert zero_points.shape == scale_b.shape, "zero_points must have the shape of scale_b"
        zp = zero_points if zero_points.dtype == scale.dtype and zero_points.is_contiguous() else zero_points.to(scale.dtype).contiguous()
    tw = topk_weights if topk_weights.is_contiguous() else topk_weights.contiguous()
    if tw.dtype not in _DT:
        tw = tw.float()
    sid, eid, npp = _i32(sorted_token_ids), _i32(expert_ids), _i32(num_tokens_post_padded)
    with _on_device(A):
        L = _lib.lib()
        ws_bytes = L.fnn_fused_moe_a16w4_workspace_bytes(sid.shape[0], K, group, int(zp is not None), int(BM))
        ws = _workspace(A.device, ws_bytes) if ws_bytes else None
        _lib.check(L.fnn_fused_moe_a16w4_ws(
            a2.data_ptr(), _DT[A.dtype], a2.stride(0), b.data_ptr(), E, N, K, scale.data_ptr(),
            zp.data_ptr() if zp is not None else None, _DT[scale.dtype], group, tw.data_ptr(), _DT[tw.dtype],
            sid.data_ptr(), sid.shape[0], eid.data_ptr(), npp.data_ptr(), topk_ids.numel(), int(top_k), int(BM),
            int(bool(mul_routed_weight)), C.data_ptr(), _DT[C.dtype], C.stride(1),
            ws.data_ptr() if ws is not None else None, ws_bytes, _stream(A)))
    return C
