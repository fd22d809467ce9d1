"""CPU oracle for the quantized-GEMM path.  TEST INFRASTRUCTURE ONLY.

This module restates, with plain PyTorch CPU ops, what the reference's torch
implementations of the three operators compute.  It exists to check the CUDA
kernels; nothing in the shipped package imports it.  Only the tests, the smoke
check and the benchmark's CPU-baseline leg may call into it.

Parity status: PINNED.  `tests/golden/*.npz` hold outputs of the reference's own
classes (run on CPU with its torch backend selected) on seeded inputs;
`tests/test_oracle_golden.py` requires every function below to reproduce them
bit for bit.

Functions and the reference lines they follow (paths inside the reference
project):

* `dynamic_quantize`            flashnn/quant_gemm.py:53-57
* `gemm_a8w8`                   flashnn/quant_gemm.py:96-104
* `gemm_a8w8_acc_i32`           exact form of the product at quant_gemm.py:97-98
* `unpack_int4`                 flashnn/quant_gemm.py:175-190
* `dequantize_reference`        flashnn/quant_gemm.py:14-36
* `gemm_weight_only_reference`  flashnn/quant_gemm.py:148-206
* `gemm_weight_only_fp32`       same contraction with no 16-bit rounding of w*s
* `rms_norm_dquant`             flashnn/norm.py:39-63
* `layer_norm_dquant`           flashnn/norm.py:94-124
* `fused_moe_a8w8`              flashnn/triton_kernels/fused_moe_a8w8.py:96-170.  The reference has neither a torch
                                implementation nor a test of its fused-MoE kernels, so this restates the Triton
                                kernel's arithmetic from its source; it is pinned by tests/golden/fused_moe_a8w8.npz,
                                outputs of that Triton kernel itself run on a B200 by tests/golden/make_moe_golden.py
* `fused_moe_a16w4`             flashnn/triton_kernels/fused_moe_a16w4.py:50-323, pinned the same way by
                                tests/golden/fused_moe_a16w4.npz
"""
from __future__ import annotations

import torch


# ----------------------------------------------------------------------------
# DynamicQuantize
# ----------------------------------------------------------------------------
def dynamic_quantize_precast(x: torch.Tensor):
    """Per-token symmetric int8 quantisation, up to (not including) the int8 cast.

    Follows flashnn/quant_gemm.py:53-56: every step runs in the dtype of `x`
    (so for bf16 the scale and the quotient are each rounded to bf16), the
    rounding is half-to-even, and nothing is clamped.

    Returns (rounded quotient in x.dtype, scale in x.dtype with shape [M, 1]).
    """
    amax = x.abs().max(-1, keepdim=True)[0]
    scale = amax / 127.0
    return torch.round(x / scale), scale


def dynamic_quantize(x: torch.Tensor, saturate: bool = True):
    """DynamicQuantize as the reference's torch path computes it
    (flashnn/quant_gemm.py:53-57) -> (int8 [M, K], fp16 scale [M]).

    `saturate=False` reproduces the reference's unclamped int8 cast, which lets
    a quotient of +128 (reachable with bf16 input) wrap to -128.
    `saturate=True` is the behaviour of the CUDA kernel: identical everywhere
    except that +128 becomes +127.  Rows whose absmax is 0 give NaN quotients
    in the reference; the kernel writes q = 0 and scale = 0 there, and so does
    this function when `saturate` is set.
    """
    q, scale = dynamic_quantize_precast(x)
    if saturate:
        q = torch.nan_to_num(q.float(), nan=0.0).clamp_(-128.0, 127.0)
    return q.to(torch.int8), scale.half().squeeze(-1)


# ----------------------------------------------------------------------------
# GemmA8W8
# ----------------------------------------------------------------------------
def gemm_a8w8_acc_i32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Exact int32 accumulator of A[M,K] . B[N,K]^T.

    The reference multiplies in fp32 (flashnn/quant_gemm.py:97-98), which is
    exact only below 2**24.  fp64 is exact to 2**53, far beyond K * 128**2 for
    any K that fits in memory, so this is the integer result itself.
    """
    acc = a.double() @ b.double().t()
    return acc.to(torch.int64).to(torch.int32)


def _outer_scale(alpha_row: torch.Tensor, alpha_col: torch.Tensor) -> torch.Tensor:
    # flashnn/quant_gemm.py:99-102.  torch.matmul refuses mixed dtypes, so
    # callers hand both scales over in one dtype; a mixed pair is promoted to
    # fp32 here, which is what the CUDA epilogue does for that case.
    r = torch.squeeze(alpha_row).flatten()
    c = torch.squeeze(alpha_col).flatten()
    if r.dtype != c.dtype:
        r, c = r.float(), c.float()
    return torch.matmul(r.unsqueeze(-1), c.unsqueeze(0))


def gemm_a8w8(a, b, alpha_row, alpha_col, out_ty=torch.float16) -> torch.Tensor:
    """GemmA8W8 as the reference's torch path computes it
    (flashnn/quant_gemm.py:96-104): fp32 product, outer-product scale in the
    scales' dtype, one multiply, cast to `out_ty`."""
    x = torch.matmul(a.to(torch.float32), b.transpose(0, 1).to(torch.float32))
    out = torch.mul(x, _outer_scale(alpha_row, alpha_col))
    return out.to(out_ty)


def gemm_a8w8_from_acc(acc_i32, alpha_row, alpha_col, out_ty=torch.float16) -> torch.Tensor:
    """The epilogue of `gemm_a8w8` applied to an exact integer accumulator.
    Equal to `gemm_a8w8` whenever |acc| < 2**24; used for large-K checks where
    the reference's fp32 product is itself inexact."""
    out = torch.mul(acc_i32.to(torch.float32), _outer_scale(alpha_row, alpha_col))
    return out.to(out_ty)


# ----------------------------------------------------------------------------
# GemmWeightOnly
# ----------------------------------------------------------------------------
def weight_kind(quant_w: torch.Tensor, scale_w: torch.Tensor) -> str:
    """'int8' or 'int4', decided from shapes alone as at
    flashnn/quant_gemm.py:150-155."""
    if quant_w.size(0) * 2 == scale_w.size(-1):
        return "int4"
    if quant_w.size(0) == scale_w.size(-1):
        return "int8"
    raise AssertionError("Gemm WeightOnly only support int8 or int4x2")


def unpack_int4(quant_w: torch.Tensor) -> torch.Tensor:
    """Packed [N/2, K] bytes -> signed int8 [N, K].

    Byte (j, k) carries channel 2j in its low nibble and channel 2j+1 in its
    high nibble, both two's complement (flashnn/quant_gemm.py:175-190)."""
    w = quant_w.view(torch.uint8).to(torch.int16)
    lo = w & 0xF
    hi = (w >> 4) & 0xF
    lo = torch.where(lo > 7, lo - 16, lo)
    hi = torch.where(hi > 7, hi - 16, hi)
    return torch.stack((lo, hi), dim=1).reshape(-1, quant_w.shape[1]).to(torch.int8)


def pack_int4(w: torch.Tensor) -> torch.Tensor:
    """Inverse of `unpack_int4`: signed int8 [N, K] in [-8, 7] -> int8 [N/2, K]."""
    u = w.to(torch.int16) & 0xF
    return (u[0::2] | (u[1::2] << 4)).to(torch.uint8).view(torch.int8)


def dequantize_reference(w_kn, scale_w, zero_points=None) -> torch.Tensor:
    """(w - zp) * s as the reference forms it: per channel in the promoted
    dtype of the operands (flashnn/quant_gemm.py:14-17), per K-group written
    into an fp16 buffer whatever the scale dtype (flashnn/quant_gemm.py:20-36).
    `w_kn` is the integer weight transposed to [K, N]."""
    s = scale_w.squeeze()
    if s.dim() == 1:
        s = s.unsqueeze(0)
        zp = torch.zeros_like(s) if zero_points is None else zero_points
        return (w_kn - zp) * s
    zp = torch.zeros_like(s) if zero_points is None else zero_points
    group = w_kn.shape[0] // s.shape[0]
    assert group * s.shape[0] == w_kn.shape[0]
    out = torch.zeros_like(w_kn, dtype=torch.half)
    for g in range(s.shape[0]):
        out[g * group:(g + 1) * group] = (w_kn[g * group:(g + 1) * group] - zp[g]) * s[g]
    return out


def gemm_weight_only_reference(act, quant_w, scale_w, bias=None, zero_points=None,
                               out_ty=torch.float16) -> torch.Tensor:
    """GemmWeightOnly as the reference's torch path computes it
    (flashnn/quant_gemm.py:148-206), including where it rounds: the int8 branch
    casts to `out_ty` before adding the bias, the int4 branch adds in fp32."""
    assert act.shape[1] == quant_w.shape[1], "Matrix B must be transposed"
    kind = weight_kind(quant_w, scale_w)
    w = quant_w if kind == "int8" else unpack_int4(quant_w)
    dq = dequantize_reference(w.transpose(0, 1), scale_w, zero_points)
    out = torch.matmul(act.to(torch.float32), dq.to(torch.float32))
    if kind == "int8":
        out = out.to(out_ty)
    if bias is not None:
        out += bias
    return out.to(out_ty)


def gemm_weight_only_fp32(act, quant_w, scale_w, bias=None, zero_points=None,
                          out_ty=None) -> torch.Tensor:
    """The same contraction with the dequantised weight kept in fp32:
    act.float() @ ((w - zp) * s) + bias, rounded once at the end (or not at
    all when `out_ty` is None).  This is the bound the weight-only kernels are
    held to; `gemm_weight_only_reference` differs from it only by the 16-bit
    rounding of w*s."""
    kind = weight_kind(quant_w, scale_w)
    w = (quant_w if kind == "int8" else unpack_int4(quant_w)).transpose(0, 1).float()
    s = scale_w.squeeze().float()
    zp = None if zero_points is None else zero_points.squeeze().float()
    if s.dim() == 1:
        s = s.unsqueeze(0)
        zp = None if zp is None else zp.reshape(1, -1)
    else:
        group = w.shape[0] // s.shape[0]
        s = s.repeat_interleave(group, dim=0)
        zp = None if zp is None else zp.repeat_interleave(group, dim=0)
    dq = (w if zp is None else w - zp) * s
    out = torch.matmul(act.float(), dq)
    if bias is not None:
        out = out + bias.float()
    return out if out_ty is None else out.to(out_ty)


# ----------------------------------------------------------------------------
# Norm + dynamic quantisation (the producers of the A8W8 activation operand)
# ----------------------------------------------------------------------------
def rms_norm_dquant(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6):
    """fp32 throughout: n = x * rsqrt(mean(x^2) + eps) * weight, scale = max|n| / 127,
    q = clamp(round(n / scale), -128, 127).  Returns (int8 like x, scale x.shape[:-1] in x's dtype)."""
    xf = x.float()
    n = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    n = n * weight  # fp32 * (16-bit or fp32) parameter promotes to fp32
    scale = n.abs().max(dim=-1, keepdim=True)[0] / 127.0
    q = torch.clamp(torch.round(n / scale), -128.0, 127.0)
    # a NaN quotient (row of zeros, or a row holding a NaN / an infinity, whose scale is NaN) is cast to 0: what the
    # reference's .to(torch.int8) yields on x86 hosts, made explicit here so that it does not depend on the host
    return torch.nan_to_num(q, nan=0.0).to(torch.int8), scale.reshape(x.shape[:-1]).type_as(x)


def layer_norm_dquant(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-5):
    """layer_norm in x's dtype, then absmax / 127, the quotient and its rounding all in that dtype.
    Returns (int8 like x, scale [rows, 1] in x's dtype)."""
    n = torch.nn.functional.layer_norm(x, (x.shape[-1],), weight, bias, eps)
    scale = n.abs().max(dim=-1, keepdim=True)[0] / 127.0
    q = torch.clamp(torch.round(n / scale), -128.0, 127.0)
    return torch.nan_to_num(q.float(), nan=0.0).to(torch.int8), scale.reshape(-1, 1)  # NaN -> 0 as above


# ----------------------------------------------------------------------------
# Fused MoE (pinned by outputs of the reference's Triton kernels, see the header)
# ----------------------------------------------------------------------------
def fused_moe_a8w8(A, B, alpha_row, alpha_col, topk_weights, sorted_token_ids, expert_ids, num_tokens_post_padded,
                   num_valid_tokens, mul_routed_weight, top_k, BM, out_ty=torch.float16, C=None):
    """Block by block as the kernel walks the expert-sorted slots: exact int32 accumulator, then
    acc * alpha_row * alpha_col (* routing weight) in fp32, in that order, cast to `out_ty`, scattered to the flat
    (token, choice) rows of C [M, top_k, N].  Rows that no slot names keep what C held (zeros if C is None)."""
    E, N, K = B.shape
    M = A.shape[0]
    if C is None:
        C = torch.zeros(M, top_k, N, dtype=out_ty)
    flat_out = C.view(M * top_k, N)
    padded = int(num_tokens_post_padded.reshape(-1)[0])
    tw = topk_weights.reshape(-1)
    for blk in range(padded // BM):
        e = int(expert_ids[blk])
        slots = sorted_token_ids[blk * BM:(blk + 1) * BM].long()
        flat = slots[slots < num_valid_tokens]
        if flat.numel() == 0:
            continue
        rows = flat // top_k
        acc = gemm_a8w8_acc_i32(A[rows], B[e])
        v = acc.float() * alpha_row.reshape(-1)[rows].float()[:, None]
        v = v * alpha_col[e].float()[None, :]
        if mul_routed_weight:
            v = v * tw[flat].float()[:, None]
        # the kernel casts to fp16 whatever C's dtype is (fused_moe_a8w8.py:165); storing into a bf16 C rounds again
        flat_out[flat] = v.to(torch.float16).to(C.dtype)
    return C


def fused_moe_a16w4(A, B, scale_b, zero_points, topk_weights, sorted_token_ids, expert_ids, num_tokens_post_padded,
                    num_valid_tokens, mul_routed_weight, top_k, BM, C=None, exact_scales=False):
    """Fused-MoE A16W4 as the reference's Triton kernels compute it (flashnn/triton_kernels/fused_moe_a16w4.py).

    A [M, K] fp16/bf16; B [E, N/2, K] packed int4 (byte (j, k): channel 2j in the low nibble, 2j+1 in the high one,
    `:137,151`); scale_b / zero_points [E, N] (per channel) or [E, N, K/group]; C [M, top_k, N] in A's dtype.
    Per channel (`:50-183`): the integer weight minus the zero-point, in A's dtype, goes into an fp32-accumulated
    product; the accumulator is multiplied by the fp32 scale, then by the routing weight, and cast.
    Per group (`:186-323`): (w - zp) * s is formed in the scale's 16-bit dtype for every K group (one rounding per
    weight, `:289-303`), the product is accumulated in fp32, multiplied by the routing weight and cast.
    `exact_scales=True` keeps (w - zp) * s in fp32 instead: the fp32 dequant-matmul bound the CUDA kernels are held to.
    Rows that no slot names keep what C held (zeros if C is None).  The fp32 summation order of a tensor-core dot
    product is not defined, so outputs of the Triton kernel are reproduced to within a rounding of the result."""
    E, NP, K = B.shape
    N = 2 * NP
    M = A.shape[0]
    dt = A.dtype
    if C is None:
        C = torch.zeros(M, top_k, N, dtype=dt)
    flat_out = C.view(M * top_k, N)
    padded = int(num_tokens_post_padded.reshape(-1)[0])
    tw = topk_weights.reshape(-1)
    per_channel = scale_b.dim() == 2
    for blk in range(padded // BM):
        e = int(expert_ids[blk])
        slots = sorted_token_ids[blk * BM:(blk + 1) * BM].long()
        flat = slots[slots < num_valid_tokens]
        if flat.numel() == 0:
            continue
        rows = flat // top_k
        w = unpack_int4(B[e])  # [N, K] int8
        a = A[rows].float()
        if per_channel:
            wq = w.to(dt) if zero_points is None else (w.to(dt) - zero_points[e].to(dt)[:, None])
            if exact_scales:
                wq = w.float() if zero_points is None else (w.float() - zero_points[e].float()[:, None])
            acc = a @ wq.float().t()
            acc = acc * scale_b[e].float()[None, :]
        else:
            groups = scale_b.shape[-1]
            g = K // groups
            s = scale_b[e].repeat_interleave(g, dim=1)  # [N, K]
            z = None if zero_points is None else zero_points[e].repeat_interleave(g, dim=1)
            if exact_scales:
                wq = (w.float() if z is None else w.float() - z.float()) * s.float()
            else:
                wq = w.to(s.dtype) if z is None else (w.to(s.dtype) - z)
                wq = (wq * s).float()
            acc = a @ wq.t()
        if mul_routed_weight:
            acc = acc * tw[flat].float()[:, None]
        flat_out[flat] = acc.to(dt)
    return C
