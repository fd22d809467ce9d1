"""DynamicQuantize, GemmA8W8 and GemmWeightOnly with the reference's module
signatures (flashnn/quant_gemm.py:39-209), computing on the sm_100a kernels
behind the C ABI.  Tensors are validated the way the reference's launchers
validate them; outputs are allocated here and the kernels run on the current
CUDA stream."""
import collections
import warnings

import torch

from . import _lib
from .kernel_backend import BackendKernel

_DT = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.float32: _lib.F32}

# scratch per (device, stream): weight-only zero-point path.  Work on one stream is ordered, so one buffer per stream
# is enough; the least recently used entries are dropped beyond a handful of streams.
_workspaces = collections.OrderedDict()
_MAX_WORKSPACES = 8


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
        while len(_workspaces) > _MAX_WORKSPACES:
            _workspaces.popitem(last=False)
    else:
        _workspaces.move_to_end(key)
    return buf


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


class _on_device:
    """`with _on_device(t):` makes t's device current for the C call; free when it already is (the usual case)."""

    def __init__(self, t):
        self.index = t.device.index
        self.ctx = None

    def __enter__(self):
        if torch.cuda.current_device() != self.index:
            self.ctx = torch.cuda.device(self.index)
            self.ctx.__enter__()

    def __exit__(self, *exc):
        if self.ctx is not None:
            self.ctx.__exit__(*exc)


_warned_strided_b = False


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("flashnn_b200 operators need CUDA tensors; there is no CPU path")


class DynamicQuantize(BackendKernel):
    """Per-token dynamic int8 quantisation.

    forward(input [M, K] fp16/bf16) -> (int8 [M, K], fp16 scale [M])
    (flashnn/quant_gemm.py:39-66)."""

    def __init__(self):
        super().__init__()

    def _cuda_impl(self, input):
        _require_cuda(input)
        assert input.dim() == 2, "input must be 2-D"
        assert input.is_contiguous(), "input must be contiguous"
        assert input.dtype in (torch.float16, torch.bfloat16), "input must be float16 or bfloat16"
        out = torch.empty(input.shape, dtype=torch.int8, device=input.device)
        scale = torch.empty(input.shape[0], dtype=torch.half, device=input.device)
        m, k = input.shape
        with _on_device(input):
            _lib.check(_lib.lib().fnn_dynamic_quant(
                input.data_ptr(), _DT[input.dtype], m, k, input.stride(0) if m > 0 else k,
                out.data_ptr(), k, scale.data_ptr(), _stream(input)))
        return out, scale

    def forward(self, input):
        return BackendKernel.forward(self, input)


class GemmA8W8(BackendKernel):
    """out[m, n] = (A[m, :] . B[n, :]) * (alpha_row[m] * alpha_col[n]) in `out_ty`.

    forward(a int8 [M, K], b int8 [N, K], alpha_row [M] or [M, 1], alpha_col [N] or [1, N])
    (flashnn/quant_gemm.py:69-107).  Scales may be fp16, bf16 or fp32."""

    def __init__(self, out_ty: torch.dtype = torch.float16):
        super().__init__()
        self.out_ty = out_ty

    def _cuda_impl(self, a, b, alpha_row, alpha_col, acc_out=None):
        _require_cuda(a, b, alpha_row, alpha_col)
        assert a.dtype == torch.int8 and b.dtype == torch.int8, "Matrix A/B must be int8 type"
        assert a.is_contiguous(), "Matrix A must be contiguous"
        assert self.out_ty in (torch.float16, torch.bfloat16), "Output type must be float16 or bfloat16"
        assert a.shape[1] == b.shape[1], "Matrix B must be transposed"
        if b.dim() == 2 and b.stride(1) != 1:
            # the kernels read K contiguously; any row pitch is taken as it is, but a B stored K-strided (for
            # instance a transposed view) has to be copied, N * K bytes on every call: say so once
            global _warned_strided_b
            if not _warned_strided_b:
                warnings.warn("GemmA8W8: matrix B has a non-unit stride along K and is copied on every call; "
                              "store it as [N, K] with K contiguous to avoid the copy")
                _warned_strided_b = True
            b = b.contiguous()
        m, k = a.shape
        n = b.shape[0]
        row = torch.squeeze(alpha_row).reshape(-1).contiguous()
        col = torch.squeeze(alpha_col).reshape(-1).contiguous()
        assert row.numel() == m and col.numel() == n, "scale shapes must be [M] and [N]"
        assert row.dtype in _DT and col.dtype in _DT, "scales must be float16, bfloat16 or float32"
        out = torch.empty([m, n], dtype=self.out_ty, device=a.device)
        L = _lib.lib()
        with _on_device(a):
            ws_bytes = L.fnn_gemm_a8w8_workspace_bytes(m, n, k)
            ws = _workspace(a.device, ws_bytes) if ws_bytes else None
            _lib.check(L.fnn_gemm_a8w8(
                a.data_ptr(), a.stride(0) if m > 1 else k, b.data_ptr(), b.stride(0) if n > 1 else k,
                row.data_ptr(), _DT[row.dtype], col.data_ptr(), _DT[col.dtype],
                out.data_ptr(), _DT[self.out_ty], n, m, n, k,
                acc_out.data_ptr() if acc_out is not None else None, n,
                ws.data_ptr() if ws is not None else None, ws_bytes, _stream(a)))
        return out

    def forward(self, a, b, alpha_row, alpha_col):
        return BackendKernel.forward(self, a, b, alpha_row, alpha_col)


class GemmWeightOnly(BackendKernel):
    """out = act . dequant(quant_w)^T (+ bias) with int8 or packed-int4 weights.

    forward(act [M, K] fp16/bf16, quant_w int8 [N, K] or packed [N/2, K],
            scale_w [N] or [K/group, N], bias=None, zero_points=None)
    (flashnn/quant_gemm.py:110-209).  Whether the weight is int8 or int4 is
    inferred from the shapes exactly as the reference does."""

    def __init__(self, out_ty: torch.dtype = torch.float16):
        super().__init__()
        self.out_ty = out_ty

    # Weight-side arguments that passed validation and are used exactly as they were handed in (no converted copy):
    # (pointers, shapes, dtypes) -> (bits, n, group).  Decode loops call with the same weights every step; the shape
    # checks then cost one dictionary look-up.  Nothing that depends on tensor contents is kept.
    _validated = collections.OrderedDict()

    def _weight_side(self, k, quant_w, scale_w, bias, zero_points):
        key = (quant_w.data_ptr(), tuple(quant_w.shape), quant_w.dtype, scale_w.data_ptr(), tuple(scale_w.shape), scale_w.dtype,
               None if bias is None else (bias.data_ptr(), tuple(bias.shape), bias.dtype),
               None if zero_points is None else (zero_points.data_ptr(), tuple(zero_points.shape), zero_points.dtype), k)
        hit = self._validated.get(key)
        if hit is not None:
            return hit + (scale_w, zero_points, bias)
        assert quant_w.dtype in (torch.int8, torch.uint8), "Weight must be int8 type"
        assert quant_w.is_contiguous(), "Weight must be contiguous"
        assert k == quant_w.shape[1], "Matrix B must be transposed"
        if quant_w.size(0) * 2 == scale_w.size(-1):
            bits = 4
        elif quant_w.size(0) == scale_w.size(-1):
            bits = 8
        else:
            raise AssertionError("Gemm WeightOnly only support int8 or int4x2")
        n = quant_w.shape[0] * (2 if bits == 4 else 1)
        scale = scale_w.squeeze()
        if scale.dim() == 0:
            scale = scale.reshape(1)
        if scale.dim() == 1:
            group = 0
        else:
            assert scale.dim() == 2 and k % scale.shape[0] == 0, "group scales must be [K/group, N]"
            group = k // scale.shape[0]
        direct = scale.is_contiguous()
        scale = scale.contiguous()
        assert scale.dtype in _DT, "scales must be float16, bfloat16 or float32"
        zp = None
        if zero_points is not None:
            zp = zero_points.squeeze()
            if zp.dim() == 0:
                zp = zp.reshape(1)
            assert zp.shape == scale.shape, "zero_points must have the shape of scale_w"
            direct = direct and zp.dtype == scale.dtype and zp.is_contiguous()
            zp = zp.to(scale.dtype).contiguous()  # the kernels read scales and zero-points in one dtype
        if bias is not None:
            direct = direct and bias.is_contiguous()
            bias = bias.reshape(-1).contiguous()
            assert bias.numel() == n and bias.dtype in _DT, "bias must be [N] in a float dtype"
        if direct:
            self._validated[key] = (bits, n, group)
            while len(self._validated) > 256:
                self._validated.popitem(last=False)
        return bits, n, group, scale, zp, bias

    def _cuda_impl(self, act, quant_w, scale_w, bias=None, zero_points=None):
        _require_cuda(act, quant_w, scale_w, bias, zero_points)
        assert act.is_contiguous(), "Activation must be contiguous"
        assert act.dtype in (torch.float16, torch.bfloat16), "Activation must be float16 or bfloat16"
        assert self.out_ty == act.dtype, "Output type must match the activation type"
        m, k = act.shape
        assert k == quant_w.shape[1], "Matrix B must be transposed"
        bits, n, group, scale, zp, bias = self._weight_side(k, quant_w, scale_w, bias, zero_points)
        out = torch.empty([m, n], dtype=self.out_ty, device=act.device)
        L = _lib.lib()
        with _on_device(act):
            ws_bytes = L.fnn_gemm_weight_only_workspace_bytes(m, n, k, bits, group) if (m > 16 and zp is not None) else 0
            ws = _workspace(act.device, ws_bytes) if ws_bytes else None
            _lib.check(L.fnn_gemm_weight_only(
                act.data_ptr(), _DT[act.dtype], k, quant_w.data_ptr(), bits,
                scale.data_ptr(), zp.data_ptr() if zp is not None else None, _DT[scale.dtype], group,
                bias.data_ptr() if bias is not None else None, _DT[bias.dtype] if bias is not None else 0,
                out.data_ptr(), _DT[self.out_ty], n, m, n, k,
                ws.data_ptr() if ws is not None else None, ws_bytes, _stream(act)))
        return out

    def forward(self, act, quant_w, scale_w, bias=None, zero_points=None):
        return BackendKernel.forward(self, act, quant_w, scale_w, bias, zero_points)
