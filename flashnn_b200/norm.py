"""RMSNormDquant and LayernormDquant with the reference's module signatures
(flashnn/norm.py:39-63 and :94-124): a normalisation fused with the per-token
int8 quantisation that feeds GemmA8W8.  One kernel launch reads each row once."""
import numbers

import torch

from . import _lib
from .kernel_backend import BackendKernel
from .quant_gemm import _DT, _on_device, _require_cuda, _stream


def _rows(x):
    assert x.dtype in (torch.float16, torch.bfloat16), "input must be float16 or bfloat16"
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    return x2, k


_affine_cache = {}


def _affine(x, *params):
    """Norm parameters on x's device in a dtype the kernel reads: x's own, or fp32.  Parameters that already are
    (the usual case) are passed as they are; a converted copy is made once per parameter version and kept."""
    dt = x.dtype if params[0].dtype in (torch.float16, torch.bfloat16) else torch.float32
    out = []
    for p in params:
        if p.device == x.device and p.dtype == dt and p.is_contiguous():
            out.append(p.detach())
            continue
        key = (id(p), p._version, p.data_ptr(), x.device, dt)
        t = _affine_cache.get(key)
        if t is None:
            for stale in [k for k in _affine_cache if k[0] == id(p)]:
                del _affine_cache[stale]
            t = p.detach().to(device=x.device, dtype=dt).contiguous()
            _affine_cache[key] = t
        out.append(t)
    return out


class RMSNormDquant(BackendKernel):
    """forward(x [..., dim] fp16/bf16) -> (int8 [..., dim], scale [...] in x's dtype)
    (flashnn/norm.py:39-63)."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = torch.nn.Parameter(torch.ones(dim))

    def _cuda_impl(self, x):
        _require_cuda(x)
        x2, k = _rows(x)
        assert self.weight.numel() == k, "last dimension of x must equal dim"
        (w,) = _affine(x, self.weight)
        q = torch.empty(x2.shape, dtype=torch.int8, device=x.device)
        scale = torch.empty(x2.shape[0], dtype=x.dtype, device=x.device)
        with _on_device(x):
            _lib.check(_lib.lib().fnn_rms_norm_dquant(
                x2.data_ptr(), _DT[x.dtype], x2.shape[0], k, k, w.data_ptr(), _DT[w.dtype], float(self.eps),
                q.data_ptr(), k, scale.data_ptr(), _stream(x)))
        return q.reshape(x.shape), scale.reshape(x.shape[:-1])

    def forward(self, x):
        return BackendKernel.forward(self, x)


class LayernormDquant(BackendKernel):
    """forward(x [..., dim] fp16/bf16) -> (int8 [..., dim], scale [rows, 1] in x's dtype)
    (flashnn/norm.py:94-124).  `dim` may be an int or a one-element shape."""

    def __init__(self, dim, eps: float = 1e-5):
        super().__init__()
        self.dim = (dim,) if isinstance(dim, numbers.Integral) else tuple(dim)
        self.eps = eps
        self.weight = torch.nn.Parameter(torch.ones(self.dim))
        self.bias = torch.nn.Parameter(torch.zeros(self.dim))

    def _cuda_impl(self, x):
        _require_cuda(x)
        if len(self.dim) != 1:
            raise NotImplementedError("LayernormDquant normalises over the last dimension only")
        x2, k = _rows(x)
        assert self.dim[0] == k, "last dimension of x must equal dim"
        w, b = _affine(x, self.weight, self.bias)
        q = torch.empty(x2.shape, dtype=torch.int8, device=x.device)
        scale = torch.empty(x2.shape[0], dtype=x.dtype, device=x.device)
        with _on_device(x):
            _lib.check(_lib.lib().fnn_layer_norm_dquant(
                x2.data_ptr(), _DT[x.dtype], x2.shape[0], k, k, w.data_ptr(), b.data_ptr(), _DT[w.dtype],
                float(self.eps), q.data_ptr(), k, scale.data_ptr(), _stream(x)))
        return q.reshape(x.shape), scale.reshape(-1, 1)

    def forward(self, x):
        return BackendKernel.forward(self, x)
