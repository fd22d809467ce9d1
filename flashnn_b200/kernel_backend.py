"""Backend switches with the reference's names (flashnn/kernel_backend.py:10-69).

This build has exactly one backend for the quantized-GEMM operators: the
sm_100a kernels behind the C ABI.  `set_use_triton` and
`set_autotune_triton_kernels` are kept so that code written against the
reference keeps importing and running, but they cannot select another
implementation: asking for the torch backend makes the operators raise instead
of computing on a fallback path.
"""
import torch

_use_native = True
_autotune = False


def get_autotune_triton_kernels():
    return _autotune


def set_autotune_triton_kernels(v: bool):
    """Accepted for compatibility; the kernels pick their tiles from the problem shape."""
    global _autotune
    _autotune = bool(v)


def get_use_triton():
    return _use_native


def set_use_triton(v: bool):
    """True (default): operators run the CUDA kernels.  False: operators raise, because
    this package ships no torch implementation to fall back to."""
    global _use_native
    _use_native = bool(v)


class BackendKernel(torch.nn.Module):
    """Base class of the operators: `forward` dispatches to `_cuda_impl`
    (the role `_triton_impl` has at flashnn/kernel_backend.py:62-69)."""

    def _cuda_impl(self, *args, **kwargs):
        raise NotImplementedError

    def forward(self, *args, **kwargs):
        if not _use_native:
            raise ValueError("No valid backend found: set_use_triton(False) selects the torch backend, "
                             "which this build does not contain")
        return self._cuda_impl(*args, **kwargs)
