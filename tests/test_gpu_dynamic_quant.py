"""DynamicQuantize on the GPU (through the C ABI) against the CPU oracle and the
golden vectors produced by the reference."""
import numpy as np
import pytest
import torch

from oracle import quant_oracle as O
from tests import golden_io as G

pytestmark = pytest.mark.gpu
DQ = G.load("dynamic_quant.npz")


def run(x_cpu):
    import flashnn_b200
    q, s = flashnn_b200.DynamicQuantize()(x_cpu.cuda())
    torch.cuda.synchronize()
    return q.cpu(), s.cpu()


@pytest.mark.parametrize("name", sorted(DQ))
def test_golden_bit_exact(name):
    c = DQ[name]
    x = G.tensor(c["x"], G.dtype_of(c["dtype"]))
    q, s = run(x)
    assert s.dtype == torch.float16 and q.dtype == torch.int8 and s.shape == (x.shape[0],)
    np.testing.assert_array_equal(s.view(torch.int16).numpy().view(np.uint16), c["scale"])
    wrap = c["precast"] == 128  # the reference's unclamped cast wraps these to -128
    np.testing.assert_array_equal(q.numpy()[~wrap], c["q"][~wrap])
    assert (q.numpy()[wrap] == 127).all()


# the shapes of the reference's own test (tests/quant_gemm/test_dynamic_quant.py:29-35) and the
# hidden sizes of its benchmark (benchmark/benchmark_dynamic_quant.py:11)
@pytest.mark.parametrize("m,k", [(32, 32), (64, 64), (128, 128), (117, 987), (2560, 8000),
                                 (7, 1664), (3, 3328), (5, 8896), (2, 13312), (3, 17792), (2, 35584),
                                 (1, 8), (1, 8192), (64, 28672)])
@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_matches_oracle(m, k, dt):
    g = torch.Generator().manual_seed(m * 131 + k)
    x = (torch.rand(m, k, generator=g) * 2 - 1).to(dt)
    q, s = run(x)
    qo, so = O.dynamic_quantize(x, saturate=True)
    assert torch.equal(s.view(torch.int16), so.view(torch.int16))
    assert torch.equal(q, qo)
    # the reference's own pass criterion against its unclamped torch path
    qr, sr = O.dynamic_quantize(x, saturate=False)
    assert int((~torch.isclose(q.int(), qr.int(), atol=1)).sum()) < 10 or dt == torch.bfloat16
    assert int((~torch.isclose(s, sr, rtol=1e-2)).sum()) < 10


def test_prefill_shape_with_outliers():
    from flashnn_b200 import workloads as W
    x = W.dq_a8w8_prefill()["x"]
    q, s = run(x)
    qo, so = O.dynamic_quantize(x, saturate=True)
    assert torch.equal(s.view(torch.int16), so.view(torch.int16))
    assert torch.equal(q, qo)
    # dequantised rows stay within one quantisation step of the input (size-independent property)
    err = (q.float() * s.float()[:, None] - x.float()).abs()
    assert bool((err <= s.float()[:, None] * 1.01 + 1e-6).all())


def test_zero_rows_and_strided_rows():
    import flashnn_b200
    from flashnn_b200 import _lib
    x = torch.zeros(4, 256, dtype=torch.float16)
    x[1] = torch.linspace(-3, 3, 256).half()
    q, s = run(x)
    assert (q[0] == 0).all() and float(s[0]) == 0.0 and (q[2:] == 0).all()
    qo, so = O.dynamic_quantize(x[1:2], saturate=True)
    assert torch.equal(q[1:2], qo) and torch.equal(s[1:2], so)
    # leading dimension larger than K, called through the C ABI directly
    big = torch.randn(16, 512, dtype=torch.bfloat16).cuda()
    view = big[:, :264]
    qd = torch.empty(16, 264, dtype=torch.int8, device="cuda")
    sd = torch.empty(16, dtype=torch.float16, device="cuda")
    _lib.check(_lib.lib().fnn_dynamic_quant(view.data_ptr(), _lib.BF16, 16, 264, 512, qd.data_ptr(), 264,
                                            sd.data_ptr(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    qo, so = O.dynamic_quantize(view.cpu().contiguous(), saturate=True)
    assert torch.equal(qd.cpu(), qo) and torch.equal(sd.cpu(), so)


def test_rows_with_subnormal_scale():
    """Rows whose scale is subnormal in bf16 (its reciprocal overflows fp32) take the exact division."""
    g = torch.Generator().manual_seed(5)
    x = (torch.rand(6, 512, generator=g) * 2 - 1)
    x[:3] *= 1e-37
    x[3:] *= 3e-39
    x = x.to(torch.bfloat16)
    x[1, :7] = 0
    q, s = run(x)
    qo, so = O.dynamic_quantize(x, saturate=True)
    assert torch.equal(s.view(torch.int16), so.view(torch.int16))
    assert torch.equal(q, qo)


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("k", [264, 8192, 10001])  # vector kernel (short and long rows) and the generic kernel
def test_rows_with_a_nan_or_an_infinity(dt, k):
    """A NaN in a row makes that row's scale NaN, an infinity makes it infinite, exactly as the reference's torch
    path does; the quantised values of such a row are 0 (a NaN quotient cast to int8), the other rows are untouched."""
    g = torch.Generator().manual_seed(k)
    x = torch.randn(5, k, generator=g).to(dt)
    x[1, k // 3] = float("nan")
    x[2, k - 1] = float("inf")
    x[3, 0] = float("-inf")
    x[3, 5] = float("nan")
    q, s = run(x)
    qo, so = O.dynamic_quantize(x, saturate=True)
    assert torch.isnan(s[1]) and torch.isinf(s[2]) and torch.isnan(s[3])
    assert torch.equal(torch.isnan(s), torch.isnan(so)) and torch.equal(torch.isinf(s), torch.isinf(so))
    assert torch.equal(s[[0, 4]].view(torch.int16), so[[0, 4]].view(torch.int16))
    assert torch.equal(q, qo)
    assert (q[1:4] == 0).all()
