"""RMSNormDquant / LayernormDquant on the GPU (through the C ABI) against the CPU oracle and the golden
vectors produced by the reference.

The kernels add up a row's fp32 statistics in a different order than torch does, so bit equality is not
defined for this pair of operators: a statistic can differ in its last bit, which moves the 16-bit scale by
at most one unit in the last place and a quantised value that sat on a rounding boundary by one step.  The
bars below are tighter than the reference's own (tests/norm/test_rms_norm_dquant.py: |dq| <= 1, scale within
1e-3; tests/norm/test_layer_norm_dquant.py: |dq| <= 2, scale within 1e-2)."""
import pytest
import torch

from oracle import quant_oracle as O
from tests import golden_io as G

pytestmark = pytest.mark.gpu
ND = G.load("norm_dquant.npz")


def ulp_distance(a, b):
    """Distance in units of the last place between two same-dtype 16-bit float tensors of one sign."""
    return (a.contiguous().view(torch.int16).int() - b.contiguous().view(torch.int16).int()).abs()


def check(q, s, qo, so, max_dq, min_exact):
    assert q.dtype == torch.int8 and s.dtype == so.dtype and q.shape == qo.shape and s.shape == so.shape
    assert int(ulp_distance(s, so).max()) <= 1
    dq = (q.int() - qo.int()).abs()
    assert int(dq.max()) <= max_dq
    # rows whose scale came out identical must agree almost everywhere
    same = (ulp_distance(s, so).reshape(-1) == 0)
    rows = dq.reshape(-1, dq.shape[-1])[same]
    if rows.numel():
        assert float((rows == 0).float().mean()) >= min_exact


def run_rms(x, w, eps):
    import flashnn_b200
    op = flashnn_b200.RMSNormDquant(x.shape[-1], eps).to(w.dtype)
    with torch.no_grad():
        op.weight.copy_(w)
    q, s = op.cuda()(x.cuda())
    torch.cuda.synchronize()
    return q.cpu(), s.cpu()


def run_ln(x, w, b, eps):
    import flashnn_b200
    op = flashnn_b200.LayernormDquant(x.shape[-1], eps).to(w.dtype)
    with torch.no_grad():
        op.weight.copy_(w)
        op.bias.copy_(b)
    q, s = op.cuda()(x.cuda())
    torch.cuda.synchronize()
    return q.cpu(), s.cpu()


@pytest.mark.parametrize("name", sorted(ND))
def test_golden(name):
    c = ND[name]
    dt = G.dtype_of(c["dtype"])
    x, w = G.tensor(c["x"], dt), G.tensor(c["weight"], dt)
    qg, sg = torch.from_numpy(c["q"].copy()), G.tensor(c["scale"], dt)
    if str(c["kind"]) == "rms":
        q, s = run_rms(x, w, float(c["eps"]))
        check(q, s, qg, sg, 1, 0.999)
    else:
        q, s = run_ln(x, w, G.tensor(c["bias"], dt), float(c["eps"]))
        check(q, s, qg, sg, 2, 0.97)


# the reference tests' shapes, the hidden sizes of its benchmark models and the A8W8 bench shapes
SHAPES = [(4, 128), (3, 32, 1024), (7, 8), (5, 1664), (3, 3328), (2, 8896), (2, 13312), (64, 8192), (3, 28672), (2, 32768)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_rms_matches_oracle(shape, dt):
    g = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(*shape, generator=g).to(dt)
    w = (torch.rand(shape[-1], generator=g) + 0.5).to(dt)
    q, s = run_rms(x, w, 1e-5)
    qo, so = O.rms_norm_dquant(x, w, 1e-5)
    check(q, s, qo, so, 1, 0.999)
    # the reference's own criterion
    torch.testing.assert_close(q.float(), qo.float(), rtol=1e-2, atol=1)
    torch.testing.assert_close(s.float(), so.float(), rtol=1e-2 if dt == torch.bfloat16 else 1e-3, atol=1e-3)


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_layer_norm_matches_oracle(shape, dt):
    g = torch.Generator().manual_seed(sum(shape) + 1)
    x = (torch.randn(*shape, generator=g) * 2 + 0.5).to(dt)
    w = (torch.rand(shape[-1], generator=g) + 0.5).to(dt)
    b = (torch.randn(shape[-1], generator=g) * 0.1).to(dt)
    q, s = run_ln(x, w, b, 1e-5)
    qo, so = O.layer_norm_dquant(x, w, b, 1e-5)
    check(q, s, qo, so, 2, 0.97)
    torch.testing.assert_close(q.float(), qo.float(), rtol=0.01, atol=2.0)
    torch.testing.assert_close(s.float(), so.float(), rtol=0.01, atol=0.01)


def test_fp32_parameters_and_feeding_a8w8():
    """Default-constructed modules hold fp32 parameters; the int8 rows and scales go straight into GemmA8W8."""
    import flashnn_b200
    g = torch.Generator().manual_seed(5)
    x = torch.randn(48, 1024, generator=g).half()
    wq = torch.randint(-127, 128, (256, 1024), generator=g, dtype=torch.int8)
    col = (torch.rand(256, generator=g) * 0.01).half()
    op = flashnn_b200.RMSNormDquant(1024, 1e-5).cuda()
    q, s = op(x.cuda())
    qo, so = O.rms_norm_dquant(x, torch.ones(1024), 1e-5)
    check(q.cpu(), s.cpu(), qo, so, 1, 0.999)
    out = flashnn_b200.GemmA8W8(torch.float16)(q, wq.cuda(), s, col.cuda())
    ref = O.gemm_a8w8(q.cpu(), wq, s.cpu(), col, torch.float16)
    assert torch.equal(out.cpu().view(torch.int16), ref.view(torch.int16))


def test_rejects_bad_arguments():
    import flashnn_b200
    from flashnn_b200 import _lib
    x = torch.randn(4, 100, device="cuda").half()  # row length not a multiple of 8
    with pytest.raises(_lib.FlashNNError):
        flashnn_b200.RMSNormDquant(100).cuda()(x)
    with pytest.raises(RuntimeError):
        flashnn_b200.LayernormDquant(128)(torch.randn(4, 128).half())  # CPU tensor: no CPU path


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("kind", ["rms", "ln"])
def test_rows_with_a_nan_or_an_infinity(kind, dt):
    """A row that holds a NaN or an infinity comes out with a NaN scale and q = 0 (every quotient is NaN), as the
    reference's torch path gives; it does not turn into plausible finite data.  Other rows are unaffected."""
    g = torch.Generator().manual_seed(11)
    x = torch.randn(4, 1024, generator=g).to(dt)
    w = (torch.rand(1024, generator=g) + 0.5).to(dt)
    b = (torch.randn(1024, generator=g) * 0.1).to(dt)
    clean_q, clean_s = run_rms(x, w, 1e-5) if kind == "rms" else run_ln(x, w, b, 1e-5)
    x[1, 77] = float("nan")
    x[2, 1000] = float("inf")
    q, s = run_rms(x, w, 1e-5) if kind == "rms" else run_ln(x, w, b, 1e-5)
    qo, so = O.rms_norm_dquant(x, w, 1e-5) if kind == "rms" else O.layer_norm_dquant(x, w, b, 1e-5)
    s, so, clean_s = s.reshape(-1), so.reshape(-1), clean_s.reshape(-1)
    assert bool(torch.isnan(s[1])) and bool(torch.isnan(s[2]))
    assert bool(torch.isnan(so[1])) and bool(torch.isnan(so[2]))
    assert (q[1:3] == 0).all() and (qo[1:3] == 0).all()
    assert torch.equal(q[[0, 3]], clean_q[[0, 3]]) and torch.equal(s[[0, 3]].view(torch.int16), clean_s[[0, 3]].view(torch.int16))
