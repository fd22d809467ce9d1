"""GemmA8W8 on the GPU (through the C ABI): exact int32 accumulators and scaled
outputs against the CPU oracle and the golden vectors produced by the reference."""
import numpy as np
import pytest
import torch

from oracle import quant_oracle as O
from tests import golden_io as G

pytestmark = pytest.mark.gpu
A8 = G.load("gemm_a8w8.npz")


def run(a, b, row, col, out_ty, want_acc=True):
    import flashnn_b200
    op = flashnn_b200.GemmA8W8(out_ty)
    acc = torch.empty(a.shape[0], b.shape[0], dtype=torch.int32, device="cuda") if want_acc else None
    out = op._cuda_impl(a.cuda(), b.cuda(), row.cuda(), col.cuda(), acc_out=acc)
    torch.cuda.synchronize()
    from flashnn_b200 import _lib
    assert _lib.device_status() == 0
    return out.cpu(), (acc.cpu() if want_acc else None)


def bits16(t):
    return t.contiguous().view(torch.int16)


@pytest.mark.parametrize("name", sorted(A8))
def test_golden_bit_exact(name):
    c = A8[name]
    st, ot = G.dtype_of(c["scale_ty"]), G.dtype_of(c["out_ty"])
    a, b = G.tensor(c["a"]), G.tensor(c["b"])
    row, col = G.tensor(c["row"], st), G.tensor(c["col"], st)
    out, acc = run(a, b, row, col, ot)
    assert torch.equal(acc, O.gemm_a8w8_acc_i32(a, b))
    np.testing.assert_array_equal(bits16(out).numpy().view(np.uint16), c["out"])


def make(m, n, k, seed, scale_ty=torch.float32, lo=-127):
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(lo, 128, (m, k), generator=g, dtype=torch.int8)
    b = torch.randint(lo, 128, (n, k), generator=g, dtype=torch.int8)
    row = (torch.rand(m, generator=g) * 0.015 + 0.005).to(scale_ty)
    col = (torch.rand(n, generator=g) * 0.009 + 0.001).to(scale_ty)
    return a, b, row, col


# ragged M / N / K (tile multiples are 128 or 256 / 64..256 / 128; the last three shapes are large enough for
# the CTA-pair kernel), tiny sizes, K with a 16-byte but not
# 128-byte pitch (TMA zero fill), K not a multiple of 16 (generic kernel), -128 operands
@pytest.mark.parametrize("m,n,k", [(1, 64, 128), (3, 200, 336), (17, 520, 1040), (129, 130, 144),
                                   (128, 128, 128), (256, 512, 4096), (300, 1000, 8896), (16, 4096, 4096),
                                   (5, 48, 100), (33, 17, 7), (64, 8192, 1024), (1000, 264, 7392),
                                   (2500, 2100, 1040), (2049, 2560, 144), (1290, 4200, 2064)])
@pytest.mark.parametrize("out_ty", [torch.float16, torch.bfloat16])
def test_shapes_exact(m, n, k, out_ty):
    a, b, row, col = make(m, n, k, seed=m + n + k, lo=-128)
    out, acc = run(a, b, row, col, out_ty)
    ref_acc = O.gemm_a8w8_acc_i32(a, b)
    assert torch.equal(acc, ref_acc)
    assert torch.equal(bits16(out), bits16(O.gemm_a8w8_from_acc(ref_acc, row, col, out_ty)))


@pytest.mark.parametrize("scale_ty", [torch.float16, torch.bfloat16])
def test_sixteen_bit_scales_follow_the_reference_rounding(scale_ty):
    a, b, row, col = make(70, 300, 512, seed=11, scale_ty=scale_ty)
    out, _ = run(a, b, row, col, scale_ty)
    assert torch.equal(bits16(out), bits16(O.gemm_a8w8(a, b, row, col, scale_ty)))
    # mixed dtypes (fp16 per-token scale from DynamicQuantize, fp32 per-channel scale)
    out, _ = run(a, b, row, col.float(), torch.bfloat16)
    assert torch.equal(bits16(out), bits16(O.gemm_a8w8(a, b, row.float(), col.float(), torch.bfloat16)))


def test_first_config_matches_reference_torch_path():
    from flashnn_b200 import workloads as W
    w = W.a8w8_small()
    out, acc = run(w["a"], w["b"], w["alpha_row"], w["alpha_col"], w["out_ty"])
    assert torch.equal(acc, O.gemm_a8w8_acc_i32(w["a"], w["b"]))
    ref = O.gemm_a8w8(w["a"], w["b"], w["alpha_row"], w["alpha_col"], w["out_ty"])
    assert torch.equal(bits16(out), bits16(ref))
    torch.testing.assert_close(out.float(), ref.float(), rtol=1e-2, atol=1e-3)


def test_non_contiguous_weight_view():
    a, b, row, col = make(40, 96, 256, seed=5)
    wide = torch.zeros(96, 512, dtype=torch.int8)
    wide[:, :256] = b
    import flashnn_b200
    out = flashnn_b200.GemmA8W8(torch.float16)(a.cuda(), wide.cuda()[:, :256], row.cuda(), col.cuda())
    assert torch.equal(bits16(out.cpu()), bits16(O.gemm_a8w8(a, b, row, col, torch.float16)))
    bt = b.t().contiguous()  # [K, N]; .t() gives an [N, K] view with unit stride along N
    out = flashnn_b200.GemmA8W8(torch.float16)(a.cuda(), bt.cuda().t(), row.cuda(), col.cuda())
    assert torch.equal(bits16(out.cpu()), bits16(O.gemm_a8w8(a, b, row, col, torch.float16)))


def check_sampled_rows(a, b, row, col, out, acc, out_ty, rows):
    idx = torch.tensor(rows)
    ref_acc = O.gemm_a8w8_acc_i32(a[idx], b)
    assert torch.equal(acc[idx], ref_acc)
    assert torch.equal(bits16(out[idx]), bits16(O.gemm_a8w8_from_acc(ref_acc, row[idx], col, out_ty)))


def test_prefill_chain_full_size():
    """DynamicQuant -> A8W8 at M=4096, N=11008, K=4096: the chain's int8 activations and scales are
    exact, the accumulator and output are exact on sampled rows, and a checksum ties the rest."""
    import flashnn_b200
    from flashnn_b200 import workloads as W
    w = W.dq_a8w8_prefill()
    x, wt, col = w["x"], w["w"], w["alpha_col"]
    q, s = flashnn_b200.DynamicQuantize()(x.cuda())
    qo, so = O.dynamic_quantize(x, saturate=True)
    assert torch.equal(q.cpu(), qo) and torch.equal(s.cpu(), so)
    out, acc = run(qo, wt, so, col, torch.bfloat16)
    rows = list(range(0, 4096, 257)) + [127, 128, 4095]
    check_sampled_rows(qo, wt, so.float(), col, out, acc, torch.bfloat16, rows)
    # column sums of the accumulator equal (sum of rows of A) . W^T  -- exact in fp64
    colsum = qo.double().sum(0) @ wt.double().t()
    assert torch.equal(acc.double().sum(0), colsum)


def test_headline_shape_8192_cubed():
    a, b, row, col = make(8192, 8192, 8192, seed=1)
    out, acc = run(a, b, row, col, torch.bfloat16)
    check_sampled_rows(a, b, row, col, out, acc, torch.bfloat16, list(range(5, 8192, 683)) + [0, 8191])
    colsum = a.double().sum(0) @ b.double().t()
    assert torch.equal(acc.double().sum(0), colsum)


def test_large_k_beyond_fp32_exactness():
    # worst-case operands: |acc| = K * 127 * 127 > 2**24, where an fp32 product is no longer exact
    m, n, k = 8, 64, 28672
    a = torch.full((m, k), 127, dtype=torch.int8)
    b = torch.full((n, k), -127, dtype=torch.int8)
    b[::2] = 127
    row = torch.full((m,), 0.01)
    col = torch.full((n,), 0.002)
    out, acc = run(a, b, row, col, torch.bfloat16)
    ref_acc = O.gemm_a8w8_acc_i32(a, b)
    assert int(ref_acc.abs().max()) > 2 ** 24
    assert torch.equal(acc, ref_acc)
    assert torch.equal(bits16(out), bits16(O.gemm_a8w8_from_acc(ref_acc, row, col, torch.bfloat16)))


# Up to 8 tokens against a wide weight matrix run on the per-lane streaming kernel (int8 activations as MMA columns,
# exact int32 sums through the reducer): accumulator and scaled output bit for bit, all scale dtype combinations,
# -128 operands, the long K of the down projection.
@pytest.mark.parametrize("m,n,k", [(1, 8192, 4096), (3, 8192, 8192), (8, 16384, 4096), (5, 8192, 28672), (2, 8208, 8192)])
@pytest.mark.parametrize("out_ty", [torch.float16, torch.bfloat16])
def test_decode_streaming_kernel_exact(m, n, k, out_ty):
    a, b, row, col = make(m, n, k, seed=m + n + k, lo=-128)
    out, acc = run(a, b, row, col, out_ty)
    ref_acc = O.gemm_a8w8_acc_i32(a, b)
    assert torch.equal(acc, ref_acc)
    assert torch.equal(bits16(out), bits16(O.gemm_a8w8_from_acc(ref_acc, row, col, out_ty)))
    # same 16-bit dtype on both scales: their product is rounded to that dtype first
    a, b, row, col = make(m, n, k, seed=m + k, scale_ty=out_ty)
    out, _ = run(a, b, row, col, out_ty, want_acc=False)
    assert torch.equal(bits16(out), bits16(O.gemm_a8w8(a, b, row, col, out_ty)))
    # worst-case operands: |acc| = k * 128 * 128 exceeds 2^24 for every k here
    a2 = torch.full((m, k), -128, dtype=torch.int8)
    b2 = torch.full((n, k), -128, dtype=torch.int8)
    b2[1::2] = 127
    out, acc = run(a2, b2, row.float(), col.float(), out_ty)
    assert torch.equal(acc, O.gemm_a8w8_acc_i32(a2, b2))


# ---- the CTA-pair kernel with its K blocks dealt out evenly (partial sums handed from pair to pair) ----
@pytest.fixture
def balanced_mode():
    from flashnn_b200 import _lib
    _lib.set_option(_lib.OPT_A8W8_BALANCED, 1)
    yield
    _lib.set_option(_lib.OPT_A8W8_BALANCED, 0)


# fewer tiles than pairs (every tile split over several pairs), a few more tiles than pairs, ragged M / N / K, short K
# (units per pair below and above the K blocks of a tile), the narrow-shard shape of the down projection
@pytest.mark.parametrize("m,n,k", [(256, 512, 4096), (300, 1000, 8896), (1000, 264, 7392), (2500, 2100, 1040),
                                   (2049, 2560, 400), (4096, 1024, 7168), (1290, 4200, 2064), (129, 64, 256)])
@pytest.mark.parametrize("out_ty", [torch.float16, torch.bfloat16])
def test_balanced_mode_exact(balanced_mode, m, n, k, out_ty):
    from flashnn_b200 import _lib
    assert _lib.a8w8_plan(m, n, k)[0] == 3
    a, b, row, col = make(m, n, k, seed=m + n + k + 1, lo=-128)
    ref_acc = O.gemm_a8w8_acc_i32(a, b)
    want = bits16(O.gemm_a8w8_from_acc(ref_acc, row, col, out_ty))
    for _ in range(3):  # the hand-over flags are reused call after call
        out, acc = run(a, b, row, col, out_ty)
        assert torch.equal(acc, ref_acc)
        assert torch.equal(bits16(out), want)


def test_balanced_mode_replayed_from_a_cuda_graph(balanced_mode):
    import flashnn_b200
    m, n, k = 1024, 1024, 4096
    a, b, row, col = make(m, n, k, seed=5)
    want = bits16(O.gemm_a8w8(a, b, row, col, torch.bfloat16))
    op = flashnn_b200.GemmA8W8(torch.bfloat16)
    a, b, row, col = a.cuda(), b.cuda(), row.cuda(), col.cuda()
    op(a, b, row, col)  # first call outside the capture (workspace allocation)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        op(a, b, row, col)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            out = op(a, b, row, col)
    for _ in range(3):
        out.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(bits16(out.cpu()), want)
    from flashnn_b200 import _lib
    assert _lib.device_status() == 0


def test_balanced_mode_is_picked_for_narrow_shards_and_matches():
    """Down projection of the 70B FFN on 1/4 of the columns: 128 tiles for 74 CTA pairs."""
    from flashnn_b200 import _lib
    m, n, k = 4096, 2048, 28672
    assert _lib.a8w8_plan(m, n, k)[0] == 3
    assert _lib.a8w8_plan(m, 8192, 8192)[0] == 1  # full waves: whole tiles
    a, b, row, col = make(m, n, k, seed=9)
    out, acc = run(a, b, row, col, torch.bfloat16)
    rows = [0, 1, 127, 128, 255, 256, 1000, 2047, 2048, 4095]
    ref_acc = O.gemm_a8w8_acc_i32(a[rows], b)
    assert torch.equal(acc[rows], ref_acc)
    assert torch.equal(bits16(out[rows]), bits16(O.gemm_a8w8_from_acc(ref_acc, row[rows], col, torch.bfloat16)))
    # the whole accumulator against the same kernel without the hand-over
    _lib.set_option(_lib.OPT_A8W8_BALANCED, 2)
    try:
        out2, acc2 = run(a, b, row, col, torch.bfloat16)
    finally:
        _lib.set_option(_lib.OPT_A8W8_BALANCED, 0)
    assert torch.equal(acc, acc2) and torch.equal(bits16(out), bits16(out2))
