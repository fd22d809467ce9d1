"""GemmWeightOnly on the GPU (through the C ABI) against the fp32 dequant-matmul
oracle (bound: |d| <= 1e-3 + 1e-2 |ref|) and the golden vectors of the reference."""
import pytest
import torch

from oracle import quant_oracle as O
from tests import golden_io as G

pytestmark = pytest.mark.gpu
WO = G.load("gemm_weight_only.npz")
RTOL, ATOL = 1e-2, 1e-3  # the bound on weight-only outputs versus fp32 dequant-matmul


def run(act, qw, scale, bias=None, zp=None):
    import flashnn_b200
    from flashnn_b200 import _lib
    dev = lambda t: None if t is None else t.cuda()
    out = flashnn_b200.GemmWeightOnly(act.dtype)(dev(act), dev(qw), dev(scale), dev(bias), dev(zp))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    return out.cpu()


def assert_within_bound(out, act, qw, scale, bias, zp, max_last_bit_mismatch=0.02):
    ref = O.gemm_weight_only_fp32(act, qw, scale, bias, zp)
    # the kernel rounds once to the 16-bit output; allow that rounding on top of the stated bound
    err = (out.float() - ref).abs()
    bound = ATOL + RTOL * ref.abs()
    assert bool((err <= bound).all()), f"max excess {(err - bound).max():.3e}"
    # and it is at least as close as one final rounding of the fp32 result almost everywhere
    exact = ref.to(out.dtype)
    assert float((out != exact).float().mean()) < max_last_bit_mismatch


def assert_rows_within_bound(out, ref, row_factor=None, mask=None):
    """The stated bound |d| <= 1e-3 + 1e-2 |ref| on every element.  A row that a test multiplied by a factor f > 1
    (to reach the top of the dtype's range) is the same problem in units f times larger, so its absolute term is
    f * 1e-3; every other row gets the plain bound."""
    atol = torch.full((out.shape[0], 1), ATOL)
    if row_factor:
        for r, f in row_factor.items():
            if r < out.shape[0]:
                atol[r] = ATOL * max(1.0, f)
    err = (out.float() - ref).abs()
    bound = atol + RTOL * ref.abs()
    ok = err <= bound
    if mask is not None:
        ok = ok | ~mask
    assert bool(ok.all()), f"max excess {(err - bound)[~ok].max():.3e}"


@pytest.mark.parametrize("name", sorted(WO))
def test_golden_cases(name):
    c = WO[name]
    dt = G.dtype_of(c["dtype"])
    act, qw, scale = G.tensor(c["act"], dt), G.tensor(c["qw"]), G.tensor(c["scale"], dt)
    bias = G.tensor(c["bias"], dt) if "bias" in c else None
    zp = G.tensor(c["zp"], dt) if "zp" in c else None
    out = run(act, qw, scale, bias, zp)
    assert_within_bound(out, act, qw, scale, bias, zp)
    # against the reference's own output: it rounds w*s to 16 bits, so only a coarse bound holds
    ref = G.tensor(c["out"], dt).float()
    assert float((out.float() - ref).abs().max()) <= 0.02 * float(ref.abs().max())


def make(kind, m, n, k, dt, group, use_bias, use_zp, seed):
    g = torch.Generator().manual_seed(seed)
    act = torch.randn(m, k, generator=g).to(dt)
    if kind == 8:
        qw = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8)
    else:
        qw = O.pack_int4(torch.randint(-8, 8, (n, k), generator=g, dtype=torch.int8))
    sshape = (n,) if group == 0 else (k // group, n)
    scale = (torch.rand(*sshape, generator=g) * 0.045 + 0.005).to(dt)
    bias = torch.randn(n, generator=g).to(dt) if use_bias else None
    zp = torch.randint(-3, 4, sshape, generator=g).to(dt) if use_zp else None
    return act, qw, scale, bias, zp


# the reference's test shape (3, 1024, 4096) with group 64, all eight option combinations, int8
# (tests/quant_gemm/test_gemm_weight_only.py:160-181), plus the same sweep for packed int4
@pytest.mark.parametrize("kind", [8, 4])
@pytest.mark.parametrize("use_bias", [False, True])
@pytest.mark.parametrize("group", [0, 64])
@pytest.mark.parametrize("use_zp", [False, True])
def test_reference_test_shape(kind, use_bias, group, use_zp):
    act, qw, scale, bias, zp = make(kind, 3, 1024, 4096, torch.float16, group, use_bias, use_zp, seed=kind + group)
    out = run(act, qw, scale, bias, zp)
    assert_within_bound(out, act, qw, scale, bias, zp)


@pytest.mark.parametrize("kind,dt,group", [(4, torch.bfloat16, 128), (4, torch.float16, 128), (8, torch.bfloat16, 0),
                                           (8, torch.float16, 128), (4, torch.bfloat16, 0), (8, torch.bfloat16, 256)])
@pytest.mark.parametrize("m", [1, 2, 8, 9, 16])
def test_decode_shapes(kind, dt, group, m):
    act, qw, scale, bias, zp = make(kind, m, 272, 1024, dt, group, True, m % 2 == 0, seed=m)
    out = run(act, qw, scale, bias, zp)
    assert_within_bound(out, act, qw, scale, bias, zp)


@pytest.mark.parametrize("kind,m,n,k,group", [(4, 17, 64, 256, 32), (8, 40, 50, 200, 0), (4, 3, 30, 96, 32),
                                              (8, 2, 7, 33, 0), (4, 130, 128, 480, 96)])
def test_generic_path_shapes(kind, m, n, k, group):
    act, qw, scale, bias, zp = make(kind, m, n, k, torch.float16, group, True, True, seed=k)
    out = run(act, qw, scale, bias, zp)
    assert_within_bound(out, act, qw, scale, bias, zp)


# prefill shapes with per-channel scales run on the tensor-core kernel: ragged M / N / K (tiles are 256 x 256 x 64),
# int8 and packed int4, both activation dtypes, bias and zero-points
@pytest.mark.parametrize("kind", [8, 4])
@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,n,k,use_bias,use_zp", [(17, 64, 256, False, False), (130, 264, 528, True, True),
                                                   (300, 1000, 2064, True, False), (513, 258, 1024, False, True)])
def test_prefill_per_channel_shapes(kind, dt, m, n, k, use_bias, use_zp):
    act, qw, scale, bias, zp = make(kind, m, n, k, dt, 0, use_bias, use_zp, seed=m + kind)
    out = run(act, qw, scale, bias, zp)
    assert_within_bound(out, act, qw, scale, bias, zp)


def test_a16w8_prefill_config():
    """A16W8 weight-only GEMM at M=2048, N=8192, K=8192 (fp16, per-channel fp16 scales): sampled rows against the
    fp32 dequant-matmul, and a checksum over all rows (column sums are linear in the activations)."""
    from flashnn_b200 import workloads as W
    w = W.a16w8_prefill()
    out = run(w["x"], w["w"], w["scale"])
    rows = torch.tensor(list(range(0, 2048, 97)) + [127, 128, 255, 256, 2047])
    # with K = 8192 the fp32 summation order alone moves a few per cent of the fp16 results by one ulp
    assert_within_bound(out[rows], w["x"][rows], w["w"], w["scale"], None, None, max_last_bit_mismatch=0.08)
    ref_colsum = (w["x"].double().sum(0) @ w["w"].double().t()) * w["scale"].double()
    got = out.double().sum(0)
    # each output carries one fp16 rounding (relative 2^-11 of |out|); the sum of 2048 of them stays far inside this bound
    tol = 2048 ** 0.5 * 2.0 ** -10 * out.double().abs().max()
    assert float((got - ref_colsum).abs().max()) <= float(tol)


@pytest.mark.parametrize("m", [1, 4, 16])
def test_a16w4_decode_config(m):
    """A16W4 decode GEMV at N=28672, K=8192, group 128 (bf16)."""
    from flashnn_b200 import workloads as W
    w = W.a16w4_decode(m)
    out = run(w["x"], w["qw"], w["scale"])
    assert_within_bound(out, w["x"], w["qw"], w["scale"], None, None)


def test_linearity_in_the_activations():
    # size-independent property: f(2x) == 2 f(x) exactly (scaling by a power of two commutes with every rounding)
    from flashnn_b200 import workloads as W
    w = W.a16w4_decode(4, n=4096, k=4096)
    o1 = run(w["x"], w["qw"], w["scale"])
    o2 = run(w["x"] * 2, w["qw"], w["scale"])
    assert torch.equal(o2.float(), o1.float() * 2)


def test_weight_kind_is_inferred_from_shapes():
    import flashnn_b200
    act = torch.randn(2, 128, dtype=torch.float16).cuda()
    qw = torch.zeros(24, 128, dtype=torch.int8).cuda()
    with pytest.raises(AssertionError, match="only support int8 or int4x2"):
        flashnn_b200.GemmWeightOnly()(act, qw, torch.ones(100, dtype=torch.float16).cuda())
    with pytest.raises(AssertionError, match="Matrix B must be transposed"):
        flashnn_b200.GemmWeightOnly()(act, torch.zeros(24, 64, dtype=torch.int8).cuda(),
                                      torch.ones(24, dtype=torch.float16).cuda())


# The one-to-five-token packed-int4 kernel (integer tensor pipe, activations as three int8 digit planes): every
# option it handles, K slices of one and many steps, an outlier-heavy row, a tiny and a huge row, and rows of zeros.
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m", [1, 2, 3, 5])
@pytest.mark.parametrize("n,k,group,use_bias,use_zp", [
    (272, 1024, 64, True, True), (64, 2048, 128, False, False), (48, 4096, 256, True, False), (32, 2048, 0, True, True),
    (96, 3072, 0, False, False), (16, 8192, 128, False, True), (112, 1024, 0, False, True), (32, 28672, 128, False, False)])
def test_int4_few_tokens(dt, m, n, k, group, use_bias, use_zp):
    act, qw, scale, bias, zp = make(4, m, n, k, dt, group, use_bias, use_zp, seed=m + n + k)
    g = torch.Generator().manual_seed(k)
    act = torch.where(torch.rand(m, k, generator=g) < 0.002, act * 30, act)  # outliers
    if m >= 2:
        act[1] = 0  # a row of zeros gives the bias (or 0)
    if m >= 3:
        act[2] = act[2] * (1e-3 if dt == torch.float16 else 1e-30)  # a tiny row
    if m >= 5:
        act[4] = act[4] * (50 if dt == torch.float16 else 1e30)  # a huge row
    out = run(act, qw, scale, bias, zp)
    ref = O.gemm_weight_only_fp32(act, qw, scale, bias, zp)
    finite = torch.isfinite(ref.to(dt).float())
    assert_rows_within_bound(out, ref, {4: 50.0 if dt == torch.float16 else 1e30}, mask=finite)
    exact = ref.to(dt)
    assert int((out != exact)[finite].sum()) <= max(3, 0.02 * out.numel())
    if m >= 2:
        want = torch.zeros(n) if bias is None else bias.float()
        assert torch.equal(out[1].float(), want.to(dt).float())


@pytest.mark.parametrize("bad", [float("inf"), float("nan")])
def test_int4_few_tokens_non_finite_row(bad):
    """A NaN or an infinity in a row makes that whole output row NaN; the other rows are unaffected."""
    act, qw, scale, bias, zp = make(4, 2, 64, 4096, torch.bfloat16, 128, False, False, seed=3)
    clean = run(act, qw, scale)
    act2 = act.clone()
    act2[0, 100] = bad
    out = run(act2, qw, scale)
    assert bool(torch.isnan(out[0].float()).all())
    assert torch.equal(out[1].view(torch.int16), clean[1].view(torch.int16))


def test_static_weights_option_keeps_stream_order():
    """FNN_OPT_STATIC_WEIGHTS lets the int4 decode kernel start before the preceding kernel has finished; it must
    still see the activations that kernel wrote and must not overwrite an output that kernel still reads."""
    import flashnn_b200
    from flashnn_b200 import _lib
    act, qw, scale, bias, zp = make(4, 2, 512, 8192, torch.bfloat16, 128, False, False, seed=11)
    op = flashnn_b200.GemmWeightOnly(torch.bfloat16)
    a, q, s = act.cuda(), qw.cuda(), scale.cuda()
    base = [op(a * float(i + 1), q, s).cpu() for i in range(4)]
    _lib.set_option(_lib.OPT_STATIC_WEIGHTS, 1)
    try:
        assert _lib.lib().fnn_get_option(_lib.OPT_STATIC_WEIGHTS) == 1
        outs = []
        for rep in range(3):
            for i in range(4):
                x = a * float(i + 1)  # produced by the kernel right before the call
                y = op(x, q, s)
                outs.append((i, y, y.float().sum()))  # consumed by the kernel right after it
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        for i, y, _ in outs:
            assert torch.equal(y.cpu().view(torch.int16), base[i].view(torch.int16))
    finally:
        _lib.set_option(_lib.OPT_STATIC_WEIGHTS, 0)


# Prefill shapes (M > 16) with group-wise scales run on the tensor-core kernel that gives every scale group its own
# fp32 accumulator and applies s[g, n] (and the zero-point term) in fp32: w * s is never rounded to 16 bits, so the
# strict bound against the fp32 dequant-matmul holds, as it does for every other weight-only path.
@pytest.mark.parametrize("kind", [8, 4])
@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,n,k,group,use_bias,use_zp", [
    (17, 64, 256, 64, False, False), (130, 128, 512, 128, True, True), (300, 1000, 2048, 128, True, False),
    (513, 258, 1024, 256, False, True), (64, 512, 4096, 64, True, True), (700, 520, 1536, 512, True, True)])
def test_prefill_group_wise_shapes(kind, dt, m, n, k, group, use_bias, use_zp):
    act, qw, scale, bias, zp = make(kind, m, n, k, dt, group, use_bias, use_zp, seed=m + kind + group)
    out = run(act, qw, scale, bias, zp)
    assert_within_bound(out, act, qw, scale, bias, zp)


def test_prefill_group_wise_fp32_scales_and_fractional_zero_points():
    """Scales and zero-points in fp32 (not rounded to the activation dtype on the way in) and zero-points that are
    not integers: the zero-point term goes through the per-group row sums in fp32, so neither is a special case."""
    act, qw, scale, bias, _ = make(4, 200, 264, 1024, torch.bfloat16, 128, True, False, seed=77)
    g = torch.Generator().manual_seed(78)
    scale32 = torch.rand(8, 264, generator=g) * 0.045 + 0.005
    zp32 = torch.rand(8, 264, generator=g) * 4 - 2
    out = run(act, qw, scale32, bias, zp32)
    assert_within_bound(out, act, qw, scale32, bias, zp32)


def test_prefill_group_wise_full_size():
    """A16W4 prefill at the decode config's weight shape (N=28672, K=8192, group 128) with 256 tokens: sampled rows
    against the fp32 dequant-matmul, and a checksum over all rows (column sums are linear in the activations)."""
    from flashnn_b200 import workloads as W
    w = W.a16w4_decode(16)
    g = torch.Generator().manual_seed(9)
    x = torch.randn(256, 8192, generator=g).to(torch.bfloat16)
    out = run(x, w["qw"], w["scale"])
    rows = [0, 17, 100, 127, 128, 255]
    assert_within_bound(out[rows], x[rows], w["qw"], w["scale"], None, None, max_last_bit_mismatch=0.08)
    dq = O.unpack_int4(w["qw"]).double() * w["scale"].double().repeat_interleave(128, dim=0).t()  # [N, K]
    ref_colsum = x.double().sum(0) @ dq.t()
    tol = 256 ** 0.5 * 2.0 ** -7 * out.double().abs().max()  # one bf16 rounding per output, 256 of them per column
    assert float((out.double().sum(0) - ref_colsum).abs().max()) <= float(tol)


# Six to sixteen tokens of packed int4 (the 16-bit-fragment decode kernel): group size 128 and per-channel scales,
# bias, ragged N, short and long K, outlier-heavy rows, a row of zeros and a tiny row.
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m", [6, 9, 13, 16])
@pytest.mark.parametrize("n,k,group,use_bias", [(272, 1024, 128, True), (64, 128, 128, False), (130, 2048, 0, True),
                                                (1024, 4096, 128, False), (96, 8192, 0, False), (48, 28672, 128, True)])
def test_int4_six_to_sixteen_tokens(dt, m, n, k, group, use_bias):
    act, qw, scale, bias, zp = make(4, m, n, k, dt, group, use_bias, False, seed=m + n + k)
    g = torch.Generator().manual_seed(k + 1)
    act = torch.where(torch.rand(m, k, generator=g) < 0.002, act * 30, act)  # outliers
    act[1] = 0  # a row of zeros gives the bias (or 0)
    act[2] = act[2] * (1e-3 if dt == torch.float16 else 1e-30)  # a tiny row
    out = run(act, qw, scale, bias, zp)
    ref = O.gemm_weight_only_fp32(act, qw, scale, bias, zp)
    assert_rows_within_bound(out, ref)
    exact = ref.to(dt)
    assert int((out != exact).sum()) <= max(3, 0.02 * out.numel())
    want = torch.zeros(n) if bias is None else bias.float()
    assert torch.equal(out[1].float(), want.to(dt).float())


# The same token counts at K = 4096 and 8192 run the kernel that keeps the activations on the SM (tokens as the MMA's
# row operand, fragments in registers and shared memory): every group size it takes, zero-points, bias, both dtypes.
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m", [6, 8, 11, 16])
@pytest.mark.parametrize("n,k,group,use_bias,use_zp", [
    (272, 8192, 128, True, True), (64, 8192, 64, False, False), (1024, 8192, 256, True, False), (48, 4096, 0, True, True),
    (160, 4096, 64, False, True), (3584, 8192, 128, False, False), (32, 4096, 256, True, False), (96, 8192, 0, False, True)])
def test_int4_resident_activations(dt, m, n, k, group, use_bias, use_zp):
    act, qw, scale, bias, zp = make(4, m, n, k, dt, group, use_bias, use_zp, seed=m + n + k + group)
    g = torch.Generator().manual_seed(k + 3)
    act = torch.where(torch.rand(m, k, generator=g) < 0.002, act * 30, act)  # outliers
    act[1] = 0  # a row of zeros gives the bias (or 0)
    act[2] = act[2] * (1e-3 if dt == torch.float16 else 1e-30)  # a tiny row
    out = run(act, qw, scale, bias, zp)
    ref = O.gemm_weight_only_fp32(act, qw, scale, bias, zp)
    assert_rows_within_bound(out, ref)
    exact = ref.to(dt)
    assert int((out != exact).sum()) <= max(3, 0.02 * out.numel())
    want = torch.zeros(n) if bias is None else bias.float()
    assert torch.equal(out[1].float(), want.to(dt).float())


def test_int4_sixteen_tokens_non_finite_row_resident():
    act, qw, scale, bias, zp = make(4, 16, 256, 8192, torch.bfloat16, 128, False, False, seed=5)
    clean = run(act, qw, scale)
    for bad in (float("nan"), float("inf")):
        act2 = act.clone()
        act2[7, 5000] = bad
        out = run(act2, qw, scale)
        assert bool(torch.isnan(out[7].float()).all())
        keep = [i for i in range(16) if i != 7]
        assert torch.equal(out[keep].view(torch.int16), clean[keep].view(torch.int16))


def test_int4_sixteen_tokens_non_finite_row():
    act, qw, scale, bias, zp = make(4, 16, 256, 2048, torch.bfloat16, 128, False, False, seed=5)
    clean = run(act, qw, scale)
    act2 = act.clone()
    act2[7, 100] = float("nan")
    out = run(act2, qw, scale)
    assert bool(torch.isnan(out[7].float()).all())
    keep = [i for i in range(16) if i != 7]
    assert torch.equal(out[keep].view(torch.int16), clean[keep].view(torch.int16))


# Decode shapes whose K the tensor-core kernels decline (not a multiple of 512): the coalesced warp-per-row kernel.
@pytest.mark.parametrize("kind,m,n,k,group,use_bias,use_zp", [
    (4, 1, 512, 11008, 128, False, False), (4, 4, 256, 11008, 128, True, True), (4, 16, 64, 1104, 48, True, False),
    (8, 3, 100, 1040, 0, True, True), (8, 9, 48, 2064, 16, False, True), (4, 2, 32, 80, 0, False, False)])
@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_decode_odd_k_shapes(kind, m, n, k, group, use_bias, use_zp, dt):
    act, qw, scale, bias, zp = make(kind, m, n, k, dt, group, use_bias, use_zp, seed=k + m)
    out = run(act, qw, scale, bias, zp)
    assert_within_bound(out, act, qw, scale, bias, zp)


# int8 weights, one to five tokens, on the integer tensor pipe (the weight bytes are the MMA operand as they are).
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m", [1, 2, 3, 5])
@pytest.mark.parametrize("n,k,group,use_bias,use_zp", [
    (1024, 4096, 64, True, True), (64, 8192, 128, False, False), (48, 4096, 256, True, False), (32, 8192, 0, True, True),
    (96, 12288, 0, False, False), (16, 8192, 128, False, True), (32, 28672, 128, True, False)])
def test_int8_few_tokens(dt, m, n, k, group, use_bias, use_zp):
    act, qw, scale, bias, zp = make(8, m, n, k, dt, group, use_bias, use_zp, seed=m + n + k)
    g = torch.Generator().manual_seed(k)
    act = torch.where(torch.rand(m, k, generator=g) < 0.002, act * 30, act)  # outliers
    if m >= 2:
        act[1] = 0
    out = run(act, qw, scale, bias, zp)
    ref = O.gemm_weight_only_fp32(act, qw, scale, bias, zp)
    assert_rows_within_bound(out, ref)
    exact = ref.to(dt)
    assert int((out != exact).sum()) <= max(3, 0.02 * out.numel())
    if m >= 2:
        want = torch.zeros(n) if bias is None else bias.float()
        assert torch.equal(out[1].float(), want.to(dt).float())
