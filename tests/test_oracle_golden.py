"""The CPU oracle must reproduce, bit for bit, what the reference's own classes
produced for the committed golden inputs (tests/golden/make_golden.py)."""
import numpy as np
import pytest
import torch

from oracle import quant_oracle as O
from tests import golden_io as G

DQ = G.load("dynamic_quant.npz")
A8 = G.load("gemm_a8w8.npz")
WO = G.load("gemm_weight_only.npz")
ND = G.load("norm_dquant.npz")


def same_bits(t: torch.Tensor, arr: np.ndarray):
    got = t.contiguous()
    if got.dtype in (torch.float16, torch.bfloat16):
        got = got.view(torch.int16).numpy().view(np.uint16)
    else:
        got = got.numpy()
    np.testing.assert_array_equal(got, arr)


@pytest.mark.parametrize("name", sorted(DQ))
def test_dynamic_quant_matches_reference(name):
    c = DQ[name]
    x = G.tensor(c["x"], G.dtype_of(c["dtype"]))
    q, s = O.dynamic_quantize(x, saturate=False)
    same_bits(q, c["q"])
    same_bits(s, c["scale"])
    pre, _ = O.dynamic_quantize_precast(x)
    np.testing.assert_array_equal(pre.float().numpy().astype(np.int16), c["precast"])
    # the saturating form differs only where the reference's quotient was +128
    qs, _ = O.dynamic_quantize(x, saturate=True)
    wrap = c["precast"] == 128
    np.testing.assert_array_equal(qs.numpy()[~wrap], c["q"][~wrap])
    assert (qs.numpy()[wrap] == 127).all() and (c["q"][wrap] == -128).all()


def test_bf16_golden_contains_wraps():
    # the fixture must actually exercise the +128 wrap that bf16 arithmetic produces
    assert sum(int((c["precast"] == 128).sum()) for c in DQ.values()) > 0


@pytest.mark.parametrize("name", sorted(A8))
def test_gemm_a8w8_matches_reference(name):
    c = A8[name]
    st, ot = G.dtype_of(c["scale_ty"]), G.dtype_of(c["out_ty"])
    a, b = G.tensor(c["a"]), G.tensor(c["b"])
    row, col = G.tensor(c["row"], st), G.tensor(c["col"], st)
    same_bits(O.gemm_a8w8(a, b, row, col, ot), c["out"])
    # the exact accumulator + epilogue form gives the same bits at these sizes
    acc = O.gemm_a8w8_acc_i32(a, b)
    assert acc.dtype == torch.int32
    assert torch.equal(acc, (a.int() @ b.int().t()))
    same_bits(O.gemm_a8w8_from_acc(acc, row, col, ot), c["out"])


@pytest.mark.parametrize("name", sorted(WO))
def test_gemm_weight_only_matches_reference(name):
    c = WO[name]
    dt = G.dtype_of(c["dtype"])
    act, qw, scale = G.tensor(c["act"], dt), G.tensor(c["qw"]), G.tensor(c["scale"], dt)
    bias = G.tensor(c["bias"], dt) if "bias" in c else None
    zp = G.tensor(c["zp"], dt) if "zp" in c else None
    if zp is not None and zp.dim() == 1:
        zp = zp.unsqueeze(0)
    torch.set_num_threads(1)
    out = O.gemm_weight_only_reference(act, qw, scale, bias, zp, dt)
    same_bits(out, c["out"])
    assert O.weight_kind(qw, scale) == str(c["kind"])
    # the fp32-dequant form differs from the reference output only by the reference's
    # 16-bit rounding of w*s: a coarse bound relative to the output range
    ref = G.tensor(c["out"], dt).float()
    o2 = O.gemm_weight_only_fp32(act, qw, scale, bias, zp)
    assert float((o2 - ref).abs().max()) <= 0.02 * float(ref.abs().max())


def test_int4_pack_roundtrip():
    g = torch.Generator().manual_seed(7)
    w = torch.randint(-8, 8, (64, 48), generator=g, dtype=torch.int8)
    assert torch.equal(O.unpack_int4(O.pack_int4(w)), w)
    # byte (j, k): low nibble = channel 2j, high nibble = channel 2j+1
    p = O.pack_int4(w).view(torch.uint8)
    assert int(p[3, 5]) == ((int(w[6, 5]) & 0xF) | ((int(w[7, 5]) & 0xF) << 4))


@pytest.mark.parametrize("name", sorted(ND))
def test_norm_dquant_matches_reference(name):
    c = ND[name]
    dt = G.dtype_of(c["dtype"])
    x = G.tensor(c["x"], dt)
    w = G.tensor(c["weight"], dt)
    if str(c["kind"]) == "rms":
        q, s = O.rms_norm_dquant(x, w, float(c["eps"]))
        assert s.shape == x.shape[:-1]
    else:
        q, s = O.layer_norm_dquant(x, w, G.tensor(c["bias"], dt), float(c["eps"]))
        assert s.shape == (x.numel() // x.shape[-1], 1)
    assert q.shape == x.shape and s.dtype == dt
    same_bits(q, c["q"])
    same_bits(s, c["scale"])
