"""The fused-MoE oracles against (a) outputs of the reference's own Triton kernels, run on a B200 by
tests/golden/make_moe_golden.py and stored in tests/golden/fused_moe_*.npz -- the pin: the reference has no CPU
implementation of these operators -- and (b) a token-by-token formulation that does not use the sorted layout."""
import pytest
import torch

from oracle import quant_oracle as O
from tests import golden_io as G
from tests.moe_util import make_moe_case

A8 = G.load("fused_moe_a8w8.npz")
W4 = G.load("fused_moe_a16w4.npz")


def _t(c, key, dt_name=None):
    dt = None if dt_name is None or dt_name == "float32" else G.dtype_of(dt_name)
    return G.tensor(c[key], dt)


@pytest.mark.parametrize("name", sorted(A8))
def test_a8w8_oracle_reproduces_the_reference_kernel_bit_for_bit(name):
    c = A8[name]
    assert "error" not in c, str(c.get("error"))
    odt, sdt = G.dtype_of(c["out_dtype"]), str(c["scale_dtype"])
    m, top_k, n, bm = int(c["m"]), int(c["top_k"]), int(c["n"]), int(c["bm"])
    out = O.fused_moe_a8w8(_t(c, "a"), _t(c, "b"), _t(c, "alpha_row", sdt), _t(c, "alpha_col", sdt), _t(c, "topk_w"),
                           _t(c, "sorted_ids"), _t(c, "expert_ids"), _t(c, "npp"), m * top_k, bool(c["mul"]), top_k, bm, odt,
                           C=torch.full((m, top_k, n), 7.0, dtype=odt))
    ref = G.tensor(c["out"], odt)
    assert torch.equal(out.view(torch.int16), ref.view(torch.int16))


def w4_args(c):
    dt = G.dtype_of(c["dtype"])
    m, top_k, bm = int(c["m"]), int(c["top_k"]), int(c["bm"])
    zp = G.tensor(c["zp"], dt) if "zp" in c else None
    return (G.tensor(c["a"], dt), _t(c, "b"), G.tensor(c["scale"], dt), zp, _t(c, "topk_w"), _t(c, "sorted_ids"),
            _t(c, "expert_ids"), _t(c, "npp"), m * top_k, bool(c["mul"]), top_k, bm)


@pytest.mark.parametrize("name", sorted(W4))
def test_a16w4_oracle_reproduces_the_reference_kernel(name):
    """A floating-point product: the tensor core's fp32 summation order is not defined, so the bar is a rounding of
    the 16-bit result (at most 2 units in the last place, at least 99 % of the outputs identical)."""
    c = W4[name]
    if "error" in c:
        # Triton 3.6 cannot compile the reference's sub-channel kernel for bf16 (int8 * bf16 has no common type there);
        # the recorded failure keeps the case visible
        assert str(c["dtype"]) == "bfloat16" and int(c["group"]) > 0 and "CompilationError" in str(c["error"])
        pytest.skip("the reference kernel does not compile for this case")
    dt = G.dtype_of(c["dtype"])
    m, top_k, n = int(c["m"]), int(c["top_k"]), int(c["n"])
    out = O.fused_moe_a16w4(*w4_args(c), C=torch.full((m, top_k, n), 7.0, dtype=dt))
    ref = G.tensor(c["out"], dt)
    ulp = (out.view(torch.int16).int() - ref.view(torch.int16).int()).abs()
    assert int(ulp.max()) <= 2
    assert float((ulp == 0).float().mean()) >= 0.99
    # and the fp32 dequant-matmul form (no 16-bit rounding of w*s), which the CUDA kernels are held to, stays within
    # the weight-only bound of the reference kernel's own output
    exact = O.fused_moe_a16w4(*w4_args(c), C=torch.full((m, top_k, n), 7.0, dtype=dt), exact_scales=True).float()
    assert bool(((exact - ref.float()).abs() <= 1e-3 + 1e-2 * ref.float().abs()).all())


@pytest.mark.parametrize("m,e,n,k,top_k,bm,mul", [(5, 4, 32, 64, 2, 16, True), (33, 8, 48, 128, 2, 16, False),
                                                  (7, 3, 16, 32, 1, 32, True), (64, 8, 64, 96, 4, 64, True)])
def test_block_walk_equals_token_by_token(m, e, n, k, top_k, bm, mul):
    c = make_moe_case(m, e, n, k, top_k, bm, seed=m + e)
    out = O.fused_moe_a8w8(c["a"], c["b"], c["alpha_row"], c["alpha_col"], c["topk_w"], c["sorted_ids"], c["expert_ids"],
                           c["npp"], m * top_k, mul, top_k, bm, torch.float16)
    want = torch.zeros(m, top_k, n, dtype=torch.float16)
    for t in range(m):
        for j in range(top_k):
            ex = int(c["topk_ids"][t, j])
            acc = O.gemm_a8w8_acc_i32(c["a"][t:t + 1], c["b"][ex]).float()
            v = acc * c["alpha_row"][t].float() * c["alpha_col"][ex].float()[None, :]
            if mul:
                v = v * c["topk_w"][t, j]
            want[t, j] = v[0].to(torch.float16)
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    # every valid flat index appears exactly once among the slots in use
    used = c["sorted_ids"][:int(c["npp"])]
    valid = used[used < m * top_k]
    assert sorted(valid.tolist()) == list(range(m * top_k))
