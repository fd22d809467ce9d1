"""fused_moe_a8w8_forward on the GPU (through the C ABI) against the CPU oracle.  The accumulator is exact and the
fp32 scale multiplications follow the reference kernel's order, so the 16-bit outputs are compared bit for bit."""
import pytest
import torch

from oracle import quant_oracle as O
from tests.moe_util import make_moe_case

pytestmark = pytest.mark.gpu


def run(c, top_k, bm, mul, out_ty, m, n):
    import flashnn_b200
    from flashnn_b200 import _lib
    dev = {k: v.cuda() for k, v in c.items()}
    out = torch.full((m, top_k, n), 7.0, dtype=out_ty, device="cuda")  # untouched rows must keep this value
    flashnn_b200.fused_moe_a8w8_forward(dev["a"], dev["b"], out, dev["alpha_row"], dev["alpha_col"], dev["topk_w"],
                                        dev["topk_ids"], dev["sorted_ids"], dev["expert_ids"], dev["npp"], mul, top_k, bm)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    return out.cpu()


@pytest.mark.parametrize("out_ty", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,e,n,k,top_k,bm,mul", [
    (5, 4, 32, 64, 2, 16, True), (33, 8, 48, 128, 2, 16, False), (7, 3, 16, 32, 1, 32, True), (64, 8, 64, 96, 4, 64, True),
    (300, 8, 1024, 512, 2, 128, True), (1, 16, 256, 1024, 4, 16, True), (513, 4, 272, 2064 // 16 * 16, 2, 256, False),
    (64, 8, 2048, 4096, 2, 16, True)])
def test_matches_oracle(out_ty, m, e, n, k, top_k, bm, mul):
    c = make_moe_case(m, e, n, k, top_k, bm, seed=m + e + n)
    out = run(c, top_k, bm, mul, out_ty, m, n)
    ref = O.fused_moe_a8w8(c["a"], c["b"], c["alpha_row"], c["alpha_col"], c["topk_w"], c["sorted_ids"], c["expert_ids"],
                           c["npp"], m * top_k, mul, top_k, bm, out_ty, C=torch.full((m, top_k, n), 7.0, dtype=out_ty))
    assert torch.equal(out.view(torch.int16), ref.view(torch.int16))


# blocks of 256 slots and enough tiles for every CTA pair: the CTA-pair kernel's fused-MoE mode (ragged N, an expert
# count that leaves some experts with an odd number of half-filled blocks, with and without the routing weights)
@pytest.mark.parametrize("out_ty", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,e,n,k,top_k,mul", [(2000, 4, 1024, 512, 2, True), (1800, 6, 1008, 272, 2, False),
                                               (4400, 8, 768, 128, 1, True)])
def test_blocks_of_256_on_the_cta_pair_kernel(out_ty, m, e, n, k, top_k, mul):
    bm = 256
    c = make_moe_case(m, e, n, k, top_k, bm, seed=m + e + n)
    assert (c["sorted_ids"].numel() // 256) * ((n + 255) // 256) >= 74
    out = run(c, top_k, bm, mul, out_ty, m, n)
    ref = O.fused_moe_a8w8(c["a"], c["b"], c["alpha_row"], c["alpha_col"], c["topk_w"], c["sorted_ids"], c["expert_ids"],
                           c["npp"], m * top_k, mul, top_k, bm, out_ty, C=torch.full((m, top_k, n), 7.0, dtype=out_ty))
    assert torch.equal(out.view(torch.int16), ref.view(torch.int16))



def test_sixteen_bit_scales_and_dropped_tokens():
    """fp16 scales; some slots in use are padding-valued in the middle of a block (tokens dropped by the router)."""
    m, e, n, k, top_k, bm = 40, 4, 64, 256, 2, 16
    c = make_moe_case(m, e, n, k, top_k, bm, seed=3, scale_dt=torch.float16)
    c["sorted_ids"][1] = m * top_k
    c["sorted_ids"][5] = m * top_k + 3
    out = run(c, top_k, bm, True, torch.float16, m, n)
    ref = O.fused_moe_a8w8(c["a"], c["b"], c["alpha_row"], c["alpha_col"], c["topk_w"], c["sorted_ids"], c["expert_ids"],
                           c["npp"], m * top_k, True, top_k, bm, torch.float16, C=torch.full((m, top_k, n), 7.0, dtype=torch.float16))
    assert torch.equal(out.view(torch.int16), ref.view(torch.int16))


# Outputs of the reference's own Triton kernel on a B200 (tests/golden/make_moe_golden.py): the CUDA kernel must
# reproduce them bit for bit, including the fp16 rounding the reference applies before a bf16 store.
from tests import golden_io as G  # noqa: E402

A8 = G.load("fused_moe_a8w8.npz")


@pytest.mark.parametrize("name", sorted(A8))
def test_reproduces_the_reference_kernel(name):
    c = A8[name]
    odt = G.dtype_of(c["out_dtype"])
    sdt = None if str(c["scale_dtype"]) == "float32" else G.dtype_of(c["scale_dtype"])
    m, top_k, n, bm = int(c["m"]), int(c["top_k"]), int(c["n"]), int(c["bm"])
    case = dict(a=G.tensor(c["a"]), b=G.tensor(c["b"]), alpha_row=G.tensor(c["alpha_row"], sdt),
                alpha_col=G.tensor(c["alpha_col"], sdt), topk_w=G.tensor(c["topk_w"]), topk_ids=G.tensor(c["topk_ids"]),
                sorted_ids=G.tensor(c["sorted_ids"]), expert_ids=G.tensor(c["expert_ids"]), npp=G.tensor(c["npp"]))
    out = run(case, top_k, bm, bool(c["mul"]), odt, m, n)
    ref = G.tensor(c["out"], odt)
    assert torch.equal(out.view(torch.int16), ref.view(torch.int16))


# ---------------------------------------------------------------------------------------------------------------
# fused_moe_a16w4_forward: packed-int4 expert weights, per-channel and per-group scales.  The bar is the weight-only
# bound (|d| <= 1e-3 + 1e-2 |ref|) against the oracle's fp32 dequant-matmul form, plus the outputs of the reference's
# own Triton kernel on a B200 (tests/golden/fused_moe_a16w4.npz).
# ---------------------------------------------------------------------------------------------------------------
from tests.moe_util import make_moe_w4_case  # noqa: E402

W4 = G.load("fused_moe_a16w4.npz")
RTOL, ATOL = 1e-2, 1e-3


def run_w4(c, top_k, bm, mul, m, n):
    import flashnn_b200
    from flashnn_b200 import _lib
    dev = {k: (None if v is None else v.cuda()) for k, v in c.items() if k != "w4"}
    out = torch.full((m, top_k, n), 7.0, dtype=c["a"].dtype, device="cuda")
    flashnn_b200.fused_moe_a16w4_forward(dev["a"], dev["b"], out, dev["scale"], dev["zp"], dev["topk_w"], dev["topk_ids"],
                                         dev["sorted_ids"], dev["expert_ids"], dev["npp"], mul, top_k, bm)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    return out.cpu()


def check_w4(out, c, top_k, bm, mul, m, n):
    dt = c["a"].dtype
    ref = O.fused_moe_a16w4(c["a"], c["b"], c["scale"], c["zp"], c["topk_w"], c["sorted_ids"], c["expert_ids"], c["npp"],
                            m * top_k, mul, top_k, bm, C=torch.full((m, top_k, n), 7.0, dtype=torch.float32).to(dt),
                            exact_scales=True)
    # the oracle keeps fp32 until its final cast; compare in fp32 against an fp32 copy of that result
    ref32 = O.fused_moe_a16w4(c["a"].float(), c["b"], c["scale"].float(), None if c["zp"] is None else c["zp"].float(),
                              c["topk_w"], c["sorted_ids"], c["expert_ids"], c["npp"], m * top_k, mul, top_k, bm,
                              C=torch.full((m, top_k, n), 7.0, dtype=torch.float32), exact_scales=True)
    err = (out.float() - ref32).abs()
    bound = ATOL + RTOL * ref32.abs()
    assert bool((err <= bound).all()), f"max excess {(err - bound).max():.3e}"
    assert float((out != ref).float().mean()) < 0.02  # almost everywhere the same 16-bit value


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,e,n,k,top_k,bm,mul,group,use_zp", [
    (5, 4, 64, 128, 2, 16, True, 0, False), (33, 8, 96, 256, 2, 16, False, 0, True), (20, 4, 64, 256, 2, 32, True, 64, False),
    (48, 4, 128, 512, 2, 16, True, 128, True), (9, 4, 64, 208, 2, 8, True, 0, True), (300, 8, 1024, 512, 2, 64, True, 128, False),
    (1, 16, 256, 1024, 4, 16, True, 256, True), (513, 4, 288, 2048, 2, 128, False, 128, True), (64, 8, 2048, 4096, 2, 16, True, 128, False),
    (40, 4, 96, 256, 1, 64, True, 0, False)])
def test_a16w4_matches_the_fp32_dequant_oracle(dt, m, e, n, k, top_k, bm, mul, group, use_zp):
    c = make_moe_w4_case(m, e, n, k, top_k, bm, seed=m + e + n, dtype=dt, group=group, use_zp=use_zp)
    out = run_w4(c, top_k, bm, mul, m, n)
    check_w4(out, c, top_k, bm, mul, m, n)


# blocks of 256 slots and enough tiles for every CTA pair: the tcgen05 prefill kernels in their fused-MoE mode
# (per-channel and per-group scales, with and without zero-points, ragged N, an expert count that leaves padding tiles)
@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,e,n,k,top_k,mul,group,use_zp", [
    (2000, 4, 1024, 512, 2, True, 0, False), (1800, 6, 1056, 256, 2, False, 0, True), (2000, 4, 1024, 512, 2, True, 128, False),
    (1800, 6, 1056, 512, 2, True, 64, True), (4400, 8, 768, 256, 1, True, 256, False)])
def test_a16w4_blocks_of_256_on_the_prefill_kernels(dt, m, e, n, k, top_k, mul, group, use_zp):
    bm = 256
    c = make_moe_w4_case(m, e, n, k, top_k, bm, seed=m + e + n, dtype=dt, group=group, use_zp=use_zp)
    assert (c["sorted_ids"].numel() // 256) * ((n + 255) // 256) >= 74
    from flashnn_b200 import _lib
    assert _lib.lib().fnn_fused_moe_a16w4_workspace_bytes(c["sorted_ids"].numel(), k, group, int(use_zp), bm) > 0
    out = run_w4(c, top_k, bm, mul, m, n)
    check_w4(out, c, top_k, bm, mul, m, n)


def test_a16w4_dropped_tokens_and_fractional_zero_points():
    m, e, n, k, top_k, bm = 40, 4, 64, 256, 2, 16
    c = make_moe_w4_case(m, e, n, k, top_k, bm, seed=3, dtype=torch.float16, group=64, use_zp=True)
    c["zp"] = (c["zp"].float() + 0.37).half()
    c["sorted_ids"][1] = m * top_k
    c["sorted_ids"][5] = m * top_k + 3
    out = run_w4(c, top_k, bm, True, m, n)
    check_w4(out, c, top_k, bm, True, m, n)


@pytest.mark.parametrize("name", sorted(W4))
def test_a16w4_against_the_reference_kernel(name):
    c = W4[name]
    if "error" in c:
        pytest.skip("the reference kernel does not compile for this case")
    dt = G.dtype_of(c["dtype"])
    m, top_k, n, bm = int(c["m"]), int(c["top_k"]), int(c["n"]), int(c["bm"])
    case = dict(a=G.tensor(c["a"], dt), b=G.tensor(c["b"]), scale=G.tensor(c["scale"], dt),
                zp=G.tensor(c["zp"], dt) if "zp" in c else None, topk_w=G.tensor(c["topk_w"]), topk_ids=G.tensor(c["topk_ids"]),
                sorted_ids=G.tensor(c["sorted_ids"]), expert_ids=G.tensor(c["expert_ids"]), npp=G.tensor(c["npp"]))
    out = run_w4(case, top_k, bm, bool(c["mul"]), m, n)
    ref = G.tensor(c["out"], dt).float()
    assert bool(((out.float() - ref).abs() <= ATOL + RTOL * ref.abs()).all())
    if int(c["group"]) == 0:  # per channel the reference itself scales in fp32: the same 16-bit value almost everywhere
        assert float((out.float() != ref).float().mean()) < 0.02
