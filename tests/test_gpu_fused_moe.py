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
