"""The fused-MoE oracle (block walk over expert-sorted slots) against a token-by-token formulation that does not
use the sorted layout at all.  The reference has no CPU implementation of this op, so this is a consistency check
of the restatement, not a pin."""
import pytest
import torch

from oracle import quant_oracle as O
from tests.moe_util import make_moe_case


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
