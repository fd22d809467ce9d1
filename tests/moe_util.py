"""Block-aligned expert sort used by the fused-MoE tests: the layout the reference kernel's docstring describes
(flashnn/triton_kernels/fused_moe_a8w8.py:191-209; the reference itself ships no routine that produces it)."""
import torch


def moe_align_block_size(topk_ids: torch.Tensor, num_experts: int, block_m: int):
    """topk_ids [M, top_k] -> (sorted_token_ids [EM] int32, expert_ids [EM / block_m] int32,
    num_tokens_post_padded [1] int32).  Flat (token * top_k + choice) indices are grouped by expert, each group
    padded to a multiple of block_m with the value M * top_k; EM is the worst-case length, the unused tail holds
    padding values and expert 0."""
    flat = topk_ids.reshape(-1)
    num_valid = flat.numel()
    em = num_valid + num_experts * (block_m - 1)
    em = (em + block_m - 1) // block_m * block_m
    sorted_ids = torch.full((em,), num_valid, dtype=torch.int32)
    expert_ids = torch.zeros(em // block_m, dtype=torch.int32)
    pos = 0
    for e in range(num_experts):
        idx = torch.nonzero(flat == e).reshape(-1).to(torch.int32)
        if idx.numel() == 0:
            continue
        n_blocks = (idx.numel() + block_m - 1) // block_m
        sorted_ids[pos:pos + idx.numel()] = idx
        expert_ids[pos // block_m:pos // block_m + n_blocks] = e
        pos += n_blocks * block_m
    return sorted_ids, expert_ids, torch.tensor([pos], dtype=torch.int32)


def make_moe_case(m, e, n, k, top_k, block_m, seed, scale_dt=torch.float32):
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8)
    b = torch.randint(-127, 128, (e, n, k), generator=g, dtype=torch.int8)
    alpha_row = (torch.rand(m, generator=g) * 0.015 + 0.005).to(scale_dt)
    alpha_col = (torch.rand(e, n, generator=g) * 0.009 + 0.001).to(scale_dt)
    logits = torch.rand(m, e, generator=g)
    topk_w, topk_ids = torch.topk(torch.softmax(logits, dim=-1), top_k, dim=-1)
    sorted_ids, expert_ids, npp = moe_align_block_size(topk_ids, e, block_m)
    return dict(a=a, b=b, alpha_row=alpha_row, alpha_col=alpha_col, topk_w=topk_w.float().contiguous(),
                topk_ids=topk_ids.to(torch.int32), sorted_ids=sorted_ids, expert_ids=expert_ids, npp=npp)
