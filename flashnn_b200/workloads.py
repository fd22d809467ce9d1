"""Seeded synthetic inputs for the benchmark configurations of the quantized-GEMM
path.  Every tensor is generated on the CPU with its own `torch.Generator`, so
the CUDA kernels and any CPU check see identical bits.

Distributions: int8 operands uniform in [-127, 127]; per-token scales uniform
[0.005, 0.02]; per-channel scales uniform [0.001, 0.01]; activations N(0, 1)
(with 0.1 % of entries multiplied by 20 where a configuration asks for outliers);
int4 weights uniform in [-8, 7]; group scales uniform [0.005, 0.05].
"""
import torch


def _gen(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


def rand_int8(shape, seed, lo=-127, hi=127) -> torch.Tensor:
    return torch.randint(lo, hi + 1, shape, generator=_gen(seed), dtype=torch.int8)


def rand_uniform(shape, seed, lo, hi, dtype=torch.float32) -> torch.Tensor:
    return (torch.rand(shape, generator=_gen(seed)) * (hi - lo) + lo).to(dtype)


def rand_normal(shape, seed, dtype, outliers: bool = False) -> torch.Tensor:
    g = _gen(seed)
    x = torch.randn(shape, generator=g)
    if outliers:
        x = torch.where(torch.rand(shape, generator=g) < 0.001, x * 20, x)
    return x.to(dtype)


def pack_int4(w: torch.Tensor) -> torch.Tensor:
    """int8 [N, K] with values in [-8, 7] -> packed int8 [N/2, K]: byte (j, k) holds channel 2j in
    its low nibble and channel 2j+1 in its high nibble (the reference's layout,
    flashnn/quant_gemm.py:175-190)."""
    u = w.to(torch.int16) & 0xF
    return (u[0::2] | (u[1::2] << 4)).to(torch.uint8).view(torch.int8)


def a8w8_small(m=16, n=4096, k=4096, out_ty=torch.bfloat16):
    """A8W8 GEMM with int8 operands and fp32 scales (first benchmark configuration)."""
    return dict(a=rand_int8((m, k), 0), b=rand_int8((n, k), 1),
                alpha_row=rand_uniform((m,), 2, 0.005, 0.02), alpha_col=rand_uniform((n,), 3, 0.001, 0.01),
                out_ty=out_ty)


def dq_a8w8_prefill(m=4096, n=11008, k=4096):
    """DynamicQuant -> A8W8 prefill chain: bf16 activations with outliers, int8 weights."""
    return dict(x=rand_normal((m, k), 0, torch.bfloat16, outliers=True), w=rand_int8((n, k), 1),
                alpha_col=rand_uniform((n,), 3, 0.001, 0.01), out_ty=torch.bfloat16)


def a16w8_prefill(m=2048, n=8192, k=8192):
    """A16W8 weight-only GEMM: fp16 activations, int8 weights, per-channel fp16 scales."""
    return dict(x=rand_normal((m, k), 0, torch.float16), w=rand_int8((n, k), 1),
                scale=rand_uniform((n,), 2, 0.001, 0.01, torch.float16), out_ty=torch.float16)


def a16w4_decode(m=1, n=28672, k=8192, group=128, dtype=torch.bfloat16):
    """A16W4 decode GEMV: bf16 activations, packed int4 weights, group-wise bf16 scales, no zero-points."""
    w4 = torch.randint(-8, 8, (n, k), generator=_gen(1), dtype=torch.int8)
    return dict(x=rand_normal((m, k), 0, dtype), qw=pack_int4(w4),
                scale=rand_uniform((k // group, n), 2, 0.005, 0.05, dtype), group=group, out_ty=dtype)


def ffn_layer(m, rank=0, world=1, hidden=8192, inter=28672, weights=True):
    """Llama-2-70B-shaped FFN, A8W8, column-sharded: rank `rank` of `world` owns output columns
    [r*N/world, (r+1)*N/world) of both projections (gate/up: hidden -> 2*inter; down: inter -> hidden).
    Activations are replicated; the down projection gets its own N(0,1) input.  `weights=False` returns
    the activations only."""
    n_gu, n_dn = 2 * inter, hidden
    if not weights:
        return dict(x=rand_normal((m, hidden), 0, torch.bfloat16), h=rand_normal((m, inter), 3, torch.bfloat16),
                    out_ty=torch.bfloat16)
    assert n_gu % world == 0 and n_dn % world == 0
    s_gu, s_dn = n_gu // world, n_dn // world

    def shard_rows(n_total, k, seed, lo, hi):
        # generate only this rank's rows, reproducibly: one generator per 1024-row block of the full matrix
        out = torch.empty((hi - lo, k), dtype=torch.int8)
        blk = 1024
        for b0 in range((lo // blk) * blk, hi, blk):
            rows = rand_int8((min(blk, n_total - b0), k), seed * 100003 + b0 // blk)
            a, b = max(lo, b0), min(hi, b0 + blk)
            out[a - lo:b - lo] = rows[a - b0:b - b0]
        return out

    return dict(
        x=rand_normal((m, hidden), 0, torch.bfloat16), h=rand_normal((m, inter), 3, torch.bfloat16),
        w_gu=shard_rows(n_gu, hidden, 1, rank * s_gu, (rank + 1) * s_gu),
        w_dn=shard_rows(n_dn, inter, 2, rank * s_dn, (rank + 1) * s_dn),
        col_gu=rand_uniform((n_gu,), 4, 0.001, 0.01)[rank * s_gu:(rank + 1) * s_gu].contiguous(),
        col_dn=rand_uniform((n_dn,), 5, 0.001, 0.01)[rank * s_dn:(rank + 1) * s_dn].contiguous(),
        out_ty=torch.bfloat16)


def reference_sweep_shapes():
    """The (N, K) pairs and the M values of the reference's own A8W8 benchmark sweep
    (benchmark/benchmark_gemm_a8w8.py:13-44): four projections (FFN layer 1, FFN layer 2, attention output, QKV) of
    five tensor-parallel model configurations.  Returns (list of (N, K), list of M)."""
    nk = []
    for hidden, inter, tp, heads, kv_heads in [(13312, 71168, 8, 104, 8), (13312, 71168, 4, 104, 4), (8192, 29568, 4, 64, 8),
                                               (8192, 29568, 2, 64, 8), (3584, 18944, 1, 28, 4)]:
        gqa = heads // kv_heads
        nk += [(hidden, inter // tp), ((inter // tp) * 2, hidden), (hidden, hidden // tp),
               ((hidden // tp) + ((hidden // tp) // gqa) * 2, hidden)]
    return nk, [1, 10, 20, 30, 40, 764, 1024, 2048, 4096, 8192]


DYNAMIC_QUANT_SWEEP_K = [1664, 3328, 8896, 13312, 17792, 35584]  # benchmark/benchmark_dynamic_quant.py:11


# Algorithmic work of each op (what the roofline figures are computed from).
def a8w8_ops(m, n, k) -> int:
    return 2 * m * n * k


def a8w8_bytes(m, n, k) -> int:
    return m * k + n * k + 2 * m * n + 4 * (m + n)


def dynamic_quant_bytes(m, k) -> int:
    return 2 * m * k + m * k + 2 * m


def a16w4_bytes(m, n, k, group) -> int:
    return n * k // 2 + 2 * (k // group) * n + 2 * m * k + 2 * m * n


# ----------------------------------------------------------------------------
# Fused mixture-of-experts cases
# ----------------------------------------------------------------------------
def moe_align_block_size(topk_ids: torch.Tensor, num_experts: int, block_m: int):
    """The block-aligned expert sort the reference's fused-MoE kernels expect as input
    (flashnn/triton_kernels/fused_moe_a8w8.py:191-209 describes the layout; the reference ships no routine that
    produces it).  topk_ids [M, top_k] -> (sorted_token_ids [EM] int32, expert_ids [EM / block_m] int32,
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
    """Seeded fused-MoE A8W8 problem: int8 tokens [m, k], expert weights [e, n, k], scales, softmax routing."""
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


def make_moe_w4_case(m, e, n, k, top_k, block_m, seed, dtype=torch.float16, group=0, use_zp=False):
    """Seeded fused-MoE A16W4 problem: 16-bit tokens [m, k], packed int4 expert weights [e, n/2, k] (channel 2j in the
    low nibble of byte (j, k), 2j+1 in the high nibble), scales [e, n] (group == 0) or [e, n, k/group], optional
    zero-points of the same shape."""
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g).to(dtype)
    w4 = torch.randint(-8, 8, (e, n, k), generator=g, dtype=torch.int8)
    u = w4.to(torch.int16) & 0xF
    b = (u[:, 0::2] | (u[:, 1::2] << 4)).to(torch.uint8).view(torch.int8).contiguous()
    sshape = (e, n) if group == 0 else (e, n, k // group)
    scale = (torch.rand(*sshape, generator=g) * 0.045 + 0.005).to(dtype)
    zp = torch.randint(-2, 3, sshape, generator=g).to(dtype) if use_zp else None
    logits = torch.rand(m, e, generator=g)
    topk_w, topk_ids = torch.topk(torch.softmax(logits, dim=-1), top_k, dim=-1)
    sorted_ids, expert_ids, npp = moe_align_block_size(topk_ids, e, block_m)
    return dict(a=a, b=b, w4=w4, scale=scale, zp=zp, topk_w=topk_w.float().contiguous(), topk_ids=topk_ids.to(torch.int32),
                sorted_ids=sorted_ids, expert_ids=expert_ids, npp=npp)
