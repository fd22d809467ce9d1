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


def ffn_layer(m, rank=0, world=1, hidden=8192, inter=28672):
    """Llama-2-70B-shaped FFN, A8W8, column-sharded: rank `rank` of `world` owns output columns
    [r*N/world, (r+1)*N/world) of both projections (gate/up: hidden -> 2*inter; down: inter -> hidden).
    Activations are replicated; the down projection gets its own N(0,1) input."""
    n_gu, n_dn = 2 * inter, hidden
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


# Algorithmic work of each op (what the roofline figures are computed from).
def a8w8_ops(m, n, k) -> int:
    return 2 * m * n * k


def a8w8_bytes(m, n, k) -> int:
    return m * k + n * k + 2 * m * n + 4 * (m + n)


def dynamic_quant_bytes(m, k) -> int:
    return 2 * m * k + m * k + 2 * m


def a16w4_bytes(m, n, k, group) -> int:
    return n * k // 2 + 2 * (k // group) * n + 2 * m * k + 2 * m * n
