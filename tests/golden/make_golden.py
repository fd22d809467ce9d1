"""Generate the golden vectors under tests/golden/ from the reference itself.

Run once, in a container that has the reference checkout (CPU only):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference <checkout>

It imports the reference package, selects its torch backend
(`set_use_triton(False)`, flashnn/kernel_backend.py:27-29) and calls the
unmodified operator classes (flashnn/quant_gemm.py:39-209, flashnn/norm.py:39-124) on small seeded CPU
tensors.  Inputs and outputs are stored as raw bits (16-bit floats as uint16)
so the files are independent of the torch version that reads them.
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().contiguous()
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def gen(seed):
    return torch.Generator().manual_seed(seed)


def dq_cases(flashnn):
    op = flashnn.DynamicQuantize()
    cases = {}
    # shapes of the reference's own test (tests/quant_gemm/test_dynamic_quant.py:29-35),
    # the largest one cut down, in both input dtypes, plus an outlier-heavy case.
    for name, (m, k), dt, kind in [
        ("dq_f16_32x32", (32, 32), torch.float16, "uniform"),
        ("dq_f16_117x987", (117, 987), torch.float16, "uniform"),
        ("dq_bf16_64x64", (64, 64), torch.bfloat16, "uniform"),
        ("dq_bf16_29x987", (29, 987), torch.bfloat16, "normal"),
        ("dq_bf16_24x4096_outliers", (24, 4096), torch.bfloat16, "outliers"),
        ("dq_f16_8x8000", (8, 8000), torch.float16, "normal"),
    ]:
        g = gen(len(cases))
        if kind == "uniform":
            x = torch.rand(m, k, generator=g) * 2 - 1
        else:
            x = torch.randn(m, k, generator=g)
            if kind == "outliers":
                x = torch.where(torch.rand(m, k, generator=g) < 0.001, x * 20, x)
        x = x.to(dt)
        q, s = op(x)
        # the value before the unclamped int8 cast, to mark where the reference wraps
        amax = x.abs().max(-1, keepdim=True)[0]
        pre = torch.round(x / (amax / 127.0)).float()
        cases[name] = dict(x=bits(x), q=bits(q), scale=bits(s), precast=pre.to(torch.int16).numpy(),
                           dtype=str(dt).split(".")[-1])
    return cases


def a8w8_cases(flashnn):
    cases = {}
    for name, (m, n, k), out_ty, scale_ty, lo in [
        ("a8w8_128x128x128_f16", (128, 128, 128), torch.float16, torch.float16, -128),
        ("a8w8_16x256x512_bf16_f32scale", (16, 256, 512), torch.bfloat16, torch.float32, -127),
        ("a8w8_33x200x336_bf16_bf16scale", (33, 200, 336), torch.bfloat16, torch.bfloat16, -128),
        ("a8w8_130x136x1040_f16_f32scale", (130, 136, 1040), torch.float16, torch.float32, -127),
    ]:
        g = gen(100 + len(cases))
        a = torch.randint(lo, 128, (m, k), generator=g, dtype=torch.int8)
        b = torch.randint(lo, 128, (n, k), generator=g, dtype=torch.int8)
        row = (torch.rand(m, 1, generator=g) * 0.015 + 0.005).to(scale_ty)
        col = (torch.rand(1, n, generator=g) * 0.009 + 0.001).to(scale_ty)
        out = flashnn.GemmA8W8(out_ty)(a, b, row, col)
        cases[name] = dict(a=bits(a), b=bits(b), row=bits(row), col=bits(col), out=bits(out),
                           out_ty=str(out_ty).split(".")[-1], scale_ty=str(scale_ty).split(".")[-1])
    return cases


def pack_int4(w):
    u = w.to(torch.int16) & 0xF
    return (u[0::2] | (u[1::2] << 4)).to(torch.uint8).view(torch.int8)


def wo_cases(flashnn):
    cases = {}
    for name, kind, (m, n, k), dt, group, use_bias, use_zp in [
        ("wo_int8_pc_f16", "int8", (3, 256, 512), torch.float16, 0, False, False),
        ("wo_int8_pc_f16_bias_zp", "int8", (3, 256, 512), torch.float16, 0, True, True),
        ("wo_int8_g64_f16_bias", "int8", (3, 256, 512), torch.float16, 64, True, False),
        ("wo_int8_g64_f16_zp", "int8", (5, 128, 256), torch.float16, 64, False, True),
        ("wo_int8_pc_bf16", "int8", (17, 128, 384), torch.bfloat16, 0, False, False),
        ("wo_int4_g128_bf16", "int4", (4, 256, 512), torch.bfloat16, 128, False, False),
        ("wo_int4_g128_bf16_bias_zp", "int4", (1, 256, 512), torch.bfloat16, 128, True, True),
        ("wo_int4_pc_f16", "int4", (16, 128, 256), torch.float16, 0, False, False),
        ("wo_int4_pc_f16_bias_zp", "int4", (2, 128, 256), torch.float16, 0, True, True),
        ("wo_int4_g64_f16", "int4", (7, 64, 256), torch.float16, 64, False, False),
    ]:
        g = gen(200 + len(cases))
        act = torch.randn(m, k, generator=g).to(dt)
        if kind == "int8":
            w = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8)
            qw = w
            zlo, zhi = -20, 21
        else:
            w = torch.randint(-8, 8, (n, k), generator=g, dtype=torch.int8)
            qw = pack_int4(w)
            zlo, zhi = -3, 4
        sshape = (n,) if group == 0 else (k // group, n)
        scale = (torch.rand(*sshape, generator=g) * 0.045 + 0.005).to(dt)
        bias = torch.randn(n, generator=g).to(dt) if use_bias else None
        zp = None
        if use_zp:
            zp = torch.randint(zlo, zhi, sshape, generator=g).to(dt)
            # the per-channel helper subtracts a [1, N] zero-point row
            zp_arg = zp.unsqueeze(0) if group == 0 else zp
        else:
            zp_arg = None
        out = flashnn.GemmWeightOnly(dt)(act, qw, scale, bias, zp_arg)
        d = dict(act=bits(act), qw=bits(qw), scale=bits(scale), out=bits(out),
                 dtype=str(dt).split(".")[-1], kind=kind, group=group)
        if bias is not None:
            d["bias"] = bits(bias)
        if zp is not None:
            d["zp"] = bits(zp)
        cases[name] = d
    return cases


def norm_cases(flashnn):
    """RMSNormDquant / LayernormDquant on the shapes of the reference's tests
    (tests/norm/test_rms_norm_dquant.py, tests/norm/test_layer_norm_dquant.py: [4, 128] and [3, 32, 1024],
    the second one cut to 8 middle rows) with non-trivial weights."""
    cases = {}
    for name, kind, shape, dt, eps in [
        ("rms_f16_4x128", "rms", (4, 128), torch.float16, 1e-5),
        ("rms_f16_3x8x1024", "rms", (3, 8, 1024), torch.float16, 1e-5),
        ("rms_bf16_16x4096", "rms", (16, 4096), torch.bfloat16, 1e-6),
        ("ln_f16_4x128", "ln", (4, 128), torch.float16, 1e-5),
        ("ln_f16_3x8x1024", "ln", (3, 8, 1024), torch.float16, 1e-5),
        ("ln_bf16_16x4096", "ln", (16, 4096), torch.bfloat16, 1e-5),
    ]:
        g = gen(300 + len(cases))
        x = torch.randn(*shape, generator=g).to(dt)
        dim = shape[-1]
        w = (torch.rand(dim, generator=g) + 0.5).to(dt)
        if kind == "rms":
            op = flashnn.RMSNormDquant(dim, eps).to(dt)
            with torch.no_grad():
                op.weight.copy_(w)
                q, s = op(x)
            d = dict(x=bits(x), weight=bits(w), q=bits(q), scale=bits(s))
        else:
            b = (torch.randn(dim, generator=g) * 0.1).to(dt)
            op = flashnn.LayernormDquant(dim, eps).to(dt)
            with torch.no_grad():
                op.weight.copy_(w)
                op.bias.copy_(b)
                q, s = op(x)
            d = dict(x=bits(x), weight=bits(w), bias=bits(b), q=bits(q), scale=bits(s))
        d.update(dtype=str(dt).split(".")[-1], kind=kind, eps=np.float64(eps))
        cases[name] = d
    return cases


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import flashnn  # the reference package

    flashnn.set_use_triton(False)
    torch.set_num_threads(1)  # fixed reduction order inside the CPU matmul
    for fname, cases in [("dynamic_quant.npz", dq_cases(flashnn)),
                         ("gemm_a8w8.npz", a8w8_cases(flashnn)),
                         ("gemm_weight_only.npz", wo_cases(flashnn)),
                         ("norm_dquant.npz", norm_cases(flashnn))]:
        flat = {}
        for cname, d in cases.items():
            for key, val in d.items():
                flat[f"{cname}/{key}"] = np.asarray(val)
        np.savez_compressed(os.path.join(HERE, fname), **flat)
        print(fname, len(cases), "cases", os.path.getsize(os.path.join(HERE, fname)), "bytes")


if __name__ == "__main__":
    main()
