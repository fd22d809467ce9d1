"""Generates tests/golden/fused_moe_a8w8.npz and tests/golden/fused_moe_a16w4.npz by running the reference's own
fused-MoE Triton kernels (flashnn/triton_kernels/fused_moe_a8w8.py:176-290, fused_moe_a16w4.py:326-466) on a CUDA
GPU.  The reference has no CPU implementation and no test of these two operators, so outputs of its kernels on
seeded inputs are the only thing that can pin the CPU oracle's restatement of them.

    python tests/golden/make_moe_golden.py [--ref DIR] [--out DIR]

DIR for --ref is a directory that holds the unmodified reference package `flashnn/` (default: baseline/_ref next to
this repository's root, else what the environment variable FLASHNN_REFERENCE names); --out defaults to tests/golden.  Every case stores its inputs and the
reference's output; 16-bit floats are stored as their raw uint16 bits.  A case whose kernel fails to compile or run
is recorded under `<case>/error` instead of being dropped silently.

Two facts about the reference launchers shape the cases.  With autotuning off, `fused_moe_a8w8_forward` launches its
kernel with BLOCK_SIZE_M fixed at 32 whatever `BM` says (fused_moe_a8w8.py:266), so its expert_ids are only read
correctly when BM == 32: the A8W8 cases use BM = 32.  `fused_moe_a16w4_forward` uses BM itself.
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=None)
    ap.add_argument("--out", default=HERE)
    args = ap.parse_args()
    ref = args.ref
    if ref is None:
        for cand in (os.path.join(ROOT, "baseline", "_ref"), os.environ.get("FLASHNN_REFERENCE", "")):
            if cand and os.path.exists(os.path.join(cand, "flashnn", "quant_gemm.py")):
                ref = cand
                break
    if ref is None:
        raise SystemExit("no reference tree found; pass --ref")
    from flashnn_b200.workloads import make_moe_case, make_moe_w4_case  # before the reference shadows nothing of ours
    for name in [n for n in sys.modules if n == "flashnn" or n.startswith("flashnn.")]:
        del sys.modules[name]
    sys.path.insert(0, ref)
    from flashnn.triton_kernels.fused_moe_a8w8 import fused_moe_a8w8_forward
    from flashnn.triton_kernels.fused_moe_a16w4 import fused_moe_a16w4_forward
    import flashnn
    assert os.path.abspath(flashnn.__file__).startswith(os.path.abspath(ref))
    dev = torch.device("cuda", 0)
    os.makedirs(args.out, exist_ok=True)

    # ---------------- A8W8 ----------------
    a8 = {}
    #        m, e,  n,   k, top_k, mul,   out dtype,      scale dtype
    cases = [(5, 4, 64, 64, 2, True, torch.float16, torch.float32),
             (33, 8, 48, 128, 2, False, torch.float16, torch.float32),
             (40, 4, 128, 208, 1, True, torch.float16, torch.float16),
             (64, 8, 64, 96, 4, True, torch.bfloat16, torch.float32),
             (100, 6, 80, 512, 2, True, torch.bfloat16, torch.bfloat16),
             (1, 16, 32, 1024, 4, True, torch.float16, torch.float32)]
    for i, (m, e, n, k, top_k, mul, out_ty, sdt) in enumerate(cases):
        name = f"a8w8_{i}"
        bm = 32
        c = make_moe_case(m, e, n, k, top_k, bm, seed=100 + i, scale_dt=sdt)
        if i == 2:  # two slots in use that name no token (dropped by the router): padding values inside a block
            c["sorted_ids"][1] = m * top_k
            c["sorted_ids"][3] = m * top_k + 2
        d = {kk: v.to(dev) for kk, v in c.items()}
        out = torch.full((m, top_k, n), 7.0, dtype=out_ty, device=dev)
        rec = {"m": m, "e": e, "n": n, "k": k, "top_k": top_k, "bm": bm, "mul": int(mul),
               "out_dtype": str(out_ty).split(".")[-1], "scale_dtype": str(sdt).split(".")[-1]}
        for kk, v in c.items():
            rec[kk] = bits(v)
        try:
            fused_moe_a8w8_forward(d["a"], d["b"], out, d["alpha_row"], d["alpha_col"], d["topk_w"], d["topk_ids"],
                                   d["sorted_ids"], d["expert_ids"], d["npp"], mul, top_k, bm)
            torch.cuda.synchronize()
            rec["out"] = bits(out)
        except Exception as ex:  # recorded, not hidden
            rec["error"] = np.array(f"{type(ex).__name__}: {str(ex)[:500]}")
            print(name, "FAILED", rec["error"], file=sys.stderr)
        for kk, v in rec.items():
            a8[f"{name}/{kk}"] = np.asarray(v)
    np.savez_compressed(os.path.join(args.out, "fused_moe_a8w8.npz"), **a8)

    # ---------------- A16W4 ----------------
    w4 = {}
    #        m, e,  n,   k, top_k, bm, mul,  dtype,        group, zp
    cases = [(5, 4, 64, 128, 2, 16, True, torch.float16, 0, False),
             (33, 8, 96, 256, 2, 16, False, torch.float16, 0, True),
             (20, 4, 64, 256, 2, 32, True, torch.float16, 64, False),
             (48, 4, 128, 512, 2, 16, True, torch.float16, 128, True),
             (17, 8, 64, 256, 4, 16, True, torch.bfloat16, 0, False),
             (40, 4, 96, 256, 1, 64, True, torch.bfloat16, 128, False),
             (9, 4, 64, 128, 2, 16, False, torch.bfloat16, 64, True)]
    for i, (m, e, n, k, top_k, bm, mul, dt, group, use_zp) in enumerate(cases):
        name = f"a16w4_{i}"
        c = make_moe_w4_case(m, e, n, k, top_k, bm, seed=200 + i, dtype=dt, group=group, use_zp=use_zp)
        d = {kk: (None if v is None else v.to(dev)) for kk, v in c.items()}
        out = torch.full((m, top_k, n), 7.0, dtype=dt, device=dev)
        rec = {"m": m, "e": e, "n": n, "k": k, "top_k": top_k, "bm": bm, "mul": int(mul), "group": group,
               "dtype": str(dt).split(".")[-1]}
        for kk, v in c.items():
            if v is not None and kk != "w4":
                rec[kk] = bits(v)
        try:
            fused_moe_a16w4_forward(d["a"], d["b"], out, d["scale"], d["zp"], d["topk_w"], d["topk_ids"], d["sorted_ids"],
                                    d["expert_ids"], d["npp"], mul, top_k, bm)
            torch.cuda.synchronize()
            rec["out"] = bits(out)
        except Exception as ex:
            rec["error"] = np.array(f"{type(ex).__name__}: {str(ex)[:500]}")
            print(name, "FAILED", rec["error"], file=sys.stderr)
        for kk, v in rec.items():
            w4[f"{name}/{kk}"] = np.asarray(v)
    np.savez_compressed(os.path.join(args.out, "fused_moe_a16w4.npz"), **w4)
    print("wrote", os.path.join(args.out, "fused_moe_a8w8.npz"), "and fused_moe_a16w4.npz")


if __name__ == "__main__":
    main()
