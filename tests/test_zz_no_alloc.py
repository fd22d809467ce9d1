"""fnn_gemm_weight_only_prefill_static: the entry point for callers that cannot hand the library any device
memory (a plugin in a process that owns all allocations, a server with a fixed pool).  It must give what
fnn_gemm_weight_only gives with a caller workspace, on repeated calls that share the built-in scratch, and both
must stay inside the weight-only bound against the CPU oracle's fp32 dequant-matmul."""
import pytest
import torch

from flashnn_b200 import _lib

RTOL, ATOL = 1e-2, 1e-3  # the bound the weight-only tests use


def test_rows_beyond_the_built_in_scratch_are_refused():
    # checked before any CUDA call, so this needs no GPU
    L = _lib.lib()
    st = L.fnn_gemm_weight_only_prefill_static(None, _lib.BF16, 64, None, 8, None, None, _lib.BF16, None, 0,
                                               None, _lib.BF16, 64, 65537, 64, 64, None)
    assert st == 6 and b"65536" in L.fnn_last_error_string()
    assert L.fnn_gemm_weight_only_prefill_static(None, _lib.BF16, 64, None, 8, None, None, _lib.BF16, None, 0,
                                                 None, _lib.BF16, 64, 128, 64, 64, None) == 1  # null tensors


def _problem(m, n, k, bits, dt, seed, use_zp=True):
    g = torch.Generator().manual_seed(seed)
    act = torch.randn(m, k, generator=g).to(dt)
    if bits == 8:
        qw = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8)
    else:
        w = torch.randint(-8, 8, (n, k), generator=g, dtype=torch.int8).to(torch.int16) & 0xF
        qw = (w[0::2] | (w[1::2] << 4)).to(torch.uint8).view(torch.int8)
    scale = (torch.rand(n, generator=g) * 0.045 + 0.005).to(dt)
    zp = torch.randint(-3, 4, (n,), generator=g).to(dt) if use_zp else None
    bias = torch.randn(n, generator=g).to(dt)
    return act, qw, scale, zp, bias


def _ptr(t):
    return None if t is None else t.data_ptr()


def _call_both(m, n, k, bits, dt, seed, use_zp=True):
    from oracle import quant_oracle as O
    L = _lib.lib()
    code = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}[dt]
    host = _problem(m, n, k, bits, dt, seed, use_zp)
    act, qw, scale, zp, bias = [None if t is None else t.cuda() for t in host]
    stream = torch.cuda.current_stream().cuda_stream
    # existing entry point, scratch handed in by the caller
    ws_bytes = L.fnn_gemm_weight_only_workspace_bytes(m, n, k, bits, 0)
    ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device="cuda")
    ref = torch.empty(m, n, dtype=dt, device="cuda")
    _lib.check(L.fnn_gemm_weight_only(act.data_ptr(), code, k, qw.data_ptr(), bits, scale.data_ptr(), _ptr(zp), code, 0,
                                      bias.data_ptr(), code, ref.data_ptr(), code, n, m, n, k, ws.data_ptr(), ws_bytes, stream))
    # new entry point: inputs and outputs only
    out = torch.full((m, n), float("nan"), dtype=dt, device="cuda")
    _lib.check(L.fnn_gemm_weight_only_prefill_static(act.data_ptr(), code, k, qw.data_ptr(), bits, scale.data_ptr(),
                                                     _ptr(zp), code, bias.data_ptr(), code, out.data_ptr(), code, n,
                                                     m, n, k, stream))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    oracle = O.gemm_weight_only_fp32(host[0], host[1], host[2], host[4], host[3])
    return out.float().cpu(), ref.float().cpu(), oracle


@pytest.mark.gpu
def test_matches_the_workspace_entry_point_and_the_oracle_on_consecutive_calls():
    # calls in a row on the shared scratch: sizes and data change from call to call, so anything an earlier call
    # left behind in the array would show up as a wrong zero-point term.  Covered besides: a call without
    # zero-points (the scratch is not touched) and one with fewer than 17 rows.
    for m, n, k, bits, dt, seed, use_zp in [(300, 520, 1024, 8, torch.bfloat16, 1, True), (130, 264, 528, 4, torch.float16, 2, True),
                                            (300, 520, 1024, 8, torch.bfloat16, 3, True), (200, 256, 512, 4, torch.bfloat16, 4, False),
                                            (9, 128, 1024, 8, torch.float16, 5, True)]:
        out, ref, oracle = _call_both(m, n, k, bits, dt, seed, use_zp)
        assert not torch.isnan(out).any()
        assert bool(((out - oracle).abs() <= ATOL + RTOL * oracle.abs()).all()), "static entry point outside the oracle's bound"
        assert bool(((ref - oracle).abs() <= ATOL + RTOL * oracle.abs()).all())
        if m > 16:  # above 16 rows both entry points run the same kernel: identical bits
            assert torch.equal(out, ref)
        else:       # below, the workspace entry point takes a decode kernel: same bound, other rounding order
            assert bool(((out - ref).abs() <= ATOL + RTOL * ref.abs()).all())


@pytest.mark.gpu
def test_misaligned_operands_are_refused():
    L = _lib.lib()
    act, qw, scale, zp, bias = [t.cuda() for t in _problem(64, 128, 264, 8, torch.bfloat16, 7)]
    out = torch.empty(64, 128, dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    # K = 264 is not a multiple of 16, and a row pitch of 260 elements would break the 16-byte rule as well
    st = L.fnn_gemm_weight_only_prefill_static(act.data_ptr(), _lib.BF16, 264, qw.data_ptr(), 8, scale.data_ptr(), zp.data_ptr(),
                                               _lib.BF16, bias.data_ptr(), _lib.BF16, out.data_ptr(), _lib.BF16, 128, 64, 128, 264, stream)
    assert st == 4 and b"aligned" in L.fnn_last_error_string()
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
