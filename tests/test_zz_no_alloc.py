"""fnn_gemm_weight_only_prefill_static: the entry point for callers that cannot hand the library any device
memory (a plugin in a process that owns all allocations, a server with a fixed pool).  It must give what
fnn_gemm_weight_only gives with a caller workspace, on repeated calls that share the built-in scratch."""
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


def _problem(m, n, k, bits, dt, seed):
    g = torch.Generator().manual_seed(seed)
    act = torch.randn(m, k, generator=g).to(dt)
    if bits == 8:
        qw = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8)
    else:
        w = torch.randint(-8, 8, (n, k), generator=g, dtype=torch.int8).to(torch.int16) & 0xF
        qw = (w[0::2] | (w[1::2] << 4)).to(torch.uint8).view(torch.int8)
    scale = (torch.rand(n, generator=g) * 0.045 + 0.005).to(dt)
    zp = torch.randint(-3, 4, (n,), generator=g).to(dt)
    bias = torch.randn(n, generator=g).to(dt)
    return [t.cuda() for t in (act, qw, scale, zp, bias)]


def _call_both(m, n, k, bits, dt, seed):
    L = _lib.lib()
    code = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}[dt]
    act, qw, scale, zp, bias = _problem(m, n, k, bits, dt, seed)
    stream = torch.cuda.current_stream().cuda_stream
    # existing entry point, scratch handed in by the caller
    ws_bytes = L.fnn_gemm_weight_only_workspace_bytes(m, n, k, bits, 0)
    ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device="cuda")
    ref = torch.empty(m, n, dtype=dt, device="cuda")
    _lib.check(L.fnn_gemm_weight_only(act.data_ptr(), code, k, qw.data_ptr(), bits, scale.data_ptr(), zp.data_ptr(), code, 0,
                                      bias.data_ptr(), code, ref.data_ptr(), code, n, m, n, k, ws.data_ptr(), ws_bytes, stream))
    # new entry point: inputs and outputs only
    out = torch.full((m, n), float("nan"), dtype=dt, device="cuda")
    _lib.check(L.fnn_gemm_weight_only_prefill_static(act.data_ptr(), code, k, qw.data_ptr(), bits, scale.data_ptr(),
                                                     zp.data_ptr(), code, bias.data_ptr(), code, out.data_ptr(), code, n,
                                                     m, n, k, stream))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    return out.float().cpu(), ref.float().cpu()


@pytest.mark.gpu
def test_matches_the_workspace_entry_point_on_consecutive_calls():
    # two calls in a row on the shared scratch: the second is smaller and carries different data, so anything the
    # first call left behind in the array would show up as a wrong zero-point term
    for m, n, k, bits, dt, seed in [(300, 520, 1024, 8, torch.bfloat16, 1), (130, 264, 528, 4, torch.float16, 2),
                                    (300, 520, 1024, 8, torch.bfloat16, 3)]:
        out, ref = _call_both(m, n, k, bits, dt, seed)
        assert not torch.isnan(out).any()
        assert bool(((out - ref).abs() <= ATOL + RTOL * ref.abs()).all())
