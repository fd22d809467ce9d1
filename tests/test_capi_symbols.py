"""The C-ABI library loads without a GPU, exports every symbol that include/flashnn_b200.h declares, and rejects
bad arguments with the documented status codes before touching the device (host-side failure injection)."""
import ctypes
import os
import re

import pytest

from flashnn_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "flashnn_b200.h")


@pytest.fixture(scope="module")
def lib():
    from flashnn_b200 import build
    build.build()  # cross-compiles for sm_100a; needs nvcc, not a GPU
    return _lib.lib()


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fnn_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_functions()
    assert len(names) >= 9
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes signatures and header declarations differ"


def test_version_and_status_strings(lib):
    assert lib.fnn_version() == 100
    assert lib.fnn_status_string(0) == b"ok"
    assert lib.fnn_status_string(8) == b"device-side wait timed out"
    assert lib.fnn_status_string(1234) == b"unknown status"


def test_dynamic_quant_argument_errors(lib):
    f = lib.fnn_dynamic_quant
    assert f(None, _lib.BF16, 4, 8, 8, None, 8, None, None) == 1  # null pointers
    assert b"null" in lib.fnn_last_error_string()
    assert f(None, _lib.F32, 4, 8, 8, None, 8, None, None) == 2  # fp32 input is not accepted
    assert f(None, _lib.BF16, 4, 8, 4, None, 8, None, None) == 3  # ldx < K
    assert f(None, _lib.BF16, -1, 8, 8, None, 8, None, None) == 3
    assert f(None, _lib.BF16, 0, 8, 8, None, 8, None, None) == 0  # empty input: nothing to do
    with pytest.raises(_lib.FlashNNError) as e:
        _lib.check(f(None, 7, 4, 8, 8, None, 8, None, None))
    assert e.value.status == 2 and "dtype" in str(e.value)


def test_gemm_a8w8_argument_errors(lib):
    f = lib.fnn_gemm_a8w8
    args = dict(a=None, lda=64, b=None, ldb=64, row=None, rdt=_lib.F32, col=None, cdt=_lib.F32, out=None,
                odt=_lib.BF16, ldo=32, M=16, N=32, K=64, acc=None, ldacc=0, ws=None, wsb=0, st=None)

    def call(**kw):
        v = dict(args, **kw)
        return f(v["a"], v["lda"], v["b"], v["ldb"], v["row"], v["rdt"], v["col"], v["cdt"], v["out"], v["odt"],
                 v["ldo"], v["M"], v["N"], v["K"], v["acc"], v["ldacc"], v["ws"], v["wsb"], v["st"])

    assert call() == 1                      # null tensors
    assert call(odt=_lib.F32) == 2          # fp32 output is not accepted
    assert call(rdt=5) == 2
    assert call(lda=32) == 3                # lda < K
    assert call(ldo=8) == 3                 # ldo < N
    assert call(M=0) == 0 and call(N=0) == 0
    # scratch only where the K-balanced mode of the CTA-pair kernel is planned: 8192^3 fills its rounds of CTA pairs,
    # 4096 x 2048 x 28672 (128 tiles on 74 pairs) does not; 16 KB of flags and two 256 x 256 int32 slots per pair of the 148 SMs
    assert lib.fnn_gemm_a8w8_workspace_bytes(8192, 8192, 8192) == 0
    assert lib.fnn_gemm_a8w8_workspace_bytes(16, 4096, 4096) == 0
    assert lib.fnn_gemm_a8w8_workspace_bytes(4096, 2048, 28672) == 16384 + 148 * 256 * 256 * 4


def test_gemm_weight_only_argument_errors(lib):
    f = lib.fnn_gemm_weight_only

    def call(bits=4, M=2, N=64, K=256, group=128, adt=_lib.BF16, odt=_lib.BF16, sdt=_lib.BF16, lda=256, ldo=64):
        return f(None, adt, lda, None, bits, None, None, sdt, group, None, 0, None, odt, ldo, M, N, K, None, 0, None)

    assert call() == 1
    assert call(bits=3) == 5                # only 4 and 8 bit weights exist
    assert call(N=63) == 3                  # packed int4 needs an even N
    assert call(group=100) == 3             # K not a multiple of the group
    assert call(adt=_lib.F32) == 2
    assert call(odt=_lib.F16) == 2          # output dtype must equal the activation dtype
    assert call(lda=128) == 3
    assert call(M=0) == 0
    assert lib.fnn_gemm_weight_only_workspace_bytes(1, 28672, 8192, 4, 128) == 0


def test_device_status_needs_an_output_pointer(lib):
    assert lib.fnn_device_status(None) == 1


def test_fused_moe_a16w4_workspace_and_argument_errors(lib):
    # scratch only for blocks of 256 slots (the prefill kernels): the expert-sorted 16-bit copy of the token rows,
    # plus their row sums per scale group when zero-points are given
    ws = lib.fnn_fused_moe_a16w4_workspace_bytes
    assert ws(4096, 4096, 128, 0, 64) == 0 and ws(4096, 4096, 128, 0, 128) == 0
    assert ws(4096, 4096, 128, 0, 256) == 4096 * 4096 * 2
    assert ws(4096, 4096, 128, 1, 256) == 4096 * 4096 * 2 + 4096 * 4 * 32
    assert ws(4096, 4096, 0, 1, 512) == 4096 * 4096 * 2 + 4096 * 4
    f = lib.fnn_fused_moe_a16w4_ws

    def call(N=64, K=128, EM=256, bm=256, group=0, adt=_lib.BF16, odt=_lib.BF16, top_k=2):
        return f(None, adt, K, None, 4, N, K, None, None, _lib.BF16, group, None, _lib.F32, None, EM, None, None, 64, top_k, bm, 1,
                 None, odt, N, None, 0, None)

    assert call() == 1                # null tensors
    assert call(N=63) == 3            # packed int4 needs an even N
    assert call(EM=200) == 3          # slots not a multiple of block_m
    assert call(bm=100, EM=200) == 5  # block size
    assert call(group=96) == 5        # group size
    assert call(odt=_lib.F16) == 2    # output dtype must equal the token dtype
