"""Host-side behaviour of the operator classes that needs no GPU: the reference's names are importable, the backend
switches exist, and nothing falls back to a CPU computation."""
import pytest
import torch


def test_reference_names_are_importable():
    import flashnn
    from flashnn import DynamicQuantize, GemmA8W8, GemmWeightOnly, set_use_triton  # noqa: F401
    import flashnn_b200
    assert flashnn.GemmA8W8 is flashnn_b200.GemmA8W8
    assert isinstance(flashnn.DynamicQuantize(), torch.nn.Module)
    assert flashnn.GemmA8W8().out_ty == torch.float16 and flashnn.GemmWeightOnly().out_ty == torch.float16
    assert flashnn.GemmA8W8(torch.bfloat16).out_ty == torch.bfloat16


def test_cpu_tensors_are_rejected_not_computed():
    import flashnn_b200
    x = torch.randn(4, 64).half()
    with pytest.raises(RuntimeError, match="no CPU path"):
        flashnn_b200.DynamicQuantize()(x)
    a = torch.zeros(4, 64, dtype=torch.int8)
    with pytest.raises(RuntimeError, match="no CPU path"):
        flashnn_b200.GemmA8W8()(a, a, torch.ones(4), torch.ones(4))
    with pytest.raises(RuntimeError, match="no CPU path"):
        flashnn_b200.GemmWeightOnly()(x, a, torch.ones(4).half())


def test_selecting_the_torch_backend_raises():
    import flashnn_b200
    from flashnn_b200 import kernel_backend as kb
    assert kb.get_use_triton() is True
    flashnn_b200.set_use_triton(False)
    try:
        with pytest.raises(ValueError, match="No valid backend found"):
            flashnn_b200.DynamicQuantize()(torch.randn(2, 8).half())
    finally:
        flashnn_b200.set_use_triton(True)
    flashnn_b200.set_autotune_triton_kernels(True)  # accepted, has no effect on these operators
    assert kb.get_autotune_triton_kernels() is True
    flashnn_b200.set_autotune_triton_kernels(False)


def test_package_does_not_import_the_oracle():
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dirpath, _, files in os.walk(os.path.join(root, "flashnn_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.replace("the oracle", ""), f"{f} refers to the oracle package"


def test_workload_byte_and_op_counts():
    from flashnn_b200 import workloads as W
    assert W.a8w8_ops(8192, 8192, 8192) == 2 * 8192 ** 3
    assert W.a8w8_bytes(16, 4096, 4096) == 16990272
    assert W.dynamic_quant_bytes(4096, 4096) == 50339840
    assert W.a16w4_bytes(1, 28672, 8192, 128) == 121184256
    assert W.a16w4_bytes(4, 28672, 8192, 128) == 121405440 and W.a16w4_bytes(16, 28672, 8192, 128) == 122290176


def test_norm_and_moe_entry_points_reject_cpu_tensors():
    import flashnn
    import flashnn_b200
    assert flashnn.RMSNormDquant is flashnn_b200.RMSNormDquant and flashnn.LayernormDquant is flashnn_b200.LayernormDquant
    assert flashnn.fused_moe_a8w8_forward is flashnn_b200.fused_moe_a8w8_forward
    rms, ln = flashnn_b200.RMSNormDquant(64, 1e-5), flashnn_b200.LayernormDquant((64,), 1e-5)
    assert rms.weight.shape == (64,) and ln.weight.shape == (64,) and ln.bias.shape == (64,) and ln.dim == (64,)
    x = torch.randn(4, 64).half()
    with pytest.raises(RuntimeError, match="no CPU path"):
        rms(x)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ln(x)
    a = torch.zeros(4, 64, dtype=torch.int8)
    b = torch.zeros(2, 16, 64, dtype=torch.int8)
    c = torch.zeros(4, 1, 16, dtype=torch.float16)
    ids = torch.zeros(16, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="no CPU path"):
        flashnn_b200.fused_moe_a8w8_forward(a, b, c, torch.ones(4), torch.ones(2, 16), torch.ones(4, 1), torch.zeros(4, 1, dtype=torch.int32),
                                            ids, torch.zeros(1, dtype=torch.int32), torch.tensor([16], dtype=torch.int32), True, 1, 16)


def test_options_round_trip_without_a_gpu():
    from flashnn_b200 import _lib
    assert _lib.lib().fnn_get_option(_lib.OPT_STATIC_WEIGHTS) == 0
    _lib.set_option(_lib.OPT_STATIC_WEIGHTS, 1)
    assert _lib.lib().fnn_get_option(_lib.OPT_STATIC_WEIGHTS) == 1
    _lib.set_option(_lib.OPT_STATIC_WEIGHTS, 0)
    assert _lib.lib().fnn_get_option(12345) == -1
    with pytest.raises(_lib.FlashNNError):
        _lib.set_option(12345, 1)


def test_a8w8_shape_to_tile_plan():
    """The shape -> kernel / tile table (needs no GPU: 148 SMs are assumed without a device).  The cases are the ones
    the plan was introduced for: shards of the FFN layer over 8 GPUs, the headline shape, decode shapes."""
    import torch
    from flashnn_b200 import _lib
    if torch.cuda.is_available() and torch.cuda.get_device_properties(0).multi_processor_count != 148:
        pytest.skip("the expected tiles are for 148 SMs")
    assert _lib.a8w8_plan(8192, 8192, 8192) == (1, 256)
    assert _lib.a8w8_plan(4096, 57344, 8192) == (1, 256)
    assert _lib.a8w8_plan(4096, 7168, 8192) == (1, 224)     # 512 tiles = 6.92 waves instead of 448 = 6.05 -> 7
    assert _lib.a8w8_plan(4096, 1024, 28672) == (1, 256)    # 64 pair tiles in one wave, not 256 single-CTA tiles
    assert _lib.a8w8_plan(4096, 2048, 28672) == (3, 256)    # 128 tiles = 1.73 rounds: the ragged round's K blocks are shared
    assert _lib.a8w8_plan(4096, 4096, 28672) == (3, 256)    # 256 tiles = 3.46 rounds
    assert _lib.a8w8_plan(764, 8192, 8192) == (1, 192)      # the hand-over would cost what the even split gains
    assert _lib.a8w8_plan(4096, 4096, 4096)[0] == 1         # short K: the extra epilogues would not hide behind the MMAs
    _lib.set_option(_lib.OPT_A8W8_BALANCED, 2)
    try:
        assert _lib.a8w8_plan(4096, 2048, 28672) == (1, 256)  # whole tiles: two rounds
    finally:
        _lib.set_option(_lib.OPT_A8W8_BALANCED, 0)
    assert _lib.a8w8_plan(256, 512, 4096) == (0, 64)        # too small for the pair kernel to fill the GPU
    assert _lib.a8w8_plan(64, 57344, 8192) == (0, 256)      # decode: the widest tile that still gives every SM work
    assert _lib.a8w8_plan(16, 4096, 4096) == (0, 64)
    assert _lib.a8w8_plan(1, 57344, 8192) == (2, 16)
    with pytest.raises(_lib.FlashNNError):
        _lib.a8w8_plan(0, 16, 16)
