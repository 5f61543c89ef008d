"""C-ABI checks that need no GPU: the library loads, exports every declared symbol, and
validates arguments / reports CUDA_UNAVAILABLE without launching anything.

Modelled on the reference's native CPU self-test (native/tests/native_selftest.cc:10-112:
version string, error propagation through glmrt_last_error, clean *_UNAVAILABLE statuses).
"""
import ctypes as C
import os

import pytest
import torch

HAS_GPU = torch.cuda.is_available()


@pytest.fixture(scope="module")
def lib(pkg):
    from glmrt_b200 import native as N
    path = N.DEFAULT_LIB
    if not os.path.exists(path):
        import importlib.util
        spec = importlib.util.spec_from_file_location("_b", os.path.join(N.HERE, "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
    return N.NativeLibrary(path)


def test_every_declared_symbol_is_exported(lib, pkg):
    from glmrt_b200 import native as N
    names = N.declared_symbols()
    assert len(names) >= 40
    missing = [n for n in names if not hasattr(lib.lib, n)]
    assert missing == []


def test_version_and_last_error(lib):
    assert "glmrt-b200" in lib.version()
    small = C.create_string_buffer(4)
    assert lib.call_status("glmrt_native_version", small, C.c_size_t(4)) == 2  # BUFFER_TOO_SMALL
    assert lib.call_status("glmrt_native_version", None, C.c_size_t(4)) == 1
    assert "null" in lib.last_error()


def test_invalid_arguments_are_rejected_before_any_launch(lib, pkg):
    from glmrt_b200 import native as N
    null = N.DeviceBuffer.null()
    # router: null pointers, zero rows, top_k > experts (router.cu:259-281 rules)
    assert lib.call_status("glmrt_cuda_router_topk_bf16_async", None, None, None, None, None, None,
                           C.c_size_t(1), C.c_size_t(16), C.c_size_t(4), C.c_size_t(2), None) == 1
    one = C.c_void_p(16)
    assert lib.call_status("glmrt_cuda_router_topk_f32_async", one, one, one, one, one, one,
                           C.c_size_t(0), C.c_size_t(16), C.c_size_t(4), C.c_size_t(2), None) == 1
    assert lib.call_status("glmrt_cuda_router_topk_f32_async", one, one, one, one, one, one,
                           C.c_size_t(1), C.c_size_t(16), C.c_size_t(4), C.c_size_t(5), None) == 1
    # payload quantiser: hidden_dim not a multiple of 16, too-small buffers
    buf = N.DeviceBuffer.of(4096, 64)
    assert lib.call_status("glmrt_cuda_b12x_quantize_bf16_nvfp4_row_payload_async", buf, buf,
                           C.c_size_t(1), C.c_size_t(24), None) == 1
    assert lib.call_status("glmrt_cuda_b12x_quantize_bf16_nvfp4_row_payload_async", buf, buf,
                           C.c_size_t(8), C.c_size_t(64), None) == 2
    assert "too small" in lib.last_error()
    assert lib.call_status("glmrt_cuda_b12x_quantize_bf16_nvfp4_row_payload_async", null, buf,
                           C.c_size_t(1), C.c_size_t(16), None) == 1
    # layer create: bad shapes
    out = C.c_void_p()
    for cfg in (N.MoeConfig(100, 256, 16, 4, 8, 1, 0, 0, 2.5), N.MoeConfig(256, 256, 16, 32, 8, 1, 0, 0, 2.5),
                N.MoeConfig(256, 256, 16, 4, 0, 1, 0, 0, 2.5), N.MoeConfig(256, 256, 16, 4, 8, 2, 2, 0, 2.5)):
        assert lib.call_status("glmrt_b200_moe_layer_create", C.byref(cfg), C.byref(out)) == 1
    assert lib.call_status("glmrt_b200_moe_layer_destroy", None) == 1
    assert lib.call_status("glmrt_cuda_event_elapsed_ms", None, None, None) == 1


@pytest.mark.skipif(HAS_GPU, reason="checks the no-device behaviour")
def test_without_a_device_compute_calls_report_cuda_unavailable(lib, pkg):
    from glmrt_b200 import native as N
    b = N.DeviceBuffer()
    assert lib.call_status("glmrt_alloc_device_buffer", C.c_size_t(1024), C.byref(b)) == 3
    assert "CUDA" in lib.last_error()
    out = C.c_void_p()
    cfg = N.MoeConfig(256, 256, 16, 4, 8, 1, 0, 0, 2.5)
    assert lib.call_status("glmrt_b200_moe_layer_create", C.byref(cfg), C.byref(out)) == 3
    info = N.DeviceInfo()
    assert lib.call_status("glmrt_cuda_device_info", C.c_int(0), C.byref(info)) == 3
    buf = N.DeviceBuffer.of(4096, 1 << 20)
    assert lib.call_status("glmrt_cuda_b12x_quantize_bf16_nvfp4_row_payload_async", buf, buf,
                           C.c_size_t(1), C.c_size_t(64), None) == 3


def test_missing_library_fails_loudly(pkg):
    from glmrt_b200 import native as N
    with pytest.raises(FileNotFoundError):
        N.NativeLibrary("/nonexistent/libglmrt_b200.so")


def test_nccl_wrappers_validate_or_report_unavailable(lib, pkg):
    """native/tests/native_selftest.cc checks that the NCCL ABI answers cleanly without NCCL; here the
    library is resolved at run time, so either answer is legal: NCCL_UNAVAILABLE (8) everywhere, or
    the reference's argument validation."""
    n = C.c_size_t(0)
    st = lib.call_status("glmrt_nccl_unique_id_bytes", C.byref(n))
    assert st in (0, 8)
    assert lib.call_status("glmrt_nccl_unique_id_bytes", None) == 1
    if st == 8:
        assert n.value == 0 and "NCCL" in lib.last_error()
        out = C.c_void_p()
        assert lib.call_status("glmrt_nccl_comm_init_rank", None, C.c_size_t(0), C.c_int(1), C.c_int(0), C.byref(out)) == 8
    else:
        assert n.value == 128
        buf = C.create_string_buffer(64)
        assert lib.call_status("glmrt_nccl_get_unique_id", buf, C.c_size_t(64)) == 1      # wrong size
        out = C.c_void_p()
        assert lib.call_status("glmrt_nccl_comm_init_rank", None, C.c_size_t(128), C.c_int(1), C.c_int(0), C.byref(out)) == 1
        from glmrt_b200 import native as N
        nb = N.DeviceBuffer.null()
        assert lib.call_status("glmrt_nccl_all_reduce_bf16_async", None, nb, nb, C.c_size_t(4), None) == 1


def test_protocol_codec_validates_its_arguments(lib, pkg):
    """The ExpertProtocolV2 codec is host code: it must answer without a GPU, reject null pointers
    and report the size it needs when the output buffer is too small."""
    from glmrt_b200 import protocol_v2 as P
    n = C.c_size_t()
    assert lib.call_status("glmrt_b200_pv2_row_bytes", C.c_uint32(1), C.c_size_t(8), None) == 1
    assert lib.call_status("glmrt_b200_pv2_row_bytes", C.c_uint32(9), C.c_size_t(8), C.byref(n)) == 1
    assert "unknown dtype" in lib.last_error()
    assert lib.call_status("glmrt_b200_pv2_parse_request", None, C.c_size_t(0), None, None) == 1
    assert lib.call_status("glmrt_b200_pv2_compact_id", None, None) == 1
    req = P.ExpertProtocolV2Request(1, 1, 0, 32, P.ExpertV2Dtype.Bf16,
                                    [P.ExpertProtocolV2RowDescriptor(0, P.ExpertV2SourceKind.Decode, 0, 0, 0, 0)], [],
                                    b"\0" * 64)
    frame = req.encode(lib)
    assert len(frame) == 96 + 40 + 64
    h = P._RequestHeader()
    h.request_id, h.hidden_dim, h.hidden_dtype = 1, 32, 1
    row = P._Row(0, 0, 0, 0, 0, 1, 0)
    small = C.create_string_buffer(16)
    st = lib.call_status("glmrt_b200_pv2_encode_request", C.byref(h), C.byref(row), C.c_size_t(1), None, C.c_size_t(0),
                         b"\0" * 64, C.c_size_t(64), small, C.c_size_t(16), C.byref(n))
    assert st == 2 and n.value == len(frame)
    # the executor refuses a null layer before it looks at the frame
    assert lib.call_status("glmrt_b200_pv2_execute", None, frame, C.c_size_t(len(frame)), small, C.c_size_t(16),
                           C.byref(n), None) == 1


def test_row_scaled_fp8_packers_refuse_a_misaligned_destination(lib, pkg):
    """The row-scaled FP8 packers store each row's float32 scale behind the row's bytes: the
    destination itself must be 4-byte aligned like the width and the stride, or the store would
    fault on the device.  Checked before any CUDA call, so it answers without a GPU."""
    aligned, odd = C.c_void_p(4096), C.c_void_p(4098)
    for sym, extra in (("glmrt_cuda_bf16_rows_to_fp8_e4m3_row_scaled_async", ()),
                       ("glmrt_cuda_gather_rows_f32_to_fp8_e4m3_row_scaled_async", (C.c_void_p(8192),))):
        args = (C.c_size_t(2), C.c_size_t(64), C.c_size_t(68), None)
        assert lib.call_status(sym, aligned, *extra, odd, *args) == 1
        assert "4-byte aligned" in lib.last_error()
    # lanes and stacked layers validate their arguments without a device as well
    out = C.c_void_p()
    assert lib.call_status("glmrt_b200_moe_layer_create_lane", None, C.c_uint32(0), C.byref(out)) == 1
    assert lib.call_status("glmrt_b200_moe_layer_create_stacked", None, None, C.byref(out)) == 1
