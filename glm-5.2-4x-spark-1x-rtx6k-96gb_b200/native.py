"""ctypes binding of libglmrt_b200.so.

Host-side mirror of the reference's FFI crate (rust/crates/glmrt-ffi/src/lib.rs:
``NativeLibrary`` dlopens the library named by ``GLMRT_NATIVE_LIB``, resolves symbols
by name and turns every non-OK ``glmrt_status_t`` into an error that carries
``glmrt_last_error``), written with ctypes as the reference's own Python tools do
(python/tools/bench_b12x_spark_w4a16_native.py:34-112).

There is no fallback: if the shared library is missing or a symbol cannot be
resolved, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_LIB = os.path.join(HERE, "libglmrt_b200.so")
HEADER = os.path.join(os.path.dirname(HERE), "include", "glmrt_b200.h")

STATUS_NAMES = {
    0: "OK", 1: "INVALID_ARGUMENT", 2: "BUFFER_TOO_SMALL", 3: "CUDA_UNAVAILABLE",
    4: "ALLOCATION_FAILED", 5: "COPY_FAILED", 6: "INTERNAL_ERROR", 7: "RDMA_UNAVAILABLE",
    8: "NCCL_UNAVAILABLE",
}


class GlmrtError(RuntimeError):
    """A native call returned a non-OK status (mirrors the FFI crate's status -> anyhow error)."""

    def __init__(self, symbol: str, status: int, message: str):
        self.symbol, self.status, self.message = symbol, status, message
        super().__init__(f"{symbol} failed: {STATUS_NAMES.get(status, status)}: {message}")


class DeviceBuffer(C.Structure):
    """glmrt_device_buffer_t (native/include/glmrt_native.h:77-82)."""
    _fields_ = [("ptr", C.c_void_p), ("bytes", C.c_size_t), ("device_id", C.c_int), ("flags", C.c_uint64)]

    @staticmethod
    def of(ptr: int, nbytes: int, device: int = 0) -> "DeviceBuffer":
        return DeviceBuffer(C.c_void_p(ptr), nbytes, device, 0)

    @staticmethod
    def null() -> "DeviceBuffer":
        return DeviceBuffer(None, 0, 0, 0)


class DeviceInfo(C.Structure):
    _fields_ = [("device_id", C.c_int), ("cuda_available", C.c_int), ("compute_capability_major", C.c_int),
                ("compute_capability_minor", C.c_int), ("integrated", C.c_int), ("can_map_host_memory", C.c_int),
                ("unified_addressing", C.c_int), ("total_memory_bytes", C.c_uint64), ("name", C.c_char * 128),
                ("driver_version", C.c_char * 64), ("runtime_version", C.c_char * 64)]


class MoeConfig(C.Structure):
    """glmrt_b200_moe_config_t."""
    _fields_ = [("hidden_dim", C.c_uint32), ("intermediate_dim", C.c_uint32), ("experts", C.c_uint32),
                ("top_k", C.c_uint32), ("max_tokens", C.c_uint32), ("ep_world", C.c_uint32),
                ("ep_rank", C.c_uint32), ("flags", C.c_uint32), ("routed_scaling", C.c_float)]


class LayerStats(C.Structure):
    _fields_ = [("launches_total", C.c_uint64), ("launches_last_forward", C.c_uint32), ("chunks", C.c_uint32),
                ("slots", C.c_uint32), ("distinct_experts", C.c_uint32), ("device_error", C.c_uint32),
                ("reserved", C.c_uint32)]


LAYER_ORDERED_COMBINE = 8
LAYER_ENGINE_SIMT = 1
LAYER_PAIR_FC1 = 2
LAYER_PAIR_FC2 = 4
LAYER_PAIR_TILES = 6
FP4_RULE_RNE_PAYLOAD = 0
FP4_RULE_NEAREST_LOW = 1

DEBUG = {name: i for i, name in enumerate(
    ["PAYLOAD", "ROUTE_SLOT", "ACT1_CODES", "ACT1_SF", "ACT2_CODES", "ACT2_SF", "ROUTE_ROWS", "COUNTERS",
     "CHUNKS", "EXPERT_COUNTS", "GATE_CODES", "UP_CODES", "DOWN_CODES", "GATE_SF", "UP_SF", "DOWN_SF",
     "SCALE2", "TOPK_IDX", "TOPK_W"])}


class RouteBatchedMetadata(C.Structure):
    """glmrt_nvfp4_route_batched_metadata_t (native/include/glmrt_native.h:114-127)."""
    _fields_ = [("gate_weight", C.c_size_t), ("gate_scale", C.c_size_t), ("up_weight", C.c_size_t),
                ("up_scale", C.c_size_t), ("down_weight", C.c_size_t), ("down_scale", C.c_size_t),
                ("intermediate", C.c_size_t), ("down_weight_row_stride_bytes", C.c_size_t),
                ("down_scale_row_stride_bytes", C.c_size_t), ("gate_scale_2", C.c_float), ("up_scale_2", C.c_float),
                ("down_scale_2", C.c_float)]


class RouteShardReductionBuffers(C.Structure):
    """glmrt_route_shard_reduction_buffers_t (native/include/glmrt_native.h:101-105)."""
    _fields_ = [("local", DeviceBuffer), ("peers", DeviceBuffer * 3), ("output_f32", DeviceBuffer)]


def declared_symbols(header_path: str = HEADER) -> list[str]:
    """Every function name declared in include/glmrt_b200.h."""
    text = open(header_path).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"glmrt_status_t\s+(glmrt_\w+)\s*\(", text)))


class NativeLibrary:
    """Loads the shared library and exposes checked calls: ``lib.call("symbol", *args)``."""

    def __init__(self, path: str | None = None):
        self.path = path or os.environ.get("GLMRT_NATIVE_LIB") or DEFAULT_LIB
        if not os.path.exists(self.path):
            raise FileNotFoundError(
                f"{self.path} not found: build it with `python {os.path.join(HERE, 'build.py')}` "
                "(there is no CPU fallback)")
        self.lib = C.CDLL(self.path)
        self._fn = {}

    def symbol(self, name: str):
        fn = self._fn.get(name)
        if fn is None:
            fn = getattr(self.lib, name)  # AttributeError when the symbol is missing
            fn.restype = C.c_int
            self._fn[name] = fn
        return fn

    def last_error(self) -> str:
        buf = C.create_string_buffer(1024)
        self.symbol("glmrt_last_error")(buf, C.c_size_t(len(buf)))
        return buf.value.decode("utf-8", "replace")

    def call_status(self, name: str, *args) -> int:
        return int(self.symbol(name)(*args))

    def call(self, name: str, *args) -> None:
        st = self.call_status(name, *args)
        if st != 0:
            raise GlmrtError(name, st, self.last_error())

    def version(self) -> str:
        buf = C.create_string_buffer(256)
        self.call("glmrt_native_version", buf, C.c_size_t(len(buf)))
        return buf.value.decode()


_LIB: NativeLibrary | None = None


def library() -> NativeLibrary:
    global _LIB
    if _LIB is None:
        _LIB = NativeLibrary()
    return _LIB
