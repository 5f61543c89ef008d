"""Host mirror of the reference's ExpertProtocolV2 types and executor contract, over the C codec.

Names follow rust/crates/glmrt-transport/src/protocol_v2.rs (request / response structs
:236-310, dtypes :44-83, flags :16-31) and the plugin trait ``ProtocolV2ExpertExecutor``
(glmrt-transport/src/synthetic.rs:51-107).  Every byte is produced and checked by the C
functions ``glmrt_b200_pv2_*`` of the shared library; this module only carries the values.
"""
from __future__ import annotations

import ctypes as C
import enum
import struct
from dataclasses import dataclass, field

from . import native as N

EXPERT_PROTOCOL_V2_REQUEST_HEADER_LEN = 96
EXPERT_PROTOCOL_V2_RESPONSE_HEADER_LEN = 96
EXPERT_PROTOCOL_V2_REQUEST_DEBUG_HEADER_LEN = 128
EXPERT_PROTOCOL_V2_ROW_DESCRIPTOR_LEN = 40
EXPERT_PROTOCOL_V2_ROUTE_ENTRY_LEN = 10
EXPERT_PROTOCOL_V2_FLAG_DEBUG_CHECKSUM = 1 << 0
EXPERT_PROTOCOL_V2_FLAG_PRECOMPILE_WARMUP = 1 << 1
EXPERT_PROTOCOL_V2_FLAG_RESPONSE_ROW_INDICES = 1 << 2
EXPERT_PROTOCOL_V2_FLAG_RESPONSE_MORE_CHUNKS = 1 << 3
EXPERT_PROTOCOL_V2_FLAG_RESPONSE_FP8_E4M3_ROW_SCALED = 1 << 4
EXPERT_PROTOCOL_V2_FLAG_RESPONSE_NVFP4_E2M1_FP8_E4M3 = 1 << 5
EXPERT_PROTOCOL_V2_FLAG_STREAM_PLAN = 1 << 6
EXPERT_PROTOCOL_V2_FLAG_STREAM_DATA = 1 << 7
EXPERT_PROTOCOL_V2_FLAG_STREAM_FINAL = 1 << 8
EXPERT_PROTOCOL_V2_FLAG_SPARK_REDUCTION = 1 << 9
EXPERT_PROTOCOL_V2_FLAG_LAYER_BLOCK = 1 << 10
EXPERT_PROTOCOL_V2_FLAG_SPARK_ROW_SHARDED_REDUCTION = 1 << 11
B200_EXECUTOR_NAME = "b200-nvfp4-tcgen05-executor"


class ExpertV2Dtype(enum.IntEnum):
    Bf16 = 1
    F16 = 2
    Fp8Debug = 3
    Nvfp4E2m1Fp8E4m3 = 4
    Fp8E4m3RowScaled = 5

    def row_bytes(self, elements: int, lib: N.NativeLibrary | None = None) -> int:
        out = C.c_size_t()
        (lib or N.library()).call("glmrt_b200_pv2_row_bytes", C.c_uint32(int(self)), C.c_size_t(elements), C.byref(out))
        return out.value


class ExpertV2SourceKind(enum.IntEnum):
    Decode = 1
    Prefill = 2
    MtpVerify = 3
    Benchmark = 4


class ExpertProtocolV2Status(enum.IntEnum):
    Ok = 0
    Error = 1


class _RequestHeader(C.Structure):
    _fields_ = [("request_id", C.c_uint64), ("placement_version", C.c_uint64), ("layer_id", C.c_uint32),
                ("row_count", C.c_uint32), ("hidden_dim", C.c_uint32), ("hidden_dtype", C.c_uint32),
                ("hidden_row_stride_bytes", C.c_uint32), ("route_count", C.c_uint32),
                ("row_descriptor_bytes", C.c_uint32), ("route_bytes", C.c_uint32),
                ("hidden_payload_bytes", C.c_uint64), ("flags", C.c_uint32), ("header_len", C.c_uint32)]


class _Row(C.Structure):
    _fields_ = [("row_id", C.c_uint64), ("source_request_id", C.c_uint64), ("token_position", C.c_uint64),
                ("route_offset", C.c_uint32), ("route_count", C.c_uint32), ("source_kind", C.c_uint32),
                ("reserved", C.c_uint32)]


class _Route(C.Structure):
    _fields_ = [("row_index", C.c_uint32), ("expert_id", C.c_uint32), ("gate_weight", C.c_float)]


class _ResponseHeader(C.Structure):
    _fields_ = [("request_id", C.c_uint64), ("placement_version", C.c_uint64), ("layer_id", C.c_uint32),
                ("row_count", C.c_uint32), ("output_dim", C.c_uint32), ("output_dtype", C.c_uint32),
                ("output_row_stride_bytes", C.c_uint32), ("status", C.c_uint32),
                ("output_payload_bytes", C.c_uint64), ("flags", C.c_uint32), ("header_len", C.c_uint32),
                ("executor_id", C.c_uint64)]


class _Sections(C.Structure):
    _fields_ = [("rows_offset", C.c_uint64), ("routes_offset", C.c_uint64), ("payload_offset", C.c_uint64),
                ("payload_bytes", C.c_uint64)]


def expert_protocol_v2_compact_id(value: str, lib: N.NativeLibrary | None = None) -> int:
    out = C.c_uint64()
    (lib or N.library()).call("glmrt_b200_pv2_compact_id", value.encode(), C.byref(out))
    return out.value


@dataclass
class ExpertProtocolV2RowDescriptor:
    row_id: int
    source_kind: ExpertV2SourceKind
    source_request_id: int
    token_position: int
    route_offset: int
    route_count: int


@dataclass
class ExpertProtocolV2RouteEntry:
    row_index: int
    expert_id: int
    gate_weight: float


@dataclass
class ExpertProtocolV2WireStats:
    logical_payload_bytes: int
    wire_bytes: int


@dataclass
class ExpertProtocolV2Request:
    request_id: int
    placement_version: int
    layer_id: int
    hidden_dim: int
    hidden_dtype: ExpertV2Dtype
    rows: list
    routes: list
    hidden_payload: bytes
    hidden_row_stride_bytes: int = 0      # 0: the dtype's row size
    flags: int = 0

    def _header(self) -> _RequestHeader:
        h = _RequestHeader()
        h.request_id, h.placement_version, h.layer_id = self.request_id, self.placement_version, self.layer_id
        h.hidden_dim, h.hidden_dtype = self.hidden_dim, int(self.hidden_dtype)
        h.hidden_row_stride_bytes, h.flags = self.hidden_row_stride_bytes, self.flags
        return h

    def encode(self, lib: N.NativeLibrary | None = None) -> bytes:
        lib = lib or N.library()
        rows = (_Row * max(1, len(self.rows)))()
        for i, r in enumerate(self.rows):
            rows[i] = _Row(r.row_id, r.source_request_id, r.token_position, r.route_offset, r.route_count,
                           int(r.source_kind), 0)
        routes = (_Route * max(1, len(self.routes)))()
        for i, r in enumerate(self.routes):
            routes[i] = _Route(r.row_index, r.expert_id, r.gate_weight)
        payload = bytes(self.hidden_payload)
        cap = (EXPERT_PROTOCOL_V2_REQUEST_DEBUG_HEADER_LEN + 40 * len(self.rows) + 10 * len(self.routes) + len(payload))
        out = C.create_string_buffer(cap)
        n = C.c_size_t()
        lib.call("glmrt_b200_pv2_encode_request", C.byref(self._header()), rows, C.c_size_t(len(self.rows)), routes,
                 C.c_size_t(len(self.routes)), payload, C.c_size_t(len(payload)), out, C.c_size_t(cap), C.byref(n))
        return out.raw[:n.value]

    def wire_stats(self) -> ExpertProtocolV2WireStats:
        header = (EXPERT_PROTOCOL_V2_REQUEST_DEBUG_HEADER_LEN if self.flags & EXPERT_PROTOCOL_V2_FLAG_DEBUG_CHECKSUM
                  else EXPERT_PROTOCOL_V2_REQUEST_HEADER_LEN)
        return ExpertProtocolV2WireStats(len(self.hidden_payload), header + 40 * len(self.rows) + 10 * len(self.routes)
                                         + len(self.hidden_payload))

    @classmethod
    def decode(cls, frame: bytes, lib: N.NativeLibrary | None = None) -> "ExpertProtocolV2Request":
        """Request::decode: parse, validate and check the checksum when the frame carries one."""
        view = ExpertProtocolV2RequestView.parse(frame, lib)
        view.verify_checksum()
        h = view.header
        return cls(h.request_id, h.placement_version, h.layer_id, h.hidden_dim, ExpertV2Dtype(h.hidden_dtype),
                   [view.row(i) for i in range(view.row_descriptor_count)],
                   [view.route(i) for i in range(view.route_entry_count)],
                   view.hidden_payload(), h.hidden_row_stride_bytes, h.flags)


@dataclass
class ExpertProtocolV2StreamRouteGroup:
    """protocol_v2/stream.rs:14-19: routes that can run once ``ready_after_rows`` rows have arrived."""
    ready_after_rows: int
    route_indices: list
    completed_rows: list


@dataclass
class ExpertProtocolV2StreamPlan:
    """The "GLMSTRM2" payload of a stream-plan frame (protocol_v2/stream.rs:21-27, encode :86-150):
    the order in which the hidden rows will arrive and the completion-first route groups.  This is
    the sender's side of streamed ingress; the library parses it in ``glmrt_b200_pv2_execute``."""
    row_count: int
    route_count: int
    activation_row_order: list
    groups: list = field(default_factory=list)

    def encode(self) -> bytes:
        route_indices = [r for g in self.groups for r in g.route_indices]
        completed = [r for g in self.groups for r in g.completed_rows]
        wire = 40 + 20 * len(self.groups) + 4 * (len(self.activation_row_order) + len(route_indices) + len(completed))
        out = b"GLMSTRM2" + struct.pack("<HHIIIIIII", 1, 40, wire, self.row_count, self.route_count,
                                        len(self.activation_row_order), len(self.groups), len(route_indices),
                                        len(completed))
        r_off = c_off = 0
        for g in self.groups:
            out += struct.pack("<IIIII", g.ready_after_rows, r_off, len(g.route_indices), c_off, len(g.completed_rows))
            r_off += len(g.route_indices)
            c_off += len(g.completed_rows)
        for seq in (self.activation_row_order, route_indices, completed):
            out += struct.pack(f"<{len(seq)}I", *seq)
        assert len(out) == wire
        return out


def streamed_request_frames(request: "ExpertProtocolV2Request", plan: ExpertProtocolV2StreamPlan, rows_per_frame: int,
                            lib: N.NativeLibrary | None = None) -> list:
    """The frames of a streamed request: the stream-plan frame (the request's rows and routes, the
    plan as payload), then stream-data frames with runs of hidden rows in the plan's activation
    order, the last one flagged final (protocol_v2/request.rs:183-230, 521-531: a data frame has
    no descriptors and its route_count field is the position of its first row)."""
    stride = request.hidden_row_stride_bytes or request.hidden_dtype.row_bytes(request.hidden_dim, lib)
    base_flags = request.flags & ~(EXPERT_PROTOCOL_V2_FLAG_STREAM_PLAN | EXPERT_PROTOCOL_V2_FLAG_STREAM_DATA |
                                   EXPERT_PROTOCOL_V2_FLAG_STREAM_FINAL | EXPERT_PROTOCOL_V2_FLAG_DEBUG_CHECKSUM)
    head = ExpertProtocolV2Request(request.request_id, request.placement_version, request.layer_id, request.hidden_dim,
                                   request.hidden_dtype, request.rows, request.routes, plan.encode(), stride,
                                   base_flags | EXPERT_PROTOCOL_V2_FLAG_STREAM_PLAN)
    frames = [head.encode(lib)]
    order = plan.activation_row_order
    for first in range(0, len(order), rows_per_frame):
        run = order[first:first + rows_per_frame]
        payload = b"".join(request.hidden_payload[r * stride:(r + 1) * stride] for r in run)
        flags = base_flags | EXPERT_PROTOCOL_V2_FLAG_STREAM_DATA
        if first + rows_per_frame >= len(order):
            flags |= EXPERT_PROTOCOL_V2_FLAG_STREAM_FINAL
        h = b"GLMRTE2\0" + struct.pack("<HHI", 2, 1, EXPERT_PROTOCOL_V2_REQUEST_HEADER_LEN)
        h += struct.pack("<QQIIIHHIIIQQQII", request.request_id, request.placement_version, request.layer_id, len(run),
                         request.hidden_dim, int(request.hidden_dtype), 0, first, 0, 0, len(payload), len(payload),
                         EXPERT_PROTOCOL_V2_REQUEST_HEADER_LEN + len(payload), flags, stride) + b"\0" * 4
        frames.append(h + payload)
    return frames


class ExpertProtocolV2RequestView:
    """Borrowing view of an encoded request (protocol_v2/view.rs:24-330)."""

    def __init__(self, frame: bytes, header: _RequestHeader, sections: _Sections, lib: N.NativeLibrary):
        self.frame, self.header, self.sections, self.lib = frame, header, sections, lib

    @classmethod
    def parse(cls, frame: bytes, lib: N.NativeLibrary | None = None) -> "ExpertProtocolV2RequestView":
        lib = lib or N.library()
        frame = bytes(frame)
        h, s = _RequestHeader(), _Sections()
        lib.call("glmrt_b200_pv2_parse_request", frame, C.c_size_t(len(frame)), C.byref(h), C.byref(s))
        return cls(frame, h, s, lib)

    @property
    def row_descriptor_count(self) -> int:
        return self.header.row_descriptor_bytes // EXPERT_PROTOCOL_V2_ROW_DESCRIPTOR_LEN

    @property
    def route_entry_count(self) -> int:
        return self.header.route_bytes // EXPERT_PROTOCOL_V2_ROUTE_ENTRY_LEN

    def header_len(self) -> int:
        return self.header.header_len

    def row(self, index: int) -> ExpertProtocolV2RowDescriptor:
        r = _Row()
        self.lib.call("glmrt_b200_pv2_request_row", self.frame, C.c_size_t(len(self.frame)), C.c_size_t(index), C.byref(r))
        return ExpertProtocolV2RowDescriptor(r.row_id, ExpertV2SourceKind(r.source_kind), r.source_request_id,
                                             r.token_position, r.route_offset, r.route_count)

    def route(self, index: int) -> ExpertProtocolV2RouteEntry:
        r = _Route()
        self.lib.call("glmrt_b200_pv2_request_route", self.frame, C.c_size_t(len(self.frame)), C.c_size_t(index),
                      C.byref(r))
        return ExpertProtocolV2RouteEntry(r.row_index, r.expert_id, r.gate_weight)

    def row_descriptor_bytes(self) -> bytes:
        return self.frame[self.sections.rows_offset:self.sections.routes_offset]

    def route_bytes(self) -> bytes:
        return self.frame[self.sections.routes_offset:self.sections.payload_offset]

    def hidden_payload(self) -> bytes:
        s = self.sections
        return self.frame[s.payload_offset:s.payload_offset + s.payload_bytes]

    def hidden_row_payload(self, index: int) -> bytes:
        stride = self.header.hidden_row_stride_bytes
        logical = ExpertV2Dtype(self.header.hidden_dtype).row_bytes(self.header.hidden_dim, self.lib)
        if index >= self.header.row_count:
            raise IndexError(index)
        start = self.sections.payload_offset + index * stride
        return self.frame[start:start + logical]

    def debug_checksum_enabled(self) -> bool:
        return bool(self.header.flags & EXPERT_PROTOCOL_V2_FLAG_DEBUG_CHECKSUM)

    def verify_checksum(self) -> None:
        self.lib.call("glmrt_b200_pv2_verify_request_checksum", self.frame, C.c_size_t(len(self.frame)))


@dataclass
class ExpertProtocolV2Response:
    request_id: int
    placement_version: int
    layer_id: int
    row_count: int
    output_dim: int
    output_dtype: ExpertV2Dtype
    status: ExpertProtocolV2Status
    partial_output_payload: bytes
    output_row_stride_bytes: int = 0
    flags: int = 0
    executor_id: int = 0
    row_indices: list | None = field(default=None)

    def with_executor_name(self, name: str) -> "ExpertProtocolV2Response":
        self.executor_id = expert_protocol_v2_compact_id(name)
        return self

    def with_debug_checksum(self) -> "ExpertProtocolV2Response":
        self.flags |= EXPERT_PROTOCOL_V2_FLAG_DEBUG_CHECKSUM
        return self

    def with_row_indices(self, row_indices: list, more_chunks: bool) -> "ExpertProtocolV2Response":
        self.flags |= EXPERT_PROTOCOL_V2_FLAG_RESPONSE_ROW_INDICES
        if more_chunks:
            self.flags |= EXPERT_PROTOCOL_V2_FLAG_RESPONSE_MORE_CHUNKS
        else:
            self.flags &= ~EXPERT_PROTOCOL_V2_FLAG_RESPONSE_MORE_CHUNKS
        self.row_indices = list(row_indices)
        return self

    def row_indexed(self) -> bool:
        return bool(self.flags & EXPERT_PROTOCOL_V2_FLAG_RESPONSE_ROW_INDICES)

    def more_chunks(self) -> bool:
        return bool(self.flags & EXPERT_PROTOCOL_V2_FLAG_RESPONSE_MORE_CHUNKS)

    def encode(self, lib: N.NativeLibrary | None = None) -> bytes:
        lib = lib or N.library()
        h = _ResponseHeader()
        h.request_id, h.placement_version, h.layer_id = self.request_id, self.placement_version, self.layer_id
        h.row_count, h.output_dim, h.output_dtype = self.row_count, self.output_dim, int(self.output_dtype)
        h.output_row_stride_bytes, h.status, h.flags = self.output_row_stride_bytes, int(self.status), self.flags
        h.executor_id = self.executor_id
        idx = None
        if self.row_indices is not None:
            idx = (C.c_uint32 * max(1, len(self.row_indices)))(*self.row_indices)
            if len(self.row_indices) != self.row_count:
                raise N.GlmrtError("glmrt_b200_pv2_encode_response", 1,
                                   "ExpertProtocolV2 response row index count mismatch: expected="
                                   f"{self.row_count} actual={len(self.row_indices)}")
        payload = bytes(self.partial_output_payload)
        cap = EXPERT_PROTOCOL_V2_REQUEST_DEBUG_HEADER_LEN + 4 * self.row_count + len(payload)
        out = C.create_string_buffer(cap)
        n = C.c_size_t()
        lib.call("glmrt_b200_pv2_encode_response", C.byref(h), idx, payload, C.c_size_t(len(payload)), out,
                 C.c_size_t(cap), C.byref(n))
        return out.raw[:n.value]

    def wire_stats(self) -> ExpertProtocolV2WireStats:
        header = (EXPERT_PROTOCOL_V2_REQUEST_DEBUG_HEADER_LEN if self.flags & EXPERT_PROTOCOL_V2_FLAG_DEBUG_CHECKSUM
                  else EXPERT_PROTOCOL_V2_RESPONSE_HEADER_LEN)
        idx = 4 * len(self.row_indices) if self.row_indices is not None else 0
        return ExpertProtocolV2WireStats(len(self.partial_output_payload), header + idx + len(self.partial_output_payload))

    @classmethod
    def decode(cls, frame: bytes, lib: N.NativeLibrary | None = None) -> "ExpertProtocolV2Response":
        lib = lib or N.library()
        frame = bytes(frame)
        h, s = _ResponseHeader(), _Sections()
        lib.call("glmrt_b200_pv2_parse_response", frame, C.c_size_t(len(frame)), C.byref(h), C.byref(s))
        lib.call("glmrt_b200_pv2_verify_response_checksum", frame, C.c_size_t(len(frame)))
        idx = None
        if h.flags & EXPERT_PROTOCOL_V2_FLAG_RESPONSE_ROW_INDICES:
            raw = frame[s.rows_offset:s.payload_offset]
            idx = [int.from_bytes(raw[4 * i:4 * i + 4], "little") for i in range(h.row_count)]
        return cls(h.request_id, h.placement_version, h.layer_id, h.row_count, h.output_dim,
                   ExpertV2Dtype(h.output_dtype), ExpertProtocolV2Status(h.status),
                   frame[s.payload_offset:s.payload_offset + s.payload_bytes], h.output_row_stride_bytes, h.flags,
                   h.executor_id, idx)

    def partial_output_row_payload(self, index: int) -> bytes:
        stride = self.output_row_stride_bytes or self.output_dtype.row_bytes(self.output_dim)
        logical = self.output_dtype.row_bytes(self.output_dim)
        return self.partial_output_payload[index * stride:index * stride + logical]


class ProtocolV2ExpertExecutor:
    """The plugin contract of glmrt-transport/src/synthetic.rs:51-107: ``name`` and ``execute``;
    ``execute_with_identity`` stamps the response with the compact id of the name."""

    def name(self) -> str:
        raise NotImplementedError

    def execute(self, request: ExpertProtocolV2RequestView) -> ExpertProtocolV2Response:
        raise NotImplementedError

    def execute_with_identity(self, request: ExpertProtocolV2RequestView) -> ExpertProtocolV2Response:
        return self.execute(request).with_executor_name(self.name())


class B200MoeExecutor(ProtocolV2ExpertExecutor):
    """Runs request frames through a ``MoeLayer`` (``glmrt_b200_pv2_execute``): the role of
    RealNvfp4ProtocolV2Executor (real_full/expert_probe/protocol_v2_executor.rs:1882-2493)."""

    def __init__(self, layer):
        self.layer = layer

    def name(self) -> str:
        return B200_EXECUTOR_NAME

    def execute_frame(self, frame: bytes) -> bytes:
        """Request frame in, response frame out (empty for a stream-plan frame and for every
        stream-data frame but the final one: their rows are staged, nothing is sent back yet)."""
        frame = bytes(frame)
        cap = EXPERT_PROTOCOL_V2_REQUEST_DEBUG_HEADER_LEN + self.layer.max_tokens * self.layer.hidden * 2
        out = C.create_string_buffer(cap)
        n = C.c_size_t()
        import torch
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        self.layer.lib.call("glmrt_b200_pv2_execute", self.layer.handle, frame, C.c_size_t(len(frame)), out,
                            C.c_size_t(cap), C.byref(n), stream)
        return out.raw[:n.value]

    def execute(self, request: ExpertProtocolV2RequestView) -> ExpertProtocolV2Response:
        return ExpertProtocolV2Response.decode(self.execute_frame(request.frame), self.layer.lib)
