"""ExpertProtocolV2 frames through the C codec (no GPU): the cases of the reference's own tests
(rust/crates/glmrt-transport/src/protocol_v2/tests.rs) restated against the Python mirror, plus
byte-level checks against an independent ``struct``/``hashlib`` restatement of the wire layout.

The reference's tests hold no golden byte strings (they are round trips and rejections), and its
Rust cannot be built here.  What pins the bytes: the frame header (magic, version, kind, header
length rule, flags and wire-bytes offsets) by the reference's own C++ frame validator, compiled
from the reference tree (last tests of this file); row descriptors, route entries and payload only
by the layout documented in protocol_v2.rs, restated twice (C and this file), and SHA-256 /
compact ids checked against hashlib.
"""
import hashlib
import struct

import numpy as np
import pytest


@pytest.fixture(scope="module")
def P(pkg):
    from glmrt_b200 import protocol_v2
    return protocol_v2


@pytest.fixture(scope="module")
def Err(pkg):
    from glmrt_b200 import native
    return native.GlmrtError


def make_request(P, row_count, source_kind, hidden_dim=6144, dtype=None, flags=0, stride=0, weights=(0.25, 0.75)):
    """tests.rs:10-43: rows with two routes each, experts 7 and 19 + row, bf16 hidden rows."""
    dtype = dtype or P.ExpertV2Dtype.Bf16
    rows, routes = [], []
    for r in range(row_count):
        rows.append(P.ExpertProtocolV2RowDescriptor(1000 + r, source_kind, 77, 4096 + r, len(routes), 2))
        routes.append(P.ExpertProtocolV2RouteEntry(r, 7, weights[0]))
        routes.append(P.ExpertProtocolV2RouteEntry(r, 19 + r, weights[1]))
    row_bytes = stride or dtype.row_bytes(hidden_dim)
    payload = bytes((i * 31 + 7) % 251 for i in range(row_count * row_bytes))
    return P.ExpertProtocolV2Request(42, 9, 3, hidden_dim, dtype, rows, routes, payload, stride, flags)


def reference_layout_request(req, P):
    """The request layout of protocol_v2/request.rs:333-379 written with struct.pack."""
    stride = req.hidden_row_stride_bytes or req.hidden_dtype.row_bytes(req.hidden_dim)
    debug = bool(req.flags & P.EXPERT_PROTOCOL_V2_FLAG_DEBUG_CHECKSUM)
    header_len = 128 if debug else 96
    rows = b"".join(struct.pack("<QHHQQIII", r.row_id, int(r.source_kind), 0, r.source_request_id, r.token_position,
                                r.route_offset, r.route_count, 0) for r in req.rows)
    routes = b"".join(struct.pack("<II", r.row_index, r.expert_id) +
                      struct.pack("<H", struct.unpack("<I", struct.pack("<f", r.gate_weight))[0] >> 16) for r in req.routes)
    wire = header_len + len(rows) + len(routes) + len(req.hidden_payload)
    head = b"GLMRTE2\0" + struct.pack("<HHI", 2, 1, header_len)
    head += struct.pack("<QQIIIHHIIIQQQII", req.request_id, req.placement_version, req.layer_id, len(req.rows),
                        req.hidden_dim, int(req.hidden_dtype), 0, len(req.routes), len(rows), len(routes),
                        len(req.hidden_payload), len(req.hidden_payload), wire, req.flags, stride)
    assert len(head) == 92
    if debug:
        head += hashlib.sha256(rows + routes + req.hidden_payload).digest()
    head += b"\0" * (header_len - len(head))
    return head + rows + routes + req.hidden_payload


def test_constants_and_row_bytes(P, Err):
    assert P.EXPERT_PROTOCOL_V2_REQUEST_HEADER_LEN == 96 and P.EXPERT_PROTOCOL_V2_ROW_DESCRIPTOR_LEN == 40
    assert P.EXPERT_PROTOCOL_V2_ROUTE_ENTRY_LEN == 10
    D = P.ExpertV2Dtype
    assert D.Bf16.row_bytes(6144) == 12288 and D.F16.row_bytes(6144) == 12288 and D.Fp8Debug.row_bytes(6144) == 6144
    assert D.Nvfp4E2m1Fp8E4m3.row_bytes(6144) == 3456          # 3072 code bytes + 384 scale bytes
    assert D.Fp8E4m3RowScaled.row_bytes(6144) == 6148           # values + one float32 scale
    for bad in (0, 24):
        with pytest.raises(Err, match="multiple of 16"):
            D.Nvfp4E2m1Fp8E4m3.row_bytes(bad)


def test_sha256_and_compact_id_match_hashlib(P, pkg):
    import ctypes as C
    from glmrt_b200 import native as N
    lib = N.library()
    for msg in (b"", b"abc", b"a" * 55, b"a" * 56, b"a" * 64, bytes(range(256)) * 5):
        out = (C.c_uint8 * 32)()
        lib.call("glmrt_b200_pv2_sha256", msg, C.c_size_t(len(msg)), out)
        assert bytes(out) == hashlib.sha256(msg).digest()
    for name in ("protocol-v2-echo-loopback", P.B200_EXECUTOR_NAME, ""):
        want = int.from_bytes(hashlib.sha256(name.encode()).digest()[:8], "little")   # protocol_v2.rs:229-232
        assert P.expert_protocol_v2_compact_id(name) == want


def test_encode_decode_one_row_decode_request_has_12288_payload_bytes(P):
    """tests.rs:45-60"""
    req = make_request(P, 1, P.ExpertV2SourceKind.Decode)
    frame = req.encode()
    assert len(frame) == 96 + 40 + 2 * 10 + 12288 == req.wire_stats().wire_bytes
    assert frame == reference_layout_request(req, P)
    back = P.ExpertProtocolV2Request.decode(frame)
    assert back.hidden_payload == req.hidden_payload and len(back.hidden_payload) == 12288
    assert back.rows == req.rows and back.hidden_row_stride_bytes == 12288
    assert [(r.row_index, r.expert_id) for r in back.routes] == [(0, 7), (0, 19)]


@pytest.mark.parametrize("rows,kind", [(2, "MtpVerify"), (4, "MtpVerify"), (8, "MtpVerify"), (16, "Prefill"), (257, "Prefill")])
def test_encode_decode_mtp_and_prefill_request_shapes(P, rows, kind):
    """tests.rs:544-580"""
    req = make_request(P, rows, getattr(P.ExpertV2SourceKind, kind), hidden_dim=64)
    frame = req.encode()
    assert frame == reference_layout_request(req, P)
    back = P.ExpertProtocolV2Request.decode(frame)
    assert len(back.rows) == rows and len(back.routes) == 2 * rows
    assert back.rows[-1].source_kind == getattr(P.ExpertV2SourceKind, kind)
    assert back.rows[-1].route_offset == 2 * (rows - 1)


def test_nvfp4_hidden_exchange_uses_packed_values_plus_fp8_scales(P):
    """tests.rs:249-282: 6144 elements travel as 3072 + 384 bytes per row."""
    req = make_request(P, 3, P.ExpertV2SourceKind.Decode, dtype=P.ExpertV2Dtype.Nvfp4E2m1Fp8E4m3)
    frame = req.encode()
    view = P.ExpertProtocolV2RequestView.parse(frame)
    assert view.header.hidden_row_stride_bytes == 3456 and len(view.hidden_payload()) == 3 * 3456
    assert view.hidden_row_payload(2) == req.hidden_payload[2 * 3456:3 * 3456]
    assert frame == reference_layout_request(req, P)


def test_route_entries_carry_gate_weights_as_bf16_on_wire(P):
    """tests.rs:449-502: weights are truncated to bf16 by the encoder, so a decoded request
    compares equal to the canonical form, and a route entry is 10 bytes."""
    w = 0.333333343267
    req = make_request(P, 1, P.ExpertV2SourceKind.Decode, hidden_dim=16, weights=(w, 1.0))
    view = P.ExpertProtocolV2RequestView.parse(req.encode())
    assert len(view.route_bytes()) == 2 * 10
    bits = struct.unpack("<I", struct.pack("<f", w))[0] & 0xFFFF0000
    canonical = struct.unpack("<f", struct.pack("<I", bits))[0]
    assert view.route(0).gate_weight == canonical != w
    assert view.route(1).gate_weight == 1.0
    assert view.route_bytes()[8:10] == struct.pack("<H", bits >> 16)


def test_request_header_carries_explicit_hidden_stride(P, Err):
    """tests.rs:504-542 and :596-608"""
    req = make_request(P, 2, P.ExpertV2SourceKind.Prefill, hidden_dim=64, stride=160)
    frame = req.encode()
    view = P.ExpertProtocolV2RequestView.parse(frame)
    assert view.header.hidden_row_stride_bytes == 160 and len(view.hidden_payload()) == 320
    assert view.hidden_row_payload(1) == req.hidden_payload[160:160 + 128]
    assert struct.unpack_from("<I", frame, 88)[0] == 160
    small = make_request(P, 2, P.ExpertV2SourceKind.Prefill, hidden_dim=64, stride=127)
    with pytest.raises(Err, match="smaller than logical row bytes"):
        small.encode()


def test_malformed_frames_are_rejected(P, Err):
    """tests.rs:582-619"""
    req = make_request(P, 2, P.ExpertV2SourceKind.Decode, hidden_dim=32)
    frame = req.encode()
    for broken, msg in ((frame[:-1], "wire bytes mismatch"), (frame + b"\0", "wire bytes mismatch"),
                        (frame[:50], "too short"), (b"XLMRTE2\0" + frame[8:], "invalid magic"),
                        (frame[:8] + struct.pack("<H", 3) + frame[10:], "unsupported version"),
                        (frame[:10] + struct.pack("<H", 2) + frame[12:], "unexpected message kind")):
        with pytest.raises(Err, match=msg):
            P.ExpertProtocolV2RequestView.parse(broken)
    # a row whose route range leaves the route table
    req.rows[1].route_count = 3
    with pytest.raises(Err, match="exceeds route count"):
        req.encode()
    req.rows[1].route_count = 2
    req.routes[3].row_index = 2
    with pytest.raises(Err, match="exceeds row count"):
        req.encode()
    req.routes[3].row_index = 1
    req.routes[3].gate_weight = float("inf")
    with pytest.raises(Err, match="finite"):
        req.encode()


def test_flag_rules(P, Err):
    """protocol_v2.rs:431-497 and tests.rs:62-104, 179-247, 357-367"""
    F = P
    ok = [F.EXPERT_PROTOCOL_V2_FLAG_SPARK_REDUCTION,
          F.EXPERT_PROTOCOL_V2_FLAG_SPARK_REDUCTION | F.EXPERT_PROTOCOL_V2_FLAG_SPARK_ROW_SHARDED_REDUCTION,
          F.EXPERT_PROTOCOL_V2_FLAG_SPARK_REDUCTION | F.EXPERT_PROTOCOL_V2_FLAG_SPARK_ROW_SHARDED_REDUCTION | (3 << 12),
          F.EXPERT_PROTOCOL_V2_FLAG_RESPONSE_FP8_E4M3_ROW_SCALED, F.EXPERT_PROTOCOL_V2_FLAG_RESPONSE_NVFP4_E2M1_FP8_E4M3,
          F.EXPERT_PROTOCOL_V2_FLAG_PRECOMPILE_WARMUP]
    for flags in ok:
        req = make_request(P, 1, P.ExpertV2SourceKind.Decode, hidden_dim=32, flags=flags)
        assert P.ExpertProtocolV2Request.decode(req.encode()).flags == flags
    bad = [(F.EXPERT_PROTOCOL_V2_FLAG_RESPONSE_FP8_E4M3_ROW_SCALED | F.EXPERT_PROTOCOL_V2_FLAG_RESPONSE_NVFP4_E2M1_FP8_E4M3, "multiple low-precision"),
           (F.EXPERT_PROTOCOL_V2_FLAG_SPARK_ROW_SHARDED_REDUCTION, "requires Spark reduction"),
           (F.EXPERT_PROTOCOL_V2_FLAG_SPARK_REDUCTION | F.EXPERT_PROTOCOL_V2_FLAG_SPARK_ROW_SHARDED_REDUCTION | (1 << 12), "at least two parts"),
           (F.EXPERT_PROTOCOL_V2_FLAG_SPARK_REDUCTION | (2 << 12), "requires row-sharded"),
           (F.EXPERT_PROTOCOL_V2_FLAG_STREAM_FINAL, "requires a stream data frame"),
           (F.EXPERT_PROTOCOL_V2_FLAG_STREAM_PLAN | F.EXPERT_PROTOCOL_V2_FLAG_STREAM_DATA, "both a stream plan"),
           (F.EXPERT_PROTOCOL_V2_FLAG_RESPONSE_ROW_INDICES, "unknown flags"), (1 << 20, "unknown flags")]
    for flags, msg in bad:
        with pytest.raises(Err, match=msg):
            make_request(P, 1, P.ExpertV2SourceKind.Decode, hidden_dim=32, flags=flags).encode()


def test_debug_checksum_is_explicit_validation(P, Err):
    """tests.rs:737-815, 910-963: hot frames carry no checksum (96-byte header); a debug frame has a
    128-byte header whose SHA-256 covers rows, routes and payload; views check it only on request."""
    hot = make_request(P, 2, P.ExpertV2SourceKind.Decode, hidden_dim=32)
    assert P.ExpertProtocolV2RequestView.parse(hot.encode()).header_len() == 96
    req = make_request(P, 2, P.ExpertV2SourceKind.Decode, hidden_dim=32, flags=P.EXPERT_PROTOCOL_V2_FLAG_DEBUG_CHECKSUM)
    frame = req.encode()
    assert frame == reference_layout_request(req, P) and len(frame) == len(hot.encode()) + 32
    view = P.ExpertProtocolV2RequestView.parse(frame)
    assert view.header_len() == 128 and view.debug_checksum_enabled()
    view.verify_checksum()
    corrupt = bytearray(frame)
    corrupt[-1] ^= 1
    bad_view = P.ExpertProtocolV2RequestView.parse(bytes(corrupt))      # parsing alone does not hash
    with pytest.raises(Err, match="checksum mismatch"):
        bad_view.verify_checksum()
    with pytest.raises(Err, match="checksum mismatch"):
        P.ExpertProtocolV2Request.decode(bytes(corrupt))


def test_response_encode_decode_reports_wire_and_logical_bytes(P, Err):
    """tests.rs:621-689"""
    payload = bytes(range(256)) * 48                      # one bf16 row of 6144
    resp = P.ExpertProtocolV2Response(42, 9, 3, 1, 6144, P.ExpertV2Dtype.Bf16, P.ExpertProtocolV2Status.Ok, payload)
    resp.with_executor_name("protocol-v2-echo-loopback")
    frame = resp.encode()
    assert len(frame) == 96 + 12288 == resp.wire_stats().wire_bytes and resp.wire_stats().logical_payload_bytes == 12288
    want_head = b"GLMRTE2\0" + struct.pack("<HHIQQIIHHQQQIIIQ", 2, 2, 96, 42, 9, 3, 1, 1, 0, 12288, 12288, 96 + 12288, 0,
                                           6144, 12288, resp.executor_id)
    assert frame[:88] == want_head and frame[88:96] == b"\0" * 8 and frame[96:] == payload
    back = P.ExpertProtocolV2Response.decode(frame)
    assert back.partial_output_payload == payload and back.output_row_stride_bytes == 12288
    assert back.executor_id == int.from_bytes(hashlib.sha256(b"protocol-v2-echo-loopback").digest()[:8], "little")
    strided = P.ExpertProtocolV2Response(1, 1, 0, 2, 64, P.ExpertV2Dtype.Bf16, P.ExpertProtocolV2Status.Ok, b"\x11" * 320, 160)
    assert P.ExpertProtocolV2Response.decode(strided.encode()).partial_output_row_payload(1) == b"\x11" * 128
    with pytest.raises(Err, match="payload bytes mismatch"):
        P.ExpertProtocolV2Response(1, 1, 0, 2, 64, P.ExpertV2Dtype.Bf16, P.ExpertProtocolV2Status.Ok, b"\0" * 100).encode()
    with pytest.raises(Err, match="unknown flags"):   # a request-only flag on a response (tests.rs:848-868)
        P.ExpertProtocolV2Response(1, 1, 0, 1, 64, P.ExpertV2Dtype.Bf16, P.ExpertProtocolV2Status.Ok, b"\0" * 128,
                                   flags=P.EXPERT_PROTOCOL_V2_FLAG_PRECOMPILE_WARMUP).encode()


def test_low_precision_response_payloads_roundtrip(P):
    """tests.rs:179-247: row-scaled FP8 rows are elements + 4 bytes, NVFP4 rows elements/2 + elements/16."""
    for dtype, row in ((P.ExpertV2Dtype.Fp8E4m3RowScaled, 6148), (P.ExpertV2Dtype.Nvfp4E2m1Fp8E4m3, 3456)):
        payload = bytes([0x35]) * (2 * row)
        resp = P.ExpertProtocolV2Response(7, 1, 2, 2, 6144, dtype, P.ExpertProtocolV2Status.Ok, payload)
        back = P.ExpertProtocolV2Response.decode(resp.encode())
        assert back.output_dtype == dtype and back.output_row_stride_bytes == row and back.partial_output_payload == payload


def test_row_indexed_response_chunk_round_trips(P, Err):
    """tests.rs:691-735"""
    payload = b"\x22" * (3 * 128)
    resp = P.ExpertProtocolV2Response(5, 1, 0, 3, 64, P.ExpertV2Dtype.Bf16, P.ExpertProtocolV2Status.Ok, payload)
    plain = resp.encode()
    assert len(plain) == 96 + 384
    resp.with_row_indices([4, 0, 9], more_chunks=True)
    frame = resp.encode()
    assert len(frame) == 96 + 12 + 384 and frame[96:108] == struct.pack("<III", 4, 0, 9)
    back = P.ExpertProtocolV2Response.decode(frame)
    assert back.row_indices == [4, 0, 9] and back.row_indexed() and back.more_chunks()
    with pytest.raises(Err, match="unique"):
        resp.with_row_indices([4, 4, 9], more_chunks=False).encode()
    with pytest.raises(Err, match="count mismatch"):
        resp.with_row_indices([4, 9], more_chunks=False).encode()
    lonely = P.ExpertProtocolV2Response(5, 1, 0, 3, 64, P.ExpertV2Dtype.Bf16, P.ExpertProtocolV2Status.Ok, payload,
                                        flags=P.EXPERT_PROTOCOL_V2_FLAG_RESPONSE_MORE_CHUNKS)
    with pytest.raises(Err, match="disagree|requires row indices"):
        lonely.encode()
    checked = P.ExpertProtocolV2Response(5, 1, 0, 3, 64, P.ExpertV2Dtype.Bf16, P.ExpertProtocolV2Status.Ok, payload)
    checked.with_debug_checksum().with_row_indices([2, 1, 0], False)
    cframe = checked.encode()
    assert cframe[88:120] == hashlib.sha256(struct.pack("<III", 2, 1, 0) + payload).digest()   # response.rs:644-656
    P.ExpertProtocolV2Response.decode(cframe)
    with pytest.raises(Err, match="checksum mismatch"):
        P.ExpertProtocolV2Response.decode(cframe[:-1] + b"\x23")


def test_stream_data_frames_parse_with_their_own_rules(P, Err):
    """request.rs:183-230, 521-531: no descriptors, route_count is the row offset into the plan."""
    stride, rows, offset = 128, 2, 5
    payload = b"\x37" * (rows * stride)
    flags = P.EXPERT_PROTOCOL_V2_FLAG_STREAM_DATA | P.EXPERT_PROTOCOL_V2_FLAG_STREAM_FINAL
    head = b"GLMRTE2\0" + struct.pack("<HHI", 2, 1, 96)
    head += struct.pack("<QQIIIHHIIIQQQII", 1, 1, 0, rows, 64, 1, 0, offset, 0, 0, len(payload), len(payload),
                        96 + len(payload), flags, stride) + b"\0" * 4
    view = P.ExpertProtocolV2RequestView.parse(head + payload)
    assert view.header.route_count == offset and view.row_descriptor_count == 0 and view.hidden_payload() == payload
    with pytest.raises(Err, match="not built by this encoder"):
        make_request(P, 1, P.ExpertV2SourceKind.Decode, hidden_dim=32, flags=flags).encode()


def test_streamed_request_frames_parse_and_carry_the_plan(P):
    """Sender side of streamed ingress (protocol_v2/stream.rs:9-27, 86-150; request.rs:183-230): a
    stream-plan frame with the request's rows and routes and the GLMSTRM2 plan as payload, then
    stream-data frames with runs of rows in the plan's order; the last one is flagged final."""
    rows, hidden = 5, 64
    req = make_request(P, rows, P.ExpertV2SourceKind.MtpVerify, hidden_dim=hidden)
    stride = 2 * hidden
    req.hidden_payload = bytes((r * 16 + (i % 16)) & 0xff for r in range(rows) for i in range(stride))
    order = [3, 0, 4, 1, 2]
    groups = [P.ExpertProtocolV2StreamRouteGroup(2, [6, 7, 0, 1], [3, 0]),
              P.ExpertProtocolV2StreamRouteGroup(5, [8, 9, 2, 3, 4, 5], [4, 1, 2])]
    plan = P.ExpertProtocolV2StreamPlan(rows, len(req.routes), order, groups)
    blob = plan.encode()
    assert blob[:8] == b"GLMSTRM2" and struct.unpack_from("<HHI", blob, 8) == (1, 40, len(blob))
    assert struct.unpack_from("<IIIIII", blob, 16) == (rows, len(req.routes), rows, 2, 10, 5)
    assert len(blob) == 40 + 2 * 20 + 4 * (5 + 10 + 5)
    assert struct.unpack_from("<IIIII", blob, 60) == (5, 4, 6, 2, 3)          # second group: offsets follow the first
    assert list(struct.unpack_from("<5I", blob, 80)) == order

    frames = P.streamed_request_frames(req, plan, 2)
    assert len(frames) == 1 + 3
    head = P.ExpertProtocolV2RequestView.parse(frames[0])
    assert head.header.flags & P.EXPERT_PROTOCOL_V2_FLAG_STREAM_PLAN
    assert head.header.row_count == rows and head.header.route_count == len(req.routes)
    assert head.hidden_payload() == blob
    seen = []
    for k, frame in enumerate(frames[1:]):
        v = P.ExpertProtocolV2RequestView.parse(frame)
        final = bool(v.header.flags & P.EXPERT_PROTOCOL_V2_FLAG_STREAM_FINAL)
        assert v.header.flags & P.EXPERT_PROTOCOL_V2_FLAG_STREAM_DATA and final == (k == 2)
        assert v.header.route_count == 2 * k and v.row_descriptor_count == 0      # position of the run's first row
        run = order[2 * k:2 * k + 2]
        assert v.header.row_count == len(run)
        assert v.hidden_payload() == b"".join(req.hidden_payload[r * stride:(r + 1) * stride] for r in run)
        seen += run
    assert seen == order


# ---------------------------------------------------------------------------------------------
# The reference's own frame validator (native/src/glmrt_native.cc, compiled by oracle/build_ref.py
# into oracle/_ref/) on the frames this repository encodes: pins magic, version, kind, the header
# length rule (96, or 128 with the debug-checksum flag), the flags offset (84 in requests, 68 in
# responses) and the wire-bytes offset (76 / 60).  Row descriptors, route entries and the payload
# are not looked at by that validator and stay pinned only by the restated layout above.
# ---------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def ref_validate():
    import ctypes
    import os
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    from oracle import build_ref
    path = build_ref.build()
    if path is None:
        pytest.skip("the reference tree is not present and oracle/_ref holds no built validator")
    lib = ctypes.CDLL(path)
    fn = lib.glmrt_ref_validate_protocol_v2_frame
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.c_uint, ctypes.c_char_p, ctypes.c_size_t]

    def validate(frame: bytes, kind: int):
        msg = ctypes.create_string_buffer(256)
        st = fn(frame, len(frame), kind, msg, 256)
        return st, msg.value.decode()
    return validate


def all_test_frames(P):
    """(frame, kind) for every shape of request and response frame the tests of this file build."""
    K = P.ExpertV2SourceKind
    D = P.ExpertV2Dtype
    out = []
    for rows, kind in ((1, K.Decode), (2, K.MtpVerify), (8, K.MtpVerify), (16, K.Prefill), (257, K.Prefill)):
        out.append((make_request(P, rows, kind, hidden_dim=64).encode(), 1))
    out.append((make_request(P, 1, K.Decode).encode(), 1))
    out.append((make_request(P, 3, K.Decode, dtype=D.Nvfp4E2m1Fp8E4m3).encode(), 1))
    out.append((make_request(P, 2, K.Decode, hidden_dim=32, flags=P.EXPERT_PROTOCOL_V2_FLAG_DEBUG_CHECKSUM).encode(), 1))
    out.append((make_request(P, 2, K.Decode, hidden_dim=64, stride=160).encode(), 1))
    ok = P.ExpertProtocolV2Status.Ok
    out.append((P.ExpertProtocolV2Response(42, 9, 3, 1, 6144, D.Bf16, ok, bytes(range(256)) * 48).encode(), 2))
    out.append((P.ExpertProtocolV2Response(1, 1, 0, 2, 64, D.Bf16, ok, b"\x11" * 320, 160).encode(), 2))
    for dtype, row in ((D.Fp8E4m3RowScaled, 6148), (D.Nvfp4E2m1Fp8E4m3, 3456)):
        out.append((P.ExpertProtocolV2Response(7, 1, 2, 2, 6144, dtype, ok, bytes([0x35]) * (2 * row)).encode(), 2))
    chunk = P.ExpertProtocolV2Response(5, 1, 0, 3, 64, D.Bf16, ok, b"\x22" * 384)
    chunk.with_row_indices([4, 0, 9], more_chunks=True)
    out.append((chunk.encode(), 2))
    checked = P.ExpertProtocolV2Response(5, 1, 0, 3, 64, D.Bf16, ok, b"\x22" * 384)
    checked.with_debug_checksum().with_row_indices([2, 1, 0], False)
    out.append((checked.encode(), 2))
    streamed = make_request(P, 4, K.MtpVerify, hidden_dim=64)
    plan = P.ExpertProtocolV2StreamPlan(4, len(streamed.routes), [2, 0, 3, 1],
                                        [P.ExpertProtocolV2StreamRouteGroup(4, list(range(len(streamed.routes))), [0, 1, 2, 3])])
    out += [(f, 1) for f in P.streamed_request_frames(streamed, plan, 3)]
    return out


def test_frames_pass_the_reference_validator(P, ref_validate):
    frames = all_test_frames(P)
    assert len(frames) >= 15
    for frame, kind in frames:
        st, msg = ref_validate(frame, kind)
        assert st == 0, f"reference validator refused a kind-{kind} frame of {len(frame)} bytes: {msg}"
        # the other kind's offsets must not fit: a request is no response
        assert ref_validate(frame, 3 - kind)[0] != 0


def test_reference_validator_and_this_codec_reject_the_same_malformed_frames(P, Err, ref_validate):
    good = make_request(P, 2, P.ExpertV2SourceKind.Decode, hidden_dim=64).encode()
    resp = P.ExpertProtocolV2Response(1, 1, 0, 2, 64, P.ExpertV2Dtype.Bf16, P.ExpertProtocolV2Status.Ok, b"\x11" * 256).encode()
    cases = {
        "short": good[:80],
        "magic": b"X" + good[1:],
        "version": good[:8] + struct.pack("<H", 3) + good[10:],
        "header_len": good[:12] + struct.pack("<I", 128) + good[16:],
        "wire_bytes": good[:76] + struct.pack("<Q", len(good) + 1) + good[84:],
        "truncated": good[:-1],
    }
    for name, frame in cases.items():
        st, msg = ref_validate(frame, 1)
        assert st != 0, name
        with pytest.raises(Err):
            P.ExpertProtocolV2Request.decode(frame)
    bad_resp = resp[:60] + struct.pack("<Q", len(resp) + 4) + resp[68:]
    assert ref_validate(bad_resp, 2)[0] != 0
    with pytest.raises(Err):
        P.ExpertProtocolV2Response.decode(bad_resp)
    # the debug-checksum flag decides the header length: setting it on a 96-byte header is refused by both
    flagged = good[:84] + struct.pack("<I", P.EXPERT_PROTOCOL_V2_FLAG_DEBUG_CHECKSUM) + good[88:]
    assert ref_validate(flagged, 1)[0] != 0
    with pytest.raises(Err):
        P.ExpertProtocolV2Request.decode(flagged)
