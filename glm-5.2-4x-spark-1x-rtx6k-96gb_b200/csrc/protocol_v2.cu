// ExpertProtocolV2 frames (host side): encode, parse and validate regular request and response
// frames in the reference's wire format, and the executor entry point that runs a request frame
// through a layer object.
//
// Wire format restated from rust/crates/glmrt-transport/src/protocol_v2.rs (constants :5-34,
// dtypes :44-83, flag rules :431-497, row descriptor / route entry :515-575, checksum :577-601)
// and protocol_v2/{request.rs:327-633, response.rs:130-277,577-656, view.rs:33-136,299-330}.
// Everything is little-endian.
//
//   request header (96 bytes, 128 with the debug checksum)
//     0 magic "GLMRTE2\0"   8 u16 version = 2   10 u16 kind = 1   12 u32 header_len
//    16 u64 request_id     24 u64 placement_version   32 u32 layer_id   36 u32 row_count
//    40 u32 hidden_dim     44 u16 hidden_dtype  46 u16 0   48 u32 route_count
//    52 u32 row_descriptor_bytes   56 u32 route_bytes   60 u64 hidden_payload_bytes
//    68 u64 logical_payload_bytes  76 u64 wire_bytes    84 u32 flags  88 u32 hidden_row_stride_bytes
//    92 [32-byte SHA-256 of rows, routes, payload when FLAG_DEBUG_CHECKSUM], zero padding
//   then row descriptors (40 bytes: u64 row_id, u16 source_kind, u16 0, u64 source_request_id,
//   u64 token_position, u32 route_offset, u32 route_count, u32 0), route entries (10 bytes: u32
//   row_index, u32 expert_id, bf16 gate weight) and the hidden payload (row_count rows of
//   hidden_row_stride_bytes).
//
//   response header (96 / 128 bytes)
//     0 magic, version, kind = 2, header_len   16 request_id   24 placement_version
//    32 layer_id   36 row_count   40 u16 output_dtype   42 u16 status   44 u64 output_payload_bytes
//    52 u64 logical_payload_bytes   60 u64 wire_bytes   68 u32 flags   72 u32 output_dim
//    76 u32 output_row_stride_bytes   80 u64 executor_id   88 [checksum]
//   then the optional u32 row-index table and the payload.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"
#include "internal.h"

namespace glmrt {
namespace {

constexpr uint8_t kMagic[8] = {'G', 'L', 'M', 'R', 'T', 'E', '2', 0};
constexpr uint16_t kVersion = 2, kRequestKind = 1, kResponseKind = 2;
constexpr size_t kChecksumLen = 32, kRequestChecksumOffset = 92, kResponseChecksumOffset = 88;
constexpr uint32_t kPartCountMask = 0x0fu << GLMRT_B200_PV2_SPARK_COLLECTIVE_PART_COUNT_SHIFT;
constexpr const char* kExecutorName = "b200-nvfp4-tcgen05-executor";

// ---- SHA-256 (FIPS 180-4) ------------------------------------------------------------------
struct Sha256 {
  uint32_t h[8] = {0x6a09e667u, 0xbb67ae85u, 0x3c6ef372u, 0xa54ff53au, 0x510e527fu, 0x9b05688cu, 0x1f83d9abu, 0x5be0cd19u};
  uint8_t block[64];
  size_t fill = 0;
  uint64_t total = 0;

  static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
  void compress(const uint8_t* p) {
    static const uint32_t k[64] = {
        0x428a2f98u, 0x71374491u, 0xb5c0fbcfu, 0xe9b5dba5u, 0x3956c25bu, 0x59f111f1u, 0x923f82a4u, 0xab1c5ed5u,
        0xd807aa98u, 0x12835b01u, 0x243185beu, 0x550c7dc3u, 0x72be5d74u, 0x80deb1feu, 0x9bdc06a7u, 0xc19bf174u,
        0xe49b69c1u, 0xefbe4786u, 0x0fc19dc6u, 0x240ca1ccu, 0x2de92c6fu, 0x4a7484aau, 0x5cb0a9dcu, 0x76f988dau,
        0x983e5152u, 0xa831c66du, 0xb00327c8u, 0xbf597fc7u, 0xc6e00bf3u, 0xd5a79147u, 0x06ca6351u, 0x14292967u,
        0x27b70a85u, 0x2e1b2138u, 0x4d2c6dfcu, 0x53380d13u, 0x650a7354u, 0x766a0abbu, 0x81c2c92eu, 0x92722c85u,
        0xa2bfe8a1u, 0xa81a664bu, 0xc24b8b70u, 0xc76c51a3u, 0xd192e819u, 0xd6990624u, 0xf40e3585u, 0x106aa070u,
        0x19a4c116u, 0x1e376c08u, 0x2748774cu, 0x34b0bcb5u, 0x391c0cb3u, 0x4ed8aa4au, 0x5b9cca4fu, 0x682e6ff3u,
        0x748f82eeu, 0x78a5636fu, 0x84c87814u, 0x8cc70208u, 0x90befffau, 0xa4506cebu, 0xbef9a3f7u, 0xc67178f2u};
    uint32_t w[64];
    for (int i = 0; i < 16; ++i)
      w[i] = (uint32_t(p[4 * i]) << 24) | (uint32_t(p[4 * i + 1]) << 16) | (uint32_t(p[4 * i + 2]) << 8) | p[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
      const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
      const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
    for (int i = 0; i < 64; ++i) {
      const uint32_t t1 = hh + (rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25)) + ((e & f) ^ (~e & g)) + k[i] + w[i];
      const uint32_t t2 = (rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
      hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
  }
  void update(const void* data, size_t len) {
    const uint8_t* p = static_cast<const uint8_t*>(data);
    total += len;
    while (len > 0) {
      const size_t take = std::min(len, sizeof(block) - fill);
      std::memcpy(block + fill, p, take);
      fill += take; p += take; len -= take;
      if (fill == sizeof(block)) { compress(block); fill = 0; }
    }
  }
  void finish(uint8_t out[32]) {
    const uint64_t bits = total * 8;
    const uint8_t one = 0x80, zero = 0;
    update(&one, 1);
    while (fill != 56) update(&zero, 1);
    uint8_t len_be[8];
    for (int i = 0; i < 8; ++i) len_be[i] = static_cast<uint8_t>(bits >> (56 - 8 * i));
    update(len_be, 8);
    for (int i = 0; i < 8; ++i)
      for (int j = 0; j < 4; ++j) out[4 * i + j] = static_cast<uint8_t>(h[i] >> (24 - 8 * j));
  }
};

// ---- little-endian access ------------------------------------------------------------------
void put16(uint8_t* p, uint16_t v) { p[0] = uint8_t(v); p[1] = uint8_t(v >> 8); }
void put32(uint8_t* p, uint32_t v) { for (int i = 0; i < 4; ++i) p[i] = uint8_t(v >> (8 * i)); }
void put64(uint8_t* p, uint64_t v) { for (int i = 0; i < 8; ++i) p[i] = uint8_t(v >> (8 * i)); }
uint16_t get16(const uint8_t* p) { return uint16_t(p[0] | (p[1] << 8)); }
uint32_t get32(const uint8_t* p) { uint32_t v = 0; for (int i = 0; i < 4; ++i) v |= uint32_t(p[i]) << (8 * i); return v; }
uint64_t get64(const uint8_t* p) { uint64_t v = 0; for (int i = 0; i < 8; ++i) v |= uint64_t(p[i]) << (8 * i); return v; }

uint16_t bf16_trunc_bits(float v) { uint32_t b; std::memcpy(&b, &v, 4); return uint16_t(b >> 16); }
float bf16_bits_value(uint16_t bits) { const uint32_t b = uint32_t(bits) << 16; float v; std::memcpy(&v, &b, 4); return v; }

glmrt_status_t bad(const std::string& msg) { return fail(GLMRT_STATUS_INVALID_ARGUMENT, "ExpertProtocolV2 " + msg); }

bool dtype_known(uint32_t d) { return d >= GLMRT_B200_PV2_DTYPE_BF16 && d <= GLMRT_B200_PV2_DTYPE_FP8_E4M3_ROW_SCALED; }

glmrt_status_t row_bytes(uint32_t dtype, size_t elements, size_t* out) {
  switch (dtype) {
    case GLMRT_B200_PV2_DTYPE_BF16:
    case GLMRT_B200_PV2_DTYPE_F16:
      if (elements > SIZE_MAX / 2) return bad("16-bit row byte count overflow");
      *out = elements * 2;
      return GLMRT_STATUS_OK;
    case GLMRT_B200_PV2_DTYPE_FP8_DEBUG:
      *out = elements;
      return GLMRT_STATUS_OK;
    case GLMRT_B200_PV2_DTYPE_NVFP4_E2M1_FP8_E4M3:
      if (elements == 0 || elements % 16 != 0)
        return bad("NVFP4 E2M1 + FP8 E4M3 row width must be a nonzero multiple of 16, got " + std::to_string(elements));
      *out = elements / 2 + elements / 16;
      return GLMRT_STATUS_OK;
    case GLMRT_B200_PV2_DTYPE_FP8_E4M3_ROW_SCALED:
      if (elements > SIZE_MAX - 4) return bad("row-scaled FP8 E4M3 row byte count overflow");
      *out = elements + 4;
      return GLMRT_STATUS_OK;
    default:
      return bad("unknown dtype " + std::to_string(dtype));
  }
}

// validate_flags (protocol_v2.rs:431-497)
glmrt_status_t validate_flags(uint32_t flags, bool request) {
  const uint32_t allowed =
      request ? (GLMRT_B200_PV2_FLAG_DEBUG_CHECKSUM | GLMRT_B200_PV2_FLAG_PRECOMPILE_WARMUP |
                 GLMRT_B200_PV2_FLAG_RESPONSE_FP8_E4M3_ROW_SCALED | GLMRT_B200_PV2_FLAG_RESPONSE_NVFP4_E2M1_FP8_E4M3 |
                 GLMRT_B200_PV2_FLAG_STREAM_PLAN | GLMRT_B200_PV2_FLAG_STREAM_DATA | GLMRT_B200_PV2_FLAG_STREAM_FINAL |
                 GLMRT_B200_PV2_FLAG_SPARK_REDUCTION | GLMRT_B200_PV2_FLAG_SPARK_ROW_SHARDED_REDUCTION | kPartCountMask |
                 GLMRT_B200_PV2_FLAG_LAYER_BLOCK)
              : (GLMRT_B200_PV2_FLAG_DEBUG_CHECKSUM | GLMRT_B200_PV2_FLAG_RESPONSE_ROW_INDICES |
                 GLMRT_B200_PV2_FLAG_RESPONSE_MORE_CHUNKS);
  const char* label = request ? "request" : "response";
  if (flags & ~allowed) {
    char buf[16];
    snprintf(buf, sizeof(buf), "0x%08x", flags & ~allowed);
    return bad(std::string(label) + " has unknown flags " + buf);
  }
  if (!request) return GLMRT_STATUS_OK;
  auto on = [&](uint32_t f) { return (flags & f) != 0; };
  if (on(GLMRT_B200_PV2_FLAG_RESPONSE_FP8_E4M3_ROW_SCALED) && on(GLMRT_B200_PV2_FLAG_RESPONSE_NVFP4_E2M1_FP8_E4M3))
    return bad("request selects multiple low-precision response dtypes");
  const bool plan = on(GLMRT_B200_PV2_FLAG_STREAM_PLAN), data = on(GLMRT_B200_PV2_FLAG_STREAM_DATA);
  if (plan && data) return bad("request cannot be both a stream plan and stream data frame");
  if (on(GLMRT_B200_PV2_FLAG_STREAM_FINAL) && !data) return bad("stream-final flag requires a stream data frame");
  const bool spark = on(GLMRT_B200_PV2_FLAG_SPARK_REDUCTION), sharded = on(GLMRT_B200_PV2_FLAG_SPARK_ROW_SHARDED_REDUCTION);
  if (sharded && !spark) return bad("row-sharded reduction requires Spark reduction");
  const uint32_t parts = (flags & kPartCountMask) >> GLMRT_B200_PV2_SPARK_COLLECTIVE_PART_COUNT_SHIFT;
  if (parts == 1) return bad("striped Spark collective requires at least two parts");
  if (parts > 0 && !sharded) return bad("striped Spark collective requires row-sharded reduction");
  const bool warm = on(GLMRT_B200_PV2_FLAG_PRECOMPILE_WARMUP);
  if (warm && (plan || data)) return bad("precompile warmup cannot use streamed ingress frames");
  if (on(GLMRT_B200_PV2_FLAG_LAYER_BLOCK) && (plan || data || spark || warm))
    return bad("layer-block requests cannot be stream, Spark-reduction, or precompile frames");
  return GLMRT_STATUS_OK;
}

size_t header_len_for(uint32_t flags) {
  return (flags & GLMRT_B200_PV2_FLAG_DEBUG_CHECKSUM) ? GLMRT_B200_PV2_DEBUG_HEADER_LEN : GLMRT_B200_PV2_REQUEST_HEADER_LEN;
}

// validate_common_header (protocol_v2.rs:499-513)
glmrt_status_t common_header(const uint8_t* b, uint16_t kind, size_t* header_len) {
  if (std::memcmp(b, kMagic, 8) != 0) return bad("invalid magic");
  if (get16(b + 8) != kVersion) return bad("unsupported version " + std::to_string(get16(b + 8)));
  if (get16(b + 10) != kind) return bad("unexpected message kind " + std::to_string(get16(b + 10)));
  *header_len = get32(b + 12);
  return GLMRT_STATUS_OK;
}

void encode_row(uint8_t* p, const glmrt_b200_pv2_row_t& r) {
  put64(p, r.row_id); put16(p + 8, uint16_t(r.source_kind)); put16(p + 10, 0); put64(p + 12, r.source_request_id);
  put64(p + 20, r.token_position); put32(p + 28, r.route_offset); put32(p + 32, r.route_count); put32(p + 36, 0);
}
glmrt_status_t decode_row(const uint8_t* p, glmrt_b200_pv2_row_t* r) {
  r->row_id = get64(p); r->source_kind = get16(p + 8); r->source_request_id = get64(p + 12);
  r->token_position = get64(p + 20); r->route_offset = get32(p + 28); r->route_count = get32(p + 32); r->reserved = 0;
  if (r->source_kind < 1 || r->source_kind > 4) return bad("unknown source kind " + std::to_string(r->source_kind));
  return GLMRT_STATUS_OK;
}
void encode_route(uint8_t* p, const glmrt_b200_pv2_route_t& r) {
  put32(p, r.row_index); put32(p + 4, r.expert_id); put16(p + 8, bf16_trunc_bits(r.gate_weight));
}
void decode_route(const uint8_t* p, glmrt_b200_pv2_route_t* r) {
  r->row_index = get32(p); r->expert_id = get32(p + 4); r->gate_weight = bf16_bits_value(get16(p + 8));
}

// The row / route / payload rules of Request::validate (request.rs:516-633) for a regular,
// stream-plan or layer-block frame whose sections are laid out in memory as on the wire.
glmrt_status_t validate_request_body(const glmrt_b200_pv2_request_header_t& h, const uint8_t* rows, const uint8_t* routes) {
  const bool plan = h.flags & GLMRT_B200_PV2_FLAG_STREAM_PLAN, layer_block = h.flags & GLMRT_B200_PV2_FLAG_LAYER_BLOCK;
  if (plan && h.row_count == 0) return bad("stream plan must contain at least one row");
  if (layer_block && h.route_count != 0) return bad("layer-block request cannot contain precomputed routes");
  if (h.hidden_dim == 0) return bad("request hidden_dim must be non-zero");
  size_t logical = 0;
  GLMRT_RETURN_IF_ERROR(row_bytes(h.hidden_dtype, h.hidden_dim, &logical));
  if (h.hidden_row_stride_bytes < logical)
    return bad("request hidden row stride bytes " + std::to_string(h.hidden_row_stride_bytes) +
               " smaller than logical row bytes " + std::to_string(logical));
  if (plan) {
    if (h.hidden_payload_bytes == 0) return bad("stream plan payload must be non-empty");
  } else {
    const uint64_t expected = uint64_t(h.row_count) * h.hidden_row_stride_bytes;
    if (expected != h.hidden_payload_bytes)
      return bad("request hidden payload bytes mismatch: expected=" + std::to_string(expected) +
                 " actual=" + std::to_string(h.hidden_payload_bytes));
  }
  for (uint32_t i = 0; i < h.row_count; ++i) {
    glmrt_b200_pv2_row_t r;
    GLMRT_RETURN_IF_ERROR(decode_row(rows + size_t(i) * GLMRT_B200_PV2_ROW_DESCRIPTOR_LEN, &r));
    if (layer_block && (r.route_offset != 0 || r.route_count != 0))
      return bad("layer-block row " + std::to_string(i) + " must not contain precomputed routes");
    const uint64_t end = uint64_t(r.route_offset) + r.route_count;
    if (end > 0xffffffffull) return bad("row route range overflow");
    if (end > h.route_count)
      return bad("row " + std::to_string(i) + " route range " + std::to_string(r.route_offset) + ".." +
                 std::to_string(end) + " exceeds route count " + std::to_string(h.route_count));
  }
  for (uint32_t i = 0; i < h.route_count; ++i) {
    glmrt_b200_pv2_route_t r;
    decode_route(routes + size_t(i) * GLMRT_B200_PV2_ROUTE_ENTRY_LEN, &r);
    if (r.row_index >= h.row_count)
      return bad("route row_index " + std::to_string(r.row_index) + " exceeds row count " + std::to_string(h.row_count));
    if (!std::isfinite(r.gate_weight)) return bad("route gate_weight must be finite");
  }
  return GLMRT_STATUS_OK;
}

void request_checksum(const uint8_t* rows, size_t rows_bytes, const uint8_t* routes, size_t routes_bytes,
                      const uint8_t* payload, size_t payload_bytes, uint8_t out[32]) {
  Sha256 s;   // payload_checksum (protocol_v2.rs:577-601): the encoded rows, the encoded routes, the payload
  s.update(rows, rows_bytes);
  s.update(routes, routes_bytes);
  s.update(payload, payload_bytes);
  s.finish(out);
}

}  // namespace
}  // namespace glmrt

using namespace glmrt;

extern "C" glmrt_status_t glmrt_b200_pv2_row_bytes(uint32_t dtype, size_t elements, size_t* out_bytes) {
  if (out_bytes == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "pv2_row_bytes: null output");
  GLMRT_RETURN_IF_ERROR(row_bytes(dtype, elements, out_bytes));
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_pv2_sha256(const void* bytes, size_t len, uint8_t out_digest[32]) {
  if ((bytes == nullptr && len != 0) || out_digest == nullptr)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "pv2_sha256: null pointer argument");
  Sha256 s;
  s.update(bytes, len);
  s.finish(out_digest);
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_pv2_compact_id(const char* name, uint64_t* out_id) {
  if (name == nullptr || out_id == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "pv2_compact_id: null pointer argument");
  uint8_t d[32];
  Sha256 s;
  s.update(name, std::strlen(name));
  s.finish(d);
  *out_id = get64(d);
  return ok();
}

// ---- request frames ------------------------------------------------------------------------
extern "C" glmrt_status_t glmrt_b200_pv2_encode_request(const glmrt_b200_pv2_request_header_t* header,
                                                        const glmrt_b200_pv2_row_t* rows, size_t row_count,
                                                        const glmrt_b200_pv2_route_t* routes, size_t route_count,
                                                        const void* hidden_payload, size_t hidden_payload_bytes,
                                                        void* out, size_t out_capacity, size_t* out_len) {
  if (header == nullptr || out_len == nullptr || (rows == nullptr && row_count != 0) ||
      (routes == nullptr && route_count != 0) || (hidden_payload == nullptr && hidden_payload_bytes != 0))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "pv2_encode_request: null pointer argument");
  if (row_count > 0xffffffffull / GLMRT_B200_PV2_ROW_DESCRIPTOR_LEN) return bad("row descriptor bytes exceeds u32");
  if (route_count > 0xffffffffull / GLMRT_B200_PV2_ROUTE_ENTRY_LEN) return bad("route bytes exceeds u32");
  glmrt_b200_pv2_request_header_t h = *header;
  GLMRT_RETURN_IF_ERROR(validate_flags(h.flags, true));
  if (h.flags & GLMRT_B200_PV2_FLAG_STREAM_DATA)
    return bad("stream data frames are not built by this encoder");
  if (!dtype_known(h.hidden_dtype)) return bad("unknown dtype " + std::to_string(h.hidden_dtype));
  if (h.hidden_row_stride_bytes == 0) {   // default_hidden_row_stride_bytes (request.rs:643-651)
    size_t logical = 0;
    if (h.hidden_dim == 0) return bad("request hidden_dim must be non-zero");
    GLMRT_RETURN_IF_ERROR(row_bytes(h.hidden_dtype, h.hidden_dim, &logical));
    if (logical > 0xffffffffull) return bad("hidden row stride bytes exceeds u32");
    h.hidden_row_stride_bytes = static_cast<uint32_t>(logical);
  }
  h.row_count = static_cast<uint32_t>(row_count);
  h.route_count = static_cast<uint32_t>(route_count);
  h.row_descriptor_bytes = static_cast<uint32_t>(row_count * GLMRT_B200_PV2_ROW_DESCRIPTOR_LEN);
  h.route_bytes = static_cast<uint32_t>(route_count * GLMRT_B200_PV2_ROUTE_ENTRY_LEN);
  h.hidden_payload_bytes = hidden_payload_bytes;
  h.header_len = static_cast<uint32_t>(header_len_for(h.flags));

  const size_t prefix = h.header_len + h.row_descriptor_bytes + h.route_bytes;
  const size_t wire = prefix + hidden_payload_bytes;
  // rows and routes in wire form first: validation and the checksum read the encoded bytes
  std::vector<uint8_t> body(h.row_descriptor_bytes + h.route_bytes);
  for (size_t i = 0; i < row_count; ++i) {
    if (rows[i].source_kind < 1 || rows[i].source_kind > 4)
      return bad("unknown source kind " + std::to_string(rows[i].source_kind));
    encode_row(body.data() + i * GLMRT_B200_PV2_ROW_DESCRIPTOR_LEN, rows[i]);
  }
  uint8_t* route_bytes = body.data() + h.row_descriptor_bytes;
  for (size_t i = 0; i < route_count; ++i) encode_route(route_bytes + i * GLMRT_B200_PV2_ROUTE_ENTRY_LEN, routes[i]);
  GLMRT_RETURN_IF_ERROR(validate_request_body(h, body.data(), route_bytes));
  *out_len = wire;
  if (out == nullptr || out_capacity < wire)
    return fail(GLMRT_STATUS_BUFFER_TOO_SMALL, "pv2_encode_request: output buffer too small for " + std::to_string(wire) + " bytes");

  uint8_t* b = static_cast<uint8_t*>(out);
  std::memset(b, 0, h.header_len);
  std::memcpy(b, kMagic, 8);
  put16(b + 8, kVersion); put16(b + 10, kRequestKind); put32(b + 12, h.header_len);
  put64(b + 16, h.request_id); put64(b + 24, h.placement_version); put32(b + 32, h.layer_id);
  put32(b + 36, h.row_count); put32(b + 40, h.hidden_dim); put16(b + 44, uint16_t(h.hidden_dtype)); put16(b + 46, 0);
  put32(b + 48, h.route_count); put32(b + 52, h.row_descriptor_bytes); put32(b + 56, h.route_bytes);
  put64(b + 60, h.hidden_payload_bytes); put64(b + 68, hidden_payload_bytes /* logical payload bytes */);
  put64(b + 76, wire); put32(b + 84, h.flags); put32(b + 88, h.hidden_row_stride_bytes);
  if (h.flags & GLMRT_B200_PV2_FLAG_DEBUG_CHECKSUM)
    request_checksum(body.data(), h.row_descriptor_bytes, route_bytes, h.route_bytes,
                     static_cast<const uint8_t*>(hidden_payload), hidden_payload_bytes, b + kRequestChecksumOffset);
  std::memcpy(b + h.header_len, body.data(), body.size());
  if (hidden_payload_bytes != 0) std::memcpy(b + prefix, hidden_payload, hidden_payload_bytes);
  return ok();
}

namespace glmrt {
namespace {

glmrt_status_t parse_request(const uint8_t* b, size_t n, glmrt_b200_pv2_request_header_t* h, glmrt_b200_pv2_sections_t* s) {
  if (n < GLMRT_B200_PV2_REQUEST_HEADER_LEN) return bad("request frame too short: " + std::to_string(n));
  size_t header_len = 0;
  GLMRT_RETURN_IF_ERROR(common_header(b, kRequestKind, &header_len));
  h->request_id = get64(b + 16); h->placement_version = get64(b + 24); h->layer_id = get32(b + 32);
  h->row_count = get32(b + 36); h->hidden_dim = get32(b + 40); h->hidden_dtype = get16(b + 44);
  h->route_count = get32(b + 48); h->row_descriptor_bytes = get32(b + 52); h->route_bytes = get32(b + 56);
  h->hidden_payload_bytes = get64(b + 60);
  const uint64_t wire = get64(b + 76);
  h->flags = get32(b + 84); h->hidden_row_stride_bytes = get32(b + 88);
  h->header_len = static_cast<uint32_t>(header_len);
  if (!dtype_known(h->hidden_dtype)) return bad("unknown dtype " + std::to_string(h->hidden_dtype));
  GLMRT_RETURN_IF_ERROR(validate_flags(h->flags, true));
  if (header_len != header_len_for(h->flags))
    return bad("header length mismatch: header=" + std::to_string(header_len) + " expected=" + std::to_string(header_len_for(h->flags)));
  if (n < header_len) return bad("request frame shorter than declared header");
  if (wire != n) return bad("request wire bytes mismatch: header=" + std::to_string(wire) + " actual=" + std::to_string(n));
  const bool data = h->flags & GLMRT_B200_PV2_FLAG_STREAM_DATA;
  const uint64_t rows_len = data ? 0 : h->row_count, routes_len = data ? 0 : h->route_count;
  if (h->row_descriptor_bytes != rows_len * GLMRT_B200_PV2_ROW_DESCRIPTOR_LEN)
    return bad("request row descriptor bytes mismatch: header=" + std::to_string(h->row_descriptor_bytes));
  if (h->route_bytes != routes_len * GLMRT_B200_PV2_ROUTE_ENTRY_LEN)
    return bad("request route bytes mismatch: header=" + std::to_string(h->route_bytes));
  const uint64_t rows_start = header_len, routes_start = rows_start + h->row_descriptor_bytes,
                 payload_start = routes_start + h->route_bytes;
  if (h->hidden_payload_bytes > n || payload_start + h->hidden_payload_bytes != n)
    return bad("request length mismatch: sections end at " + std::to_string(payload_start + h->hidden_payload_bytes) +
               ", frame has " + std::to_string(n));
  if (data) {   // request.rs:521-531: no descriptors, route_count is the row offset into the plan
    if (h->row_count == 0) return bad("stream data frame must contain at least one row");
    if (uint64_t(h->route_count) + h->row_count > 0xffffffffull) return bad("stream data row range overflow");
    if (h->hidden_dim == 0) return bad("request hidden_dim must be non-zero");
    size_t logical = 0;
    GLMRT_RETURN_IF_ERROR(row_bytes(h->hidden_dtype, h->hidden_dim, &logical));
    if (h->hidden_row_stride_bytes < logical) return bad("request hidden row stride bytes smaller than logical row bytes");
    if (uint64_t(h->row_count) * h->hidden_row_stride_bytes != h->hidden_payload_bytes)
      return bad("request hidden payload bytes mismatch");
  } else {
    GLMRT_RETURN_IF_ERROR(validate_request_body(*h, b + rows_start, b + routes_start));
  }
  if (s != nullptr) {
    s->rows_offset = rows_start; s->routes_offset = routes_start; s->payload_offset = payload_start;
    s->payload_bytes = h->hidden_payload_bytes;
  }
  return GLMRT_STATUS_OK;
}

glmrt_status_t validate_response(const glmrt_b200_pv2_response_header_t& h, const uint32_t* row_indices, bool have_indices,
                                 size_t payload_bytes) {
  // validate_response_shape (response.rs:585-642)
  GLMRT_RETURN_IF_ERROR(validate_flags(h.flags, false));
  if (h.status > 1) return bad("unknown response status " + std::to_string(h.status));
  const bool indexed = h.flags & GLMRT_B200_PV2_FLAG_RESPONSE_ROW_INDICES;
  if (indexed != have_indices) return bad("response row-index flag and row index table disagree");
  if ((h.flags & GLMRT_B200_PV2_FLAG_RESPONSE_MORE_CHUNKS) && !indexed) return bad("response more-chunks flag requires row indices");
  if (indexed) {
    std::vector<uint32_t> sorted(row_indices, row_indices + h.row_count);
    std::sort(sorted.begin(), sorted.end());
    if (std::adjacent_find(sorted.begin(), sorted.end()) != sorted.end())
      return bad("response row indices must be unique within a chunk");
  }
  if (h.output_dim == 0) return bad("response output_dim must be non-zero");
  size_t logical = 0;
  GLMRT_RETURN_IF_ERROR(row_bytes(h.output_dtype, h.output_dim, &logical));
  if (h.output_row_stride_bytes < logical)
    return bad("response output row stride bytes " + std::to_string(h.output_row_stride_bytes) +
               " smaller than logical row bytes " + std::to_string(logical));
  if (uint64_t(h.row_count) * h.output_row_stride_bytes != payload_bytes)
    return bad("response output payload bytes mismatch: expected=" +
               std::to_string(uint64_t(h.row_count) * h.output_row_stride_bytes) + " actual=" + std::to_string(payload_bytes));
  if (h.output_payload_bytes != payload_bytes) return bad("response output_payload_bytes mismatch");
  return GLMRT_STATUS_OK;
}

void response_checksum(const uint8_t* index_bytes, size_t index_len, const uint8_t* payload, size_t payload_bytes, uint8_t out[32]) {
  Sha256 s;   // frame_content_checksum (response.rs:644-656): the row-index table as on the wire, then the payload
  s.update(index_bytes, index_len);
  s.update(payload, payload_bytes);
  s.finish(out);
}

glmrt_status_t parse_response(const uint8_t* b, size_t n, glmrt_b200_pv2_response_header_t* h, glmrt_b200_pv2_sections_t* s) {
  if (n < GLMRT_B200_PV2_RESPONSE_HEADER_LEN) return bad("response frame too short: " + std::to_string(n));
  size_t header_len = 0;
  GLMRT_RETURN_IF_ERROR(common_header(b, kResponseKind, &header_len));
  h->request_id = get64(b + 16); h->placement_version = get64(b + 24); h->layer_id = get32(b + 32);
  h->row_count = get32(b + 36); h->output_dtype = get16(b + 40); h->status = get16(b + 42);
  h->output_payload_bytes = get64(b + 44);
  const uint64_t wire = get64(b + 60);
  h->flags = get32(b + 68); h->output_dim = get32(b + 72); h->output_row_stride_bytes = get32(b + 76);
  h->executor_id = get64(b + 80); h->header_len = static_cast<uint32_t>(header_len);
  if (!dtype_known(h->output_dtype)) return bad("unknown dtype " + std::to_string(h->output_dtype));
  GLMRT_RETURN_IF_ERROR(validate_flags(h->flags, false));
  if (header_len != header_len_for(h->flags)) return bad("header length mismatch: header=" + std::to_string(header_len));
  if (n < header_len) return bad("response frame shorter than declared header");
  if (wire != n) return bad("response wire bytes mismatch: header=" + std::to_string(wire) + " actual=" + std::to_string(n));
  const bool indexed = h->flags & GLMRT_B200_PV2_FLAG_RESPONSE_ROW_INDICES;
  const uint64_t index_bytes = indexed ? uint64_t(h->row_count) * 4 : 0;
  const uint64_t payload_start = header_len + index_bytes;
  if (h->output_payload_bytes > n || payload_start + h->output_payload_bytes != n)
    return bad("response length mismatch: sections end at " + std::to_string(payload_start + h->output_payload_bytes) +
               ", frame has " + std::to_string(n));
  std::vector<uint32_t> idx(indexed ? h->row_count : 0);
  for (size_t i = 0; i < idx.size(); ++i) idx[i] = get32(b + header_len + 4 * i);
  GLMRT_RETURN_IF_ERROR(validate_response(*h, idx.data(), indexed, h->output_payload_bytes));
  if (s != nullptr) {
    s->rows_offset = header_len; s->routes_offset = payload_start; s->payload_offset = payload_start;
    s->payload_bytes = h->output_payload_bytes;
  }
  return GLMRT_STATUS_OK;
}

}  // namespace
}  // namespace glmrt

extern "C" glmrt_status_t glmrt_b200_pv2_parse_request(const void* frame, size_t frame_bytes,
                                                       glmrt_b200_pv2_request_header_t* out_header,
                                                       glmrt_b200_pv2_sections_t* out_sections) {
  if (frame == nullptr || out_header == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "pv2_parse_request: null pointer argument");
  GLMRT_RETURN_IF_ERROR(parse_request(static_cast<const uint8_t*>(frame), frame_bytes, out_header, out_sections));
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_pv2_request_row(const void* frame, size_t frame_bytes, size_t index,
                                                     glmrt_b200_pv2_row_t* out_row) {
  if (frame == nullptr || out_row == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "pv2_request_row: null pointer argument");
  glmrt_b200_pv2_request_header_t h;
  glmrt_b200_pv2_sections_t s;
  const uint8_t* b = static_cast<const uint8_t*>(frame);
  GLMRT_RETURN_IF_ERROR(parse_request(b, frame_bytes, &h, &s));
  if (index >= h.row_descriptor_bytes / GLMRT_B200_PV2_ROW_DESCRIPTOR_LEN)
    return bad("row index " + std::to_string(index) + " out of range");
  GLMRT_RETURN_IF_ERROR(decode_row(b + s.rows_offset + index * GLMRT_B200_PV2_ROW_DESCRIPTOR_LEN, out_row));
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_pv2_request_route(const void* frame, size_t frame_bytes, size_t index,
                                                       glmrt_b200_pv2_route_t* out_route) {
  if (frame == nullptr || out_route == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "pv2_request_route: null pointer argument");
  glmrt_b200_pv2_request_header_t h;
  glmrt_b200_pv2_sections_t s;
  const uint8_t* b = static_cast<const uint8_t*>(frame);
  GLMRT_RETURN_IF_ERROR(parse_request(b, frame_bytes, &h, &s));
  if (index >= h.route_bytes / GLMRT_B200_PV2_ROUTE_ENTRY_LEN) return bad("route index " + std::to_string(index) + " out of range");
  decode_route(b + s.routes_offset + index * GLMRT_B200_PV2_ROUTE_ENTRY_LEN, out_route);
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_pv2_verify_request_checksum(const void* frame, size_t frame_bytes) {
  if (frame == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "pv2_verify_request_checksum: null frame");
  glmrt_b200_pv2_request_header_t h;
  glmrt_b200_pv2_sections_t s;
  const uint8_t* b = static_cast<const uint8_t*>(frame);
  GLMRT_RETURN_IF_ERROR(parse_request(b, frame_bytes, &h, &s));
  if (!(h.flags & GLMRT_B200_PV2_FLAG_DEBUG_CHECKSUM)) return ok();
  uint8_t d[32];
  request_checksum(b + s.rows_offset, h.row_descriptor_bytes, b + s.routes_offset, h.route_bytes, b + s.payload_offset,
                   s.payload_bytes, d);
  if (std::memcmp(d, b + kRequestChecksumOffset, kChecksumLen) != 0) return bad("request checksum mismatch");
  return ok();
}

// ---- response frames -----------------------------------------------------------------------
extern "C" glmrt_status_t glmrt_b200_pv2_encode_response(const glmrt_b200_pv2_response_header_t* header,
                                                         const uint32_t* row_indices, const void* payload,
                                                         size_t payload_bytes, void* out, size_t out_capacity,
                                                         size_t* out_len) {
  if (header == nullptr || out_len == nullptr || (payload == nullptr && payload_bytes != 0))
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "pv2_encode_response: null pointer argument");
  glmrt_b200_pv2_response_header_t h = *header;
  if (!dtype_known(h.output_dtype)) return bad("unknown dtype " + std::to_string(h.output_dtype));
  if (h.output_row_stride_bytes == 0 && h.output_dim != 0) {   // default_output_row_stride_bytes (response.rs:658-665)
    size_t logical = 0;
    GLMRT_RETURN_IF_ERROR(row_bytes(h.output_dtype, h.output_dim, &logical));
    h.output_row_stride_bytes = static_cast<uint32_t>(logical);
  }
  h.output_payload_bytes = payload_bytes;
  h.header_len = static_cast<uint32_t>(header_len_for(h.flags));
  GLMRT_RETURN_IF_ERROR(validate_response(h, row_indices, row_indices != nullptr, payload_bytes));
  const bool indexed = h.flags & GLMRT_B200_PV2_FLAG_RESPONSE_ROW_INDICES;
  const size_t index_bytes = indexed ? size_t(h.row_count) * 4 : 0;
  const size_t wire = h.header_len + index_bytes + payload_bytes;
  *out_len = wire;
  if (out == nullptr || out_capacity < wire)
    return fail(GLMRT_STATUS_BUFFER_TOO_SMALL, "pv2_encode_response: output buffer too small for " + std::to_string(wire) + " bytes");
  uint8_t* b = static_cast<uint8_t*>(out);
  std::memset(b, 0, h.header_len);
  std::memcpy(b, kMagic, 8);
  put16(b + 8, kVersion); put16(b + 10, kResponseKind); put32(b + 12, h.header_len);
  put64(b + 16, h.request_id); put64(b + 24, h.placement_version); put32(b + 32, h.layer_id); put32(b + 36, h.row_count);
  put16(b + 40, uint16_t(h.output_dtype)); put16(b + 42, uint16_t(h.status)); put64(b + 44, h.output_payload_bytes);
  put64(b + 52, payload_bytes /* logical payload bytes */); put64(b + 60, wire); put32(b + 68, h.flags);
  put32(b + 72, h.output_dim); put32(b + 76, h.output_row_stride_bytes); put64(b + 80, h.executor_id);
  for (size_t i = 0; i < index_bytes / 4; ++i) put32(b + h.header_len + 4 * i, row_indices[i]);
  if (payload_bytes != 0 && payload != b + h.header_len + index_bytes)
    std::memmove(b + h.header_len + index_bytes, payload, payload_bytes);   // the payload may already be in place
  if (h.flags & GLMRT_B200_PV2_FLAG_DEBUG_CHECKSUM)
    response_checksum(b + h.header_len, index_bytes, b + h.header_len + index_bytes, payload_bytes, b + kResponseChecksumOffset);
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_pv2_parse_response(const void* frame, size_t frame_bytes,
                                                        glmrt_b200_pv2_response_header_t* out_header,
                                                        glmrt_b200_pv2_sections_t* out_sections) {
  if (frame == nullptr || out_header == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "pv2_parse_response: null pointer argument");
  GLMRT_RETURN_IF_ERROR(parse_response(static_cast<const uint8_t*>(frame), frame_bytes, out_header, out_sections));
  return ok();
}

extern "C" glmrt_status_t glmrt_b200_pv2_verify_response_checksum(const void* frame, size_t frame_bytes) {
  if (frame == nullptr) return fail(GLMRT_STATUS_INVALID_ARGUMENT, "pv2_verify_response_checksum: null frame");
  glmrt_b200_pv2_response_header_t h;
  glmrt_b200_pv2_sections_t s;
  const uint8_t* b = static_cast<const uint8_t*>(frame);
  GLMRT_RETURN_IF_ERROR(parse_response(b, frame_bytes, &h, &s));
  if (!(h.flags & GLMRT_B200_PV2_FLAG_DEBUG_CHECKSUM)) return ok();
  uint8_t d[32];
  response_checksum(b + s.rows_offset, s.payload_offset - s.rows_offset, b + s.payload_offset, s.payload_bytes, d);
  if (std::memcmp(d, b + kResponseChecksumOffset, kChecksumLen) != 0) return bad("response checksum mismatch");
  return ok();
}

// ---- executor ------------------------------------------------------------------------------
namespace glmrt {
namespace {

// The layer's view of a request: [rows, top_k] route tables (unused entries kNoRoute).
struct RouteTables {
  std::vector<uint32_t> idx;
  std::vector<float> w;
};

glmrt_status_t build_route_tables(const uint8_t* b, const glmrt_b200_pv2_request_header_t& h,
                                  const glmrt_b200_pv2_sections_t& sec, const LayerDims& d, RouteTables* t) {
  const size_t rows = h.row_count;
  t->idx.assign(rows * d.top_k, kNoRoute);
  t->w.assign(rows * d.top_k, 0.0f);
  for (size_t i = 0; i < rows; ++i) {
    glmrt_b200_pv2_row_t row;
    GLMRT_RETURN_IF_ERROR(decode_row(b + sec.rows_offset + i * GLMRT_B200_PV2_ROW_DESCRIPTOR_LEN, &row));
    if (row.route_count > d.top_k)
      return bad("executor: row " + std::to_string(i) + " has " + std::to_string(row.route_count) + " routes, the layer's top_k is " +
                 std::to_string(d.top_k));
    for (uint32_t k = 0; k < row.route_count; ++k) {
      glmrt_b200_pv2_route_t r;
      decode_route(b + sec.routes_offset + (size_t(row.route_offset) + k) * GLMRT_B200_PV2_ROUTE_ENTRY_LEN, &r);
      if (r.row_index != i)
        return bad("executor: route row_index " + std::to_string(r.row_index) + " did not match row " + std::to_string(i));
      if (r.expert_id >= d.experts || r.expert_id % d.ep_world != d.ep_rank)
        return bad("executor: expert " + std::to_string(r.expert_id) + " does not live on this shard");
      t->idx[i * d.top_k + k] = r.expert_id;
      t->w[i * d.top_k + k] = r.gate_weight;
    }
  }
  return GLMRT_STATUS_OK;
}

glmrt_status_t check_request_against_layer(const glmrt_b200_pv2_request_header_t& h, const LayerDims& d, uint32_t total_rows,
                                           bool* in_payload) {
  if (h.hidden_dim != d.hidden)
    return bad("executor: request hidden_dim " + std::to_string(h.hidden_dim) + " does not match the layer's " + std::to_string(d.hidden));
  *in_payload = h.hidden_dtype == GLMRT_B200_PV2_DTYPE_NVFP4_E2M1_FP8_E4M3;
  if (!*in_payload && h.hidden_dtype != GLMRT_B200_PV2_DTYPE_BF16)
    return bad("executor: hidden dtype must be bf16 or NVFP4 E2M1 + FP8 E4M3, got " + std::to_string(h.hidden_dtype));
  if (total_rows == 0) return bad("executor: request has no rows");
  if (total_rows > d.max_tokens)
    return bad("executor: " + std::to_string(total_rows) + " rows exceed the layer's max_tokens " + std::to_string(d.max_tokens));
  return GLMRT_STATUS_OK;
}

// Runs `rows` hidden rows (host memory, `stride` bytes apart) with their route tables and frames the response.
glmrt_status_t run_and_frame(void* layer, const glmrt_b200_pv2_request_header_t& h, uint32_t rows, const uint8_t* hidden,
                             size_t stride, bool in_payload, const RouteTables& t, void* response_out, size_t response_capacity,
                             size_t* response_len, cudaStream_t stream) {
  glmrt_b200_pv2_response_header_t rh{};
  rh.request_id = h.request_id; rh.placement_version = h.placement_version; rh.layer_id = h.layer_id;
  rh.row_count = rows; rh.output_dim = h.hidden_dim;
  // response dtype negotiated by the request's flags (view.rs:258-264)
  const int out_kind = (h.flags & GLMRT_B200_PV2_FLAG_RESPONSE_NVFP4_E2M1_FP8_E4M3)   ? kOutNvfp4Payload
                       : (h.flags & GLMRT_B200_PV2_FLAG_RESPONSE_FP8_E4M3_ROW_SCALED) ? kOutFp8RowScaled
                                                                                       : kOutBf16;
  rh.output_dtype = out_kind == kOutNvfp4Payload   ? GLMRT_B200_PV2_DTYPE_NVFP4_E2M1_FP8_E4M3
                    : out_kind == kOutFp8RowScaled ? GLMRT_B200_PV2_DTYPE_FP8_E4M3_ROW_SCALED
                                                   : GLMRT_B200_PV2_DTYPE_BF16;
  size_t out_row = 0;
  GLMRT_RETURN_IF_ERROR(row_bytes(rh.output_dtype, rh.output_dim, &out_row));
  rh.output_row_stride_bytes = static_cast<uint32_t>(out_row);
  rh.status = 0;
  // a response to a checksummed request carries a checksum too (synthetic.rs with_matching_debug_checksum)
  rh.flags = h.flags & GLMRT_B200_PV2_FLAG_DEBUG_CHECKSUM;
  GLMRT_RETURN_IF_ERROR(glmrt_b200_pv2_compact_id(kExecutorName, &rh.executor_id));
  const size_t header_len = header_len_for(rh.flags), payload_bytes = size_t(rows) * out_row, wire = header_len + payload_bytes;
  *response_len = wire;
  if (response_out == nullptr || response_capacity < wire)
    return fail(GLMRT_STATUS_BUFFER_TOO_SMALL, "pv2_execute: response buffer too small for " + std::to_string(wire) + " bytes");
  uint8_t* out = static_cast<uint8_t*>(response_out);
  // the partial output rows land directly behind the header
  GLMRT_RETURN_IF_ERROR(layer_execute_host_rows(layer, hidden, in_payload, stride, rows, t.idx.data(), t.w.data(), out_kind,
                                                out + header_len, out_row, stream));
  return glmrt_b200_pv2_encode_response(&rh, nullptr, out + header_len, payload_bytes, out, response_capacity, response_len);
}

// ---- streamed ingress (protocol_v2/stream.rs:9-27; executor side: protocol_v2_executor.rs:1936-1945) ----
// A stream-plan frame carries the request's rows and routes and, as its payload, a "GLMSTRM2" plan:
// the order in which the hidden rows will arrive and, for the sender's benefit, groups of routes that
// become ready after so many rows.  Stream-data frames follow, each with a run of hidden rows in that
// order (their route_count field is the position of the first row); the last one carries the
// stream-final flag.  The reference starts expert work group by group while rows are still arriving;
// this executor stages the rows as they come and runs the request when the final frame is in, which
// gives the same response as the regular request (the reference tests exactly that equality).
struct StreamSession {
  glmrt_b200_pv2_request_header_t head{};
  RouteTables tables;
  std::vector<uint32_t> order;      // activation_row_order
  std::vector<uint8_t> hidden;      // staged rows, request order, `stride` bytes each
  std::vector<uint8_t> have;
  size_t stride = 0, received = 0;
  bool in_payload = false;
};
std::mutex g_stream_mutex;
std::map<void*, StreamSession> g_streams;    // one pending streamed request per layer handle (lane)

constexpr size_t kStreamPlanHeaderLen = 40, kStreamPlanGroupLen = 20;

glmrt_status_t parse_stream_plan(const uint8_t* p, size_t n, uint32_t rows, uint32_t routes, std::vector<uint32_t>* order) {
  if (n < kStreamPlanHeaderLen) return bad("stream plan frame too short: " + std::to_string(n));
  if (std::memcmp(p, "GLMSTRM2", 8) != 0) return bad("stream plan magic mismatch");
  if (get16(p + 8) != 1) return bad("unsupported stream plan version " + std::to_string(get16(p + 8)));
  if (get16(p + 10) != kStreamPlanHeaderLen) return bad("stream plan header length did not match 40");
  if (get32(p + 12) != n) return bad("stream plan wire bytes " + std::to_string(get32(p + 12)) + " did not match " + std::to_string(n));
  const uint32_t row_count = get32(p + 16), route_count = get32(p + 20), activation = get32(p + 24), groups = get32(p + 28),
                 route_indices = get32(p + 32), completed = get32(p + 36);
  const uint64_t expect = kStreamPlanHeaderLen + uint64_t(groups) * kStreamPlanGroupLen +
                          4ull * (uint64_t(activation) + route_indices + completed);
  if (expect != n) return bad("stream plan section bytes " + std::to_string(expect) + " did not match " + std::to_string(n));
  if (row_count != rows) return bad("stream plan rows " + std::to_string(row_count) + " did not match request rows " + std::to_string(rows));
  if (route_count != routes)
    return bad("stream plan routes " + std::to_string(route_count) + " did not match request routes " + std::to_string(routes));
  if (activation != rows) return bad("stream plan activation order must name every row once");
  const uint8_t* act = p + kStreamPlanHeaderLen + size_t(groups) * kStreamPlanGroupLen;
  const uint8_t* rts = act + 4ull * activation;
  const uint8_t* done = rts + 4ull * route_indices;
  order->resize(activation);
  std::vector<uint8_t> seen(rows, 0);
  for (uint32_t i = 0; i < activation; ++i) {
    const uint32_t r = get32(act + 4ull * i);
    if (r >= rows || seen[r]) return bad("stream plan activation order is not a permutation of the rows");
    seen[r] = 1;
    (*order)[i] = r;
  }
  for (uint32_t g = 0; g < groups; ++g) {
    const uint8_t* q = p + kStreamPlanHeaderLen + size_t(g) * kStreamPlanGroupLen;
    const uint64_t ready = get32(q), r_off = get32(q + 4), r_cnt = get32(q + 8), c_off = get32(q + 12), c_cnt = get32(q + 16);
    if (ready == 0 || ready > rows) return bad("stream group " + std::to_string(g) + " ready-after row count is out of range");
    if (r_off + r_cnt > route_indices) return bad("stream group " + std::to_string(g) + " route range is invalid");
    if (c_off + c_cnt > completed) return bad("stream group " + std::to_string(g) + " completion range is invalid");
    for (uint64_t i = 0; i < r_cnt; ++i)
      if (get32(rts + 4 * (r_off + i)) >= routes) return bad("stream group " + std::to_string(g) + " names a route outside the request");
    for (uint64_t i = 0; i < c_cnt; ++i)
      if (get32(done + 4 * (c_off + i)) >= rows) return bad("stream group " + std::to_string(g) + " names a row outside the request");
  }
  return GLMRT_STATUS_OK;
}

glmrt_status_t begin_stream(void* layer, const uint8_t* b, const glmrt_b200_pv2_request_header_t& h,
                            const glmrt_b200_pv2_sections_t& sec, const LayerDims& d) {
  StreamSession s;
  s.head = h;
  GLMRT_RETURN_IF_ERROR(check_request_against_layer(h, d, h.row_count, &s.in_payload));
  GLMRT_RETURN_IF_ERROR(build_route_tables(b, h, sec, d, &s.tables));
  GLMRT_RETURN_IF_ERROR(parse_stream_plan(b + sec.payload_offset, sec.payload_bytes, h.row_count, h.route_count, &s.order));
  s.stride = h.hidden_row_stride_bytes;
  s.hidden.assign(size_t(h.row_count) * s.stride, 0);
  s.have.assign(h.row_count, 0);
  std::lock_guard<std::mutex> lock(g_stream_mutex);
  g_streams[layer] = std::move(s);      // a plan replaces an unfinished stream on the same handle
  return GLMRT_STATUS_OK;
}

glmrt_status_t continue_stream(void* layer, const uint8_t* b, const glmrt_b200_pv2_request_header_t& h,
                               const glmrt_b200_pv2_sections_t& sec, void* response_out, size_t response_capacity,
                               size_t* response_len, cudaStream_t stream) {
  StreamSession done;
  {
    std::lock_guard<std::mutex> lock(g_stream_mutex);
    auto it = g_streams.find(layer);
    if (it == g_streams.end()) return bad("executor: stream data frame without a stream plan on this handle");
    StreamSession& s = it->second;
    if (h.request_id != s.head.request_id || h.layer_id != s.head.layer_id || h.placement_version != s.head.placement_version)
      return bad("executor: stream data frame does not belong to the pending stream plan");
    if (h.hidden_dim != s.head.hidden_dim || h.hidden_dtype != s.head.hidden_dtype || h.hidden_row_stride_bytes != s.stride)
      return bad("executor: stream data frame rows differ in shape from the stream plan");
    const uint64_t first = h.route_count;     // position of the first row in the plan's activation order
    if (first + h.row_count > s.order.size())
      return bad("executor: stream data rows " + std::to_string(first) + ".." + std::to_string(first + h.row_count) +
                 " exceed the plan's " + std::to_string(s.order.size()) + " rows");
    for (uint32_t i = 0; i < h.row_count; ++i) {
      const uint32_t row = s.order[first + i];
      if (s.have[row]) return bad("executor: stream data row " + std::to_string(row) + " arrived twice");
      std::memcpy(s.hidden.data() + size_t(row) * s.stride, b + sec.payload_offset + size_t(i) * s.stride, s.stride);
      s.have[row] = 1;
      ++s.received;
    }
    if (!(h.flags & GLMRT_B200_PV2_FLAG_STREAM_FINAL)) {
      *response_len = 0;      // nothing to send back yet
      return GLMRT_STATUS_OK;
    }
    if (s.received != s.order.size()) {
      const size_t got = s.received, want = s.order.size();
      g_streams.erase(it);
      return bad("executor: final stream data frame after " + std::to_string(got) + " of " + std::to_string(want) + " rows");
    }
    done = std::move(s);
    g_streams.erase(it);
  }
  return run_and_frame(layer, done.head, done.head.row_count, done.hidden.data(), done.stride, done.in_payload, done.tables,
                       response_out, response_capacity, response_len, stream);
}

}  // namespace

void drop_stream_session(void* layer) {
  std::lock_guard<std::mutex> lock(g_stream_mutex);
  g_streams.erase(layer);
}

}  // namespace glmrt

extern "C" glmrt_status_t glmrt_b200_pv2_execute(void* layer, const void* request_frame, size_t request_bytes,
                                                 void* response_out, size_t response_capacity, size_t* response_len,
                                                 void* cuda_stream) {
  if (layer == nullptr || request_frame == nullptr || response_len == nullptr)
    return fail(GLMRT_STATUS_INVALID_ARGUMENT, "pv2_execute: null pointer argument");
  const uint8_t* b = static_cast<const uint8_t*>(request_frame);
  glmrt_b200_pv2_request_header_t h;
  glmrt_b200_pv2_sections_t sec;
  GLMRT_RETURN_IF_ERROR(parse_request(b, request_bytes, &h, &sec));
  if (h.flags & GLMRT_B200_PV2_FLAG_LAYER_BLOCK)
    return bad("executor: layer-block requests (attention blocks on the expert hosts) are not supported, only routed-expert requests");
  // the reference's executors check the checksum of a frame that carries one (synthetic.rs:124)
  GLMRT_RETURN_IF_ERROR(glmrt_b200_pv2_verify_request_checksum(request_frame, request_bytes));
  LayerDims d;
  GLMRT_RETURN_IF_ERROR(layer_dims(layer, &d));
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (h.flags & GLMRT_B200_PV2_FLAG_STREAM_PLAN) {
    GLMRT_RETURN_IF_ERROR(begin_stream(layer, b, h, sec, d));
    *response_len = 0;
    return ok();
  }
  if (h.flags & GLMRT_B200_PV2_FLAG_STREAM_DATA) {
    const glmrt_status_t st = continue_stream(layer, b, h, sec, response_out, response_capacity, response_len, stream);
    return st == GLMRT_STATUS_OK ? ok() : st;
  }
  bool in_payload = false;
  GLMRT_RETURN_IF_ERROR(check_request_against_layer(h, d, h.row_count, &in_payload));
  RouteTables t;
  GLMRT_RETURN_IF_ERROR(build_route_tables(b, h, sec, d, &t));
  return run_and_frame(layer, h, h.row_count, b + sec.payload_offset, h.hidden_row_stride_bytes, in_payload, t, response_out,
                       response_capacity, response_len, stream);
}
