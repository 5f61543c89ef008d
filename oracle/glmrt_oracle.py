"""CPU oracle for the routed-MoE expert FFN path (TEST INFRASTRUCTURE ONLY).

This module is a numpy restatement of the reference's algorithm for the hot
path: router -> NVFP4 activation payload -> expert-sorted route plan -> NVFP4
expert FFN (gate/up + SwiGLU, down) -> weighted combine.  It exists to check
the CUDA library; nothing in the shipped library imports it, and the library
has no CPU fallback.  Only tests, the smoke check and the benchmark's CPU
baseline may call it.

Parity status: PINNED.  ``tests/golden/`` holds vectors produced by importing
the reference's own ``python/reference/glmrt_reference`` package (generator
script committed beside them) plus the known-answer vectors of the reference's
native and Rust tests; ``tests/test_oracle_golden.py`` checks this file
against all of them.

Every function cites the reference file:line it follows (paths are relative
to the reference project root).
"""
from __future__ import annotations

import numpy as np

# ---------------------------------------------------------------------------
# Formats
# ---------------------------------------------------------------------------

#: E2M1 code -> value.  python/reference/glmrt_reference/quant_ref.py:11-28,
#: native/cuda/kernels/common.h:32-38.
E2M1_VALUES = np.array(
    [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
     0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=np.float32)

ROUTED_SCALING = np.float32(2.5)  # native/cuda/kernels/common.h:20


def e4m3_decode(byte) -> np.ndarray:
    """E4M3 byte -> float32 without NaN handling (0x7f decodes as 480).

    quant_ref.py:79-88 (f8e4m3_byte_to_float), common.h:40-50,
    rust/crates/glmrt-daemon/src/commands/real_full/sparse_mlp/math.rs:149-162.
    """
    b = np.asarray(byte, dtype=np.uint8).astype(np.int32)
    sign = np.where(b & 0x80, -1.0, 1.0).astype(np.float32)
    exp = (b >> 3) & 0x0F
    man = (b & 0x07).astype(np.float32)
    sig = np.where(exp == 0, man / 8.0, 1.0 + man / 8.0).astype(np.float32)
    pw = np.where(exp == 0, -6, exp - 7)
    out = sign * sig * np.ldexp(np.float32(1.0), pw).astype(np.float32)
    out = np.where((b == 0) | (b == 0x80), np.float32(0.0), out)
    return out.astype(np.float32)


_E4M3_POS = e4m3_decode(np.arange(0x7F, dtype=np.uint8)).astype(np.float64)  # 0x00..0x7e
_E4M3_MID = (_E4M3_POS[:-1] + _E4M3_POS[1:]) / 2.0


def e4m3_encode_satfinite(x) -> np.ndarray:
    """Non-negative float32 -> E4M3 byte, round-to-nearest-even, saturating at 448.

    Behaviour of ``__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3)`` used at
    native/cuda/kernels/nvfp4_payload.cu:57-58 and mlp.cu:116-117, and of a
    clamped ``torch.float8_e4m3fn`` cast.  NaN inputs are not supported.
    """
    x = np.asarray(x, dtype=np.float32).astype(np.float64)
    neg = np.signbit(x)
    m = np.abs(x)
    idx = np.searchsorted(_E4M3_MID, m, side="left")
    idx = np.minimum(idx, 0x7E)
    tie = (idx < 0x7E) & (m == _E4M3_MID[np.minimum(idx, 0x7D)])
    idx = np.where(tie & (idx % 2 == 1), idx + 1, idx)
    return (idx | np.where(neg, 0x80, 0)).astype(np.uint8)


def bf16_round(x) -> np.ndarray:
    """float32 -> bf16 bit pattern (uint16), round-to-nearest-even (torch ``.to(bfloat16)``).

    The Python oracle rounds (moe_ref.py:21,35); the reference's native kernels
    truncate instead (common.h:64-66) -- parity follows the Python oracle.
    """
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    r = np.where(nan, (u >> 16) | 0x40, r)
    return r.astype(np.uint16)


def bf16_truncate(x) -> np.ndarray:
    """float32 -> bf16 bits by truncation (common.h:64-66)."""
    return (np.asarray(x, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)


def bf16_to_f32(bits) -> np.ndarray:
    """bf16 bit pattern -> float32 (common.h:60-62)."""
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def pack_nibbles(codes) -> np.ndarray:
    """Low-nibble-first packing, odd counts zero padded (quant_ref.py:56-63)."""
    flat = np.asarray(codes, dtype=np.uint8).reshape(-1)
    if flat.size % 2:
        flat = np.concatenate([flat, np.zeros(1, np.uint8)])
    return ((flat[0::2] & 0x0F) | ((flat[1::2] & 0x0F) << 4)).astype(np.uint8)


def unpack_nibbles(packed, count: int) -> np.ndarray:
    """quant_ref.py:66-72."""
    p = np.asarray(packed, dtype=np.uint8).reshape(-1)
    out = np.empty(p.size * 2, np.uint8)
    out[0::2] = p & 0x0F
    out[1::2] = (p >> 4) & 0x0F
    return out[:count]


# ---------------------------------------------------------------------------
# FP4 code selection rules
# ---------------------------------------------------------------------------

_THRESH = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)


def fp4_codes_nearest_low(scaled) -> np.ndarray:
    """Nearest E2M1 code, exact ties to the LOWER magnitude, -0 and NaN -> code 0.

    Equivalent to ``(scaled[..., None] - codebook).abs().argmin(-1)`` of
    quant_ref.py:41-46: the first minimum wins, so 0.75 -> 0.5 and a negative
    value that rounds to zero yields code 0, never code 8.  (Every distance in
    that expression is exact in float32, so the threshold form is identical.)
    """
    s = np.asarray(scaled, dtype=np.float32)
    m = np.abs(s)
    mag = np.zeros(s.shape, np.uint8)
    for t in _THRESH:
        mag += (m > t).astype(np.uint8)
    neg = (s < 0) & (mag > 0)
    return (mag | np.where(neg, 8, 0)).astype(np.uint8)


def fp4_codes_rne_payload(scaled) -> np.ndarray:
    """Round-to-nearest-even thresholds, sign bit from signbit() (so -0 -> code 8).

    native/cuda/kernels/nvfp4_payload.cu:11-33 (fp4_e2m1_payload_code).
    """
    s = np.asarray(scaled, dtype=np.float32)
    m = np.abs(s)
    code = np.full(s.shape, 7, np.uint8)
    code = np.where(m <= 5.0, 6, code)
    code = np.where(m < 3.5, 5, code)
    code = np.where(m <= 2.5, 4, code)
    code = np.where(m < 1.75, 3, code)
    code = np.where(m <= 1.25, 2, code)
    code = np.where(m < 0.75, 1, code)
    code = np.where(m <= 0.25, 0, code)
    return (code | np.where(np.signbit(s), 8, 0)).astype(np.uint8)


def nvfp4_quantize(x, scale) -> np.ndarray:
    """quant_ref.py:41-46: codes of x / scale (float32 division)."""
    with np.errstate(divide="ignore", invalid="ignore"):
        scaled = np.asarray(x, np.float32) / np.asarray(scale, np.float32)
    return fp4_codes_nearest_low(scaled)


def nvfp4_dequantize(codes, scale) -> np.ndarray:
    """quant_ref.py:49-53."""
    return (E2M1_VALUES[np.asarray(codes, np.int64)] * np.asarray(scale, np.float32)).astype(np.float32)


def decode_packed_nvfp4(packed, scale_bytes, scale_2, count: int) -> np.ndarray:
    """value = codebook[code] * e4m3(scale[i // 16]) * scale_2, left to right.

    quant_ref.py:108-125 (decode_packed_nvfp4_values), common.h:52-58.
    """
    codes = unpack_nibbles(packed, count)
    s = e4m3_decode(np.asarray(scale_bytes, np.uint8).reshape(-1))[np.arange(count) // 16]
    return ((E2M1_VALUES[codes] * s).astype(np.float32) * np.float32(scale_2)).astype(np.float32)


def dot_packed_nvfp4(x, packed, scale_bytes, scale_2) -> np.float32:
    """Sequential fused-multiply-add dot (sparse_mlp/math.rs:95-134).  Small inputs only."""
    w = decode_packed_nvfp4(packed, scale_bytes, scale_2, len(x)).astype(np.float64)
    acc = np.float32(0.0)
    for xi, wi in zip(np.asarray(x, np.float32).astype(np.float64), w):
        acc = np.float32(xi * wi + np.float64(acc))  # fma: one rounding
    return acc


# ---------------------------------------------------------------------------
# a2: activation payload quantiser
# ---------------------------------------------------------------------------

def quantize_rows_nvfp4(x_f32, rule: str = "nearest_low"):
    """Block-16 NVFP4 quantisation of activation rows with no global scale.

    scale byte = e4m3(amax / 6) (RN, saturating); a zero scale makes every code of
    the block 0.  ``rule``:
      * "nearest_low" -- codes from ``x / scale`` with ties to the lower magnitude:
        the python oracle's rule (quant_ref.py:41-46).  The layer path uses it.
      * "rne_payload" -- codes from ``clamp(x * (1 / scale), -6, 6)`` with the
        round-to-nearest-even thresholds of nvfp4_payload.cu:11-33,56-66.
    Returns (codes uint8 [rows, cols], scale_bytes uint8 [rows, cols // 16]).
    """
    x = np.asarray(x_f32, np.float32)
    rows, cols = x.shape
    assert cols % 16 == 0
    blk = x.reshape(rows, cols // 16, 16)
    amax = np.max(np.abs(blk), axis=-1)
    sb = e4m3_encode_satfinite(amax / np.float32(6.0))
    s = e4m3_decode(sb)
    if rule == "nearest_low":
        with np.errstate(divide="ignore", invalid="ignore"):
            scaled = blk / s[..., None]
        codes = fp4_codes_nearest_low(scaled)
        codes = np.where(s[..., None] == 0, np.uint8(0), codes)
    elif rule == "rne_payload":
        with np.errstate(divide="ignore"):
            inv = np.where(s == 0, np.float32(0.0), np.float32(1.0) / s).astype(np.float32)
        scaled = np.clip((blk * inv[..., None]).astype(np.float32), -6.0, 6.0)
        codes = fp4_codes_rne_payload(scaled)
    else:
        raise ValueError(rule)
    return codes.reshape(rows, cols).astype(np.uint8), sb.astype(np.uint8)


def payload_rows(codes, scale_bytes) -> np.ndarray:
    """Row payload = packed codes (cols/2 bytes) followed by scale bytes (cols/16).

    nvfp4_payload.cu:52-54,69-72; rust/crates/glmrt-transport/src/protocol_v2.rs:67-77.
    """
    rows, cols = codes.shape
    packed = pack_nibbles(codes).reshape(rows, cols // 2)
    return np.concatenate([packed, np.asarray(scale_bytes, np.uint8)], axis=1)


def dequantize_payload_rows(payload, cols: int) -> np.ndarray:
    """Payload rows -> float32 (code * e4m3 scale, no global scale).

    native/cuda/kernels/b12x_direct.cu:171-201.
    """
    p = np.asarray(payload, np.uint8)
    rows = p.shape[0]
    codes = np.stack([unpack_nibbles(p[r, : cols // 2], cols) for r in range(rows)])
    s = e4m3_decode(p[:, cols // 2: cols // 2 + cols // 16])
    return (E2M1_VALUES[codes].reshape(rows, cols // 16, 16) * s[..., None]).reshape(rows, cols).astype(np.float32)


# ---------------------------------------------------------------------------
# a3: weight quantisers
# ---------------------------------------------------------------------------

def quantize_weight_baseline(w_f32):
    """NVFP4 weight quantiser of the benchmark configuration.

    global scale g = amax / (6 * 448); block scale byte = e4m3(amax_blk / (6 * g));
    codes = quant_ref.nvfp4_quantize(block, e4m3(byte) * g); value = code * e4m3 * g
    (decode order of quant_ref.py:108-125).  Returns (codes, scale_bytes, g).
    """
    w = np.asarray(w_f32, np.float32)
    rows, cols = w.shape
    assert cols % 16 == 0
    amax = np.float32(np.max(np.abs(w)))
    g = np.float32(amax / np.float32(6.0 * 448.0))
    blk = w.reshape(rows, cols // 16, 16)
    bmax = np.max(np.abs(blk), axis=-1)
    with np.errstate(divide="ignore", invalid="ignore"):
        ratio = np.where(g == 0, np.float32(0.0), bmax / (np.float32(6.0) * g)).astype(np.float32)
    sb = e4m3_encode_satfinite(ratio)
    sg = (e4m3_decode(sb) * g).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        scaled = blk / sg[..., None]
    codes = fp4_codes_nearest_low(scaled)
    codes = np.where(sg[..., None] == 0, np.uint8(0), codes)
    return codes.reshape(rows, cols).astype(np.uint8), sb.astype(np.uint8), g


def fp4_codes_rn_cvt(scaled) -> np.ndarray:
    """``__nv_cvt_float_to_fp4(x, __NV_E2M1, cudaRoundNearest)``: RNE on the E2M1 grid,
    saturating at 6, sign bit kept for -0 (native/cuda/kernels/mlp.cu:126-129 and the
    known answer at native/tests/cuda_selftest.cc:2736-2765)."""
    return fp4_codes_rne_payload(np.clip(np.asarray(scaled, np.float32), -6.0, 6.0))


def quantize_weight_bf16_multiplicative(w_bf16_bits, global_scale):
    """native/cuda/kernels/mlp.cu:98-132: scale = e4m3(amax * g / 6), code = cvt_rn(v * g / scale)."""
    w = bf16_to_f32(w_bf16_bits)
    rows, cols = w.shape
    g = np.float32(global_scale)
    blk = w.reshape(rows, cols // 16, 16)
    bmax = np.max(np.abs(blk), axis=-1)
    sb = e4m3_encode_satfinite((bmax * g).astype(np.float32) / np.float32(6.0))
    s = e4m3_decode(sb)
    with np.errstate(divide="ignore", invalid="ignore"):
        scaled = np.where(s[..., None] == 0, np.float32(0.0),
                          (blk * g).astype(np.float32) / s[..., None]).astype(np.float32)
    codes = fp4_codes_rn_cvt(scaled)
    return codes.reshape(rows, cols), sb


def dequantize_weight(codes, scale_bytes, scale_2) -> np.ndarray:
    """[rows, cols] float32 = codebook[code] * e4m3(scale) * scale_2 (common.h:52-58)."""
    rows, cols = codes.shape
    s = e4m3_decode(scale_bytes)
    v = (E2M1_VALUES[codes].reshape(rows, cols // 16, 16) * s[..., None]).astype(np.float32)
    return (v * np.float32(scale_2)).reshape(rows, cols).astype(np.float32)


# ---------------------------------------------------------------------------
# a1: router
# ---------------------------------------------------------------------------

def sigmoid_f32(x) -> np.ndarray:
    """Stable two-branch float32 sigmoid (common.h:23-30)."""
    x = np.asarray(x, np.float32)
    with np.errstate(over="ignore"):
        en = np.exp(-np.abs(x)).astype(np.float32)
    pos = np.float32(1.0) / (np.float32(1.0) + en)
    neg = en / (np.float32(1.0) + en)
    return np.where(x >= 0, pos, neg).astype(np.float32)


def router_topk(hidden_f32, router_weight_f32, bias_f32, top_k: int = 8,
                scaling: float = 2.5, logits=None):
    """Sigmoid + bias top-k router.

    python/reference/glmrt_reference/glm_moe_dsa_layer_ref.py:62-83: logits = X @ W^T in
    float32; scores = sigmoid; selection = scores + bias; top-k by selection (descending);
    weights = scores[idx] / max(sum, 1e-12) * 2.5.  Ties go to the lower expert id
    (native/cuda/kernels/router.cu:136-137).  Non-finite scores count as 0 and can never
    be selected ahead of a finite one (router.cu:112-116).
    Returns (indices uint32 [T,k], weights f32 [T,k], scores f32 [T,E], selection f32 [T,E]).
    """
    x = np.asarray(hidden_f32, np.float32)
    w = np.asarray(router_weight_f32, np.float32)
    if logits is None:
        logits = (x @ w.T).astype(np.float32)
    raw = sigmoid_f32(logits)
    fin = np.isfinite(raw)
    scores = np.where(fin, raw, np.float32(0.0)).astype(np.float32)
    sel = (scores + np.asarray(bias_f32, np.float32).reshape(1, -1)).astype(np.float32)
    sel = np.where(fin & np.isfinite(sel), sel, -np.inf).astype(np.float32)
    experts = sel.shape[1]
    # descending by selection, ascending by id on ties: stable sort of -sel
    order = np.argsort(-sel.astype(np.float64), axis=1, kind="stable")[:, :top_k]
    picked = np.take_along_axis(scores, order, axis=1)
    ssum = np.zeros(picked.shape[0], np.float32)
    for j in range(top_k):  # sequential float32 sum as router.cu:52-56
        ssum = (ssum + picked[:, j]).astype(np.float32)
    ssum = np.maximum(ssum, np.float32(1e-12))
    weights = ((picked / ssum[:, None]).astype(np.float32) * np.float32(scaling)).astype(np.float32)
    assert experts >= top_k
    return order.astype(np.uint32), weights, scores, sel


def router_indices_equivalent(idx_a, idx_b, selection_f64, tol: float = 1e-6) -> bool:
    """True when two top-k index sets agree except for swaps between experts whose
    selection scores differ by at most ``tol`` (float64 adjudication)."""
    idx_a = np.asarray(idx_a, np.int64)
    idx_b = np.asarray(idx_b, np.int64)
    for r in range(idx_a.shape[0]):
        sa, sb = set(idx_a[r].tolist()), set(idx_b[r].tolist())
        if sa == sb:
            continue
        only_a = sorted(sa - sb, key=lambda e: -selection_f64[r, e])
        only_b = sorted(sb - sa, key=lambda e: -selection_f64[r, e])
        if len(only_a) != len(only_b):
            return False
        for ea, eb in zip(only_a, only_b):
            if abs(selection_f64[r, ea] - selection_f64[r, eb]) > tol:
                return False
    return True


# ---------------------------------------------------------------------------
# a4: route plan
# ---------------------------------------------------------------------------

def owner_for_expert(layer_id: int, expert_id: int, world: int, experts: int = 256) -> int:
    """rust/crates/glmrt-core/src/placement.rs:25-42; glm_moe_dsa_layer_ref.py:51-59."""
    return (layer_id * experts + expert_id) % world


def plan_routes(route_indices, experts: int, block_rows: int):
    """Stable counting sort of (row, slot) routes by expert, each expert padded to a
    multiple of ``block_rows`` with the sentinel ``route_count``.

    rust/crates/glmrt-daemon/src/commands/real_full/sparse_mlp/route.rs:3727-3828
    (plan_packed_w4a16_topk8_prefill_flat).  Returns (packed_route_indices uint32,
    block_expert_ids uint32, counts int64 [experts]).
    """
    idx = np.asarray(route_indices, np.int64)
    flat = idx.reshape(-1)
    n = flat.size
    counts = np.bincount(flat, minlength=experts).astype(np.int64)
    packed, blocks = [], []
    order = np.argsort(flat, kind="stable")
    pos = 0
    for e in range(experts):
        c = int(counts[e])
        if c == 0:
            continue
        routes = order[pos:pos + c]
        pos += c
        nb = (c + block_rows - 1) // block_rows
        pad = nb * block_rows - c
        packed.extend(routes.tolist())
        packed.extend([n] * pad)
        blocks.extend([e] * nb)
    return np.array(packed, np.uint32), np.array(blocks, np.uint32), counts


# ---------------------------------------------------------------------------
# a5/a6: expert FFN, a7: combine
# ---------------------------------------------------------------------------

def silu_f32(g) -> np.ndarray:
    """g * sigmoid(g) with the stable sigmoid (mlp.cu:195,271; torch F.silu, moe_ref.py:20)."""
    g = np.asarray(g, np.float32)
    return (g * sigmoid_f32(g)).astype(np.float32)


class ExpertWeights:
    """Dequantised float32 projections of one expert (moe_ref.py:10-14)."""

    def __init__(self, gate, up, down):
        self.gate_proj = np.asarray(gate, np.float32)   # [I, H]
        self.up_proj = np.asarray(up, np.float32)       # [I, H]
        self.down_proj = np.asarray(down, np.float32)   # [H_out, I]


def requantize_intermediate(a_f32) -> np.ndarray:
    """Quantise -> dequantise of the SwiGLU output rows with the activation format
    (block 16, e4m3(amax/6) scale, nearest-low codes).  This is the second quantisation
    point of the W4A4 path; the float32 reference has none."""
    codes, sb = quantize_rows_nvfp4(a_f32, "nearest_low")
    rows, cols = codes.shape
    s = e4m3_decode(sb)
    return (E2M1_VALUES[codes].reshape(rows, cols // 16, 16) * s[..., None]).reshape(rows, cols).astype(np.float32)


def expert_forward(x_f32, w: ExpertWeights, requant: bool = False) -> np.ndarray:
    """float32 (silu(x Wg^T) * (x Wu^T)) Wd^T (moe_ref.py:17-21, before the bf16 cast)."""
    x = np.asarray(x_f32, np.float32)
    gate = (x @ w.gate_proj.T).astype(np.float32)
    up = (x @ w.up_proj.T).astype(np.float32)
    act = (silu_f32(gate) * up).astype(np.float32)
    if requant:
        act = requantize_intermediate(act)
    return (act @ w.down_proj.T).astype(np.float32)


def moe_forward(hidden_bf16_bits, expert_weights, route_indices, route_weights,
                mode: str = "O1", only_owner=None):
    """Routed MoE forward over bf16 hidden rows; returns bf16 bits [T, H_out].

    moe_ref.py:24-37: for row, for slot: out[row] += bf16(w) * bf16(expert_forward(row)),
    every operation rounded to bf16 (torch bf16 tensor arithmetic).
      * mode "O0": reference-exact (float32 activations everywhere).
      * mode "O1": quantisation-matched: the hidden row and the SwiGLU intermediate pass
        through the NVFP4 activation quantise->dequantise first, as on the NVFP4 wire
        (nvfp4_payload.cu:35-73) and in the FP4 x FP4 tensor-core path.
      * mode "O1f": as O1 but float32 accumulation and one final bf16 rounding.
    ``expert_weights`` maps expert id -> ExpertWeights (or is a callable doing so).
    ``only_owner``: optional predicate expert_id -> bool selecting one shard's partial
    (partitioned_moe_forward, moe_ref.py:40-66).
    """
    hid = bf16_to_f32(hidden_bf16_bits)
    T = hid.shape[0]
    idx = np.asarray(route_indices, np.int64)
    wts = np.asarray(route_weights, np.float32)
    getw = expert_weights if callable(expert_weights) else expert_weights.__getitem__
    if mode in ("O1", "O1f"):
        c, s = quantize_rows_nvfp4(hid, "nearest_low")
        xin = dequantize_payload_rows(payload_rows(c, s), hid.shape[1])
    elif mode == "O0":
        xin = hid
    else:
        raise ValueError(mode)
    # group by expert so each expert's weights are materialised once
    ys = {}
    for e in np.unique(idx):
        if only_owner is not None and not only_owner(int(e)):
            continue
        rows = np.unique(np.nonzero(idx == e)[0])
        y = expert_forward(xin[rows], getw(int(e)), requant=(mode != "O0"))
        for r, yr in zip(rows, y):
            ys[(int(r), int(e))] = yr
    h_out = next(iter(ys.values())).shape[0] if ys else hid.shape[1]
    if mode == "O1f":
        acc = np.zeros((T, h_out), np.float32)
        for r in range(T):
            for k in range(idx.shape[1]):
                key = (r, int(idx[r, k]))
                if key in ys:
                    acc[r] = acc[r] + wts[r, k] * ys[key]
        return bf16_round(acc)
    out = np.zeros((T, h_out), np.uint16)
    for r in range(T):
        for k in range(idx.shape[1]):
            key = (r, int(idx[r, k]))
            if key not in ys:
                continue
            out[r] = combine_step_bf16(out[r], wts[r, k], bf16_round(ys[key]))
    return out


def combine_step_bf16(acc_bits, weight_f32, y_bits) -> np.ndarray:
    """One ``output[row] += gate.to(bf16) * y`` step in bf16 tensor arithmetic
    (moe_ref.py:35-36): product rounded to bf16, then sum rounded to bf16."""
    wb = bf16_to_f32(bf16_round(np.float32(weight_f32)))
    prod = bf16_to_f32(bf16_round(wb * bf16_to_f32(y_bits)))
    return bf16_round(bf16_to_f32(acc_bits) + prod)


def combine_routes_bf16(y_routes_bits, route_weights) -> np.ndarray:
    """[T, k, H] per-route bf16 rows -> [T, H] bf16 with the oracle's sequential
    bf16 accumulation (moe_ref.py:30-36)."""
    y = np.asarray(y_routes_bits, np.uint16)
    T, k, H = y.shape
    out = np.zeros((T, H), np.uint16)
    for j in range(k):
        for r in range(T):
            out[r] = combine_step_bf16(out[r], route_weights[r, j], y[r, j])
    return out


def sum_topk_bf16(y_routes_bits) -> np.ndarray:
    """Fixed-order float32 sum over the k per-route bf16 rows, truncated to bf16.

    native/cuda/kernels/b12x_direct.cu:203-219 (sum_w4a16_topk_bf16_kernel).
    """
    y = bf16_to_f32(np.asarray(y_routes_bits, np.uint16))
    acc = np.zeros((y.shape[0], y.shape[2]), np.float32)
    for j in range(y.shape[1]):
        acc = (acc + y[:, j]).astype(np.float32)
    return bf16_truncate(acc)


def residual_add_bf16(residual_bits, delta_bits) -> np.ndarray:
    """out = bf16(residual + delta), float32 add, truncating store
    (native/cuda/kernels/residual.cu:18-26; f32_to_bf16 truncates, common.h:64-66)."""
    r = bf16_to_f32(np.asarray(residual_bits, np.uint16))
    d = bf16_to_f32(np.asarray(delta_bits, np.uint16))
    return bf16_truncate((r + d).astype(np.float32))


def residual_add_f32_delta_bf16(residual_bits, delta_f32) -> np.ndarray:
    """out = bf16(residual + bf16(delta)) (native/cuda/kernels/residual.cu:28-38)."""
    d = bf16_truncate(np.asarray(delta_f32, np.float32))
    return residual_add_bf16(residual_bits, d)


def residual_add_shared_f32_delta_bf16(residual_bits, shared_bits, routed_f32) -> np.ndarray:
    """out = bf16(residual + bf16(shared + bf16(routed))) (native/cuda/kernels/residual.cu:40-52):
    the layer output hidden + routed + shared of glm_moe_dsa_layer_ref.py:196-198 in the
    native kernel's association and rounding."""
    routed = bf16_to_f32(bf16_truncate(np.asarray(routed_f32, np.float32)))
    shared = bf16_to_f32(np.asarray(shared_bits, np.uint16))
    mlp = bf16_truncate((shared + routed).astype(np.float32))
    return residual_add_bf16(residual_bits, mlp)


def decode_wire_rows(rows_bytes, width: int, dtype: str) -> np.ndarray:
    """[R, stride] bytes of wire rows -> [R, width] float32 (native/cuda/kernels/residual.cu:544-559):
    "bf16"; "fp8" = width E4M3 bytes then a float32 scale; "nvfp4" = width/2 code bytes (low nibble
    first) then width/16 E4M3 scale bytes."""
    b = np.asarray(rows_bytes, np.uint8)
    if dtype == "bf16":
        return bf16_to_f32(np.ascontiguousarray(b[:, :2 * width]).view(np.uint16))
    if dtype == "fp8":
        scale = np.ascontiguousarray(b[:, width:width + 4]).view(np.float32)
        return (e4m3_decode(b[:, :width]) * scale).astype(np.float32)
    packed = b[:, :width // 2]
    codes = np.empty((b.shape[0], width), np.uint8)
    codes[:, 0::2] = packed & 0x0F
    codes[:, 1::2] = packed >> 4
    scales = e4m3_decode(b[:, width // 2:width // 2 + width // 16])
    return (E2M1_VALUES[codes] * np.repeat(scales, 16, axis=1)).astype(np.float32)


def scatter_add_rows_to_f32(values_f32, row_indices, dst_f32) -> np.ndarray:
    """dst[row_indices[r]] += values[r], contributions added in source order, float32
    (native/cuda/kernels/residual.cu:438-453, the ordered form used up to 64 rows)."""
    out = np.array(dst_f32, np.float32, copy=True)
    for r, d in enumerate(np.asarray(row_indices)):
        out[int(d)] = (out[int(d)] + np.asarray(values_f32[r], np.float32)).astype(np.float32)
    return out


def reduce_route_shards_to_f32(local_f32, peers_f32) -> np.ndarray:
    """local + peers[0] + peers[1] + ... in float32, in that order (residual.cu:561-589)."""
    out = np.asarray(local_f32, np.float32).copy()
    for p in peers_f32:
        out = (out + np.asarray(p, np.float32)).astype(np.float32)
    return out


def bf16_rows_to_fp8_e4m3_row_scaled(rows_bits) -> np.ndarray:
    """[R, W] bf16 -> [R, W + 4] bytes: E4M3 values then one little-endian float32 scale per row
    (native/cuda/kernels/residual.cu:245-277): scale = max |finite| / 448, 1 for an all-zero row;
    byte = e4m3(value / scale) round-to-nearest, saturating; non-finite values encode 0."""
    x = bf16_to_f32(np.asarray(rows_bits, np.uint16))
    finite = np.isfinite(x)
    amax = np.where(finite, np.abs(x), np.float32(0)).max(axis=1).astype(np.float32)
    scale = np.where(amax > 0, (amax / np.float32(448.0)).astype(np.float32), np.float32(1.0)).astype(np.float32)
    q = np.where(finite, (x / scale[:, None]).astype(np.float32), np.float32(0)).astype(np.float32)
    out = np.zeros((x.shape[0], x.shape[1] + 4), np.uint8)
    out[:, :x.shape[1]] = e4m3_encode_satfinite(q)
    out[:, x.shape[1]:] = scale.view(np.uint8).reshape(-1, 4)
    return out


def scatter_add_rows_bf16_weighted_to_f32(src_bits, row_indices, row_weights, dst_f32) -> np.ndarray:
    """dst[row_indices[r]] += w[r] * src[r] (native/cuda/kernels/residual.cu:666-678)."""
    dst = np.array(dst_f32, np.float32, copy=True)
    src = bf16_to_f32(src_bits)
    for r, (ri, w) in enumerate(zip(row_indices, row_weights)):
        if ri < dst.shape[0]:
            dst[ri] = (dst[ri] + np.float32(w) * src[r]).astype(np.float32)
    return dst


def rel_l2_per_token(a_bits, b_bits) -> np.ndarray:
    """Per-token relative L2 error between two bf16 outputs (b is the reference)."""
    a = bf16_to_f32(a_bits).astype(np.float64)
    b = bf16_to_f32(b_bits).astype(np.float64)
    den = np.sqrt((b * b).sum(axis=1))
    den = np.where(den == 0, 1.0, den)
    return np.sqrt(((a - b) ** 2).sum(axis=1)) / den


# ---------------------------------------------------------------------------
# Scale-factor tile layout used by the tensor-core path (library-defined; the oracle
# restates it so the re-tiling kernels can be checked byte-for-byte).
# ---------------------------------------------------------------------------

def sf_tile_offsets(rows: int, kblocks: int) -> np.ndarray:
    """Byte offset of scale (row r, 16-element block j) in the tiled scale layout.

    Tiles of 128 rows x 4 blocks occupy 512 contiguous bytes; inside a tile the byte
    for (r, j) sits at (r % 32) * 16 + ((r % 128) // 32) * 4 + (j % 4).  Tiles are
    ordered row-tile major, block-tile minor.
    """
    assert kblocks % 4 == 0
    r = np.arange(rows)[:, None]
    j = np.arange(kblocks)[None, :]
    tile = (r // 128) * (kblocks // 4) + (j // 4)
    return tile * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + (j % 4)


def sf_tile(scale_bytes) -> np.ndarray:
    """Row-major scale bytes [rows, kblocks] -> tiled layout (rows padded to 128)."""
    sb = np.asarray(scale_bytes, np.uint8)
    rows, kb = sb.shape
    prow = (rows + 127) // 128 * 128
    out = np.zeros(prow * kb, np.uint8)
    out[sf_tile_offsets(rows, kb).reshape(-1)] = sb.reshape(-1)
    return out


# ---------------------------------------------------------------------------
# Seeded synthetic layers
# ---------------------------------------------------------------------------

class QuantizedLayer:
    """NVFP4 layer weights in the reference's tensor layout (a3):
    gate/up codes [E, I, H], scales [E, I, H/16]; down codes [E, H, I], scales [E, H, I/16];
    scale_2 [E, 3] = (gate, up, down)."""

    def __init__(self, router_w, bias, gate, gate_s, up, up_s, down, down_s, scale2):
        self.router_w, self.bias = router_w, bias
        self.gate, self.gate_s, self.up, self.up_s = gate, gate_s, up, up_s
        self.down, self.down_s, self.scale2 = down, down_s, scale2

    @property
    def dims(self):
        E, I, H = self.gate.shape
        return H, I, E

    def expert(self, e: int) -> ExpertWeights:
        return ExpertWeights(
            dequantize_weight(self.gate[e], self.gate_s[e], self.scale2[e, 0]),
            dequantize_weight(self.up[e], self.up_s[e], self.scale2[e, 1]),
            dequantize_weight(self.down[e], self.down_s[e], self.scale2[e, 2]))


def make_layer(seed: int, hidden: int, inter: int, experts: int, router_std=0.02,
               bias_std=0.01, weight_std=0.02) -> QuantizedLayer:
    """Seeded synthetic layer with the benchmark's distributions (numpy Generator;
    a stand-in for the torch stream of the full-size configuration)."""
    rng = np.random.default_rng(seed)
    rw = (rng.standard_normal((experts, hidden), np.float32) * np.float32(router_std)).astype(np.float32)
    bias = (rng.standard_normal(experts, np.float32) * np.float32(bias_std)).astype(np.float32)
    g = np.zeros((experts, inter, hidden), np.uint8); gs = np.zeros((experts, inter, hidden // 16), np.uint8)
    u = np.zeros_like(g); us = np.zeros_like(gs)
    d = np.zeros((experts, hidden, inter), np.uint8); ds = np.zeros((experts, hidden, inter // 16), np.uint8)
    s2 = np.zeros((experts, 3), np.float32)
    for e in range(experts):
        for t, (cw, cs, shape) in enumerate(((g, gs, (inter, hidden)), (u, us, (inter, hidden)),
                                              (d, ds, (hidden, inter)))):
            w = (rng.standard_normal(shape, np.float32) * np.float32(weight_std)).astype(np.float32)
            cw[e], cs[e], s2[e, t] = quantize_weight_baseline(w)
    return QuantizedLayer(rw, bias, g, gs, u, us, d, ds, s2)


def make_hidden(seed: int, tokens: int, hidden: int) -> np.ndarray:
    """bf16 N(0,1) activations as bit patterns."""
    rng = np.random.default_rng(seed)
    return bf16_round(rng.standard_normal((tokens, hidden), np.float32))


def layer_forward(layer: QuantizedLayer, hidden_bits, top_k: int = 8, mode: str = "O1",
                  world: int = 1, rank=None):
    """Router + MoE forward of one layer.  With ``rank`` set, returns only that
    expert-parallel shard's partial (experts with ``e % world == rank``)."""
    x = bf16_to_f32(hidden_bits)
    idx, wts, scores, sel = router_topk(x, layer.router_w, layer.bias, top_k)
    owner = None if rank is None else (lambda e: owner_for_expert(0, e, world, layer.dims[2]) == rank)
    cache = {}

    def getw(e):
        if e not in cache:
            cache[e] = layer.expert(e)
        return cache[e]

    out = moe_forward(hidden_bits, getw, idx, wts, mode=mode, only_owner=owner)
    return idx, wts, out
