"""Pin the CPU oracle against the reference's golden vectors and known answers.

The .npz files were produced by the reference's own Python (see
tests/golden/generate_golden.py); the literal vectors below are the known-answer
tests of the reference's native and Rust test suites.
"""
import os

import numpy as np

from oracle import glmrt_oracle as O


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_e4m3_decode_matches_reference_table(golden_dir):
    g = _load(golden_dir, "formats.npz")
    np.testing.assert_array_equal(O.e4m3_decode(np.arange(256, dtype=np.uint8)), g["e4m3_table"])
    # python/reference/tests/test_nvfp4_real_tensor_fixture_ref.py:22-63 and
    # sparse_mlp/math.rs:235: 0x38 -> 1.0; 0x7e -> 448 is the largest finite E4M3 value
    assert O.e4m3_decode(0x38) == 1.0 and O.e4m3_decode(0x7E) == 448.0


def test_e4m3_encode_matches_torch_float8(golden_dir):
    g = _load(golden_dir, "formats.npz")
    np.testing.assert_array_equal(O.e4m3_encode_satfinite(g["e4m3_enc_in"]), g["e4m3_enc_out"])
    assert O.e4m3_encode_satfinite(np.float32(1e9)) == 0x7E


def test_nvfp4_quantize_dequantize_match_quant_ref(golden_dir):
    g = _load(golden_dir, "formats.npz")
    for s in g["scales"]:
        codes = O.nvfp4_quantize(g["values"], s)
        np.testing.assert_array_equal(codes, g[f"codes_scale_{s}"])
        np.testing.assert_array_equal(O.nvfp4_dequantize(codes, s), g[f"deq_scale_{s}"])
    # exact ties go to the lower magnitude, -0 -> code 0
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.0, -0.75], np.float32)
    np.testing.assert_array_equal(O.fp4_codes_nearest_low(ties), [0, 1, 2, 3, 4, 5, 6, 0, 9])


def test_pack_unpack_and_decode_match_quant_ref(golden_dir):
    g = _load(golden_dir, "formats.npz")
    codes = g["codes_scale_1.0"][:4097]
    np.testing.assert_array_equal(O.pack_nibbles(codes), g["packed"])
    np.testing.assert_array_equal(O.unpack_nibbles(g["packed"], 4097), g["unpacked"])
    dec = O.decode_packed_nvfp4(g["packed"][:2048], g["decode_scale_bytes"], 0.01171875, 4096)
    np.testing.assert_allclose(dec, g["decoded"], rtol=1e-6, atol=0)
    # python/reference/tests/test_quant_pack_unpack_ref.py:13-17
    c = np.array([0, 1, 2, 15, 8], np.uint8)
    np.testing.assert_array_equal(O.unpack_nibbles(O.pack_nibbles(c), 5), c)


def test_rust_dot_packed_nvfp4_known_answer():
    # sparse_mlp/math.rs:223-237: 17 ones against these codes -> -2.5
    packed = np.array([0xA9] + [0x88] * 7 + [0x89], np.uint8)
    scale = np.array([0x38, 0x40], np.uint8)
    dot = O.dot_packed_nvfp4(np.ones(17, np.float32), packed, scale, 1.0)
    assert abs(float(dot) + 2.5) < 1e-6


def test_native_weight_quantiser_known_answer():
    # native/tests/cuda_selftest.cc:2736-2765: 16 codebook values, g = 448
    vals = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
                     -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], np.float32)
    codes, sb = O.quantize_weight_bf16_multiplicative(O.bf16_truncate(vals).reshape(1, 16), 448.0)
    np.testing.assert_array_equal(O.pack_nibbles(codes), [0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE])
    np.testing.assert_array_equal(sb.reshape(-1), [0x7E])


def test_router_small_and_glm52_match_reference(golden_dir):
    g = _load(golden_dir, "router.npz")
    for name in ("small", "glm52"):
        seed, T, H, E, K = g[f"{name}_meta"]
        r = np.random.default_rng(seed)
        rw = (r.standard_normal((E, H), np.float32) * np.float32(0.02)).astype(np.float32)
        bias = (r.standard_normal(E, np.float32) * np.float32(0.01)).astype(np.float32)
        hid = O.make_hidden(seed + 1000, T, H)
        idx, w, scores, sel = O.router_topk(O.bf16_to_f32(hid), rw, bias, int(K))
        sel64 = g[f"{name}_sel"].astype(np.float64)
        assert O.router_indices_equivalent(idx, g[f"{name}_idx"], sel64)
        same = np.all(idx.astype(np.int64) == g[f"{name}_idx"], axis=1)
        assert same.mean() > 0.9  # ordering inside the top-k agrees almost always
        np.testing.assert_allclose(w[same], g[f"{name}_w"][same], atol=1e-6, rtol=1e-5)
        np.testing.assert_allclose(w.sum(axis=1), 2.5, atol=1e-5)


def test_router_reference_generated_layer_golden(golden_dir):
    # python/reference/tests/test_glm_moe_dsa_layer_ref.py:67-96
    g = _load(golden_dir, "router.npz")
    E, H = 256, 6144
    rw = np.zeros((E, H), np.float32)
    for e in range(E):
        rw[e, e % H] = np.float32(0.03125 + e / 8192.0)
        rw[e, (e * 17 + 13) % H] = np.float32(-0.015625)
    bias = np.linspace(-0.125, 0.125, E, dtype=np.float64).astype(np.float32)
    idx, w, _, _ = O.router_topk(g["gen_normalized"], rw, bias, 8)
    assert idx[0].tolist() == [255, 254, 253, 252, 251, 250, 249, 248]
    assert idx[1].tolist() == [255, 254, 253, 252, 251, 250, 249, 248]
    np.testing.assert_allclose(w, g["gen_w"], atol=1e-6)
    np.testing.assert_allclose(w.sum(axis=1), 2.5, atol=1e-5)


def test_router_bias_selects_raw_score_weights():
    # python/reference/tests/test_glm_moe_dsa_layer_ref.py:33-64
    hidden = np.array([[1.0, 0.25, -0.5, 0.125]], np.float32)
    rw = np.array([[-2.0, 0, 0, 0], [1.5, 0, 0, 0], [1.0, 0, 0, 0], [0.5, 0, 0, 0]], np.float32)
    bias = np.array([2.0, 0, 0, 0], np.float32)
    idx, w, scores, sel = O.router_topk(hidden, rw, bias, 2)
    assert idx[0].tolist() == [0, 1]
    raw = np.array([scores[0, 0], scores[0, 1]])
    np.testing.assert_allclose(w[0], raw / raw.sum() * 2.5, rtol=1e-6)


def test_moe_layer_matches_reference_o0_and_o1(golden_dir):
    g = _load(golden_dir, "moe.npz")
    for name in ("tiny", "mid"):
        seed, T, H, I, E, K = (int(v) for v in g[f"{name}_meta"])
        layer = O.make_layer(seed, H, I, E)
        # the weight quantiser reproduces the reference-composed codes bit for bit
        for e in range(2):
            for t, (c, s) in enumerate(((layer.gate, layer.gate_s), (layer.up, layer.up_s),
                                        (layer.down, layer.down_s))):
                np.testing.assert_array_equal(c[e], g[f"{name}_w{e}_{t}_codes"])
                np.testing.assert_array_equal(s[e], g[f"{name}_w{e}_{t}_scales"])
                assert layer.scale2[e, t] == g[f"{name}_w{e}_{t}_g"]
        hid = O.make_hidden(seed + 1000, T, H)
        xc, xs = O.quantize_rows_nvfp4(O.bf16_to_f32(hid))
        np.testing.assert_array_equal(xc, g[f"{name}_xcodes"])
        np.testing.assert_array_equal(xs, g[f"{name}_xscales"])
        idx, w, out0 = O.layer_forward(layer, hid, K, mode="O0")
        np.testing.assert_array_equal(idx.astype(np.int64), g[f"{name}_idx"])
        np.testing.assert_allclose(w, g[f"{name}_w"], atol=1e-6)
        # float32 matmul summation order differs between numpy and torch: bf16 outputs agree
        # to within a few bf16 ulps, i.e. far inside the 2e-2 gate
        assert O.rel_l2_per_token(out0, g[f"{name}_o0"]).max() < 3e-3
        _, _, out1 = O.layer_forward(layer, hid, K, mode="O1")
        assert O.rel_l2_per_token(out1, g[f"{name}_o1"]).max() < 3e-3
        # expert-parallel partials (moe_ref.py:40-66) for a two-way modulo split
        for rank in range(2):
            _, _, part = O.layer_forward(layer, hid, K, mode="O0", world=2, rank=rank)
            assert O.rel_l2_per_token(part, g[f"{name}_p{rank}"]).max() < 3e-3


def test_payload_rne_rule_and_roundtrip():
    rng = np.random.default_rng(7)
    x = O.bf16_to_f32(O.bf16_round(rng.standard_normal((5, 64), np.float32)))
    codes, sb = O.quantize_rows_nvfp4(x, "rne_payload")
    p = O.payload_rows(codes, sb)
    assert p.shape == (5, 32 + 4)
    deq = O.dequantize_payload_rows(p, 64)
    assert np.abs(deq - x).max() <= 0.5 * np.abs(x).max()
    # the two code rules differ only on ties / reciprocal rounding
    codes2, sb2 = O.quantize_rows_nvfp4(x, "nearest_low")
    np.testing.assert_array_equal(sb, sb2)
    assert (codes != codes2).mean() < 0.05
    # zero block -> zero scale -> all-zero codes
    z = np.zeros((1, 16), np.float32)
    c, s = O.quantize_rows_nvfp4(z)
    assert c.sum() == 0 and s.sum() == 0


def test_plan_routes_counting_sort():
    idx = np.array([[3, 1], [1, 0], [3, 2], [1, 3]], np.int64)
    packed, blocks, counts = O.plan_routes(idx, 4, block_rows=2)
    n = idx.size
    assert counts.tolist() == [1, 3, 1, 3]
    assert blocks.tolist() == [0, 1, 1, 2, 3, 3]
    assert packed.tolist() == [3, n, 1, 2, 6, n, 5, n, 0, 4, 7, n]


def test_sf_tile_layout_is_a_permutation():
    sb = np.arange(256 * 8, dtype=np.uint32).reshape(256, 8)
    off = O.sf_tile_offsets(256, 8)
    assert sorted(off.reshape(-1).tolist()) == list(range(256 * 8))
    assert off[0, 0] == 0 and off[1, 0] == 16 and off[32, 0] == 4 and off[0, 1] == 1
    assert off[0, 4] == 512 and off[128, 0] == 1024
    del sb


def test_combine_and_sum_topk():
    rng = np.random.default_rng(3)
    y = O.bf16_round(rng.standard_normal((3, 8, 32), np.float32))
    w = rng.random((3, 8), np.float32)
    out = O.combine_routes_bf16(y, w)
    ref = (O.bf16_to_f32(y) * w[..., None]).sum(axis=1)
    assert np.abs(O.bf16_to_f32(out) - ref).max() < 0.1
    s = O.sum_topk_bf16(y)
    assert np.abs(O.bf16_to_f32(s) - O.bf16_to_f32(y).sum(axis=1)).max() < 0.05


def test_residual_adds_truncate_like_the_native_kernels():
    """native/tests/cuda_selftest.cc:1079-1093 inputs; expected values worked out by hand from
    the kernel's formula: float32 adds, results and the float32 delta truncated to bf16."""
    res = O.bf16_truncate(np.array([0.25, -0.5, 1.5, 2.0], np.float32))
    shared = O.bf16_truncate(np.array([-0.25, 0.75, 0.125, -1.5], np.float32))
    routed = np.array([-0.51, 0.26, 0.501, -1.001], np.float32)
    out = O.bf16_to_f32(O.residual_add_shared_f32_delta_bf16(res, shared, routed))
    # bf16(-0.51) = -0.5078125 (truncated), bf16(0.26) = 0.259765625, bf16(0.501) = 0.5, bf16(-1.001) = -1.0
    # mlp = bf16(shared + routed) = -0.7578125 -> trunc 8 bits: -0.7578125 = -0.11000010b -> -0.75390625
    want_mlp = O.bf16_to_f32(O.bf16_truncate(np.array([-0.25 - 0.5078125, 0.75 + 0.259765625, 0.125 + 0.5, -1.5 - 1.0], np.float32)))
    want = O.bf16_to_f32(O.bf16_truncate((O.bf16_to_f32(res) + want_mlp).astype(np.float32)))
    np.testing.assert_array_equal(out, want)
    assert out[2] == 2.125 and out[3] == -0.5            # exact cases: 1.5 + 0.625, 2.0 - 2.5
    # truncation, not rounding: 1 + 2^-8 + 2^-9 keeps only the 2^-8 bit... (7 explicit mantissa bits -> dropped entirely)
    x = np.array([1.0 + 2.0 ** -8 + 2.0 ** -9], np.float32)
    assert O.bf16_to_f32(O.bf16_truncate(x))[0] == 1.0
    assert O.bf16_to_f32(O.residual_add_f32_delta_bf16(O.bf16_truncate(np.array([0.0], np.float32)), x))[0] == 1.0
