"""GPU parity tests of the stand-alone kernels behind the reference-named C-ABI symbols:
router, NVFP4 codecs, combine.  Each compares the CUDA result with the CPU oracle on the
same seeded inputs (bit-exact for codes, indices and bf16 words), the pattern of the
reference's native/tests/cuda_selftest.cc.
"""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import glmrt_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib(pkg):
    from glmrt_b200 import native as N
    return N.library()


def dbuf(t):
    from glmrt_b200 import native as N
    return N.DeviceBuffer.of(t.data_ptr(), t.numel() * t.element_size(), 0)


def stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def bf16_tensor(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16).cuda()


def ptr(t):
    return C.c_void_p(t.data_ptr())


# ---------------------------------------------------------------------------------- router
@pytest.mark.parametrize("T,H,E,K", [(1, 256, 16, 4), (33, 256, 16, 4), (16, 6144, 256, 8), (200, 512, 64, 8)])
def test_router_bf16_f32w_matches_oracle(lib, T, H, E, K):
    rng = np.random.default_rng(T * 7 + E)
    rw = (rng.standard_normal((E, H), np.float32) * np.float32(0.02)).astype(np.float32)
    bias = (rng.standard_normal(E, np.float32) * np.float32(0.01)).astype(np.float32)
    hid = O.make_hidden(T + 5, T, H)
    x = bf16_tensor(hid)
    w = torch.from_numpy(rw).cuda()
    b = torch.from_numpy(bias).cuda()
    logits = torch.empty(T * E, dtype=torch.float32, device="cuda")
    idx = torch.empty((T, K), dtype=torch.int32, device="cuda")
    sc = torch.empty((T, K), dtype=torch.float32, device="cuda")
    wt = torch.empty((T, K), dtype=torch.float32, device="cuda")
    lib.call("glmrt_b200_router_topk_bf16_f32w_async", ptr(x), ptr(w), ptr(b), ptr(logits), ptr(idx), ptr(sc),
             ptr(wt), C.c_size_t(T), C.c_size_t(H), C.c_size_t(E), C.c_size_t(K), stream())
    torch.cuda.synchronize()
    oi, ow, oscores, osel = O.router_topk(O.bf16_to_f32(hid), rw, bias, K)
    sel64 = (1.0 / (1.0 + np.exp(-(O.bf16_to_f32(hid).astype(np.float64) @ rw.astype(np.float64).T)))) + bias
    gi = idx.cpu().numpy()
    assert O.router_indices_equivalent(gi, oi, sel64, tol=1e-6)
    same = np.all(gi == oi.astype(np.int32), axis=1)
    assert same.mean() > 0.9
    np.testing.assert_allclose(wt.cpu().numpy()[same], ow[same], atol=2e-6, rtol=1e-5)
    np.testing.assert_allclose(wt.cpu().numpy().sum(axis=1), 2.5, atol=1e-5)
    raw = np.take_along_axis(oscores, oi.astype(np.int64), axis=1)
    np.testing.assert_allclose(sc.cpu().numpy()[same], raw[same], atol=2e-6)


def test_router_reference_named_entry_points_and_golden(lib, golden_dir):
    # generated-layer golden of python/reference/tests/test_glm_moe_dsa_layer_ref.py:67-96
    g = np.load(os.path.join(golden_dir, "router.npz"))
    E, H, K = 256, 6144, 8
    rw = np.zeros((E, H), np.float32)
    for e in range(E):
        rw[e, e % H] = np.float32(0.03125 + e / 8192.0)
        rw[e, (e * 17 + 13) % H] = np.float32(-0.015625)
    bias = np.linspace(-0.125, 0.125, E, dtype=np.float64).astype(np.float32)
    x = torch.from_numpy(g["gen_normalized"]).cuda()
    w = torch.from_numpy(rw).cuda()
    b = torch.from_numpy(bias).cuda()
    idx = torch.empty((2, K), dtype=torch.int32, device="cuda")
    sc = torch.empty((2, K), dtype=torch.float32, device="cuda")
    wt = torch.empty((2, K), dtype=torch.float32, device="cuda")
    lib.call("glmrt_cuda_router_topk_f32", ptr(x), ptr(w), ptr(b), ptr(idx), ptr(sc), ptr(wt), C.c_size_t(2),
             C.c_size_t(H), C.c_size_t(E), C.c_size_t(K))
    assert idx.cpu().numpy().tolist() == [[255, 254, 253, 252, 251, 250, 249, 248]] * 2
    np.testing.assert_allclose(wt.cpu().numpy(), g["gen_w"], atol=1e-6)
    # bf16 x bf16 variant against the oracle with bf16-rounded weights
    rng = np.random.default_rng(5)
    hid = O.make_hidden(77, 9, 512)
    rwb = O.bf16_round((rng.standard_normal((32, 512), np.float32) * np.float32(0.05)).astype(np.float32))
    bias = (rng.standard_normal(32, np.float32) * np.float32(0.01)).astype(np.float32)
    idx = torch.empty((9, 4), dtype=torch.int32, device="cuda")
    sc = torch.empty((9, 4), dtype=torch.float32, device="cuda")
    wt = torch.empty((9, 4), dtype=torch.float32, device="cuda")
    xb, wb, bb = bf16_tensor(hid), bf16_tensor(rwb), torch.from_numpy(bias).cuda()
    lib.call("glmrt_cuda_router_topk_bf16", ptr(xb), ptr(wb), ptr(bb), ptr(idx), ptr(sc), ptr(wt), C.c_size_t(9),
             C.c_size_t(512), C.c_size_t(32), C.c_size_t(4))
    oi, ow, _, _ = O.router_topk(O.bf16_to_f32(hid), O.bf16_to_f32(rwb), bias, 4)
    np.testing.assert_array_equal(idx.cpu().numpy(), oi.astype(np.int32))
    np.testing.assert_allclose(wt.cpu().numpy(), ow, atol=2e-6)
    # the variant with caller-owned scratch (native/include/glmrt_native.h:1019-1030): same answer, nothing allocated
    n = 9 * 32
    f1, f2 = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    u1 = torch.zeros(n, dtype=torch.int32, device="cuda")
    u2 = torch.zeros(n, dtype=torch.int32, device="cuda")
    seg = torch.zeros(10, dtype=torch.int32, device="cuda")
    tmp = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    idx2, sc2, wt2 = torch.empty_like(idx), torch.empty_like(sc), torch.empty_like(wt)
    lib.call("glmrt_cuda_router_topk_bf16_cub_async", ptr(xb), ptr(wb), ptr(bb), ptr(f1), ptr(f2), ptr(u1), ptr(u2),
             ptr(seg), ptr(idx2), ptr(sc2), ptr(wt2), ptr(tmp), C.c_size_t(4096), C.c_size_t(9), C.c_size_t(512),
             C.c_size_t(32), C.c_size_t(4), stream())
    torch.cuda.synchronize()
    assert torch.equal(idx2, idx) and torch.equal(wt2, wt) and torch.equal(sc2, sc)
    assert lib.call_status("glmrt_cuda_router_topk_bf16_cub_async", ptr(xb), ptr(wb), ptr(bb), ptr(f1), ptr(f2), ptr(u1),
                           ptr(u2), ptr(seg), ptr(idx2), ptr(sc2), ptr(wt2), None, C.c_size_t(0), C.c_size_t(9),
                           C.c_size_t(512), C.c_size_t(32), C.c_size_t(4), stream()) == 1


@pytest.mark.parametrize("E", [40, 256, 320])
def test_router_negative_selection_scores_on_both_selection_paths(lib, E):
    """Up to 256 experts the selection runs on registers with an order-preserving integer key, above
    that on shared memory: both must rank negative selection scores (a strongly negative bias) like
    the oracle, whose arg-max is on the corrected score while the weights come from the raw one."""
    T, H, K = 12, 512, 8
    rng = np.random.default_rng(E)
    rw = (rng.standard_normal((E, H), np.float32) * np.float32(0.05)).astype(np.float32)
    bias = (-2.0 - rng.random(E)).astype(np.float32)
    hid = O.make_hidden(E, T, H)
    x = bf16_tensor(hid)
    w, b = torch.from_numpy(rw).cuda(), torch.from_numpy(bias).cuda()
    logits = torch.empty(T * E, dtype=torch.float32, device="cuda")
    idx = torch.empty((T, K), dtype=torch.int32, device="cuda")
    sc = torch.empty((T, K), dtype=torch.float32, device="cuda")
    wt = torch.empty((T, K), dtype=torch.float32, device="cuda")
    lib.call("glmrt_b200_router_topk_bf16_f32w_async", ptr(x), ptr(w), ptr(b), ptr(logits), ptr(idx), ptr(sc),
             ptr(wt), C.c_size_t(T), C.c_size_t(H), C.c_size_t(E), C.c_size_t(K), stream())
    torch.cuda.synchronize()
    oi, ow, _, _ = O.router_topk(O.bf16_to_f32(hid), rw, bias, K)
    sel64 = (1.0 / (1.0 + np.exp(-(O.bf16_to_f32(hid).astype(np.float64) @ rw.astype(np.float64).T)))) + bias
    assert (sel64 < 0).all()
    gi = idx.cpu().numpy()
    assert O.router_indices_equivalent(gi, oi, sel64, tol=1e-6)
    same = np.all(gi == oi.astype(np.int32), axis=1)
    assert same.mean() > 0.9
    np.testing.assert_allclose(wt.cpu().numpy()[same], ow[same], atol=2e-6, rtol=1e-5)


def test_router_ties_go_to_lower_expert_and_nonfinite_scores_are_skipped(lib):
    H, E, K = 256, 8, 3
    x = np.zeros((2, H), np.float32)
    x[:, 0] = 1.0
    rw = np.zeros((E, H), np.float32)
    rw[:, 0] = [0.5, 1.0, 1.0, 0.25, 1.0, -1.0, 0.0, 0.0]   # experts 1, 2, 4 tie
    bias = np.zeros(E, np.float32)
    bias[7] = np.inf                                         # non-finite corrected score: never selected
    xt = bf16_tensor(O.bf16_round(x))
    logits = torch.empty(2 * E, dtype=torch.float32, device="cuda")
    idx = torch.empty((2, K), dtype=torch.int32, device="cuda")
    sc = torch.empty((2, K), dtype=torch.float32, device="cuda")
    wt = torch.empty((2, K), dtype=torch.float32, device="cuda")
    w, b = torch.from_numpy(rw).cuda(), torch.from_numpy(bias).cuda()
    lib.call("glmrt_b200_router_topk_bf16_f32w_async", ptr(xt), ptr(w), ptr(b), ptr(logits), ptr(idx), ptr(sc),
             ptr(wt), C.c_size_t(2), C.c_size_t(H), C.c_size_t(E), C.c_size_t(K), stream())
    torch.cuda.synchronize()
    assert idx.cpu().numpy().tolist() == [[1, 2, 4], [1, 2, 4]]
    oi, _, _, _ = O.router_topk(x, rw, bias, K)
    assert oi.tolist() == [[1, 2, 4], [1, 2, 4]]


# ---------------------------------------------------------------------------------- codecs
@pytest.mark.parametrize("rule,name", [(0, "rne_payload"), (1, "nearest_low")])
@pytest.mark.parametrize("T,H", [(1, 6144), (37, 6144), (5, 48), (64, 256)])
def test_payload_quantiser_bit_exact(lib, rule, name, T, H):
    rng = np.random.default_rng(T * 31 + H)
    x = rng.standard_normal((T, H), np.float32)
    x[0, :16] = 0.0                                  # zero block -> zero scale
    if H >= 48:
        x[0, 16:32] = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0]
        x[0, 32:48] *= 1e-4                          # sub-normal E4M3 scale range
    bits = O.bf16_round(x)
    xin = bf16_tensor(bits)
    out = torch.zeros(T * (H // 2 + H // 16), dtype=torch.uint8, device="cuda")
    lib.call("glmrt_b200_quantize_bf16_nvfp4_row_payload_async", dbuf(xin), dbuf(out), C.c_size_t(T),
             C.c_size_t(H), C.c_uint32(rule), stream())
    torch.cuda.synchronize()
    codes, sb = O.quantize_rows_nvfp4(O.bf16_to_f32(bits), name)
    np.testing.assert_array_equal(out.cpu().numpy().reshape(T, -1), O.payload_rows(codes, sb))
    if rule == 0:  # the reference-named symbol is the RNE rule
        out2 = torch.zeros_like(out)
        lib.call("glmrt_cuda_b12x_quantize_bf16_nvfp4_row_payload_async", dbuf(xin), dbuf(out2), C.c_size_t(T),
                 C.c_size_t(H), stream())
        torch.cuda.synchronize()
        assert torch.equal(out, out2)


def test_payload_quantiser_many_values_including_every_tie(lib):
    # >= 10^7 values: every bf16 bit pattern with a finite value appears, scaled copies of the ties too
    allb = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    fin = allb[np.isfinite(O.bf16_to_f32(allb))]
    rng = np.random.default_rng(0)
    bits = np.concatenate([fin, O.bf16_round(rng.standard_normal(10_400_000 - fin.size, np.float32) * 3)])
    bits = bits[: bits.size // 6144 * 6144].reshape(-1, 6144)
    xin = bf16_tensor(bits)
    T = bits.shape[0]
    out = torch.zeros(T * 3456, dtype=torch.uint8, device="cuda")
    lib.call("glmrt_b200_quantize_bf16_nvfp4_row_payload_async", dbuf(xin), dbuf(out), C.c_size_t(T),
             C.c_size_t(6144), C.c_uint32(1), stream())
    torch.cuda.synchronize()
    codes, sb = O.quantize_rows_nvfp4(O.bf16_to_f32(bits), "nearest_low")
    np.testing.assert_array_equal(out.cpu().numpy().reshape(T, -1), O.payload_rows(codes, sb))


def test_weight_quantiser_known_answer_and_random(lib):
    # native/tests/cuda_selftest.cc:2736-2765
    vals = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], np.float32)
    xin = bf16_tensor(O.bf16_truncate(vals).reshape(1, 16))
    packed = torch.zeros(8, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(1, dtype=torch.uint8, device="cuda")
    lib.call("glmrt_cuda_quantize_bf16_weight_nvfp4_async", dbuf(xin), dbuf(packed), dbuf(scales), C.c_size_t(1),
             C.c_size_t(16), C.c_float(448.0), stream())
    torch.cuda.synchronize()
    assert packed.cpu().numpy().tolist() == [0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE]
    assert scales.cpu().numpy().tolist() == [0x7E]
    rng = np.random.default_rng(9)
    wb = O.bf16_round(rng.standard_normal((64, 256), np.float32) * np.float32(0.02))
    xin = bf16_tensor(wb)
    packed = torch.zeros(64 * 128, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(64 * 16, dtype=torch.uint8, device="cuda")
    lib.call("glmrt_cuda_quantize_bf16_weight_nvfp4_async", dbuf(xin), dbuf(packed), dbuf(scales), C.c_size_t(64),
             C.c_size_t(256), C.c_float(3000.0), stream())
    torch.cuda.synchronize()
    codes, sb = O.quantize_weight_bf16_multiplicative(wb, 3000.0)
    np.testing.assert_array_equal(scales.cpu().numpy().reshape(64, 16), sb)
    np.testing.assert_array_equal(packed.cpu().numpy(), O.pack_nibbles(codes))


def test_f32_weight_quantiser_matches_oracle_recipe(lib):
    rng = np.random.default_rng(4)
    w = (rng.standard_normal((256, 512), np.float32) * np.float32(0.02)).astype(np.float32)
    w[3, :16] = 0.0
    win = torch.from_numpy(w).cuda()
    packed = torch.zeros(256 * 256, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(256 * 32, dtype=torch.uint8, device="cuda")
    s2 = torch.zeros(1, dtype=torch.float32, device="cuda")
    scratch = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib.call("glmrt_b200_quantize_f32_weight_nvfp4_async", dbuf(win), dbuf(packed), dbuf(scales), dbuf(s2),
             dbuf(scratch), C.c_size_t(256), C.c_size_t(512), stream())
    torch.cuda.synchronize()
    codes, sb, g = O.quantize_weight_baseline(w)
    assert float(s2.cpu()[0]) == float(g)
    np.testing.assert_array_equal(scales.cpu().numpy().reshape(256, 32), sb)
    np.testing.assert_array_equal(packed.cpu().numpy(), O.pack_nibbles(codes))


def test_gather_payload_rows_to_bf16(lib):
    rng = np.random.default_rng(2)
    x = O.bf16_to_f32(O.bf16_round(rng.standard_normal((6, 64), np.float32)))
    codes, sb = O.quantize_rows_nvfp4(x, "rne_payload")
    pay = O.payload_rows(codes, sb)
    rows = np.array([5, 0, 3, 3], np.uint32)
    p = torch.from_numpy(pay).cuda()
    ri = torch.from_numpy(rows.view(np.int32)).cuda()
    out = torch.zeros((4, 64), dtype=torch.bfloat16, device="cuda")
    lib.call("glmrt_cuda_b12x_gather_nvfp4_rows_bf16_async", dbuf(p), C.c_size_t(6), C.c_size_t(36), dbuf(ri),
             dbuf(out), C.c_size_t(4), C.c_size_t(64), stream())
    torch.cuda.synchronize()
    want = O.bf16_truncate(O.dequantize_payload_rows(pay, 64)[rows.astype(np.int64)])
    np.testing.assert_array_equal(out.cpu().view(torch.int16).numpy().view(np.uint16), want)


# ---------------------------------------------------------------------------------- combine
def test_sum_topk8_and_weighted_scatter_and_gather(lib):
    rng = np.random.default_rng(8)
    y = O.bf16_round(rng.standard_normal((3, 8, 6144), np.float32))
    yt = bf16_tensor(y.reshape(24, 6144))
    out = torch.zeros((3, 6144), dtype=torch.bfloat16, device="cuda")
    lib.call("glmrt_cuda_b12x_spark_sum_topk8_bf16_async", dbuf(yt), dbuf(out), C.c_size_t(3), stream())
    torch.cuda.synchronize()
    np.testing.assert_array_equal(out.cpu().view(torch.int16).numpy().view(np.uint16), O.sum_topk_bf16(y))
    # weighted scatter-add: distinct destination rows -> deterministic
    src = O.bf16_round(rng.standard_normal((4, 96), np.float32))
    ri = np.array([2, 0, 3, 1], np.uint32)
    w = rng.random(4, np.float32)
    dst0 = rng.standard_normal((4, 96), np.float32)
    dst = torch.from_numpy(dst0.copy()).cuda()
    st, rt, wt = bf16_tensor(src), torch.from_numpy(ri.view(np.int32)).cuda(), torch.from_numpy(w).cuda()
    lib.call("glmrt_cuda_scatter_add_rows_bf16_weighted_to_f32", ptr(st), ptr(rt), ptr(wt), ptr(dst), C.c_size_t(4),
             C.c_size_t(96))
    want = O.scatter_add_rows_bf16_weighted_to_f32(src, ri, w, dst0)
    np.testing.assert_allclose(dst.cpu().numpy(), want, rtol=1e-6, atol=1e-7)
    g = torch.zeros((4, 96), dtype=torch.bfloat16, device="cuda")
    lib.call("glmrt_cuda_gather_rows_bf16_async", ptr(st), ptr(rt), ptr(g), C.c_size_t(4), C.c_size_t(96), stream())
    torch.cuda.synchronize()
    np.testing.assert_array_equal(g.cpu().view(torch.int16).numpy().view(np.uint16), src[ri.astype(np.int64)])


def test_residual_adds_match_oracle_bit_exactly(lib):
    """native/tests/cuda_selftest.cc:1053-1110 (same inputs, same host formula), then random data
    with values whose sums are not representable in bf16 so that truncation matters."""
    res = O.bf16_truncate(np.array([0.25, -0.5, 1.5, 2.0, -3.0, 4.5, 0.0, -0.125], np.float32))
    shared = O.bf16_truncate(np.array([-0.25, 0.75, 0.125, -1.5, 2.0, -0.5, 0.25, 0.5], np.float32))
    routed = np.array([-0.51, 0.26, 0.501, -1.001, 3.51, -2.01, 0.126, 0.251], np.float32)
    rng = np.random.default_rng(12)
    n = 100003                                                        # not a multiple of the block size
    cases = [(res, shared, routed),
             (O.bf16_round(rng.standard_normal(n, np.float32) * 3), O.bf16_round(rng.standard_normal(n, np.float32)),
              rng.standard_normal(n, np.float32))]
    for r, sh, rt in cases:
        k = r.size
        rt_t, sh_t = bf16_tensor(r), bf16_tensor(sh)
        d32 = torch.from_numpy(rt).cuda()
        out = torch.zeros(k, dtype=torch.bfloat16, device="cuda")
        bits = lambda t: t.cpu().view(torch.int16).numpy().view(np.uint16)
        lib.call("glmrt_cuda_residual_add_shared_f32_delta_bf16_async", ptr(rt_t), ptr(sh_t), ptr(d32), ptr(out),
                 C.c_size_t(k), stream())
        torch.cuda.synchronize()
        np.testing.assert_array_equal(bits(out), O.residual_add_shared_f32_delta_bf16(r, sh, rt))
        lib.call("glmrt_cuda_residual_add_f32_delta_bf16", ptr(rt_t), ptr(d32), ptr(out), C.c_size_t(k))
        np.testing.assert_array_equal(bits(out), O.residual_add_f32_delta_bf16(r, rt))
        lib.call("glmrt_cuda_residual_add_bf16", ptr(rt_t), ptr(sh_t), ptr(out), C.c_size_t(k))
        np.testing.assert_array_equal(bits(out), O.residual_add_bf16(r, sh))
    # empty range is accepted; null pointers are not
    assert lib.call_status("glmrt_cuda_residual_add_bf16_async", None, None, None, C.c_size_t(0), stream()) == 0
    assert lib.call_status("glmrt_cuda_residual_add_bf16_async", None, None, None, C.c_size_t(4), stream()) == 1


def test_w4a16_route_mlp_entry_points_match_the_float32_reference(lib, pkg):
    """The reference's float32 route MLP symbols (bf16 activations x NVFP4 weights, no activation
    quantisation; native/cuda/kernels/mlp.cu:218-420): grouped (one expert for all routes) and batched
    (an expert per route through the metadata table), against the float32 expert_forward of the
    Python reference (moe_ref.py:17-21) restated in the oracle.  A route whose row index is out of
    range is skipped."""
    from glmrt_b200 import native as N
    H, I, E = 512, 256, 3
    ref = O.make_layer(5, H, I, E)
    rows, routes = 6, 14
    rng = np.random.default_rng(2)
    hid = O.make_hidden(88, rows, H)
    stride = H + 32                                           # rows wider than hidden_dim
    xs = np.zeros((rows, stride), np.uint16)
    xs[:, :H] = hid
    row_idx = rng.integers(0, rows, routes).astype(np.uint32)
    row_idx[5] = 1000                                         # out of range: skipped
    rw = rng.random(routes, np.float32)
    experts = rng.integers(0, E, routes)

    def pack(c):
        c = np.ascontiguousarray(c, np.uint8)
        return (c[..., 0::2] | (c[..., 1::2] << 4)).astype(np.uint8)

    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    W = [dict(g=dev(pack(ref.gate[e])), gs=dev(ref.gate_s[e]), u=dev(pack(ref.up[e])), us=dev(ref.up_s[e]),
              d=dev(pack(ref.down[e])), ds=dev(ref.down_s[e])) for e in range(E)]
    x = dev(xs.view(np.int16)).view(torch.bfloat16)
    ri, rwt = dev(row_idx.view(np.int32)), dev(rw)
    x32 = O.bf16_to_f32(hid)

    def expected(expert_of_route):
        acc = np.zeros((rows, H), np.float64)
        for r in range(routes):
            if row_idx[r] >= rows:
                continue
            y = O.expert_forward(x32[row_idx[r]][None, :], ref.expert(int(expert_of_route[r])))[0]
            acc[row_idx[r]] += np.float64(rw[r]) * y.astype(np.float64)
        return acc

    work = torch.zeros(routes * I, device="cuda")
    # grouped: expert 1 for every route
    acc = torch.zeros(rows, H, device="cuda")
    s2 = ref.scale2[1]
    lib.call("glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_grouped_staged_accumulate_f32_async", ptr(x), ptr(ri), ptr(rwt),
             ptr(W[1]["g"]), ptr(W[1]["gs"]), ptr(W[1]["u"]), ptr(W[1]["us"]), ptr(W[1]["d"]), ptr(W[1]["ds"]), ptr(work),
             ptr(acc), C.c_size_t(rows), C.c_size_t(routes), C.c_size_t(H), C.c_size_t(stride), C.c_size_t(I), C.c_size_t(H),
             C.c_size_t(I // 2), C.c_size_t(I // 16), C.c_float(s2[0]), C.c_float(s2[1]), C.c_float(s2[2]), stream())
    torch.cuda.synchronize()
    want = expected(np.full(routes, 1))
    scale = np.abs(want).max()
    np.testing.assert_allclose(acc.cpu().numpy(), want, atol=2e-5 * scale, rtol=1e-4)
    assert float(work[5 * I:(5 + 1) * I].abs().max()) == 0.0      # the skipped route staged zeros
    # batched: an expert per route
    meta = (N.RouteBatchedMetadata * routes)()
    for r in range(routes):
        w, s2 = W[int(experts[r])], ref.scale2[int(experts[r])]
        meta[r] = N.RouteBatchedMetadata(w["g"].data_ptr(), w["gs"].data_ptr(), w["u"].data_ptr(), w["us"].data_ptr(),
                                         w["d"].data_ptr(), w["ds"].data_ptr(), I, I // 2, I // 16, s2[0], s2[1], s2[2])
    meta_dev = torch.from_numpy(np.frombuffer(bytes(meta), np.uint8).copy()).cuda()
    acc2 = torch.zeros(rows, H, device="cuda")
    lib.call("glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_batched_staged_accumulate_f32", ptr(x), ptr(ri), ptr(rwt),
             ptr(meta_dev), ptr(work), ptr(acc2), C.c_size_t(rows), C.c_size_t(routes), C.c_size_t(H), C.c_size_t(stride),
             C.c_size_t(I), C.c_size_t(H))
    want2 = expected(experts)
    np.testing.assert_allclose(acc2.cpu().numpy(), want2, atol=2e-5 * np.abs(want2).max(), rtol=1e-4)
    assert lib.call_status("glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_batched_staged_accumulate_f32_async", ptr(x), ptr(ri),
                           ptr(rwt), None, ptr(work), ptr(acc2), C.c_size_t(rows), C.c_size_t(routes), C.c_size_t(H),
                           C.c_size_t(stride), C.c_size_t(I), C.c_size_t(H), stream()) == 1
    # single row (mlp.cu:474-518): routes whose row index is 0 are summed in route order and the row is
    # written as truncated bf16; other routes are ignored; rows other than 1 are refused
    one_idx = np.zeros(routes, np.uint32)
    one_idx[[2, 9]] = 1
    oi = dev(one_idx.view(np.int32))
    out1 = torch.full((H,), 7.0, dtype=torch.bfloat16, device="cuda")
    lib.call("glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_batched_staged_single_row_bf16_async", ptr(x), ptr(oi), ptr(rwt),
             ptr(meta_dev), ptr(work), ptr(out1), C.c_size_t(1), C.c_size_t(routes), C.c_size_t(H), C.c_size_t(stride),
             C.c_size_t(I), C.c_size_t(H), stream())
    torch.cuda.synchronize()
    want1 = np.zeros(H, np.float64)
    for r in range(routes):
        if one_idx[r] == 0:
            want1 += np.float64(rw[r]) * O.expert_forward(x32[0][None, :], ref.expert(int(experts[r])))[0].astype(np.float64)
    got1 = out1.float().cpu().numpy()
    s1 = np.abs(want1).max()
    assert np.abs(got1 - want1).max() <= 2 ** -7 * s1         # one bf16 truncation of a float32 sum
    assert (np.abs(got1) <= np.abs(want1) + 2e-5 * s1).all()  # truncation never rounds away from zero
    assert lib.call_status("glmrt_cuda_nvfp4_silu_gated_mlp_route_bf16_batched_staged_single_row_bf16_async", ptr(x), ptr(oi),
                           ptr(rwt), ptr(meta_dev), ptr(work), ptr(out1), C.c_size_t(2), C.c_size_t(routes), C.c_size_t(H),
                           C.c_size_t(stride), C.c_size_t(I), C.c_size_t(H), stream()) == 1


@pytest.mark.parametrize("rows", [5, 200])
def test_row_gather_scatter_add_and_shard_reduce_family(lib, pkg, rows):
    """native/include/glmrt_native.h:757-836.  Up to 64 source rows the scatter-adds are ordered
    (bit-exact against the oracle's source-order sum, duplicates in the index list included); above
    that they use atomics (checked to float32 round-off)."""
    from glmrt_b200 import native as N
    rng = np.random.default_rng(rows)
    W, D = 128, 9
    idx = rng.integers(0, D, rows).astype(np.uint32)
    ridx = torch.from_numpy(idx.view(np.int32)).cuda()
    f32 = rng.standard_normal((rows, W), np.float32)
    bits = O.bf16_round(f32)
    fp8 = O.bf16_rows_to_fp8_e4m3_row_scaled(bits)
    dst0 = rng.standard_normal((D, W), np.float32)
    exact = rows <= 64

    def check(symbol, src_tensor, values, *extra):
        dst = torch.from_numpy(dst0.copy()).cuda()
        lib.call(symbol, ptr(src_tensor), *extra, ptr(ridx), ptr(dst), C.c_size_t(rows), C.c_size_t(W), stream())
        torch.cuda.synchronize()
        want = O.scatter_add_rows_to_f32(values, idx, dst0)
        if exact:
            np.testing.assert_array_equal(dst.cpu().numpy(), want)
        else:
            np.testing.assert_allclose(dst.cpu().numpy(), want, rtol=1e-5, atol=1e-5)

    check("glmrt_cuda_scatter_add_rows_f32_async", torch.from_numpy(f32).cuda(), f32)
    check("glmrt_cuda_scatter_add_rows_bf16_to_f32_async", bf16_tensor(bits), O.bf16_to_f32(bits))
    check("glmrt_cuda_scatter_add_rows_fp8_e4m3_row_scaled_to_f32_async", torch.from_numpy(fp8).cuda(),
          O.decode_wire_rows(fp8, W, "fp8"), C.c_size_t(W + 4))
    pay = torch.zeros(rows * (W // 2 + W // 16), dtype=torch.uint8, device="cuda")
    xb = bf16_tensor(bits)
    lib.call("glmrt_cuda_b12x_quantize_bf16_nvfp4_row_payload_async", N.DeviceBuffer.of(xb.data_ptr(), xb.numel() * 2),
             N.DeviceBuffer.of(pay.data_ptr(), pay.numel()), C.c_size_t(rows), C.c_size_t(W), stream())
    torch.cuda.synchronize()
    nvrows = pay.cpu().numpy().reshape(rows, W // 2 + W // 16)
    check("glmrt_cuda_scatter_add_rows_nvfp4_e2m1_fp8_e4m3_to_f32_async", pay, O.decode_wire_rows(nvrows, W, "nvfp4"),
          C.c_size_t(W // 2 + W // 16))
    # gathers
    table = rng.standard_normal((D, W), np.float32)
    t = torch.from_numpy(table).cuda()
    g = torch.zeros(rows, W, device="cuda")
    lib.call("glmrt_cuda_gather_rows_f32", ptr(t), ptr(ridx), ptr(g), C.c_size_t(rows), C.c_size_t(W))
    np.testing.assert_array_equal(g.cpu().numpy(), table[idx.astype(np.int64)])
    tb = bf16_tensor(O.bf16_round(table))
    gb = torch.zeros(rows, W, dtype=torch.bfloat16, device="cuda")
    lib.call("glmrt_cuda_gather_rows_bf16", ptr(tb), ptr(ridx), ptr(gb), C.c_size_t(rows), C.c_size_t(W))
    np.testing.assert_array_equal(gb.cpu().view(torch.int16).numpy().view(np.uint16), O.bf16_round(table)[idx.astype(np.int64)])
    # shard reduce: bf16 local + two row-scaled FP8 peers + one more, peers added in order
    local = O.bf16_round(rng.standard_normal((rows, W), np.float32))
    peers = [O.bf16_rows_to_fp8_e4m3_row_scaled(O.bf16_round(rng.standard_normal((rows, W), np.float32))) for _ in range(3)]
    lt = bf16_tensor(local)
    pts = [torch.from_numpy(p).cuda() for p in peers]
    out = torch.zeros(rows, W, device="cuda")
    bufs = N.RouteShardReductionBuffers()
    bufs.local = N.DeviceBuffer.of(lt.data_ptr(), lt.numel() * 2)
    for i, p in enumerate(pts):
        bufs.peers[i] = N.DeviceBuffer.of(p.data_ptr(), p.numel())
    bufs.output_f32 = N.DeviceBuffer.of(out.data_ptr(), out.numel() * 4)
    lib.call("glmrt_cuda_reduce_route_shards_to_f32", C.byref(bufs), C.c_size_t(rows), C.c_size_t(W), C.c_size_t(W + 4),
             C.c_uint32(2), C.c_uint32(2), C.c_uint32(3))
    want = O.reduce_route_shards_to_f32(O.bf16_to_f32(local), [O.decode_wire_rows(p, W, "fp8") for p in peers])
    np.testing.assert_array_equal(out.cpu().numpy(), want)
    assert lib.call_status("glmrt_cuda_reduce_route_shards_to_f32", C.byref(bufs), C.c_size_t(rows), C.c_size_t(W),
                           C.c_size_t(W + 4), C.c_uint32(2), C.c_uint32(2), C.c_uint32(4)) == 1


def test_bf16_rows_to_fp8_row_scaled_matches_oracle(lib):
    """native/cuda/kernels/residual.cu:245-277: E4M3 bytes + one float32 scale per row; an all-zero
    row keeps scale 1, non-finite values encode 0 and do not enter the row maximum."""
    rng = np.random.default_rng(14)
    R, W = 7, 6144
    x = rng.standard_normal((R, W), np.float32) * np.float32(3.0)
    x[1] = 0.0
    x[2, 5], x[2, 9], x[2, 100] = np.inf, -np.inf, np.nan
    x[3] *= np.float32(1e-6)
    x[4] *= np.float32(1e4)
    bits = O.bf16_round(x)
    src = bf16_tensor(bits)
    stride = W + 8                                        # wider than the row: the tail stays untouched
    dst = torch.full((R, stride), 0xAB, dtype=torch.uint8, device="cuda")
    lib.call("glmrt_cuda_bf16_rows_to_fp8_e4m3_row_scaled_async", ptr(src), ptr(dst), C.c_size_t(R), C.c_size_t(W),
             C.c_size_t(stride), stream())
    torch.cuda.synchronize()
    got = dst.cpu().numpy()
    want = O.bf16_rows_to_fp8_e4m3_row_scaled(bits)
    np.testing.assert_array_equal(got[:, :W + 4], want)
    assert (got[:, W + 4:] == 0xAB).all()
    assert want[1, W:].view(np.float32)[0] == 1.0
    assert lib.call_status("glmrt_cuda_bf16_rows_to_fp8_e4m3_row_scaled_async", ptr(src), ptr(dst), C.c_size_t(R),
                           C.c_size_t(W), C.c_size_t(W + 2), stream()) == 1
    # the response pack: float32 rows picked through an index list (residual.cu:160-196)
    table = torch.from_numpy(O.bf16_to_f32(bits)).cuda()
    pick = np.array([6, 1, 1, 3], np.uint32)
    dst2 = torch.zeros((4, W + 4), dtype=torch.uint8, device="cuda")
    lib.call("glmrt_cuda_gather_rows_f32_to_fp8_e4m3_row_scaled", ptr(table), ptr(torch.from_numpy(pick.view(np.int32)).cuda()),
             ptr(dst2), C.c_size_t(4), C.c_size_t(W), C.c_size_t(W + 4))
    np.testing.assert_array_equal(dst2.cpu().numpy(), want[pick.astype(np.int64)])


def test_gather_rows_f32_to_nvfp4_wire_rows(lib):
    """The response pack to NVFP4 wire rows (nvfp4_payload.cu:75-115): float32 accumulator rows picked through
    an index list, scale e4m3(amax/6), codes of clamp(x * (1/scale), -6, 6); bytes past the row are not touched."""
    rng = np.random.default_rng(15)
    R, W = 9, 6144
    x = rng.standard_normal((R, W), np.float32) * np.float32(2.0)
    x[1] = 0.0
    x[2] *= np.float32(1e-7)                              # scales that round to zero
    x[3] *= np.float32(1e4)                               # saturating scales
    x[4, :16] = np.array([0.25, -0.25, 0.75, -0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -5.0, 6.0, -6.0, -0.0, 0.0, 3.0, -3.0],
                         np.float32)                      # every tie of the code rule at scale 1
    pick = np.array([8, 4, 4, 0, 1, 2, 3], np.uint32)
    n = len(pick)
    stride = W // 2 + W // 16 + 5
    dst = torch.full((n, stride), 0xAB, dtype=torch.uint8, device="cuda")
    table = torch.from_numpy(x).cuda()
    idx = torch.from_numpy(pick.view(np.int32)).cuda()
    lib.call("glmrt_cuda_gather_rows_f32_to_nvfp4_e2m1_fp8_e4m3_async", ptr(table), ptr(idx), ptr(dst), C.c_size_t(n),
             C.c_size_t(W), C.c_size_t(stride), stream())
    torch.cuda.synchronize()
    codes, sb = O.quantize_rows_nvfp4(x[pick.astype(np.int64)], rule="rne_payload")
    want = O.payload_rows(codes, sb)
    got = dst.cpu().numpy()
    np.testing.assert_array_equal(got[:, :W // 2 + W // 16], want)
    assert (got[:, W // 2 + W // 16:] == 0xAB).all()
    dst2 = torch.zeros((n, W // 2 + W // 16), dtype=torch.uint8, device="cuda")
    lib.call("glmrt_cuda_gather_rows_f32_to_nvfp4_e2m1_fp8_e4m3", ptr(table), ptr(idx), ptr(dst2), C.c_size_t(n), C.c_size_t(W),
             C.c_size_t(W // 2 + W // 16))
    np.testing.assert_array_equal(dst2.cpu().numpy(), want)
    for width, st in ((W + 8, stride), (W, W // 2), (0, stride)):
        assert lib.call_status("glmrt_cuda_gather_rows_f32_to_nvfp4_e2m1_fp8_e4m3_async", ptr(table), ptr(idx), ptr(dst),
                               C.c_size_t(n), C.c_size_t(width), C.c_size_t(st), stream()) == 1


def test_infra_alloc_copy_events(lib, pkg):
    from glmrt_b200 import native as N
    b = N.DeviceBuffer()
    lib.call("glmrt_alloc_device_buffer", C.c_size_t(4096), C.byref(b))
    host = np.arange(1024, dtype=np.int32)
    lib.call("glmrt_copy_h2d", b, C.c_void_p(host.ctypes.data), C.c_size_t(4096))
    back = np.zeros_like(host)
    lib.call("glmrt_copy_d2h", C.c_void_p(back.ctypes.data), b, C.c_size_t(4096))
    np.testing.assert_array_equal(host, back)
    assert lib.call_status("glmrt_copy_h2d", b, C.c_void_p(host.ctypes.data), C.c_size_t(8192)) == 2
    ev0, ev1, ms = C.c_void_p(), C.c_void_p(), C.c_float()
    lib.call("glmrt_cuda_event_create", C.byref(ev0))
    lib.call("glmrt_cuda_event_create", C.byref(ev1))
    lib.call("glmrt_cuda_event_record", ev0, None)
    lib.call("glmrt_cuda_event_record", ev1, None)
    lib.call("glmrt_cuda_event_synchronize", ev1)
    lib.call("glmrt_cuda_event_elapsed_ms", ev0, ev1, C.byref(ms))
    assert ms.value >= 0
    lib.call("glmrt_cuda_event_destroy", ev0)
    lib.call("glmrt_cuda_event_destroy", ev1)
    lib.call("glmrt_free_device_buffer", C.byref(b))
    info = N.DeviceInfo()
    lib.call("glmrt_cuda_device_info", C.c_int(0), C.byref(info))
    assert info.cuda_available == 1 and info.compute_capability_major == 10


def test_nccl_wrappers_single_rank_communicator(lib, pkg):
    """Reference NCCL ABI on a one-rank communicator: unique id, init, bf16 all-reduce and
    reduce-to-root (identity for one rank), destroy."""
    from glmrt_b200 import native as N
    n = C.c_size_t(0)
    st = lib.call_status("glmrt_nccl_unique_id_bytes", C.byref(n))
    if st == 8:
        pytest.skip("libnccl.so.2 not loadable in this process")
    assert st == 0 and n.value == 128
    uid = C.create_string_buffer(128)
    lib.call("glmrt_nccl_get_unique_id", uid, C.c_size_t(128))
    comm = C.c_void_p()
    lib.call("glmrt_nccl_comm_init_rank", uid, C.c_size_t(128), C.c_int(1), C.c_int(0), C.byref(comm))
    x = torch.randn(1000, device="cuda").to(torch.bfloat16)
    y = torch.zeros_like(x)
    z = torch.zeros_like(x)
    s = torch.cuda.Stream()
    torch.cuda.synchronize()
    sp = C.c_void_p(s.cuda_stream)
    lib.call("glmrt_nccl_all_reduce_bf16_async", comm, dbuf(x), dbuf(y), C.c_size_t(1000), sp)
    lib.call("glmrt_nccl_reduce_bf16_async", comm, dbuf(x), dbuf(z), C.c_size_t(1000), C.c_int(0), sp)
    s.synchronize()
    assert torch.equal(x, y) and torch.equal(x, z)
    assert lib.call_status("glmrt_nccl_all_reduce_bf16_async", comm, dbuf(x), dbuf(y), C.c_size_t(1000), None) == 1
    assert lib.call_status("glmrt_nccl_reduce_bf16_async", comm, dbuf(x), dbuf(z), C.c_size_t(1000), C.c_int(3), sp) == 1
    lib.call("glmrt_nccl_comm_destroy", comm)
