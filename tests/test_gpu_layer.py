"""GPU parity tests of the layer path through the C ABI: router -> quantise -> plan/dispatch ->
tcgen05 expert GEMMs -> combine, against the CPU oracle (quantisation-matched mode O1).

Gate (from the project's statement of parity): expert indices exact up to swaps between experts
whose selection scores differ by at most 1e-6, and per-token relative L2 error of the bf16
output at most 2e-2.  The error against the float32-activation reference (mode O0) is printed
for information: it is dominated by the FP4 activation format itself.
"""
import os

import numpy as np
import pytest
import torch

from oracle import glmrt_oracle as O

pytestmark = pytest.mark.gpu

TOL = 2e-2


def to_dev(bits):
    return torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16).cuda()


def to_bits(t):
    return t.cpu().view(torch.int16).numpy().view(np.uint16)


def make(pkg, layer_ref, K, max_tokens, engine="tc", world=1, rank=0):
    from glmrt_b200.layer import MoeLayer
    H, I, E = layer_ref.dims
    layer = MoeLayer(H, I, E, K, max_tokens=max_tokens, engine=engine, ep_world=world, ep_rank=rank)
    layer.load_quantized_layer(layer_ref)
    return layer


def sel64(layer_ref, hid):
    x = O.bf16_to_f32(hid).astype(np.float64)
    return 1.0 / (1.0 + np.exp(-(x @ layer_ref.router_w.astype(np.float64).T))) + layer_ref.bias


@pytest.fixture(scope="module")
def small_layer():
    return O.make_layer(21, 512, 256, 16)


@pytest.mark.parametrize("engine", ["simt", "tc"])
@pytest.mark.parametrize("T", [1, 7, 24, 300])
def test_small_layer_matches_oracle(pkg, small_layer, engine, T):
    K = 4
    layer = make(pkg, small_layer, K, 512, engine)
    hid = O.make_hidden(1000 + T, T, 512)
    out, idx, w = layer.forward(to_dev(hid), want_routes=True)
    layer.check()
    oi, ow, oo = O.layer_forward(small_layer, hid, K, mode="O1")
    assert O.router_indices_equivalent(idx.cpu().numpy(), oi, sel64(small_layer, hid))
    err = O.rel_l2_per_token(to_bits(out), oo)
    assert err.max() <= TOL, f"{engine} T={T}: max per-token rel L2 {err.max():.3e}"
    st = layer.stats()
    assert st.device_error == 0 and st.launches_last_forward >= 6
    layer.close()


def test_tc_intermediate_codes_match_simt_and_oracle(pkg, small_layer):
    """FC1 + SwiGLU + requantisation: the tensor-core engine must write the same FP4 codes and
    scale bytes as the float64-accumulating SIMT engine (identical up to rare ties caused by
    accumulation order) and as the oracle's quantise step."""
    K, T = 4, 40
    hid = O.make_hidden(77, T, 512)
    res = {}
    for engine in ("simt", "tc"):
        layer = make(pkg, small_layer, K, 64, engine)
        out, idx, w = layer.forward(to_dev(hid), want_routes=True)
        layer.check()
        slots = layer.debug("ROUTE_SLOT", np.int32)[: T * K]
        a2 = layer.debug("ACT2_CODES", np.uint8).reshape(-1, 128)
        rr = layer.debug("ROUTE_ROWS", np.uint16)[: T * K * 512].reshape(T * K, 512)
        res[engine] = (to_bits(out), slots.copy(), a2[slots].copy(), rr.copy(), idx.cpu().numpy())
        layer.close()
    np.testing.assert_array_equal(res["simt"][4], res["tc"][4])
    mism = (res["simt"][2] != res["tc"][2]).mean()
    assert mism < 2e-3, f"intermediate code bytes differing between engines: {mism:.2e}"
    err = O.rel_l2_per_token(res["tc"][3], res["simt"][3])
    assert err.max() < 1e-2
    # oracle intermediate for route 0
    x = O.bf16_to_f32(hid)
    c, s = O.quantize_rows_nvfp4(x)
    xq = O.dequantize_payload_rows(O.payload_rows(c, s), 512)
    e0 = int(res["tc"][4][0, 0])
    w0 = small_layer.expert(e0)
    act = O.silu_f32(xq[0:1] @ w0.gate_proj.T) * (xq[0:1] @ w0.up_proj.T)
    codes, _ = O.quantize_rows_nvfp4(act.astype(np.float32))
    got = res["tc"][2][0]
    got_codes = np.stack([got & 0xF, got >> 4], axis=1).reshape(-1)
    assert (got_codes != codes[0]).mean() < 5e-3


def test_outputs_are_bit_reproducible_and_batch_invariant(pkg, small_layer):
    K = 4
    layer = make(pkg, small_layer, K, 64, "tc")
    hid = O.make_hidden(5, 48, 512)
    x = to_dev(hid)
    a = to_bits(layer.forward(x)).copy()
    b = to_bits(layer.forward(x)).copy()
    np.testing.assert_array_equal(a, b)
    # a row computed alone equals the same row inside a batch (M=1 parity of the reference's
    # m1_parity kernels, native/cuda/kernels/b12x_direct.cu:67-99)
    for r in (0, 17, 47):
        single = to_bits(layer.forward(x[r:r + 1].contiguous()))
        np.testing.assert_array_equal(single[0], a[r])
    layer.check()
    layer.close()


def test_forward_routed_and_host_entry_points(pkg, small_layer):
    K, T = 4, 20
    layer = make(pkg, small_layer, K, 64, "tc")
    hid = O.make_hidden(9, T, 512)
    x = to_dev(hid)
    out, idx, w = layer.forward(x, want_routes=True)
    ref = to_bits(out).copy()
    out2 = layer.forward_routed(x, idx, w)
    np.testing.assert_array_equal(to_bits(out2), ref)
    hin = torch.from_numpy(hid.view(np.int16)).view(torch.bfloat16).pin_memory()
    hout = torch.empty_like(hin).pin_memory()
    layer.forward_host(hin, hout)
    np.testing.assert_array_equal(hout.view(torch.int16).numpy().view(np.uint16), ref)
    # caller-supplied routes: skewed, every token to the same experts (one expert gets all rows)
    idx2 = torch.tensor([[3, 5, 7, 9]] * T, dtype=torch.int32, device="cuda")
    w2 = torch.full((T, K), 0.625, dtype=torch.float32, device="cuda")
    out3 = layer.forward_routed(x, idx2, w2)
    layer.check()
    oo = O.moe_forward(hid, lambda e: small_layer.expert(e), idx2.cpu().numpy(), w2.cpu().numpy(), mode="O1")
    assert O.rel_l2_per_token(to_bits(out3), oo).max() <= TOL
    layer.close()


@pytest.mark.parametrize("T", [5, 300])
def test_forward_residual_folds_the_layer_output_into_the_combine(pkg, small_layer, T):
    """out = bf16(residual + bf16(shared + routed)) computed inside the combine kernel equals the
    plain forward followed by the oracle's residual step, bit for bit; without a shared-expert
    row it is bf16(residual + routed).  (The residual fold lives in the ordered combine pass, so
    the plain forward it is compared with uses that pass too, also at T = 300.)"""
    K = 4
    layer = make(pkg, small_layer, K, 512, "tc-ordered")
    hid = O.make_hidden(2300 + T, T, 512)
    rng = np.random.default_rng(T)
    res = O.bf16_round(rng.standard_normal((T, 512), np.float32) * 2)
    shared = O.bf16_round(rng.standard_normal((T, 512), np.float32))
    routed = to_bits(layer.forward(to_dev(hid)))
    layer.check()
    got = to_bits(layer.forward_residual(to_dev(hid), to_dev(res), to_dev(shared)))
    layer.check()
    want = O.residual_add_shared_f32_delta_bf16(res, shared, O.bf16_to_f32(routed))
    np.testing.assert_array_equal(got, want)
    got2 = to_bits(layer.forward_residual(to_dev(hid), to_dev(res)))
    np.testing.assert_array_equal(got2, O.residual_add_bf16(res, routed))
    layer.close()


def test_decode_step_replays_from_a_cuda_graph(pkg, small_layer):
    """The forward only enqueues work on the caller's stream (no allocation, no synchronisation
    after the first call), so a decode step can be captured once and replayed on new inputs, the
    way the reference replays its routed step (native/cuda/kernels/b12x_direct.cu:1101-1256)."""
    K, T = 4, 8
    layer = make(pkg, small_layer, K, 64, "tc")
    x = to_dev(O.make_hidden(1, T, 512)).clone()
    out = torch.empty_like(x)
    layer.forward(x, out=out)                      # first call sets kernel attributes and tensor maps
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        layer.forward(x, out=out)
    for seed in (2, 3):
        hid = O.make_hidden(seed, T, 512)
        x.copy_(to_dev(hid))
        graph.replay()
        torch.cuda.synchronize()
        replayed = to_bits(out).copy()
        eager = to_bits(layer.forward(to_dev(hid)))
        np.testing.assert_array_equal(replayed, eager)
    layer.check()
    layer.close()


def test_full_size_prefill_is_row_permutation_equivariant(pkg):
    """At the full prefill size (GLM-5.2 layer, T = 8192) a property that needs no reference
    values: a token's result depends on its own row only, so with the ordered combine permuting
    the rows of the batch permutes the rows of the output bit for bit, and 64 of the rows run
    alone (decode kernels) agree with their rows in the large batch within the gate.  The default
    form (the down projection adds into the output rows as routes finish) sums the same products
    in a different order: it must agree with the ordered form within bf16 accumulation noise."""
    from glmrt_b200.layer import MoeLayer
    H, I, E, K, T = 6144, 2048, 256, 8, 8192
    layer = MoeLayer(H, I, E, K, max_tokens=T, engine="tc-ordered")
    layer.fill_synthetic(11, 0.02)
    g = torch.Generator(device="cpu").manual_seed(5)
    layer.set_router((torch.randn(E, H, generator=g) * 0.02), torch.zeros(E))
    x = (torch.randn(T, H, generator=g)).to(torch.bfloat16).cuda()
    perm = torch.randperm(T, generator=g).cuda()
    out = layer.forward(x).clone()
    out_p = layer.forward(x[perm].contiguous())
    layer.check()
    assert torch.equal(out_p.view(torch.int16), out[perm].view(torch.int16))
    assert torch.isfinite(out.float()).all() and out.float().abs().max() > 0
    rows = torch.arange(0, T, T // 64, device="cuda")[:64]
    small = layer.forward(x[rows].contiguous())
    layer.check()
    err = O.rel_l2_per_token(to_bits(small), to_bits(out[rows]))
    print(f"T=8192 rows vs the same rows alone: max per-token rel L2 {err.max():.3e}")
    assert err.max() <= 1e-2
    fused = layer.create_lane()
    fused_flags = fused.cfg.flags
    fused.close()
    assert fused_flags != 0      # lanes inherit the flags of their layer
    layer.close()
    del layer
    torch.cuda.empty_cache()
    layer = MoeLayer(H, I, E, K, max_tokens=T)          # default: fused combine above 256 rows
    layer.fill_synthetic(11, 0.02)
    g = torch.Generator(device="cpu").manual_seed(5)
    layer.set_router((torch.randn(E, H, generator=g) * 0.02), torch.zeros(E))
    out_f = layer.forward(x)
    layer.check()
    err = O.rel_l2_per_token(to_bits(out_f), to_bits(out))
    print(f"T=8192 fused combine vs ordered combine: max per-token rel L2 {err.max():.3e}")
    assert err.max() <= 1e-2
    assert layer.stats().launches_last_forward == 8      # no combine pass
    layer.close()


def test_sparse_layer_output_with_shared_expert(pkg, small_layer):
    """hidden + routed + shared (python/reference/glmrt_reference/glm_moe_dsa_layer_ref.py:190-198):
    the shared expert is one more NVFP4 expert that every row selects with weight 1; it runs through
    a second layer object (one expert, top-1, caller-supplied routes) and its rows enter the routed
    layer's combine as the shared delta.  Checked against the oracle's composition of the same
    pieces, within the gate of the layer (the residual step itself is exact, tested separately)."""
    from glmrt_b200.layer import MoeLayer
    K, T, H, I = 4, 40, 512, 256
    shared_ref = O.make_layer(77, H, I, 1)
    routed = make(pkg, small_layer, K, 64, "tc")
    shared = MoeLayer(H, I, 1, 1, max_tokens=64)
    shared.load_quantized_layer(shared_ref)
    hid = O.make_hidden(900, T, H)                # the normalised rows (input of router and experts)
    resid = O.bf16_round(np.random.default_rng(3).standard_normal((T, H), np.float32))   # the layer input
    x = to_dev(hid)
    ones = torch.ones((T, 1), dtype=torch.float32, device="cuda")
    zeros = torch.zeros((T, 1), dtype=torch.int32, device="cuda")
    shared_rows = shared.forward_routed(x, zeros, ones)
    shared.check()
    got = to_bits(routed.forward_residual(x, to_dev(resid), shared_rows))
    routed.check()
    # oracle: routed (O1) and shared (O1, weight 1) outputs, then the native residual formula
    _, _, routed_o = O.layer_forward(small_layer, hid, K, mode="O1")
    shared_o = O.moe_forward(hid, lambda e: shared_ref.expert(e), np.zeros((T, 1), np.int64), np.ones((T, 1), np.float32), mode="O1")
    want = O.residual_add_shared_f32_delta_bf16(resid, shared_o, O.bf16_to_f32(routed_o))
    delta_got = O.bf16_to_f32(got) - O.bf16_to_f32(resid)
    delta_want = O.bf16_to_f32(want) - O.bf16_to_f32(resid)
    err = np.linalg.norm(delta_got - delta_want, axis=1) / np.maximum(np.linalg.norm(delta_want, axis=1), 1e-30)
    print(f"layer output with shared expert: max per-token rel L2 of the MLP delta {err.max():.3e}")
    assert err.max() <= 3e-2       # two bf16 truncations of a value of order 1 on top of the 2e-2 gate
    routed.close()
    shared.close()


@pytest.mark.parametrize("T", [200, 256])
def test_decode_kernels_with_many_rows_per_expert(pkg, small_layer, T):
    """Batches of at most 256 rows run the decode kernels (32-slot work items).  With 16 experts
    every expert receives well over 32 rows here, so each has several work items; and with
    caller-supplied routes one expert receives every row of the batch (8 work items at T=256)."""
    K = 4
    layer = make(pkg, small_layer, K, 256, "tc")
    hid = O.make_hidden(6100 + T, T, 512)
    out, idx, w = layer.forward(to_dev(hid), want_routes=True)
    layer.check()
    oi, ow, oo = O.layer_forward(small_layer, hid, K, mode="O1")
    gi = idx.cpu().numpy()
    assert O.router_indices_equivalent(gi, oi, sel64(small_layer, hid))
    counts = np.bincount(gi.reshape(-1), minlength=16)
    assert counts.max() > 32
    chunks = layer.debug("CHUNKS", np.int32).reshape(-1, 4)
    n_chunks = int(layer.debug("COUNTERS", np.uint32)[0])
    assert n_chunks > 16 and chunks[:n_chunks, 2].max() <= 32 and (chunks[:n_chunks, 1] % 128 == 0).all()
    same = np.all(gi == oi.astype(np.int32), axis=1)
    err = O.rel_l2_per_token(to_bits(out)[same], oo[same])
    assert err.max() <= TOL, f"T={T}: max per-token rel L2 {err.max():.3e}"
    # every row to expert 3 (and three other fixed experts), weights from the router
    fixed = np.tile(np.array([[3, 0, 9, 14]], np.int32), (T, 1))
    wts = w.cpu().numpy()
    got = to_bits(layer.forward_routed(to_dev(hid), torch.from_numpy(fixed).cuda(), torch.from_numpy(wts).cuda()))
    layer.check()
    want = O.moe_forward(hid, lambda e: small_layer.expert(e), fixed.astype(np.int64), wts, mode="O1")
    err2 = O.rel_l2_per_token(got, want)
    assert err2.max() <= TOL, f"T={T} fixed routes: max per-token rel L2 {err2.max():.3e}"
    layer.close()


def test_forward_argument_edges(pkg, small_layer):
    """Empty and oversized batches, buffers that are too small or misaligned are refused before
    any launch (the reference's ABI rule: validate, then launch; native/include/glmrt_native.h:
    77-82); a batch of exactly max_tokens rows and a single row both run."""
    import ctypes as C
    from glmrt_b200 import native as N
    K, H = 4, 512
    layer = make(pkg, small_layer, K, 40, "tc")
    full = to_dev(O.make_hidden(1, 40, H))
    out = layer.forward(full)
    layer.check()
    assert torch.isfinite(out.float()).all()
    one = layer.forward(full[:1].contiguous())
    assert torch.equal(one[0].view(torch.int16), out[0].view(torch.int16))     # batch invariance at the edges
    none = N.DeviceBuffer.null()
    buf = lambda t, nbytes=None: N.DeviceBuffer.of(t.data_ptr(), t.numel() * t.element_size() if nbytes is None else nbytes)
    big = to_dev(O.make_hidden(2, 41, H))
    o41 = torch.empty_like(big)
    st = lambda rows, x, o: layer.lib.call_status("glmrt_b200_moe_layer_forward_async", layer.handle, x, C.c_size_t(rows), o,
                                                  none, none, None)
    assert st(0, buf(full), buf(out)) == 1                                    # empty
    assert st(41, buf(big), buf(o41)) == 1                                    # more than max_tokens
    assert "max_tokens" in layer.lib.last_error()
    assert st(40, buf(full, 40 * H * 2 - 2), buf(out)) == 2                   # hidden buffer too small
    assert st(40, buf(full), buf(out, 16)) == 2                               # output buffer too small
    odd = N.DeviceBuffer.of(full.data_ptr() + 2, 39 * H * 2)
    assert st(39, odd, buf(out)) == 1                                         # not 16-byte aligned
    assert st(40, none, buf(out)) in (1, 2)
    layer.check()                                                             # nothing ran, nothing broke
    again = layer.forward(full)
    assert torch.equal(again.view(torch.int16), out.view(torch.int16))
    layer.close()


def test_bad_routes_are_reported_not_faulted(pkg, small_layer):
    from glmrt_b200.native import GlmrtError
    K, T = 4, 4
    layer = make(pkg, small_layer, K, 64, "tc")
    x = to_dev(O.make_hidden(3, T, 512))
    idx = torch.tensor([[0, 1, 2, 99]] * T, dtype=torch.int32, device="cuda")   # expert 99 does not exist
    w = torch.ones((T, K), dtype=torch.float32, device="cuda")
    layer.forward_routed(x, idx, w)
    with pytest.raises(GlmrtError) as ei:
        layer.check()
    assert "expert id" in str(ei.value)
    # the layer stays usable
    out = layer.forward(x)
    layer.check()
    assert torch.isfinite(out.float()).all()
    layer.close()


def test_expert_parallel_shards_sum_to_the_full_layer(pkg, small_layer):
    """Each shard computes only routes whose expert it owns (e % world == rank,
    rust/crates/glmrt-core/src/placement.rs:25-42); partials match the oracle's
    partitioned forward (python/reference/glmrt_reference/moe_ref.py:40-66)."""
    K, T, world = 4, 24, 2
    hid = O.make_hidden(31, T, 512)
    x = to_dev(hid)
    oi, ow, _ = O.layer_forward(small_layer, hid, K, mode="O1")
    idx = torch.from_numpy(oi.astype(np.int32)).cuda()
    w = torch.from_numpy(ow).cuda()
    for rank in range(world):
        layer = make(pkg, small_layer, K, 64, "tc", world, rank)
        part = layer.forward_routed(x, idx, w)
        layer.check()
        _, _, op = O.layer_forward(small_layer, hid, K, mode="O1", world=world, rank=rank)
        err = O.rel_l2_per_token(to_bits(part), op)
        assert err.max() <= TOL
        layer.close()


def test_glm52_shape_layer_t16_matches_oracle(pkg):
    """The benchmark's reference configuration: 16 tokens, hidden 6144, 256 experts, top-8,
    intermediate 2048.  Weights are generated and quantised on the device (seeded), the experts
    that the batch touches are read back and handed to the CPU oracle."""
    from glmrt_b200.layer import MoeLayer
    H, I, E, K, T = 6144, 2048, 256, 8, 16
    layer = MoeLayer(H, I, E, K, max_tokens=64)
    layer.fill_synthetic(0, 0.02)
    rng = np.random.default_rng(0)
    rw = (rng.standard_normal((E, H), np.float32) * np.float32(0.02)).astype(np.float32)
    bias = (rng.standard_normal(E, np.float32) * np.float32(0.01)).astype(np.float32)
    layer.set_router(torch.from_numpy(rw), torch.from_numpy(bias))
    hid = O.make_hidden(1000, T, H)
    out, idx, w = layer.forward(to_dev(hid), want_routes=True)
    layer.check()
    oi, ow, _, _ = O.router_topk(O.bf16_to_f32(hid), rw, bias, K)
    x64 = O.bf16_to_f32(hid).astype(np.float64)
    s64 = 1.0 / (1.0 + np.exp(-(x64 @ rw.astype(np.float64).T))) + bias
    gi = idx.cpu().numpy()
    assert O.router_indices_equivalent(gi, oi, s64)
    cache = {}

    def getw(e):
        if e not in cache:
            (gc, gs, g2), (uc, us, u2), (dc, ds, d2) = layer.read_expert(e)
            cache.clear()  # one expert at a time keeps host memory flat
            cache[e] = O.ExpertWeights(O.dequantize_weight(gc, gs, g2), O.dequantize_weight(uc, us, u2),
                                       O.dequantize_weight(dc, ds, d2))
        return cache[e]

    oo = O.moe_forward(hid, getw, gi, w.cpu().numpy(), mode="O1")
    err = O.rel_l2_per_token(to_bits(out), oo)
    print(f"glm52 T=16: max per-token rel L2 vs O1 = {err.max():.3e}")
    assert err.max() <= TOL
    st = layer.stats()
    assert st.distinct_experts == len(np.unique(gi))
    layer.close()


@pytest.mark.parametrize("T", [64, 1024])
def test_glm52_shape_tc_matches_simt_at_bench_sizes(pkg, T):
    """At sizes beyond the CPU oracle's reach the tensor-core engine is checked against the
    float64-accumulating SIMT engine on identical device-generated weights and inputs."""
    from glmrt_b200.layer import MoeLayer
    H, I, E, K = 6144, 2048, 256, 8
    hid = O.make_hidden(50 + T, T, H)
    x = to_dev(hid)
    rng = np.random.default_rng(1)
    rw = (rng.standard_normal((E, H), np.float32) * np.float32(0.02)).astype(np.float32)
    bias = np.zeros(E, np.float32)
    outs = {}
    for engine in ("tc", "simt"):
        layer = MoeLayer(H, I, E, K, max_tokens=T, engine=engine)
        layer.fill_synthetic(7, 0.02)
        layer.set_router(torch.from_numpy(rw), torch.from_numpy(bias))
        out, idx, w = layer.forward(x, want_routes=True)
        layer.check()
        outs[engine] = (to_bits(out).copy(), idx.cpu().numpy().copy())
        layer.close()
        del layer
        torch.cuda.empty_cache()
    np.testing.assert_array_equal(outs["tc"][1], outs["simt"][1])
    err = O.rel_l2_per_token(outs["tc"][0], outs["simt"][0])
    print(f"glm52 T={T}: tc vs simt max per-token rel L2 = {err.max():.3e}")
    assert err.max() <= 1e-2


@pytest.mark.parametrize("T", [900, 1536])
def test_pair_tiles_match_oracle_and_one_cta_tiles(pkg, small_layer, T):
    """On request, above 192 routes per expert FC1 runs on CTA pairs over 256-slot work items (and
    FC2 takes each item as two halves).  The result must meet the oracle gate and agree with the
    one-CTA kernels on the same inputs; T=900 leaves many second halves empty."""
    K = 4
    hid = O.make_hidden(4200 + T, T, 512)
    oi, ow, oo = O.layer_forward(small_layer, hid, K, mode="O1")
    outs = {}
    for engine in ("tc2", "tc2-fc1", "tc2-fc2", "tc"):
        # the pair kernels write one row per route; the one-CTA reference here does the same
        layer = make(pkg, small_layer, K, 2048, "tc-ordered" if engine == "tc" else engine)
        out, idx, w = layer.forward(to_dev(hid), want_routes=True)
        layer.check()
        chunks = layer.debug("CHUNKS", np.int32).reshape(-1, 4)
        n_chunks = int(layer.debug("COUNTERS", np.uint32)[0])
        width = int(chunks[:n_chunks, 2].max())
        assert (width > 128) == engine.startswith("tc2"), f"{engine}: widest work item {width}"
        assert O.router_indices_equivalent(idx.cpu().numpy(), oi, sel64(small_layer, hid))
        err = O.rel_l2_per_token(to_bits(out), oo)
        assert err.max() <= TOL, f"{engine} T={T}: max per-token rel L2 {err.max():.3e}"
        outs[engine] = to_bits(out).copy()
        layer.close()
    for engine in ("tc2", "tc2-fc1", "tc2-fc2"):
        diff = O.rel_l2_per_token(outs[engine], outs["tc"])
        print(f"{engine} vs one-CTA tiles T={T}: max per-token rel L2 {diff.max():.3e}, "
              f"{(outs[engine] != outs['tc']).mean():.2e} of bf16 words differ")
        assert diff.max() <= 1e-3


@pytest.mark.parametrize("T", [16, 300, 1000])
def test_zipf_skewed_routing_matches_oracle(pkg, T):
    """Load-skewed routing: a router bias makes expert popularity follow rank^-1.2, so a few experts
    receive most rows (several token chunks each, some none).  T=16 is the speculative-verify
    batch 4 x (1 + 3 drafts); the larger sizes take the 128-token chunk kernels."""
    H, I, E, K = 512, 256, 16, 4
    ref = O.make_layer(33, H, I, E)
    # bias in logit space of the selection score: popular experts get a head start
    pop = (np.arange(1, E + 1, dtype=np.float64) ** -1.2)
    ref.bias = (0.35 * np.log(pop / pop.max())).astype(np.float32) * np.float32(0.25)
    layer = make(pkg, ref, K, 1024, "tc")
    hid = O.make_hidden(7000 + T, T, H)
    out, idx, w = layer.forward(to_dev(hid), want_routes=True)
    layer.check()
    oi, ow, oo = O.layer_forward(ref, hid, K, mode="O1")
    gi = idx.cpu().numpy()
    assert O.router_indices_equivalent(gi, oi, sel64(ref, hid))
    counts = np.bincount(gi.reshape(-1), minlength=E)
    assert counts.max() >= 2.5 * max(1, counts.min())          # the routing really is skewed
    same = np.all(gi == oi.astype(np.int32), axis=1)
    err = O.rel_l2_per_token(to_bits(out)[same], oo[same])
    assert err.max() <= TOL
    ec = layer.debug("EXPERT_COUNTS", np.int32)[:E]
    np.testing.assert_array_equal(ec, counts)
    layer.close()


@pytest.mark.parametrize("T", [129, 1024, 4100])
def test_tensor_core_router_matches_oracle_at_prefill_sizes(pkg, T):
    """Above 128 rows the logits come from the bf16 x (hi|mid|lo) tensor-core GEMM; indices must
    agree with the float32 oracle up to 1e-6 near-ties, weights to float32 round-off."""
    from glmrt_b200.layer import MoeLayer
    H, I, E, K = 6144, 256, 256, 8
    rng = np.random.default_rng(T)
    rw = (rng.standard_normal((E, H), np.float32) * np.float32(0.02)).astype(np.float32)
    bias = (rng.standard_normal(E, np.float32) * np.float32(0.01)).astype(np.float32)
    layer = MoeLayer(H, I, E, K, max_tokens=T)
    layer.fill_synthetic(3, 0.02)
    layer.set_router(torch.from_numpy(rw), torch.from_numpy(bias))
    hid = O.make_hidden(T, T, H)
    out, idx, w = layer.forward(to_dev(hid), want_routes=True)
    layer.check()
    oi, ow, _, _ = O.router_topk(O.bf16_to_f32(hid), rw, bias, K)
    x64 = O.bf16_to_f32(hid).astype(np.float64)
    s64 = 1.0 / (1.0 + np.exp(-(x64 @ rw.astype(np.float64).T))) + bias
    gi = idx.cpu().numpy()
    assert O.router_indices_equivalent(gi, oi, s64, tol=1e-6)
    same = np.all(gi == oi.astype(np.int32), axis=1)
    assert same.mean() > 0.98
    np.testing.assert_allclose(w.cpu().numpy()[same], ow[same], atol=3e-6, rtol=1e-5)
    assert torch.isfinite(out.float()).all()
    layer.close()


def test_layer_loaded_from_a_checkpoint_matches_the_direct_load(pkg, small_layer, tmp_path):
    """Sharded safetensors in the checkpoint's layout -> load_moe_layer: the resident weights read back
    as written and a forward is bit-equal to the same layer set through load_quantized_layer."""
    import copy
    from glmrt_b200 import checkpoint as CK
    from glmrt_b200.layer import MoeLayer
    from tests.checkpoint_fixture import write_snapshot
    H, I, E = small_layer.dims
    K, T = 4, 40
    stored_router = write_snapshot(str(tmp_path / "snap"), small_layer, layer_id=7, shards=3)
    cat = CK.TensorCatalog(str(tmp_path / "snap"))
    layer = MoeLayer(H, I, E, K, max_tokens=64)
    report = CK.load_moe_layer(layer, cat, 7)
    assert report.experts_loaded == list(range(E)) and report.weight_bytes == E * 3 * (H * I // 2 + H * I // 16 + 8)
    for e in (0, E - 1):
        (gc, gs, g2), (uc, us, u2), (dc, ds, d2) = layer.read_expert(e)
        np.testing.assert_array_equal(gc, small_layer.gate[e])
        np.testing.assert_array_equal(us, small_layer.up_s[e])
        np.testing.assert_array_equal(dc, small_layer.down[e])
        assert (g2, u2, d2) == tuple(float(v) for v in small_layer.scale2[e])
    ref = copy.copy(small_layer)
    ref.router_w = stored_router                       # the checkpoint holds the router weight as bf16
    direct = make(pkg, ref, K, 64)
    hid = to_dev(O.make_hidden(4242, T, H))
    out_a, idx_a, w_a = layer.forward(hid, want_routes=True)
    out_b, idx_b, w_b = direct.forward(hid, want_routes=True)
    layer.check(); direct.check()
    assert torch.equal(idx_a, idx_b) and torch.equal(w_a, w_b) and torch.equal(out_a, out_b)
    # a rank of a two-way expert-parallel layer takes only its own experts
    shard = MoeLayer(H, I, E, K, max_tokens=64, ep_world=2, ep_rank=1)
    assert CK.load_moe_layer(shard, cat, 7).experts_loaded == list(range(1, E, 2))
    for l in (layer, direct, shard):
        l.close()


# ---------------------------------------------------------------------------------------------
# Headline shapes against the CPU oracle: a row's arithmetic is independent of the other rows of
# its batch (mode O1), so a few rows of a large batch can be checked on the CPU by dequantising
# only the experts those rows selected.
# ---------------------------------------------------------------------------------------------
def oracle_rows_error(layer, hid_bits, idx, w, out_bits, rows):
    """Max per-token relative L2 error of `rows` of a forward pass against O.moe_forward (O1) on the
    same rows, with the weights of the selected experts read back from the device one at a time."""
    cache = {}

    def getw(e):
        if e not in cache:
            (gc, gs, g2), (uc, us, u2), (dc, ds, d2) = layer.read_expert(e)
            cache.clear()  # one expert at a time keeps host memory flat
            cache[e] = O.ExpertWeights(O.dequantize_weight(gc, gs, g2), O.dequantize_weight(uc, us, u2),
                                       O.dequantize_weight(dc, ds, d2))
        return cache[e]

    rows = np.asarray(rows)
    oo = O.moe_forward(hid_bits[rows], getw, idx[rows], w[rows], mode="O1")
    return O.rel_l2_per_token(out_bits[rows], oo)


def glm_layer(seed, T, bias=None, K=8):
    from glmrt_b200.layer import MoeLayer
    H, I, E = 6144, 2048, 256
    layer = MoeLayer(H, I, E, K, max_tokens=T)
    layer.fill_synthetic(seed, 0.02)
    rng = np.random.default_rng(seed)
    rw = (rng.standard_normal((E, H), np.float32) * np.float32(0.02)).astype(np.float32)
    b = np.zeros(E, np.float32) if bias is None else bias.astype(np.float32)
    layer.set_router(torch.from_numpy(rw), torch.from_numpy(b))
    return layer, rw, b


@pytest.mark.parametrize("T,n_rows", [(64, 8), (8192, 8)])
def test_glm52_shape_headline_sizes_match_oracle_on_sampled_rows(pkg, T, n_rows):
    """The two sizes the throughput figures are quoted on (decode T = 64, prefill T = 8192), GLM-5.2
    layer shape, uniform router: router indices of every row against the oracle, and the output
    of sampled rows against O.moe_forward within the layer gate."""
    layer, rw, bias = glm_layer(3, T)
    hid = O.make_hidden(9000 + T, T, 6144)
    out, idx, w = layer.forward(to_dev(hid), want_routes=True)
    layer.check()
    gi, gw, ob = idx.cpu().numpy(), w.cpu().numpy(), to_bits(out)
    x64 = O.bf16_to_f32(hid).astype(np.float64)
    s64 = 1.0 / (1.0 + np.exp(-(x64 @ rw.astype(np.float64).T))) + bias
    oi, ow, _, _ = O.router_topk(O.bf16_to_f32(hid), rw, bias, 8)
    assert O.router_indices_equivalent(gi, oi, s64)
    rows = np.linspace(0, T - 1, n_rows).astype(np.int64)
    np.testing.assert_allclose(gw[rows], ow[rows], rtol=2e-5, atol=1e-6)
    err = oracle_rows_error(layer, hid, gi, gw, ob, rows)
    print(f"glm52 T={T}: {n_rows} sampled rows vs O1: max per-token rel L2 = {err.max():.3e}")
    assert err.max() <= TOL
    layer.close()


@pytest.mark.parametrize("T", [16, 2048])
def test_glm52_shape_zipf_routing_matches_oracle_on_sampled_rows(pkg, T):
    """Load-skewed routing at the GLM-5.2 layer shape (popularity ~ rank^-1.2): T = 16 is the
    speculative-verify batch 4 x (1 + 3 drafts) on the decode kernels, T = 2048 puts many token
    chunks on the hot experts and none on the cold ones."""
    rng = np.random.default_rng(17)
    rw = (rng.standard_normal((256, 6144), np.float32) * np.float32(0.02)).astype(np.float32)
    hid = O.make_hidden(9100 + T, T, 6144)
    import bench   # the benchmark's calibration of the skewed router (repository root is on sys.path)
    bias = bench.zipf_bias(rw, O.bf16_to_f32(O.make_hidden(9101, 1024, 6144)), 1.2)
    from glmrt_b200.layer import MoeLayer
    layer = MoeLayer(6144, 2048, 256, 8, max_tokens=T)
    layer.fill_synthetic(5, 0.02)
    layer.set_router(torch.from_numpy(rw), torch.from_numpy(bias))
    out, idx, w = layer.forward(to_dev(hid), want_routes=True)
    layer.check()
    gi, gw, ob = idx.cpu().numpy(), w.cpu().numpy(), to_bits(out)
    x64 = O.bf16_to_f32(hid).astype(np.float64)
    s64 = 1.0 / (1.0 + np.exp(-(x64 @ rw.astype(np.float64).T))) + bias
    oi, _, _, _ = O.router_topk(O.bf16_to_f32(hid), rw, bias, 8)
    assert O.router_indices_equivalent(gi, oi, s64)
    counts = np.bincount(gi.reshape(-1), minlength=256)
    assert counts[:8].sum() > 4 * counts[-64:].sum()          # the routing really is skewed
    np.testing.assert_array_equal(layer.debug("EXPERT_COUNTS", np.int32)[:256], counts)
    rows = np.linspace(0, T - 1, 6).astype(np.int64)
    err = oracle_rows_error(layer, hid, gi, gw, ob, rows)
    print(f"glm52 zipf T={T}: max per-token rel L2 = {err.max():.3e}, hottest expert {counts.max()} of {T * 8} routes")
    assert err.max() <= TOL
    layer.close()


def test_router_choice_of_a_row_across_batch_size_classes(pkg):
    """The logits of a row come from the SIMT kernel up to 128 rows and from the tensor-core kernel
    above: the two sum in different orders, so a row's selection may differ between the classes
    only where two experts' selection scores are within 1e-6 of each other."""
    layer, rw, bias = glm_layer(4, 512)
    hid = O.make_hidden(9200, 512, 6144)
    x = to_dev(hid)
    _, idx_big, w_big = layer.forward(x, want_routes=True)
    _, idx_small, w_small = layer.forward(x[:96].contiguous(), want_routes=True)
    layer.check()
    x64 = O.bf16_to_f32(hid[:96]).astype(np.float64)
    s64 = 1.0 / (1.0 + np.exp(-(x64 @ rw.astype(np.float64).T))) + bias
    assert O.router_indices_equivalent(idx_small.cpu().numpy(), idx_big[:96].cpu().numpy().astype(np.int64), s64)
    same = (idx_small.cpu().numpy() == idx_big[:96].cpu().numpy()).all(axis=1)
    np.testing.assert_allclose(w_small.cpu().numpy()[same], w_big[:96].cpu().numpy()[same], rtol=2e-5, atol=1e-6)
    layer.close()


# ---------------------------------------------------------------------------------------------
# Lanes (shared weights, own workspace) and stacked layers (own weights, shared workspace)
# ---------------------------------------------------------------------------------------------
def test_two_lanes_on_two_streams_match_serial_execution(pkg, small_layer):
    """Two lanes of one layer run at the same time on two streams; each must give exactly what
    the layer gives when it runs the same batch alone (the reference executor's lanes share the
    resident experts and keep per-lane route tensors)."""
    K = 4
    layer = make(pkg, small_layer, K, 512, "tc-ordered")   # bit-equality below needs the ordered combine at T = 300
    lanes = [layer.create_lane(), layer.create_lane()]
    xs = [to_dev(O.make_hidden(600 + i, T, 512)) for i, T in enumerate((300, 40))]
    refs = [to_bits(layer.forward(x)).copy() for x in xs]
    layer.check()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    outs = [torch.zeros_like(x) for x in xs]
    torch.cuda.synchronize()
    for rep in range(3):
        for lane, st, x, o in zip(lanes, streams, xs, outs):
            with torch.cuda.stream(st):
                lane.forward(x, o)
    for st in streams:
        st.synchronize()
    for lane, st in zip(lanes, streams):
        with torch.cuda.stream(st):
            lane.check()
    for o, r in zip(outs, refs):
        np.testing.assert_array_equal(to_bits(o), r)
    # the weights outlive the handle that created them
    layer.close()
    again = to_bits(lanes[0].forward(xs[0]))
    lanes[0].check()
    np.testing.assert_array_equal(again, refs[0])
    for lane in lanes:
        lane.close()


def test_stacked_layers_share_one_workspace(pkg):
    """Three layers with different weights on one workspace, chained output -> input like the
    sparse layers of a model: same result as three independent layers."""
    K, H, I, E, T = 4, 512, 256, 16, 48
    refs = [O.make_layer(40 + i, H, I, E) for i in range(3)]
    x0 = to_dev(O.make_hidden(77, T, H))
    # independent layers
    y = x0
    for ref in refs:
        l = make(pkg, ref, K, 64)
        y = l.forward(y).clone()
        l.check()
        l.close()
    expect = to_bits(y)
    # one workspace
    base = make(pkg, refs[0], K, 64)
    stack = [base]
    for ref in refs[1:]:
        l = base.create_stacked()
        l.load_quantized_layer(ref)
        stack.append(l)
    y = x0
    for l in stack:
        y = l.forward(y).clone()
    for l in stack:
        l.check()
    np.testing.assert_array_equal(to_bits(y), expect)
    for l in reversed(stack):
        l.close()


def test_dense_shared_expert_beside_the_routed_path(pkg, small_layer):
    """hidden + routed + shared with the reference's DENSE shared expert (expert_forward in float32
    on unquantised weights, glm_moe_dsa_layer_ref.py:157-206): the shared rows against the
    oracle's float32 expert_forward, and the whole layer output against the oracle's composition
    (routed part in mode O1, residual step exact)."""
    from glmrt_b200.shared_expert import DenseSharedExpert, sparse_layer_forward
    K, T, H, I = 4, 40, 512, 256
    rng = np.random.default_rng(88)
    wg, wu = (O.bf16_to_f32(O.bf16_round(rng.standard_normal((I, H), np.float32) * np.float32(0.05))) for _ in range(2))
    wd = O.bf16_to_f32(O.bf16_round(rng.standard_normal((H, I), np.float32) * np.float32(0.05)))
    hid = O.make_hidden(901, T, H)
    resid = O.bf16_round(rng.standard_normal((T, H), np.float32))
    shared = DenseSharedExpert(torch.from_numpy(wg), torch.from_numpy(wu), torch.from_numpy(wd))
    delta = to_bits(shared.delta(to_dev(hid)))
    want_delta = O.bf16_round(O.expert_forward(O.bf16_to_f32(hid), O.ExpertWeights(wg, wu, wd)))
    err = O.rel_l2_per_token(delta, want_delta)
    assert err.max() <= 2e-3, f"dense shared expert vs float32 expert_forward: {err.max():.3e}"
    routed = make(pkg, small_layer, K, 64, "tc")
    got = to_bits(sparse_layer_forward(routed, shared, to_dev(resid), to_dev(hid)))
    routed.check()
    _, _, routed_ref = O.layer_forward(small_layer, hid, K, mode="O1")
    want = O.residual_add_shared_f32_delta_bf16(resid, want_delta, O.bf16_to_f32(routed_ref))
    assert O.rel_l2_per_token(got, want).max() <= TOL
    # the fold itself is exact: same routed rows and the same delta give the same bits
    routed_rows = to_bits(routed.forward(to_dev(hid)))
    np.testing.assert_array_equal(got, O.residual_add_shared_f32_delta_bf16(resid, delta, O.bf16_to_f32(routed_rows)))
    routed.close()
