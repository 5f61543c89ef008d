"""Generate the golden vectors of tests/golden/ by running the REFERENCE's own Python.

Run once in a container that has the reference checkout:

    python tests/golden/generate_golden.py /path/to/reference

It imports ``python/reference/glmrt_reference`` (torch CPU) from that checkout,
feeds it seeded inputs drawn with numpy (so the consumers can re-draw the same
inputs without the reference), and stores the reference's outputs as small
``.npz`` files.  The tests that read these files never need the reference.
"""
from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import glmrt_oracle as O  # noqa: E402  (input generators only)


def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "python", "reference"))
    import torch
    from glmrt_reference import quant_ref as Q
    from glmrt_reference.glm_moe_dsa_layer_ref import GlmMoeDsaConfig, glm_router_topk
    from glmrt_reference.moe_ref import ExpertWeights, moe_forward, partitioned_moe_forward
    from glmrt_reference.rmsnorm_ref import rmsnorm

    torch.set_num_threads(max(1, os.cpu_count() or 1))

    # ---- formats -----------------------------------------------------------
    e4m3_table = np.array([Q.f8e4m3_byte_to_float(b) for b in range(256)], np.float32)
    rng = np.random.default_rng(1234)
    vals = (rng.standard_normal(20000).astype(np.float32) * 2.5)
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 7.0, 0.0, -0.0], np.float32)
    vals = np.concatenate([vals, ties, -ties, ties * np.float32(0.375), -ties * np.float32(0.375)])
    scales = np.array([1.0, 0.375, 0.0625, 3.5], np.float32)
    q_codes = {}
    for s in scales:
        c = Q.nvfp4_quantize(torch.from_numpy(vals), float(s)).numpy()
        q_codes[f"codes_scale_{s}"] = c
        q_codes[f"deq_scale_{s}"] = Q.nvfp4_dequantize(torch.from_numpy(c), float(s)).numpy()
    packed = Q.pack_nibbles(torch.from_numpy(q_codes["codes_scale_1.0"][:4097])).numpy()
    unpacked = Q.unpack_nibbles(torch.from_numpy(packed), 4097).numpy()
    sb = rng.integers(0, 0x7F, size=(4096 + 15) // 16).astype(np.uint8)
    decoded = np.array(Q.decode_packed_nvfp4_values(bytes(packed[:2048]), bytes(sb), 0.01171875, 4096), np.float32)
    # torch float8 cast as an independent E4M3 RNE encoder (values clamped to 448 first)
    enc_in = np.concatenate([np.abs(vals) * np.float32(40.0), e4m3_table[:0x7F],
                             ((e4m3_table[:0x7E] + e4m3_table[1:0x7F]) / 2).astype(np.float32)])
    enc_out = torch.from_numpy(np.minimum(enc_in, np.float32(448.0))).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    np.savez_compressed(os.path.join(HERE, "formats.npz"), e4m3_table=e4m3_table, values=vals,
                        scales=scales, packed=packed, unpacked=unpacked, decode_scale_bytes=sb,
                        decoded=decoded, e4m3_enc_in=enc_in, e4m3_enc_out=enc_out, **q_codes)

    # ---- router ------------------------------------------------------------
    router = {}
    for name, (seed, T, H, E, K) in {"small": (11, 33, 256, 16, 4),
                                     "glm52": (0, 16, 6144, 256, 8)}.items():
        r = np.random.default_rng(seed)
        rw = (r.standard_normal((E, H), np.float32) * np.float32(0.02)).astype(np.float32)
        bias = (r.standard_normal(E, np.float32) * np.float32(0.01)).astype(np.float32)
        hid = O.make_hidden(seed + 1000, T, H)
        cfg = GlmMoeDsaConfig(hidden_size=H, routed_experts=E, experts_per_token=K)
        x = torch.from_numpy(O.bf16_to_f32(hid)).to(torch.bfloat16)
        idx, w, sc, sel = glm_router_topk(x, torch.from_numpy(rw), cfg, torch.from_numpy(bias))
        router[f"{name}_meta"] = np.array([seed, T, H, E, K], np.int64)
        router[f"{name}_idx"] = idx.numpy().astype(np.int64)
        router[f"{name}_w"] = w.numpy()
        router[f"{name}_sel"] = sel.numpy()
    # the reference's own generated-layer golden (tests/test_glm_moe_dsa_layer_ref.py:67-96)
    cfg = GlmMoeDsaConfig()
    hidden = torch.linspace(-0.75, 0.75, steps=2 * cfg.hidden_size).reshape(2, cfg.hidden_size)
    norm_w = torch.linspace(0.875, 1.125, steps=cfg.hidden_size)
    normalized = rmsnorm(hidden, norm_w)
    rw = torch.zeros(cfg.routed_experts, cfg.hidden_size)
    for e in range(cfg.routed_experts):
        rw[e, e % cfg.hidden_size] = 0.03125 + e / 8192.0
        rw[e, (e * 17 + 13) % cfg.hidden_size] = -0.015625
    bias = torch.linspace(-0.125, 0.125, steps=cfg.routed_experts)
    idx, w, sc, sel = glm_router_topk(normalized, rw, cfg, bias)
    assert idx[0].tolist() == [255, 254, 253, 252, 251, 250, 249, 248]
    router["gen_normalized"] = normalized.numpy()
    router["gen_idx"] = idx.numpy().astype(np.int64)
    router["gen_w"] = w.numpy()
    np.savez_compressed(os.path.join(HERE, "router.npz"), **router)

    # ---- NVFP4 MoE layer (small shapes) -------------------------------------
    def e4m3_cast(x):  # RNE, clamped to the largest finite E4M3 value before the cast
        return torch.clamp(x, max=448.0).to(torch.float8_e4m3fn)

    def ref_quantize_weight(w):
        amax = w.abs().max()
        g = amax / (6.0 * 448.0)
        blk = w.reshape(w.shape[0], -1, 16)
        s8 = e4m3_cast(blk.abs().amax(dim=-1) / (6.0 * g))
        sg = s8.float() * g
        codes = Q.nvfp4_quantize(blk, sg.unsqueeze(-1))
        deq = Q.nvfp4_dequantize(codes, sg.unsqueeze(-1)).reshape(w.shape)
        return codes.reshape(w.shape).numpy(), s8.view(torch.uint8).numpy(), float(g), deq

    def ref_act_qdq(x):
        blk = x.float().reshape(x.shape[0], -1, 16)
        s8 = e4m3_cast(blk.abs().amax(dim=-1) / 6.0)
        s = s8.float().unsqueeze(-1)
        codes = Q.nvfp4_quantize(blk, s)
        codes = torch.where(s == 0, torch.zeros_like(codes), codes)
        return Q.nvfp4_dequantize(codes, s).reshape(x.shape), codes.reshape(x.shape).numpy(), s8.view(torch.uint8).numpy()

    moe = {}
    for name, (seed, T, H, I, E, K) in {"tiny": (3, 6, 256, 128, 8, 2),
                                        "mid": (5, 40, 512, 256, 16, 4)}.items():
        r = np.random.default_rng(seed)
        rw = (r.standard_normal((E, H), np.float32) * np.float32(0.02)).astype(np.float32)
        bias = (r.standard_normal(E, np.float32) * np.float32(0.01)).astype(np.float32)
        experts, experts_codes = {}, {}
        for e in range(E):
            ws = []
            for t, shape in enumerate(((I, H), (I, H), (H, I))):
                w = (r.standard_normal(shape, np.float32) * np.float32(0.02)).astype(np.float32)
                c, s8, g, deq = ref_quantize_weight(torch.from_numpy(w))
                experts_codes[(e, t)] = (c, s8, g)
                ws.append(deq)
            experts[e] = ExpertWeights(*ws)
        hid = O.make_hidden(seed + 1000, T, H)
        x = torch.from_numpy(O.bf16_to_f32(hid)).to(torch.bfloat16)
        cfg = GlmMoeDsaConfig(hidden_size=H, routed_experts=E, experts_per_token=K, moe_intermediate_size=I)
        idx, w, sc, sel = glm_router_topk(x, torch.from_numpy(rw), cfg, torch.from_numpy(bias))
        out_o0 = moe_forward(x, experts, idx, w)
        total, partials = partitioned_moe_forward(x, experts, idx, w, owner_fn=lambda e: str(e % 2))
        # quantisation-matched composition out of reference functions only
        xq, xcodes, xs8 = ref_act_qdq(x)
        import torch.nn.functional as F
        out_o1 = torch.zeros_like(x)
        inter_codes = np.zeros((T, K, I), np.uint8)
        for row in range(T):
            for slot in range(K):
                ew = experts[int(idx[row, slot])]
                h = xq[row:row + 1]
                act = F.silu(h @ ew.gate_proj.T) * (h @ ew.up_proj.T)
                aq, acodes, _ = ref_act_qdq(act)
                inter_codes[row, slot] = acodes[0]
                y = (aq @ ew.down_proj.T).to(torch.bfloat16)
                out_o1[row] += w[row, slot].to(torch.bfloat16) * y.squeeze(0)
        moe[f"{name}_meta"] = np.array([seed, T, H, I, E, K], np.int64)
        moe[f"{name}_idx"] = idx.numpy().astype(np.int64)
        moe[f"{name}_w"] = w.numpy()
        moe[f"{name}_o0"] = out_o0.view(torch.uint16).numpy() if hasattr(torch, "uint16") else out_o0.view(torch.int16).numpy().view(np.uint16)
        moe[f"{name}_o1"] = out_o1.view(torch.int16).numpy().view(np.uint16)
        moe[f"{name}_p0"] = partials["0"].view(torch.int16).numpy().view(np.uint16)
        moe[f"{name}_p1"] = partials["1"].view(torch.int16).numpy().view(np.uint16)
        moe[f"{name}_xcodes"] = xcodes
        moe[f"{name}_xscales"] = xs8
        moe[f"{name}_inter_codes"] = inter_codes
        for (e, t), (c, s8, g) in experts_codes.items():
            if e < 2:
                moe[f"{name}_w{e}_{t}_codes"] = c
                moe[f"{name}_w{e}_{t}_scales"] = s8
                moe[f"{name}_w{e}_{t}_g"] = np.float32(g)
    np.savez_compressed(os.path.join(HERE, "moe.npz"), **moe)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/generate_golden.py /path/to/reference")
    main(sys.argv[1])
