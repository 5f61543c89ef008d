"""Synthetic GLM-5.2-style checkpoint shards for the loader tests (no real checkpoint is available here).

``write_snapshot`` stores an oracle layer (``oracle.glmrt_oracle.make_layer``) the way the ModelOpt
NVFP4 checkpoint the reference reads is laid out: sharded safetensors files with an index, packed
U8 codes, F8_E4M3 block scales and F32 scalars per projection, BF16 router weight, F32 router bias.
The shard writer is a plain restatement of the file format (8-byte little-endian header length,
JSON header, tensor bytes), independent of the reader under test.
"""
import json
import os
import struct

import numpy as np


def write_safetensors(path, tensors, metadata=None, pad_header_to=None):
    """tensors: list of (name, dtype string, shape, bytes-like)."""
    header, offset, blobs = {}, 0, []
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, dtype, shape, data in tensors:
        data = bytes(data)
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [offset, offset + len(data)]}
        offset += len(data)
        blobs.append(data)
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    if pad_header_to is not None:
        raw = raw + b" " * (pad_header_to - len(raw))
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for b in blobs:
            f.write(b)
    return 8 + len(raw)


def pack_codes(codes):
    c = np.ascontiguousarray(codes, np.uint8)
    return (c[..., 0::2] | (c[..., 1::2] << 4)).astype(np.uint8)


def f32_to_bf16_bits(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def expert_tensors(layer_ref, layer_id, e, input_scale=0.5):
    out = []
    for t, (proj, codes, scales) in enumerate((("gate_proj", layer_ref.gate, layer_ref.gate_s),
                                               ("up_proj", layer_ref.up, layer_ref.up_s),
                                               ("down_proj", layer_ref.down, layer_ref.down_s))):
        base = f"model.layers.{layer_id}.mlp.experts.{e}.{proj}"
        packed = pack_codes(codes[e])
        sb = np.ascontiguousarray(scales[e], np.uint8)
        out.append((base + ".weight", "U8", packed.shape, packed.tobytes()))
        out.append((base + ".weight_scale", "F8_E4M3", sb.shape, sb.tobytes()))
        out.append((base + ".weight_scale_2", "F32", (), np.float32(layer_ref.scale2[e][t]).tobytes()))
        out.append((base + ".input_scale", "F32", (), np.float32(input_scale).tobytes()))
    return out


def write_snapshot(root, layer_ref, layer_id=3, shards=2, router_dtype="BF16"):
    """Returns the router weight as the checkpoint holds it (bf16-rounded when stored as BF16)."""
    H, I, E = layer_ref.dims
    os.makedirs(root, exist_ok=True)
    per_shard = [[] for _ in range(shards)]
    if router_dtype == "BF16":
        bits = f32_to_bf16_bits(layer_ref.router_w)
        router_bytes = bits.tobytes()
        stored = (bits.astype(np.uint32) << 16).view(np.float32).reshape(E, H)
    else:
        router_bytes = np.ascontiguousarray(layer_ref.router_w, np.float32).tobytes()
        stored = np.ascontiguousarray(layer_ref.router_w, np.float32)
    per_shard[0].append((f"model.layers.{layer_id}.mlp.gate.weight", router_dtype, (E, H), router_bytes))
    per_shard[0].append((f"model.layers.{layer_id}.mlp.gate.e_score_correction_bias", "F32", (E,),
                         np.ascontiguousarray(layer_ref.bias, np.float32).tobytes()))
    # a tensor of another layer and a non-expert tensor: the loader has to leave them alone
    per_shard[-1].append((f"model.layers.{layer_id + 1}.self_attn.q_proj.weight", "BF16", (2, 4), bytes(16)))
    for e in range(E):
        per_shard[e % shards].extend(expert_tensors(layer_ref, layer_id, e))
    weight_map = {}
    for i, tensors in enumerate(per_shard):
        fname = f"model-{i + 1:05d}-of-{shards:05d}.safetensors"
        write_safetensors(os.path.join(root, fname), tensors, metadata={"format": "pt"})
        for name, *_ in tensors:
            weight_map[name] = fname
    with open(os.path.join(root, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": 0}, "weight_map": weight_map}, f)
    with open(os.path.join(root, "config.json"), "w") as f:
        json.dump({"hidden_size": H, "moe_intermediate_size": I, "n_routed_experts": E, "num_experts_per_tok": 4,
                   "quantization_config": {"quant_algo": "NVFP4"}}, f)
    return stored
