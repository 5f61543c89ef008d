"""Checkpoint reader (no GPU): the cases of the reference loader's tests
(rust/crates/glmrt-loader/src/tests.rs:56-88,199-240,318-362,573-603) restated for the Python mirror,
plus the expert-tensor validation of the route loader (sparse_mlp/route.rs:6732-6768) and the decode
formula of the reference's real-tensor fixture (python/tools/generate_nvfp4_real_tensor_decode_fixture.py).
"""
import json
import os
import struct

import numpy as np
import pytest

from oracle import glmrt_oracle as O
from tests.checkpoint_fixture import write_safetensors, write_snapshot, pack_codes

H, I, E, LAYER = 64, 32, 4, 3


@pytest.fixture(scope="module")
def CK(pkg):
    from glmrt_b200 import checkpoint
    return checkpoint


@pytest.fixture(scope="module")
def layer_ref():
    return O.make_layer(5, H, I, E)


@pytest.fixture()
def snapshot(tmp_path, layer_ref):
    root = str(tmp_path / "snap")
    stored_router = write_snapshot(root, layer_ref, LAYER, shards=2)
    return root, stored_router


def test_reads_single_file_safetensors_metadata_with_absolute_offsets(CK, tmp_path):
    # tests.rs:56-88: offsets in the header are relative to the end of the header
    path = str(tmp_path / "one.safetensors")
    data_start = write_safetensors(path, [("a", "U8", (2, 3), bytes(range(6))), ("b", "F32", (), struct.pack("<f", 1.5))],
                                   metadata={"format": "pt"})
    meta = CK.parse_safetensors_header(path)
    assert set(meta) == {"a", "b"}
    assert (meta["a"].byte_offset, meta["a"].byte_length, meta["a"].shape, meta["a"].dtype) == (data_start, 6, (2, 3), "U8")
    assert (meta["b"].byte_offset, meta["b"].byte_length, meta["b"].shape) == (data_start + 6, 4, ())


def test_malformed_shards_are_rejected(CK, tmp_path):
    p = str(tmp_path / "short.safetensors")
    open(p, "wb").write(b"\x01\x02")
    with pytest.raises(CK.CheckpointError, match="length prefix"):
        CK.parse_safetensors_header(p)
    p = str(tmp_path / "long_header.safetensors")
    open(p, "wb").write(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(CK.CheckpointError, match="header extends beyond"):
        CK.parse_safetensors_header(p)
    for name, offsets, what in (("inverted", [4, 2], "invalid safetensors offsets"), ("beyond", [0, 64], "extends beyond")):
        raw = json.dumps({"t": {"dtype": "U8", "shape": [4], "data_offsets": offsets}}).encode()
        p = str(tmp_path / (name + ".safetensors"))
        open(p, "wb").write(struct.pack("<Q", len(raw)) + raw + bytes(4))
        with pytest.raises(CK.CheckpointError, match=what):
            CK.parse_safetensors_header(p)


def test_catalog_follows_the_index_and_checks_it_against_the_headers(CK, snapshot):
    root, _ = snapshot
    cat = CK.TensorCatalog(root)
    assert cat.moe_layers() == [LAYER] and cat.experts_of(LAYER) == list(range(E))
    t = cat.info(f"model.layers.{LAYER}.mlp.experts.2.down_proj.weight_scale")
    assert (t.layer_id, t.expert_id, t.dtype, t.shape) == (LAYER, 2, "F8_E4M3", (H, I // 16))
    assert t.file == "model-00001-of-00002.safetensors"          # expert 2 lives in shard 2 % 2
    assert cat.config["n_routed_experts"] == E
    with pytest.raises(CK.CheckpointError, match="missing tensor"):
        cat.info("model.layers.9.mlp.gate.weight")
    # the index names a file that does not hold the tensor / a tensor no header has
    index_path = os.path.join(root, "model.safetensors.index.json")
    index = json.load(open(index_path))
    name = f"model.layers.{LAYER}.mlp.experts.1.up_proj.weight"
    moved = dict(index, weight_map=dict(index["weight_map"], **{name: "model-00001-of-00002.safetensors"}))
    json.dump(moved, open(index_path, "w"))
    with pytest.raises(CK.CheckpointError, match="index/header file mismatch"):
        CK.TensorCatalog(root)
    ghost = dict(index, weight_map=dict(index["weight_map"], ghost="model-00001-of-00002.safetensors"))
    json.dump(ghost, open(index_path, "w"))
    with pytest.raises(CK.CheckpointError, match="missing from safetensors header"):
        CK.TensorCatalog(root)
    # without an index every shard of the directory is scanned
    os.remove(index_path)
    assert len(CK.TensorCatalog(root).names()) == len(index["weight_map"])


def test_reads_exact_ranges_and_row_windows(CK, snapshot, layer_ref):
    # tests.rs:199-240 (exact range), 318-362 (2-D window), 573-603 (window out of bounds)
    root, _ = snapshot
    cat = CK.TensorCatalog(root)
    name = f"model.layers.{LAYER}.mlp.experts.3.gate_proj.weight"
    want = pack_codes(layer_ref.gate[3])
    np.testing.assert_array_equal(cat.read_bytes(name).reshape(I, H // 2), want)
    np.testing.assert_array_equal(cat.read_rows(name, 5, 7), want[5:12])
    assert cat.read_rows(name, I, 0).shape == (0, H // 2)
    for start, count in ((I - 1, 2), (-1, 1), (0, I + 1)):
        with pytest.raises(CK.CheckpointError, match="row window"):
            cat.read_rows(name, start, count)
    with pytest.raises(CK.CheckpointError, match="not a 2-D tensor"):
        cat.read_rows(f"model.layers.{LAYER}.mlp.experts.3.gate_proj.weight_scale_2", 0, 1)


def test_expert_tensors_decode_like_the_reference_fixture(CK, snapshot, layer_ref):
    """value = e2m1_code * f8e4m3(weight_scale[i / 16]) * weight_scale_2, low nibble first."""
    root, stored_router = snapshot
    cat = CK.TensorCatalog(root)
    x = CK.read_expert(cat, LAYER, 1, H, I)
    for t, (p, codes, scales) in enumerate(((x.gate, layer_ref.gate, layer_ref.gate_s), (x.up, layer_ref.up, layer_ref.up_s),
                                            (x.down, layer_ref.down, layer_ref.down_s))):
        np.testing.assert_array_equal(p.codes, pack_codes(codes[1]))
        np.testing.assert_array_equal(p.scales, scales[1])
        assert p.weight_scale_2 == float(layer_ref.scale2[1][t]) and p.input_scale == 0.5
        row = 7
        got = O.decode_packed_nvfp4(p.codes[row], p.scales[row], np.float32(p.weight_scale_2), p.codes.shape[1] * 2)
        want = O.dequantize_weight(codes[1], scales[1], layer_ref.scale2[1][t])[row]
        np.testing.assert_array_equal(got, want)
    w, b = CK.read_router(cat, LAYER, E, H)
    np.testing.assert_array_equal(w, stored_router)
    np.testing.assert_array_equal(b, layer_ref.bias)
    assert x.nbytes() == 3 * (H * I // 2 + H * I // 16 + 8)


def test_the_safetensors_library_writes_what_the_reader_expects(CK, tmp_path, layer_ref):
    """A shard written by the safetensors package itself (float8 and bfloat16 tensors) reads back the same."""
    torch = pytest.importorskip("torch")
    st = pytest.importorskip("safetensors.torch")
    base = f"model.layers.{LAYER}.mlp.experts.0.gate_proj"
    codes = torch.from_numpy(pack_codes(layer_ref.gate[0]))
    scales = torch.from_numpy(np.ascontiguousarray(layer_ref.gate_s[0])).view(torch.float8_e4m3fn)
    router = torch.from_numpy(layer_ref.router_w).to(torch.bfloat16)
    root = tmp_path / "lib"
    root.mkdir()
    st.save_file({base + ".weight": codes, base + ".weight_scale": scales,
                  base + ".weight_scale_2": torch.tensor(0.125, dtype=torch.float32),
                  base + ".input_scale": torch.tensor(2.0, dtype=torch.float32),
                  f"model.layers.{LAYER}.mlp.gate.weight": router}, str(root / "model.safetensors"))
    cat = CK.TensorCatalog(str(root))
    p = CK.read_projection(cat, LAYER, 0, "gate_proj", I, H)
    np.testing.assert_array_equal(p.codes, codes.numpy())
    np.testing.assert_array_equal(p.scales, layer_ref.gate_s[0])
    assert (p.weight_scale_2, p.input_scale) == (0.125, 2.0)
    w, b = CK.read_router(cat, LAYER, E, H)
    np.testing.assert_array_equal(w, router.to(torch.float32).numpy())
    assert not b.any()                                      # no bias tensor: zeros


def _rewrite(root, shard, edit):
    """Rewrite one shard with ``edit(name, dtype, shape, data) -> (dtype, shape, data)`` applied."""
    from glmrt_b200 import checkpoint as CK
    path = os.path.join(root, shard)
    meta = CK.parse_safetensors_header(path)
    blob = open(path, "rb").read()
    tensors = []
    for name, t in sorted(meta.items(), key=lambda kv: kv[1].byte_offset):
        tensors.append((name, *edit(name, t.dtype, t.shape, blob[t.byte_offset:t.byte_offset + t.byte_length])))
    write_safetensors(path, tensors)


@pytest.mark.parametrize("suffix,change,message", [
    (".gate_proj.weight", lambda d, s, b: ("I8", s, b), "unexpected tensor dtypes"),
    (".up_proj.weight_scale", lambda d, s, b: ("U8", s, b), "unexpected tensor dtypes"),
    (".down_proj.weight", lambda d, s, b: (d, (s[0] // 2, s[1] * 2), b), "expected"),
    (".down_proj.weight_scale", lambda d, s, b: (d, (s[0] * 2, s[1] // 2), b), "expected"),
    (".gate_proj.weight_scale_2", lambda d, s, b: (d, s, struct.pack("<f", float("inf"))), "not finite"),
    (".up_proj.weight_scale_2", lambda d, s, b: ("BF16", (2,), b), "must be an F32 scalar"),
    (".down_proj.input_scale", lambda d, s, b: (d, s, struct.pack("<f", 0.0)), "must be positive"),
    (".gate_proj.input_scale", lambda d, s, b: (d, s, struct.pack("<f", float("nan"))), "not finite"),
])
def test_expert_validation(CK, snapshot, suffix, change, message):
    root, _ = snapshot
    target = f"model.layers.{LAYER}.mlp.experts.0" + suffix
    _rewrite(root, "model-00001-of-00002.safetensors",
             lambda name, d, s, b: change(d, s, b) if name == target else (d, s, b))
    cat = CK.TensorCatalog(root)
    with pytest.raises(CK.CheckpointError, match=message):
        CK.read_expert(cat, LAYER, 0, H, I)
    CK.read_expert(cat, LAYER, 1, H, I)                     # the other shard is untouched


class RecordingLayer:
    """Stands in for MoeLayer: same attributes and setter signatures, records what it is given."""

    def __init__(self, world, rank):
        self.hidden, self.inter, self.experts, self.ep_world, self.ep_rank = H, I, E, world, rank
        self.router, self.set = None, {}

    def local_experts(self):
        return [e for e in range(self.experts) if e % self.ep_world == self.ep_rank]

    def set_router(self, w, b):
        self.router = (w.numpy().copy(), b.numpy().copy())

    def set_expert(self, e, gc, gs, uc, us, dc, ds, scale_2):
        self.set[e] = (gc, gs, uc, us, dc, ds, scale_2)


def test_load_moe_layer_fills_the_shard_of_the_rank(CK, snapshot, layer_ref):
    pytest.importorskip("torch")
    root, stored_router = snapshot
    cat = CK.TensorCatalog(root)
    layer = RecordingLayer(world=2, rank=1)
    report = CK.load_moe_layer(layer, cat, LAYER)
    assert report.experts_loaded == [1, 3] and sorted(layer.set) == [1, 3] and report.router_loaded
    assert report.weight_bytes == 2 * 3 * (H * I // 2 + H * I // 16 + 8)
    np.testing.assert_array_equal(layer.router[0], stored_router)
    gc, gs, uc, us, dc, ds, s2 = layer.set[3]
    np.testing.assert_array_equal(dc, pack_codes(layer_ref.down[3]))
    np.testing.assert_array_equal(us, layer_ref.up_s[3])
    assert s2 == tuple(float(v) for v in layer_ref.scale2[3])
    # an explicit subset, no router; an expert the checkpoint does not have
    layer2 = RecordingLayer(world=1, rank=0)
    CK.load_moe_layer(layer2, cat, LAYER, experts=[2], load_router=False)
    assert sorted(layer2.set) == [2] and layer2.router is None
    with pytest.raises(CK.CheckpointError, match="no tensors for experts"):
        CK.load_moe_layer(layer2, cat, LAYER, experts=[E + 1])
    with pytest.raises(CK.CheckpointError, match="no tensors for experts"):
        CK.load_moe_layer(layer2, cat, LAYER + 5)
