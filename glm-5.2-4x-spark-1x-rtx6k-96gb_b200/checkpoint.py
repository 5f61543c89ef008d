"""Checkpoint reader for the routed-MoE path: raw safetensors -> a MoeLayer's resident weights.

Mirrors the part of the reference's loader that the expert path needs
(rust/crates/glmrt-loader/src/catalog.rs:56-140,199-246 and tensors.rs:79-232, and the route
loader rust/crates/glmrt-daemon/src/commands/real_full/sparse_mlp/route.rs:6732-6768):

  * a snapshot directory holds ``model.safetensors.index.json`` (``weight_map``: tensor -> file) and
    the shard files; every shard starts with an 8-byte little-endian header length and a JSON header
    whose ``data_offsets`` are relative to the end of the header;
  * a routed expert's projections are ``model.layers.L.mlp.experts.E.{gate,up,down}_proj`` with
    ``.weight`` (U8, [out, in/2], two E2M1 codes per byte, low nibble first), ``.weight_scale``
    (F8_E4M3, [out, in/16]), ``.weight_scale_2`` and ``.input_scale`` (F32 scalars);
    value = code * e4m3(weight_scale) * weight_scale_2.  ``input_scale`` is the checkpoint's static
    activation scale; like the reference's route computation this path quantises activations per
    16-element block and only validates it;
  * the router is ``model.layers.L.mlp.gate.weight`` ([experts, hidden], BF16 or F32) and
    ``model.layers.L.mlp.gate.e_score_correction_bias`` ([experts]).

The layer keeps codes in exactly this row-major layout and re-tiles the scale bytes on the device
when an expert is set, so there is no host-side packing step and nothing worth caching on disk:
loading is a read of the tensor bytes and one host-to-device copy per tensor.
"""
from __future__ import annotations

import json
import math
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import numpy as np

# safetensors dtype names the path reads (glmrt-core/src/model.rs:43-57) and their byte widths
DTYPE_BYTES = {"U8": 1, "F8_E4M3": 1, "F32": 4, "BF16": 2, "F16": 2, "I8": 1, "I32": 4}
PROJECTIONS = ("gate_proj", "up_proj", "down_proj")


class CheckpointError(ValueError):
    """A snapshot that does not have the layout this path expects."""


@dataclass(frozen=True)
class TensorInfo:
    """One catalog entry (glmrt-core TensorInfo): offsets are absolute within the file."""
    name: str
    file: str
    dtype: str
    shape: Tuple[int, ...]
    byte_offset: int
    byte_length: int

    @property
    def layer_id(self) -> Optional[int]:
        return _number_after(self.name, "model.layers.")

    @property
    def expert_id(self) -> Optional[int]:
        return _number_after(self.name, ".mlp.experts.")


def _number_after(name: str, marker: str) -> Optional[int]:
    # catalog.rs:247-260
    pos = name.find(marker)
    if pos < 0:
        return None
    digits = ""
    for ch in name[pos + len(marker):]:
        if not ch.isdigit():
            break
        digits += ch
    return int(digits) if digits else None


def parse_safetensors_header(path: str) -> Dict[str, TensorInfo]:
    """Header of one shard with absolute offsets; the checks of catalog.rs:199-246."""
    file_len = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise CheckpointError(f"{path}: shorter than a safetensors length prefix")
        (header_len,) = struct.unpack("<Q", head)
        data_start = 8 + header_len
        if data_start > file_len:
            raise CheckpointError(
                f"safetensors header extends beyond {path}: data starts at {data_start}, file length is {file_len}")
        raw = json.loads(f.read(header_len).decode("utf-8"))
    out: Dict[str, TensorInfo] = {}
    for name, entry in raw.items():
        if name == "__metadata__":
            continue
        try:
            dtype, shape, (begin, end) = entry["dtype"], tuple(int(d) for d in entry["shape"]), entry["data_offsets"]
        except (KeyError, TypeError, ValueError) as exc:
            raise CheckpointError(f"parsing header entry {name} in {path}: {exc}") from None
        if begin > end:
            raise CheckpointError(f"invalid safetensors offsets for {name} in {path}: [{begin}, {end}]")
        if data_start + end > file_len:
            raise CheckpointError(
                f"safetensors tensor {name} extends beyond {path}: end {data_start + end}, file length {file_len}")
        out[name] = TensorInfo(name, os.path.basename(path), dtype, shape, data_start + begin, end - begin)
    return out


class TensorCatalog:
    """Tensor name -> file and byte range for one snapshot directory (catalog.rs:56-140).

    With ``model.safetensors.index.json`` present its weight map decides which file holds a tensor and
    a disagreement with the shard headers is an error; without it every ``*.safetensors`` file of the
    directory is scanned (a single-file checkpoint)."""

    def __init__(self, snapshot_path: str):
        self.snapshot_path = snapshot_path
        index_path = os.path.join(snapshot_path, "model.safetensors.index.json")
        self.tensors: Dict[str, TensorInfo] = {}
        if os.path.exists(index_path):
            with open(index_path, "r", encoding="utf-8") as f:
                try:
                    weight_map = json.load(f)["weight_map"]
                except (KeyError, json.JSONDecodeError) as exc:
                    raise CheckpointError(f"parsing {index_path}: {exc}") from None
            by_file: Dict[str, Dict[str, TensorInfo]] = {}
            for file_name in sorted(set(weight_map.values())):
                by_file[file_name] = parse_safetensors_header(os.path.join(snapshot_path, file_name))
            header_file = {name: fn for fn, entries in by_file.items() for name in entries}
            for name, file_name in weight_map.items():
                if name not in header_file:
                    raise CheckpointError(f"tensor {name} missing from safetensors header")
                if header_file[name] != file_name:
                    raise CheckpointError(
                        f"index/header file mismatch for {name}: index={file_name} header={header_file[name]}")
                self.tensors[name] = by_file[file_name][name]
        else:
            files = sorted(f for f in os.listdir(snapshot_path) if f.endswith(".safetensors"))
            if not files:
                raise CheckpointError(f"no safetensors files in {snapshot_path}")
            for file_name in files:
                self.tensors.update(parse_safetensors_header(os.path.join(snapshot_path, file_name)))
        config_path = os.path.join(snapshot_path, "config.json")
        self.config: dict = {}
        if os.path.exists(config_path):
            with open(config_path, "r", encoding="utf-8") as f:
                self.config = json.load(f)

    # ---- lookups -------------------------------------------------------------------------
    def __contains__(self, name: str) -> bool:
        return name in self.tensors

    def info(self, name: str) -> TensorInfo:
        try:
            return self.tensors[name]
        except KeyError:
            raise CheckpointError(f"missing tensor {name}") from None

    def names(self) -> List[str]:
        return sorted(self.tensors)

    def moe_layers(self) -> List[int]:
        """Layers that hold routed experts."""
        return sorted({t.layer_id for t in self.tensors.values()
                       if t.expert_id is not None and t.layer_id is not None})

    def experts_of(self, layer_id: int) -> List[int]:
        return sorted({t.expert_id for t in self.tensors.values()
                       if t.layer_id == layer_id and t.expert_id is not None})

    # ---- reads (tensors.rs:79-232) -------------------------------------------------------
    def read_bytes(self, name: str) -> np.ndarray:
        """Exactly the tensor's bytes."""
        t = self.info(name)
        data = np.fromfile(os.path.join(self.snapshot_path, t.file), dtype=np.uint8, count=t.byte_length,
                           offset=t.byte_offset)
        if data.size != t.byte_length:
            raise CheckpointError(f"read {data.size} bytes of {name}, expected {t.byte_length}")
        return data

    def read_rows(self, name: str, start_row: int, row_count: int) -> np.ndarray:
        """A window of rows of a 2-D tensor as [row_count, row_bytes] uint8."""
        t = self.info(name)
        if len(t.shape) != 2:
            raise CheckpointError(f"{name} is not a 2-D tensor: shape {list(t.shape)}")
        width = _dtype_bytes(t)
        rows, cols = t.shape
        if start_row < 0 or row_count < 0 or start_row + row_count > rows:
            raise CheckpointError(f"row window [{start_row}, {start_row + row_count}) exceeds {name} with {rows} rows")
        row_bytes = cols * width
        if rows * row_bytes != t.byte_length:
            raise CheckpointError(f"{name}: shape {list(t.shape)} does not match {t.byte_length} bytes")
        data = np.fromfile(os.path.join(self.snapshot_path, t.file), dtype=np.uint8, count=row_count * row_bytes,
                           offset=t.byte_offset + start_row * row_bytes)
        if data.size != row_count * row_bytes:
            raise CheckpointError(f"read {data.size} bytes of {name}, expected {row_count * row_bytes}")
        return data.reshape(row_count, row_bytes)

    def read_f32_scalar(self, name: str) -> float:
        """route.rs first_f32_scalar: a scalar (or one-element) F32 tensor, finite."""
        t = self.info(name)
        if t.dtype != "F32" or t.byte_length < 4 or math.prod(t.shape) != 1:
            raise CheckpointError(f"{name} must be an F32 scalar, found {t.dtype} {list(t.shape)}")
        value = float(self.read_bytes(name)[:4].view("<f4")[0])
        if not math.isfinite(value):
            raise CheckpointError(f"{name} is not finite: {value}")
        return value

    def read_f32_array(self, name: str) -> np.ndarray:
        """A BF16, F16 or F32 tensor as float32 (router weight and bias)."""
        t = self.info(name)
        raw = self.read_bytes(name)
        if t.dtype == "F32":
            out = raw.view("<f4").astype(np.float32)
        elif t.dtype == "BF16":
            out = (raw.view("<u2").astype(np.uint32) << 16).view(np.float32)
        elif t.dtype == "F16":
            out = raw.view("<f2").astype(np.float32)
        else:
            raise CheckpointError(f"{name}: {t.dtype} is not a floating-point router tensor")
        if out.size != math.prod(t.shape):
            raise CheckpointError(f"{name}: shape {list(t.shape)} does not match {t.byte_length} bytes")
        return out.reshape(t.shape)


def _dtype_bytes(t: TensorInfo) -> int:
    try:
        return DTYPE_BYTES[t.dtype]
    except KeyError:
        raise CheckpointError(f"{t.name}: unsupported dtype {t.dtype}") from None


# ---- routed experts --------------------------------------------------------------------------
@dataclass
class ExpertProjection:
    """One projection of a routed expert as the checkpoint stores it."""
    codes: np.ndarray          # uint8 [out, in/2]
    scales: np.ndarray         # uint8 (E4M3 bytes) [out, in/16]
    weight_scale_2: float
    input_scale: float


@dataclass
class ExpertWeights:
    gate: ExpertProjection
    up: ExpertProjection
    down: ExpertProjection

    def scale_2(self) -> Tuple[float, float, float]:
        return (self.gate.weight_scale_2, self.up.weight_scale_2, self.down.weight_scale_2)

    def nbytes(self) -> int:
        return sum(p.codes.nbytes + p.scales.nbytes + 8 for p in (self.gate, self.up, self.down))


def expert_base_name(layer_id: int, expert_id: int, projection: str) -> str:
    return f"model.layers.{layer_id}.mlp.experts.{expert_id}.{projection}"


def read_projection(catalog: TensorCatalog, layer_id: int, expert_id: int, projection: str, out_rows: int,
                    in_cols: int) -> ExpertProjection:
    """The four tensors of one projection, validated like route.rs:6738-6768
    (validate_packed_nvfp4_projection_width, first_f32_scalar, validate_finite_route_scalar)."""
    base = expert_base_name(layer_id, expert_id, projection)
    w, s = catalog.info(base + ".weight"), catalog.info(base + ".weight_scale")
    if w.dtype != "U8" or s.dtype != "F8_E4M3":
        raise CheckpointError(f"{base}: unexpected tensor dtypes {w.dtype}, {s.dtype} (want U8, F8_E4M3)")
    if in_cols % 16 != 0:
        raise CheckpointError(f"{base}: input width {in_cols} is not a multiple of 16")
    if tuple(w.shape) != (out_rows, in_cols // 2):
        raise CheckpointError(f"{base}.weight: shape {list(w.shape)}, expected {[out_rows, in_cols // 2]}")
    if tuple(s.shape) != (out_rows, in_cols // 16):
        raise CheckpointError(f"{base}.weight_scale: shape {list(s.shape)}, expected {[out_rows, in_cols // 16]}")
    scale_2 = catalog.read_f32_scalar(base + ".weight_scale_2")
    input_scale = catalog.read_f32_scalar(base + ".input_scale")
    return ExpertProjection(catalog.read_rows(base + ".weight", 0, out_rows),
                            catalog.read_rows(base + ".weight_scale", 0, out_rows), scale_2, input_scale)


def read_expert(catalog: TensorCatalog, layer_id: int, expert_id: int, hidden: int, inter: int) -> ExpertWeights:
    """gate/up: [inter, hidden]; down: [hidden, inter] (route.rs:6732-6735)."""
    gate = read_projection(catalog, layer_id, expert_id, "gate_proj", inter, hidden)
    up = read_projection(catalog, layer_id, expert_id, "up_proj", inter, hidden)
    down = read_projection(catalog, layer_id, expert_id, "down_proj", hidden, inter)
    # activation scales must be positive (route.rs:3103-3106)
    for label, p in (("gate_proj", gate), ("up_proj", up), ("down_proj", down)):
        if not p.input_scale > 0.0:
            raise CheckpointError(
                f"layer {layer_id} expert {expert_id} {label} activation scale must be positive, found {p.input_scale}")
    return ExpertWeights(gate, up, down)


def read_router(catalog: TensorCatalog, layer_id: int, experts: int, hidden: int) -> Tuple[np.ndarray, np.ndarray]:
    """float32 router weight [experts, hidden] and selection bias [experts]."""
    w = catalog.read_f32_array(f"model.layers.{layer_id}.mlp.gate.weight")
    if w.shape != (experts, hidden):
        raise CheckpointError(f"router weight of layer {layer_id}: shape {list(w.shape)}, expected {[experts, hidden]}")
    bias_name = f"model.layers.{layer_id}.mlp.gate.e_score_correction_bias"
    bias = catalog.read_f32_array(bias_name).reshape(-1) if bias_name in catalog else np.zeros(experts, np.float32)
    if bias.shape != (experts,):
        raise CheckpointError(f"router bias of layer {layer_id}: {bias.size} values, expected {experts}")
    return np.ascontiguousarray(w, np.float32), np.ascontiguousarray(bias, np.float32)


@dataclass
class LoadReport:
    layer_id: int
    experts_loaded: List[int]
    weight_bytes: int
    router_loaded: bool


def load_moe_layer(layer, catalog: TensorCatalog, layer_id: int, experts: Optional[Iterable[int]] = None,
                   load_router: bool = True) -> LoadReport:
    """Fill a ``MoeLayer`` from the checkpoint: the router and every expert that lives on the layer's
    shard (``layer.local_experts()``, expert e on rank e % world as in placement.rs:25-42), or the given
    subset of them.  The checkpoint must hold exactly the layer's shapes."""
    wanted = list(layer.local_experts() if experts is None else experts)
    have = set(catalog.experts_of(layer_id))
    missing = [e for e in wanted if e not in have]
    if missing:
        raise CheckpointError(f"layer {layer_id} has no tensors for experts {missing[:8]}")
    if load_router:
        import torch
        w, b = read_router(catalog, layer_id, layer.experts, layer.hidden)
        layer.set_router(torch.from_numpy(w), torch.from_numpy(b))
    total = 0
    for e in wanted:
        x = read_expert(catalog, layer_id, e, layer.hidden, layer.inter)
        layer.set_expert(e, x.gate.codes, x.gate.scales, x.up.codes, x.up.scales, x.down.codes, x.down.scales,
                         x.scale_2())
        total += x.nbytes()
    return LoadReport(layer_id, wanted, total, load_router)
