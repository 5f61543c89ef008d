"""Host-side wrapper of the layer-level C ABI.

PyTorch is used only as plumbing: device memory (tensors), the current CUDA stream and
process groups.  Every computation happens inside libglmrt_b200.so.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import native as N


def _buf(t: torch.Tensor) -> N.DeviceBuffer:
    assert t.is_cuda and t.is_contiguous()
    return N.DeviceBuffer.of(t.data_ptr(), t.numel() * t.element_size(), t.device.index or 0)


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def sf_tile_offsets(rows: int, kblocks: int) -> np.ndarray:
    """Byte offset of the scale of (row, 16-element block) in the library's tiled scale layout:
    512-byte tiles of 128 rows x 4 blocks, row-tile major (csrc/common.cuh: sf_tile_offset)."""
    r = np.arange(rows)[:, None]
    j = np.arange(kblocks)[None, :]
    return ((r // 128) * (kblocks // 4) + j // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + j % 4


class MoeLayer:
    """One routed-MoE layer resident on the current CUDA device.

    ``engine``: "tc" (tcgen05 tensor-core kernels, the product path), "tc-ordered" (the same with the
    ordered combine pass also above 256 rows), "tc2" / "tc2-fc1" / "tc2-fc2"
    (the same with both / one of the expert GEMMs of large batches on CTA pairs) or "simt" (the float64-accumulating verification kernels).
    """

    def __init__(self, hidden: int, inter: int, experts: int, top_k: int, max_tokens: int,
                 ep_world: int = 1, ep_rank: int = 0, engine: str = "tc", scaling: float = 2.5,
                 lib: N.NativeLibrary | None = None):
        self.lib = lib or N.library()
        flags = {"tc": 0, "tc-ordered": N.LAYER_ORDERED_COMBINE, "tc2": N.LAYER_PAIR_TILES,
                 "tc2-fc1": N.LAYER_PAIR_FC1, "tc2-fc2": N.LAYER_PAIR_FC2, "simt": N.LAYER_ENGINE_SIMT}[engine]
        self.cfg = N.MoeConfig(hidden, inter, experts, top_k, max_tokens, ep_world, ep_rank, flags, scaling)
        self.hidden, self.inter, self.experts, self.top_k = hidden, inter, experts, top_k
        self.max_tokens, self.ep_world, self.ep_rank = max_tokens, ep_world, ep_rank
        self.handle = C.c_void_p()
        self.lib.call("glmrt_b200_moe_layer_create", C.byref(self.cfg), C.byref(self.handle))
        self.device = torch.device("cuda", torch.cuda.current_device())

    def _clone_with_handle(self, handle: C.c_void_p) -> "MoeLayer":
        other = object.__new__(MoeLayer)
        other.__dict__.update(self.__dict__)
        other.handle = handle
        return other

    def create_lane(self, max_tokens: int = 0) -> "MoeLayer":
        """A handle on the same expert weights with a workspace of its own (glmrt_b200_moe_layer_create_lane):
        lanes can run concurrently on different streams / host threads.  ``max_tokens``: the lane's
        row capacity (0 = this layer's)."""
        h = C.c_void_p()
        self.lib.call("glmrt_b200_moe_layer_create_lane", self.handle, C.c_uint32(max_tokens), C.byref(h))
        lane = self._clone_with_handle(h)
        if max_tokens:
            lane.max_tokens = max_tokens
            lane.cfg = N.MoeConfig(self.hidden, self.inter, self.experts, self.top_k, max_tokens, self.ep_world,
                                   self.ep_rank, self.cfg.flags, self.cfg.routed_scaling)
        return lane

    def create_stacked(self) -> "MoeLayer":
        """Another layer of the same shape with weights of its own that shares this layer's workspace
        (glmrt_b200_moe_layer_create_stacked): the next sparse layer of a model."""
        h = C.c_void_p()
        self.lib.call("glmrt_b200_moe_layer_create_stacked", C.byref(self.cfg), self.handle, C.byref(h))
        return self._clone_with_handle(h)

    def close(self) -> None:
        if self.handle:
            self.lib.call("glmrt_b200_moe_layer_destroy", self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- weights ----
    def local_experts(self):
        return [e for e in range(self.experts) if e % self.ep_world == self.ep_rank]

    def set_router(self, weight_f32: torch.Tensor, bias_f32: torch.Tensor) -> None:
        w = weight_f32.to(self.device, torch.float32).contiguous()
        b = bias_f32.to(self.device, torch.float32).contiguous()
        self.lib.call("glmrt_b200_moe_layer_set_router", self.handle, _buf(w), _buf(b), _stream())
        torch.cuda.current_stream().synchronize()

    def set_expert(self, expert_id: int, gate_codes, gate_scales, up_codes, up_scales, down_codes, down_scales,
                   scale_2) -> None:
        """Packed codes (uint8, two values per byte, low nibble first) and E4M3 scale bytes in the
        reference's row-major tensor layout; ``scale_2`` = (gate, up, down)."""
        ts = [torch.as_tensor(np.ascontiguousarray(a)).to(self.device).contiguous()
              if not isinstance(a, torch.Tensor) else a.to(self.device).contiguous()
              for a in (gate_codes, gate_scales, up_codes, up_scales, down_codes, down_scales)]
        self.lib.call("glmrt_b200_moe_layer_set_expert", self.handle, C.c_uint32(expert_id),
                      *[_buf(t) for t in ts], C.c_float(scale_2[0]), C.c_float(scale_2[1]),
                      C.c_float(scale_2[2]), _stream())
        torch.cuda.current_stream().synchronize()

    def load_quantized_layer(self, layer) -> None:
        """Load every local expert from an object with unpacked NVFP4 arrays: router_w [E,H], bias [E],
        gate/up [E,I,H] codes with gate_s/up_s [E,I,H/16] scale bytes, down [E,H,I] with down_s,
        scale2 [E,3]."""
        def pack(c):
            c = np.ascontiguousarray(c, np.uint8)
            return (c[..., 0::2] | (c[..., 1::2] << 4)).astype(np.uint8)
        self.set_router(torch.from_numpy(layer.router_w), torch.from_numpy(layer.bias))
        for e in self.local_experts():
            self.set_expert(e, pack(layer.gate[e]), layer.gate_s[e], pack(layer.up[e]), layer.up_s[e],
                            pack(layer.down[e]), layer.down_s[e], tuple(float(v) for v in layer.scale2[e]))

    def fill_synthetic(self, seed: int, weight_std: float = 0.02) -> None:
        self.lib.call("glmrt_b200_moe_layer_fill_synthetic", self.handle, C.c_uint64(seed),
                      C.c_float(weight_std), _stream())
        torch.cuda.current_stream().synchronize()

    # ---- forward ----
    def forward(self, hidden_bf16: torch.Tensor, out: torch.Tensor | None = None, want_routes: bool = False):
        rows = hidden_bf16.shape[0]
        assert hidden_bf16.dtype == torch.bfloat16 and hidden_bf16.shape[1] == self.hidden
        if out is None:
            out = torch.empty_like(hidden_bf16)
        if want_routes:
            idx = torch.empty((rows, self.top_k), dtype=torch.int32, device=self.device)
            w = torch.empty((rows, self.top_k), dtype=torch.float32, device=self.device)
            bi, bw = _buf(idx), _buf(w)
        else:
            idx = w = None
            bi = bw = N.DeviceBuffer.null()
        self.lib.call("glmrt_b200_moe_layer_forward_async", self.handle, _buf(hidden_bf16), C.c_size_t(rows),
                      _buf(out), bi, bw, _stream())
        return (out, idx, w) if want_routes else out

    def forward_routed(self, hidden_bf16: torch.Tensor, idx: torch.Tensor, w: torch.Tensor,
                       out: torch.Tensor | None = None) -> torch.Tensor:
        rows = hidden_bf16.shape[0]
        if out is None:
            out = torch.empty_like(hidden_bf16)
        idx = idx.to(torch.int32).contiguous()
        w = w.to(torch.float32).contiguous()
        self.lib.call("glmrt_b200_moe_layer_forward_routed_async", self.handle, _buf(hidden_bf16),
                      C.c_size_t(rows), _buf(idx), _buf(w), _buf(out), _stream())
        return out

    def forward_residual(self, hidden_bf16: torch.Tensor, residual_bf16: torch.Tensor,
                         shared_delta_bf16: torch.Tensor | None = None,
                         out: torch.Tensor | None = None) -> torch.Tensor:
        """Forward with the layer's residual step folded into the combine:
        out = bf16(residual + bf16(shared_delta + routed)) (truncating stores)."""
        rows = hidden_bf16.shape[0]
        if out is None:
            out = torch.empty_like(hidden_bf16)
        shared = N.DeviceBuffer.null() if shared_delta_bf16 is None else _buf(shared_delta_bf16)
        self.lib.call("glmrt_b200_moe_layer_forward_residual_async", self.handle, _buf(hidden_bf16),
                      C.c_size_t(rows), _buf(residual_bf16), shared, _buf(out), _stream())
        return out

    def forward_host(self, hidden_host: torch.Tensor, out_host: torch.Tensor) -> None:
        """Host buffers in, host buffers out (pinned memory recommended); synchronises."""
        assert not hidden_host.is_cuda and not out_host.is_cuda
        rows = hidden_host.shape[0]
        self.lib.call("glmrt_b200_moe_layer_forward_host", self.handle, C.c_void_p(hidden_host.data_ptr()),
                      C.c_size_t(rows), C.c_void_p(out_host.data_ptr()), _stream())

    # ---- introspection ----
    STAGES = ("router", "quantize", "plan", "dispatch", "fc1", "fc2", "combine")

    def set_profiling(self, enable: bool) -> None:
        self.lib.call("glmrt_b200_moe_layer_set_profiling", self.handle, C.c_int(1 if enable else 0))

    def stage_times_ms(self) -> dict:
        """Device time of each stage of the last forward (CUDA events on the launching stream)."""
        arr = (C.c_float * len(self.STAGES))()
        self.lib.call("glmrt_b200_moe_layer_stage_times", self.handle, arr, C.c_size_t(len(self.STAGES)))
        return dict(zip(self.STAGES, (float(v) for v in arr)))

    def check(self) -> None:
        self.lib.call("glmrt_b200_moe_layer_check", self.handle, _stream())

    def stats(self) -> N.LayerStats:
        torch.cuda.current_stream().synchronize()
        s = N.LayerStats()
        self.lib.call("glmrt_b200_moe_layer_stats", self.handle, C.byref(s))
        return s

    def debug(self, name: str, dtype=np.uint8, nbytes: int | None = None, offset: int = 0) -> np.ndarray:
        """Copy (part of) an internal device buffer to the host: ``nbytes`` from byte ``offset``."""
        torch.cuda.current_stream().synchronize()
        b = N.DeviceBuffer()
        self.lib.call("glmrt_b200_moe_layer_debug_buffer", self.handle, C.c_uint32(N.DEBUG[name]), C.byref(b))
        assert 0 <= offset <= b.bytes
        n = b.bytes - offset if nbytes is None else min(nbytes, b.bytes - offset)
        host = np.empty(n, np.uint8)
        src = N.DeviceBuffer.of((b.ptr or 0) + offset, n, b.device_id)
        self.lib.call("glmrt_copy_d2h", C.c_void_p(host.ctypes.data), src, C.c_size_t(n))
        return host.view(dtype)

    def read_expert(self, expert_id: int):
        """Read one local expert back as (unpacked codes, row-major scale bytes, scale_2) per
        projection (gate, up, down)."""
        le = expert_id // self.ep_world
        H, I = self.hidden, self.inter
        s2 = self.debug("SCALE2", np.float32, 12, le * 12)
        out = []
        for t, (cn, sn, rows, cols) in enumerate((("GATE_CODES", "GATE_SF", I, H), ("UP_CODES", "UP_SF", I, H),
                                                 ("DOWN_CODES", "DOWN_SF", H, I))):
            packed = self.debug(cn, np.uint8, rows * cols // 2, le * rows * cols // 2).reshape(rows, cols // 2)
            codes = np.empty((rows, cols), np.uint8)
            codes[:, 0::2] = packed & 0xF
            codes[:, 1::2] = packed >> 4
            tiled = self.debug(sn, np.uint8, rows * cols // 16, le * rows * cols // 16)
            sb = tiled[sf_tile_offsets(rows, cols // 16).reshape(-1)].reshape(rows, cols // 16)
            out.append((codes, sb, float(s2[t])))
        return out
