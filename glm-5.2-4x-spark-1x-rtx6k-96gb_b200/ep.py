"""Expert-parallel set-up and forward calls.

One process per GPU (``torch.distributed`` for the rendezvous only): every rank creates a layer
shard, exchanges CUDA IPC handles of its exchange buffers, learns under which address each peer sees
its result rows, and attaches.  After that a forward step is a single collective C-ABI call per
rank; rows and results move as in-kernel stores over NVLink, no NCCL collective is on the data path.

``attach_in_process`` wires several shards that live in ONE process on one device (tests).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import native as N
from .layer import MoeLayer, _buf, _stream


class EpBuffers(C.Structure):
    """glmrt_b200_ep_buffers_t."""
    _fields_ = [("act_codes", C.c_void_p), ("act_sf", C.c_void_p), ("slot_out", C.c_void_p),
                ("route_rows", C.c_void_p), ("control", C.c_void_p), ("act_sf_rows", C.c_void_p)]


IPC_BYTES = 384


def partition_rows(total_rows: int, world: int, rank: int) -> tuple[int, int]:
    """Block partition of the batch over home ranks: (first row, row count) of ``rank``; the first
    ``total_rows % world`` ranks take one extra row (the split rule of the reference's row
    all-to-all, native/src/glmrt_native.cc:1602-1615)."""
    base, extra = divmod(total_rows, world)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


def local_buffers(layer: MoeLayer) -> EpBuffers:
    b = EpBuffers()
    layer.lib.call("glmrt_b200_ep_local_buffers", layer.handle, C.byref(b))
    return b


def attach(layer: MoeLayer, peers: list[EpBuffers], my_rows_in_peer: list[int]) -> None:
    arr = (EpBuffers * len(peers))(*peers)
    rows = (C.c_uint64 * len(peers))(*my_rows_in_peer)
    layer.lib.call("glmrt_b200_ep_attach", layer.handle, arr, C.c_size_t(len(peers)), rows)


def attach_in_process(layers: list[MoeLayer]) -> None:
    """All shards in this process, same device: peers are addressed by their own pointers."""
    bufs = [local_buffers(l) for l in layers]
    for l in layers:
        attach(l, bufs, [bufs[l.ep_rank].route_rows] * len(layers))


def attach_distributed(layer: MoeLayer, dist) -> None:
    """IPC exchange between the ranks of ``dist`` (one process per GPU on one node)."""
    world, rank = dist.get_world_size(), dist.get_rank()
    mine = C.create_string_buffer(IPC_BYTES)
    layer.lib.call("glmrt_b200_ep_ipc_export", layer.handle, mine, C.c_size_t(IPC_BYTES))
    handles = [None] * world
    dist.all_gather_object(handles, bytes(mine.raw))
    peers = []
    for p in range(world):
        if p == rank:
            peers.append(local_buffers(layer))
        else:
            b = EpBuffers()
            layer.lib.call("glmrt_b200_ep_ipc_open", layer.handle, handles[p], C.c_size_t(IPC_BYTES), C.byref(b))
            peers.append(b)
    # table[o][s] = address under which rank o sees rank s's result rows
    views = [None] * world
    dist.all_gather_object(views, [int(b.route_rows) for b in peers])
    attach(layer, peers, [views[o][rank] for o in range(world)])
    dist.barrier()


def set_global_rows(layer: MoeLayer, global_rows: int) -> None:
    """Tell the exchange how many rows the whole batch has over all ranks (same value on every
    rank): up to 256 it runs decode-sized work items, above prefill-sized ones."""
    layer.lib.call("glmrt_b200_ep_set_global_rows", layer.handle, C.c_uint32(global_rows))


def forward_ep(layer: MoeLayer, hidden: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    rows = hidden.shape[0]
    if out is None:
        out = torch.empty_like(hidden)
    hb = _buf(hidden) if rows else N.DeviceBuffer.null()
    ob = _buf(out) if rows else N.DeviceBuffer.null()
    layer.lib.call("glmrt_b200_moe_layer_forward_ep_async", layer.handle, hb, C.c_size_t(rows), ob, _stream())
    return out


def forward_ep_phase(layer: MoeLayer, phase: int, hidden: torch.Tensor, out: torch.Tensor) -> None:
    rows = hidden.shape[0]
    hb = _buf(hidden) if rows else N.DeviceBuffer.null()
    ob = _buf(out) if rows else N.DeviceBuffer.null()
    layer.lib.call("glmrt_b200_moe_layer_forward_ep_phase_async", layer.handle, C.c_uint32(phase), hb,
                   C.c_size_t(rows), ob, _stream())


def forward_ep_host(layer: MoeLayer, hidden_host: torch.Tensor, out_host: torch.Tensor) -> None:
    rows = hidden_host.shape[0]
    layer.lib.call("glmrt_b200_moe_layer_forward_ep_host", layer.handle, C.c_void_p(hidden_host.data_ptr()),
                   C.c_size_t(rows), C.c_void_p(out_host.data_ptr()), _stream())
