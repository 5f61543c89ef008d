"""Multi-process check of the expert-parallel forward: run under torchrun, one rank per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P tests/ep_selfcheck.py

Every rank loads its shard of a small seeded layer, the ranks exchange rows and results over
NVLink peer memory, and rank 0 compares the gathered output with a single-shard layer run on its
own GPU (bit for bit).  Prints ``EP_SELFCHECK_OK world=N`` on success.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

HERE = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "glm-5.2-4x-spark-1x-rtx6k-96gb_b200")


def _load():
    if "glmrt_b200" not in sys.modules:
        spec = importlib.util.spec_from_file_location("glmrt_b200", os.path.join(HERE, "__init__.py"),
                                                      submodule_search_locations=[HERE])
        mod = importlib.util.module_from_spec(spec)
        sys.modules["glmrt_b200"] = mod
        spec.loader.exec_module(mod)


class _Weights:
    """Seeded NVFP4 layer drawn on the host with numpy only (no dependency on test code)."""

    def __init__(self, seed, H, I, E):
        rng = np.random.default_rng(seed)
        self.router_w = (rng.standard_normal((E, H), np.float32) * np.float32(0.02)).astype(np.float32)
        self.bias = (rng.standard_normal(E, np.float32) * np.float32(0.01)).astype(np.float32)
        self.gate = rng.integers(0, 16, (E, I, H), dtype=np.uint8)
        self.up = rng.integers(0, 16, (E, I, H), dtype=np.uint8)
        self.down = rng.integers(0, 16, (E, H, I), dtype=np.uint8)
        self.gate_s = rng.integers(0x28, 0x48, (E, I, H // 16), dtype=np.uint8)
        self.up_s = rng.integers(0x28, 0x48, (E, I, H // 16), dtype=np.uint8)
        self.down_s = rng.integers(0x28, 0x48, (E, H, I // 16), dtype=np.uint8)
        self.scale2 = np.full((E, 3), 2.0 ** -9, np.float32)


def main() -> int:
    _load()
    from glmrt_b200 import ep as EP
    from glmrt_b200.layer import MoeLayer
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    H, I, E, K, T = 512, 256, 16, 4, 50
    w = _Weights(5, H, I, E)
    g = torch.Generator(device="cpu").manual_seed(1)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    layer = MoeLayer(H, I, E, K, max_tokens=64, ep_world=world, ep_rank=rank)
    layer.load_quantized_layer(w)
    EP.attach_distributed(layer, dist)
    s, n = EP.partition_rows(T, world, rank)
    mine = x[s:s + n].cuda()
    out = torch.zeros_like(mine)
    for _ in range(3):
        EP.forward_ep(layer, mine, out)
    layer.check()
    torch.cuda.synchronize()
    parts = [None] * world
    dist.all_gather_object(parts, out.cpu().view(torch.int16).numpy())
    ok = True
    if rank == 0:
        single = MoeLayer(H, I, E, K, max_tokens=64)
        single.load_quantized_layer(w)
        ref = single.forward(x.cuda()).cpu().view(torch.int16).numpy()
        single.check()
        got = np.concatenate([p for p in parts if p.shape[0] > 0], axis=0)
        ok = bool(np.array_equal(got, ref)) and bool(np.isfinite(ref.view(np.uint16).astype(np.float32)).all())
        print(("EP_SELFCHECK_OK" if ok else "EP_SELFCHECK_MISMATCH") + f" world={world}", flush=True)
        single.close()
    ok = nccl_row_all_to_all_check(layer.lib, rank, world) and ok
    dist.barrier()
    layer.close()
    dist.destroy_process_group()
    return 0 if ok else 1


def nccl_row_all_to_all_check(lib, rank, world) -> bool:
    """The reference-ABI NCCL row all-to-all (glmrt_nccl_row_all_to_all_u8_async) between the same
    ranks: rank r must receive every peer's copy of row slice r."""
    import ctypes as C
    from glmrt_b200 import native as N
    n = C.c_size_t(0)
    if lib.call_status("glmrt_nccl_unique_id_bytes", C.byref(n)) != 0:
        if rank == 0:
            print("NCCL_WRAPPERS_SKIPPED (library not loadable)", flush=True)
        return True
    uid = C.create_string_buffer(128)
    if rank == 0:
        lib.call("glmrt_nccl_get_unique_id", uid, C.c_size_t(128))
    box = [bytes(uid.raw)]
    dist.broadcast_object_list(box, src=0)
    uid = C.create_string_buffer(box[0], 128)
    comm = C.c_void_p()
    lib.call("glmrt_nccl_comm_init_rank", uid, C.c_size_t(128), C.c_int(world), C.c_int(rank), C.byref(comm))
    rows, stride = 4 * world + 1, 64
    send = torch.full((rows, stride), rank, dtype=torch.uint8, device="cuda")
    send[:, 0] = torch.arange(rows, dtype=torch.uint8, device="cuda")
    base, extra = divmod(rows, world)
    mine = base + (1 if rank < extra else 0)
    recv = torch.zeros(((world - 1) * mine, stride), dtype=torch.uint8, device="cuda")
    stream = torch.cuda.Stream()
    torch.cuda.synchronize()
    db = lambda t: N.DeviceBuffer.of(t.data_ptr(), t.numel(), torch.cuda.current_device())
    lib.call("glmrt_nccl_row_all_to_all_u8_async", comm, db(send), db(recv), C.c_size_t(rows), C.c_size_t(stride),
             C.c_void_p(stream.cuda_stream))
    stream.synchronize()
    start = rank * base + min(rank, extra)
    got = recv.cpu().numpy().reshape(world - 1, mine, stride)
    peers = [p for p in range(world) if p != rank]
    good = all((got[i, :, 1] == p).all() and (got[i, :, 0] == np.arange(start, start + mine)).all()
               for i, p in enumerate(peers))
    lib.call("glmrt_nccl_comm_destroy", comm)
    if rank == 0:
        print("NCCL_ROW_ALL_TO_ALL_OK" if good else "NCCL_ROW_ALL_TO_ALL_MISMATCH", flush=True)
    return bool(good)


if __name__ == "__main__":
    sys.exit(main())
