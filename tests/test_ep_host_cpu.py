"""Host-side logic of the expert-parallel path on CPU ranks (gloo, world size 2): row partition,
the all-gather of per-rank views that attach_distributed relies on, and the algebra of the
exchange itself -- partial results computed where the expert lives, pushed to the row's home rank
and combined there, equal the single-rank forward (oracle arithmetic)."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import glmrt_oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    from tests.conftest import load_package
    load_package()
    from glmrt_b200.ep import partition_rows
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    H, I, E, K, T = 256, 128, 8, 2, 11
    layer = O.make_layer(3, H, I, E)
    hid = O.make_hidden(99, T, H)
    start, n = partition_rows(T, world, rank)
    mine = hid[start:start + n]
    # phase 0: route own rows; publish the histogram to everybody (all-gather of objects)
    idx, wts, _, _ = O.router_topk(O.bf16_to_f32(mine), layer.router_w, layer.bias, K)
    hist = np.bincount(idx.reshape(-1).astype(np.int64), minlength=E)
    hists = [None] * world
    dist.all_gather_object(hists, hist)
    # every rank derives the same slot layout for every owner
    totals = np.sum(hists, axis=0)
    my_offset = np.sum(hists[:rank], axis=0) if rank else np.zeros(E, np.int64)
    base = np.zeros(E, np.int64)
    for owner in range(world):
        run = 0
        for e in range(owner, E, world):
            base[e] = run
            run += (totals[e] + 127) // 128 * 128
    layouts = [None] * world
    dist.all_gather_object(layouts, (base.tolist(), totals.tolist()))
    assert all(l == layouts[0] for l in layouts)
    # phase 1: push rows to owners; phase 2: owners compute; phase 2': push results home
    sends = [[] for _ in range(world)]
    cursor = np.zeros(E, np.int64)
    for r in range(n):
        for k in range(K):
            e = int(idx[r, k])
            slot = int(base[e] + my_offset[e] + cursor[e])
            cursor[e] += 1
            sends[e % world].append((slot, e, rank, r, k, mine[r]))
    allsends = [None] * world          # all-to-all of python objects through an all-gather
    dist.all_gather_object(allsends, sends)
    inbox = [allsends[s][rank] for s in range(world)]
    received = [item for box in inbox for item in box]
    slots = [s for s, *_ in received]
    assert len(set(slots)) == len(slots)                      # no two routes share a slot
    results = [[] for _ in range(world)]
    cache = {}
    for slot, e, src, r, k, row in received:
        assert e % world == rank
        if e not in cache:
            cache[e] = layer.expert(e)
        c, s = O.quantize_rows_nvfp4(O.bf16_to_f32(row[None, :]))
        xq = O.dequantize_payload_rows(O.payload_rows(c, s), H)
        y = O.bf16_round(O.expert_forward(xq, cache[e], requant=True))[0]
        results[src].append((r, k, y))
    allres = [None] * world
    dist.all_gather_object(allres, results)
    back = [item for o in range(world) for item in allres[o][rank]]
    # phase 3: combine at home in slot order
    rows = np.zeros((n, K, H), np.uint16)
    for r, k, y in back:
        rows[r, k] = y
    out = O.combine_routes_bf16(rows, wts) if n else np.zeros((0, H), np.uint16)
    _, _, full = O.layer_forward(layer, hid, K, mode="O1")
    ok = np.array_equal(out, full[start:start + n])
    q.put((rank, bool(ok), (start, n)))
    dist.barrier()
    dist.destroy_process_group()


def test_expert_parallel_exchange_on_two_cpu_ranks():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [r[1] for r in res] == [True, True]
    assert res[0][2] == (0, 6) and res[1][2] == (6, 5)


def test_partition_rows_covers_the_batch(pkg):
    from glmrt_b200.ep import partition_rows
    for total in (0, 1, 7, 64, 8192):
        for world in (1, 2, 4, 8):
            parts = [partition_rows(total, world, r) for r in range(world)]
            assert parts[0][0] == 0 and sum(n for _, n in parts) == total
            for (s0, n0), (s1, _) in zip(parts, parts[1:]):
                assert s0 + n0 == s1
