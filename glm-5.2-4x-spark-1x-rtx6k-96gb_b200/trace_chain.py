"""Timeline of the kernels of a forward pass, from stamps taken inside the kernels.

    python build.py --trace                                  # libglmrt_b200_trace.so (stamps compiled in)
    python trace_chain.py [--tokens 1 8 64]                  # one B200
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 trace_chain.py --tokens 64
                                                             # expert-parallel over N GPUs; rank 0 prints

The trace library is the product library built with -DGLMRT_B200_TRACE: every kernel of the chain
records, per launch, the global timer (ns) when its first and its last CTA start, when its first
CTA has passed `griddepcontrol.wait` (everything older on the stream is complete), and when its
last warp leaves (csrc/common.cuh).  The script runs a few forwards back to back and prints the
timeline of one forward in the middle, relative to the start of that forward's first kernel, plus
the distance to the same point of the next forward (the period the benchmark measures).
"""
from __future__ import annotations

import argparse
import ctypes as C
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
TRACE_LIB = os.path.join(HERE, "libglmrt_b200_trace.so")
KERNELS = ("router logits", "router select (+plan)", "quantize+dispatch", "FC1", "FC2", "combine",
           "ep plan+dispatch", "ep count", "ep retile", "route plan")
TUS = ("router", "quant", "gemm", "combine", "ep", "plan")
LAUNCHES, STAMPS = 16, 12
NONE_MIN, NONE_MAX = np.uint64(0xFFFFFFFFFFFFFFFF), np.uint64(0)


def _load_package():
    if "glmrt_b200" not in sys.modules:
        spec = importlib.util.spec_from_file_location("glmrt_b200", os.path.join(HERE, "__init__.py"),
                                                      submodule_search_locations=[HERE])
        mod = importlib.util.module_from_spec(spec)
        sys.modules["glmrt_b200"] = mod
        spec.loader.exec_module(mod)


def read_tables(lib, reset):
    """Merged table [launch, kernel, stamp]; the kernels of one translation unit fill its own table."""
    merged = None
    for tu in TUS:
        t = np.zeros((LAUNCHES, len(KERNELS), STAMPS), np.uint64)
        rc = getattr(lib, f"glmrt_b200_trace_chain_{tu}")(C.c_void_p(t.ctypes.data), C.c_int(1 if reset else 0))
        if rc != 0:
            raise SystemExit(f"reading the chain trace of {tu} failed")
        if merged is None:
            merged = t
        else:
            merged[..., 0] = np.minimum(merged[..., 0], t[..., 0])
            merged[..., 1] = np.maximum(merged[..., 1], t[..., 1])
            merged[..., 2] = np.minimum(merged[..., 2], t[..., 2])
            merged[..., 3:] = np.maximum(merged[..., 3:], t[..., 3:])
    return merged


def print_timeline(title, table, launch):
    row = table[launch]
    used = [k for k in range(len(KERNELS)) if row[k, 0] != NONE_MIN and row[k, 3] != NONE_MAX]
    if not used:
        print(f"{title}: nothing recorded")
        return
    order = sorted(used, key=lambda k: int(row[k, 0]))
    t0 = int(row[order[0], 0])
    print(title)
    print(f"  {'kernel':24s} {'first CTA in':>12s} {'last CTA in':>12s} {'past wait':>10s} {'last warp out':>14s} {'wait->out':>10s}   (µs)")
    for k in order:
        a, b, c, d = (int(v) for v in row[k, :4])
        ready = (c - t0) / 1e3 if row[k, 2] != NONE_MIN else float("nan")
        print(f"  {KERNELS[k]:24s} {(a - t0) / 1e3:12.2f} {(b - t0) / 1e3:12.2f} {ready:10.2f} {(d - t0) / 1e3:14.2f} "
              f"{(d - c) / 1e3 if row[k, 2] != NONE_MIN else float('nan'):10.2f}")
        marks = [(i, (int(row[k, 4 + i]) - t0) / 1e3) for i in range(STAMPS - 4) if row[k, 4 + i] != NONE_MAX]
        if marks:
            print("      marks (latest CTA): " + "  ".join(f"[{i}] {t:.2f}" for i, t in marks))
    end = max(int(row[k, 3]) for k in used)
    nxt = table[launch + 1]
    line = f"  first start -> last end {(end - t0) / 1e3:.2f} µs"
    if nxt[order[0], 0] != NONE_MIN:
        line += f"; the next forward's first kernel starts {(int(nxt[order[0], 0]) - t0) / 1e3:.2f} µs after this one's"
    print(line)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, nargs="+", default=[1, 8, 64])
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--forwards", type=int, default=8)
    args = ap.parse_args()
    if not os.path.exists(TRACE_LIB):
        raise SystemExit("build the trace library first: python build.py --trace")
    os.environ["GLMRT_NATIVE_LIB"] = TRACE_LIB
    import torch
    _load_package()
    from glmrt_b200.layer import MoeLayer
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        from glmrt_b200 import ep as EP
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    lib = C.CDLL(TRACE_LIB)
    H, I, K, E = 6144, 2048, 8, args.experts
    g = torch.Generator(device="cpu").manual_seed(0)
    router_w = torch.randn(E, H, generator=g) * 0.02
    for T in args.tokens:
        if T > 256 and world == 1:
            print(f"T={T}: the prefill kernels carry no chain stamps (see trace_prefill.py)")
            continue
        if world > 1:
            layer = MoeLayer(H, I, E, K, max_tokens=T, ep_world=world, ep_rank=rank)
        else:
            layer = MoeLayer(H, I, E, K, max_tokens=T)
        layer.fill_synthetic(0, 0.02)
        layer.set_router(router_w, torch.zeros(E))
        x = torch.randn(T, H, generator=g).to(torch.bfloat16)
        if world > 1:
            EP.attach_distributed(layer, dist)
            EP.set_global_rows(layer, T)
            r0, rn = EP.partition_rows(T, world, rank)
            x = x[r0:r0 + rn].contiguous()
        xd = x.cuda()
        out = torch.empty(xd.shape[0], H, dtype=torch.bfloat16, device="cuda")

        def fwd():
            if world > 1:
                EP.forward_ep(layer, xd, out)
            else:
                layer.forward(xd, out)

        for _ in range(4):
            fwd()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        read_tables(lib, reset=True)
        torch.cuda.synchronize()
        for _ in range(args.forwards):
            fwd()
        torch.cuda.synchronize()
        layer.check()
        table = read_tables(lib, reset=False)
        if rank == 0:
            mid = args.forwards // 2
            print_timeline(f"T={T}, {E} experts, {world} GPU(s), rank 0, forward {mid} of {args.forwards} (back to back)",
                           table, mid)
            print_timeline(f"T={T}: the first forward after an idle stream", table, 0)
        if dist is not None:
            dist.barrier()
        layer.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
