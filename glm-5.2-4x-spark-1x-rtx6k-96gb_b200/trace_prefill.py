"""Timeline of one CTA of the prefill expert GEMMs, from stamps taken inside the kernels.

    python build.py --trace                       # libglmrt_b200_trace.so (stamps compiled in)
    python trace_prefill.py [--tokens 8192]       # on a B200; prints the summary below

The trace library is the product library built with -DGLMRT_B200_TRACE: producer, issuer and the
first epilogue warp of CTA 5 write clock64() stamps per pipeline stage and per tile (see the macros
at the top of csrc/gemm_tc_prefill.cu).  This script runs a few forwards of the GLM-5.2-shaped layer
on synthetic weights, reads the stamps of the last forward and prints, in SM cycles:

  * the stage period of the issuer inside a tile and across a tile boundary;
  * the legs of a stage's round trip: slot seen free -> loads issued -> stage seen full -> MMAs
    issued -> slot seen free again (number of stages x period = sum of the legs when the pipeline is
    bound by that round trip);
  * at a tile boundary, relative to the issue of the previous tile's last stage: when the issuer
    starts waiting for the accumulator, when the epilogue sees it full and has read it out, when the
    issuer gets it back and when the next tile's first stage is issued.
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
KERNELS = (("FC1 <1,256>", 0, 4), ("FC2 <0,128>", 1, 5))   # name, trace index, pipeline stages


def _load_package():
    if "glmrt_b200" not in sys.modules:
        spec = importlib.util.spec_from_file_location("glmrt_b200", os.path.join(HERE, "__init__.py"),
                                                      submodule_search_locations=[HERE])
        mod = importlib.util.module_from_spec(spec)
        sys.modules["glmrt_b200"] = mod
        spec.loader.exec_module(mod)


def pct(x, q):
    return float(np.percentile(x, q))


def summarise(name, stages, tiles, k_stages, pipe_stages):
    slot_free, loads_issued, full_seen, mma_issued = stages.astype(np.float64)
    n = int((mma_issued > 0).sum())
    if n < 4 * k_stages:
        print(f"{name}: only {n} stages recorded")
        return
    d = np.diff(mma_issued[:n])
    boundary = (np.arange(1, n) % k_stages) == 0
    print(f"{name}: {n} stages = {n // k_stages} tiles of {k_stages} stages; "
          f"span {(mma_issued[n - 1] - slot_free[0]) / 1e3:.0f} k cycles")
    print(f"  stage period: inside a tile median {np.median(d[~boundary]):.0f} (p90 {pct(d[~boundary], 90):.0f}), "
          f"across a tile boundary median {np.median(d[boundary]):.0f}")
    lo, hi = k_stages, n - pipe_stages - 1
    legs = (("slot seen free -> loads issued", loads_issued[lo:hi] - slot_free[lo:hi]),
            ("loads issued -> stage seen full", full_seen[lo:hi] - loads_issued[lo:hi]),
            ("stage seen full -> MMAs issued", mma_issued[lo:hi] - full_seen[lo:hi]),
            ("MMAs issued -> slot seen free", slot_free[lo + pipe_stages:hi + pipe_stages] - mma_issued[lo:hi]))
    total = 0.0
    for label, v in legs:
        total += float(np.median(v))
        print(f"  {label:34s} median {np.median(v):6.0f}  p10 {pct(v, 10):6.0f}  p90 {pct(v, 90):6.0f}")
    print(f"  sum of the medians {total:.0f} = {total / pipe_stages:.0f} per stage with {pipe_stages} stages in flight")
    acc_wait, acc_got, epi_wait, epi_full, epi_released, epi_done = tiles.astype(np.float64)
    nt = min(int((acc_wait > 0).sum()), n // k_stages)
    rows = []
    for i in range(2, nt - 1):
        t0 = mma_issued[i * k_stages - 1]          # issue of the last stage of tile i-1
        rows.append((acc_wait[i] - t0, epi_full[i - 1] - t0, epi_released[i - 1] - t0, acc_got[i] - t0,
                     full_seen[i * k_stages] - t0, mma_issued[i * k_stages] - t0, epi_done[i - 1] - t0))
    r = np.array(rows)
    labels = ("issuer starts waiting for the accumulator", "epilogue sees the accumulator full",
              "first epilogue warp has read it out", "issuer has the accumulator back",
              "issuer sees the next tile's first stage", "next tile's first stage issued", "epilogue of the tile done")
    print("  tile boundary, cycles after the issue of the tile's last stage:")
    for j, label in enumerate(labels):
        if name.startswith("FC2") and j == 2:
            continue                                  # stamp taken in the FC1 epilogue only
        print(f"    {label:44s} median {np.median(r[:, j]):7.0f}  p90 {pct(r[:, j], 90):7.0f}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--experts", type=int, default=256)
    args = ap.parse_args()
    if not os.path.exists(TRACE_LIB):
        raise SystemExit("build the trace library first: python build.py --trace")
    os.environ["GLMRT_NATIVE_LIB"] = TRACE_LIB
    import torch
    _load_package()
    from glmrt_b200.layer import MoeLayer
    H, I, K = 6144, 2048, 8
    T, E = args.tokens, args.experts
    if T <= 256:
        raise SystemExit("the traced kernels serve batches above 256 tokens")
    torch.cuda.set_device(0)
    layer = MoeLayer(H, I, E, K, max_tokens=T)
    layer.fill_synthetic(0, 0.02)
    g = torch.Generator(device="cpu").manual_seed(0)
    layer.set_router(torch.randn(E, H, generator=g) * 0.02, torch.zeros(E))
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    for _ in range(5):
        layer.forward(x, out)
    torch.cuda.synchronize()
    layer.check()
    lib = C.CDLL(TRACE_LIB)
    stages = np.zeros((2, 4, 2048), np.int64)
    tiles = np.zeros((2, 6, 256), np.int64)
    rc = lib.glmrt_b200_debug_prefill_trace(C.c_void_p(stages.ctypes.data), C.c_void_p(tiles.ctypes.data))
    if rc != 0:
        raise SystemExit(f"reading the trace failed: CUDA error {rc}")
    print(f"layer {H}x{I}, {E} experts, top-{K}, {T} tokens; CTA 5 of 148; all figures in SM cycles (clock64)")
    for name, kind, pipe in KERNELS:
        k_stages = (H if kind == 0 else I) // 256
        summarise(name, stages[kind], tiles[kind], k_stages, pipe)
    layer.close()


if __name__ == "__main__":
    main()
