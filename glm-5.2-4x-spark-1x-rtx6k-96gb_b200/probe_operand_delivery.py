"""Measures how fast the SMs can pull operand tiles into shared memory (L2 -> SMEM and HBM -> SMEM)
with the copy shapes of the prefill FC1 kernel; prints one JSON line.

    python glm-5.2-4x-spark-1x-rtx6k-96gb_b200/probe_operand_delivery.py

The figure for an L2-resident working set is the ceiling of the token-major expert GEMMs once
their operands are L2 hits: per 256-element K stage a CTA must bring 54 KB (FC1) into shared
memory for 512 cycles of tensor-core work.
"""
from __future__ import annotations

import ctypes as C
import importlib.util
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def main() -> int:
    import torch
    if "glmrt_b200" not in sys.modules:
        spec = importlib.util.spec_from_file_location("glmrt_b200", os.path.join(HERE, "__init__.py"),
                                                      submodule_search_locations=[HERE])
        mod = importlib.util.module_from_spec(spec)
        sys.modules["glmrt_b200"] = mod
        spec.loader.exec_module(mod)
    from glmrt_b200 import native as N
    lib = N.library()
    torch.cuda.set_device(0)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    out = {}
    for name, ws in (("l2_resident_48MB", 48 << 20), ("l2_resident_24MB", 24 << 20), ("hbm_4GB", 4 << 30)):
        for stages in (4, 2):
            gbs, ms = C.c_float(), C.c_float()
            lib.call("glmrt_b200_probe_operand_delivery", C.c_size_t(ws), C.c_uint32(stages), C.c_uint32(8),
                     C.byref(gbs), C.byref(ms), stream)
            out[f"{name}_stages{stages}"] = {"gb_per_s": round(gbs.value, 1), "ms": round(ms.value, 4)}
    print(json.dumps({"probe": "operand_delivery", "stage_bytes": 55296, "sms": torch.cuda.get_device_properties(0).multi_processor_count,
                      "results": out}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
