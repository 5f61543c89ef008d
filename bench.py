"""Benchmark of the routed-MoE expert path: MoE-layer tokens/s on 1..8 B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T] [--impl reference]

One "step" is one forward pass of one GLM-5.2-shaped routed-MoE layer (hidden 6144, 256
experts, top-8, expert intermediate 2048, NVFP4 weights, uniform router) over one batch of
T synthetic bf16 N(0,1) rows (default T = 64, the decode-shaped configuration).  Prints ONE
JSON line (rank 0).  Keys beyond the usual ones:

  value     whole-job tokens/s with inputs resident in device memory, K steps between two CUDA
            events on the launching stream, max over ranks.
  e2e       the same through glmrt_b200_moe_layer_forward_host: pinned HOST buffers in and out,
            host<->device copies inside the timed region.
  roofline  dominant kernel (FC1 expert GEMM): algorithmic bytes per launch / its mean duration
            from CUDA events recorded around it on the launching stream during K further steps.
  cpu_baseline  the CPU oracle (numpy port of the reference's python/reference path) timed on
            this host on a bounded sample of the same workload.

With --impl reference only the CPU port runs (no kernel of this repository is used).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

H, I, E, K_TOP = 6144, 2048, 256, 8
EXPERT_BYTES = 3 * I * (H // 2 + H // 16)            # 21,233,664: codes + block scales of one expert
FC1_EXPERT_BYTES = 2 * I * (H // 2 + H // 16)        # gate + up
FC2_EXPERT_BYTES = H * (I // 2 + I // 16)
ROUTER_BYTES = E * H * 4


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def measured_peak_tflops():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    except Exception:
        return 1590.0, "fallback"


def layer_algorithmic_bytes(tokens: int, distinct: int) -> int:
    """Bytes one forward must move: weights of the experts actually selected, activations in and
    out, the float32 router weight and the route table."""
    return distinct * EXPERT_BYTES + tokens * (2 * H * 2) + ROUTER_BYTES + tokens * K_TOP * 8


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the benchmark runs."""

    def __init__(self, index: int, period_s: float = 0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.nv = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._halt.is_set():
            try:
                util = nv.nvmlDeviceGetUtilizationRates(self.h).gpu
                mhz = int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                self.samples.append((mhz, util))
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._halt.wait(self.period)

    def stop(self):
        self._halt.set()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        mhz = [m for m, _ in self.samples]
        return {"sm_mhz": float(np.median(mhz)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(mhz)}


# ------------------------------------------------------------------------------------------
# CPU arm: the oracle port of python/reference (router + moe_forward) on host cores
# ------------------------------------------------------------------------------------------
def cpu_port_run(tokens_total: int, sample_tokens: int, steps: int, warmup: int):
    """Times the numpy port on `sample_tokens` rows of the workload.  Weights of the touched
    experts are drawn, quantised to NVFP4 and pre-dequantised before timing, as the reference's
    baseline plan does; the timed step is router + per-route expert FFNs + combine."""
    from oracle import glmrt_oracle as O
    rng = np.random.default_rng(0)
    rw = (rng.standard_normal((E, H), np.float32) * np.float32(0.02)).astype(np.float32)
    bias = np.zeros(E, np.float32)
    hid = O.make_hidden(1000, sample_tokens, H)
    idx, wts, _, _ = O.router_topk(O.bf16_to_f32(hid), rw, bias, K_TOP)
    cache = {}
    t0 = time.perf_counter()
    for e in np.unique(idx):
        ws = []
        for shape in ((I, H), (I, H), (H, I)):
            w = (rng.standard_normal(shape, np.float32) * np.float32(0.02)).astype(np.float32)
            c, s, g = O.quantize_weight_baseline(w)
            ws.append(O.dequantize_weight(c, s, g))
        cache[int(e)] = O.ExpertWeights(*ws)
    prep_s = time.perf_counter() - t0

    def step():
        i2, w2, _, _ = O.router_topk(O.bf16_to_f32(hid), rw, bias, K_TOP)
        return O.moe_forward(hid, cache.__getitem__, i2, w2, mode="O1")

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    cores = os.cpu_count() or 1
    try:
        from threadpoolctl import threadpool_info
        cores = max([p.get("num_threads", 1) for p in threadpool_info()] + [1])
    except Exception:
        pass
    return {"tokens_per_s": sample_tokens / dt, "ms_per_step": dt * 1e3, "cores": int(cores),
            "sample": f"{sample_tokens} of {tokens_total} rows ({len(cache)} experts touched), weights "
                      f"pre-dequantised ({prep_s:.1f} s, untimed), {steps} timed steps",
            "prep_s": prep_s}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 200))
    warmup = max(0, min(args.warmup, 3))
    r = cpu_port_run(args.tokens, min(args.tokens, 2), steps, warmup)
    line = {
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": r["tokens_per_s"], "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
        "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "nvfp4", "data": "synthetic",
        "config": {"workload": f"glm52_moe_layer_{'prefill' if args.tokens > 256 else 'decode'}_T{args.tokens}", "tokens": args.tokens, "hidden": H,
                   "experts": E, "top_k": K_TOP, "intermediate": I},
        "cpu_baseline": {"value": r["tokens_per_s"], "unit": "tokens/s", "cores": r["cores"], "kind": "port",
                         "sample": r["sample"]},
        "e2e": {"value": r["tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def run_gpu(args):
    import torch
    import __graft_entry__ as entry
    entry.load_package()
    from glmrt_b200.layer import MoeLayer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        return run_ep(args, dist, rank, world, local_rank)

    T, steps, warmup = args.tokens, args.steps, max(3, args.warmup)
    sampler = ClockSampler(local_rank)
    sampler.start()
    layer = MoeLayer(H, I, E, K_TOP, max_tokens=T, engine=args.pair_tiles or "tc")
    layer.fill_synthetic(0, 0.02)
    g = torch.Generator(device="cpu").manual_seed(0)
    rw = (torch.randn(E, H, generator=g) * 0.02)
    layer.set_router(rw, torch.zeros(E))
    # a few distinct input batches so that consecutive steps select different experts
    n_batches = 4
    host_batches = [torch.randn(T, H, generator=g).to(torch.bfloat16).pin_memory() for _ in range(n_batches)]
    dev_batches = [b.cuda() for b in host_batches]
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    host_out = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()

    for i in range(warmup):
        layer.forward(dev_batches[i % n_batches], out)
    layer.check()
    st0 = layer.stats()

    # ---- device-resident timing ----
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    ev0.record()
    for i in range(steps):
        layer.forward(dev_batches[i % n_batches], out)
    ev1.record()
    torch.cuda.synchronize()
    total_ms = ev0.elapsed_time(ev1)
    st1 = layer.stats()
    launches = int(st1.launches_total - st0.launches_total)
    ms_per_step = total_ms / steps

    # ---- the same steps replayed from CUDA graphs (reported beside the stream-ordered figure) ----
    graph_ms = None
    if args.graph:
        graphs = []
        for b in dev_batches:
            gph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gph):
                layer.forward(b, out)
            graphs.append(gph)
        for i in range(warmup):
            graphs[i % n_batches].replay()
        torch.cuda.synchronize()
        ev0.record()
        for i in range(steps):
            graphs[i % n_batches].replay()
        ev1.record()
        torch.cuda.synchronize()
        graph_ms = ev0.elapsed_time(ev1) / steps
        layer.check()

    # ---- per-kernel timing (events around each kernel on the launching stream) ----
    layer.set_profiling(True)
    stage_sum = {}
    distinct_sum = 0
    for i in range(steps):
        layer.forward(dev_batches[i % n_batches], out)
        for k, v in layer.stage_times_ms().items():
            stage_sum[k] = stage_sum.get(k, 0.0) + v
        distinct_sum += layer.stats().distinct_experts
    layer.set_profiling(False)
    stage_ms = {k: v / steps for k, v in stage_sum.items()}
    distinct = distinct_sum / steps
    routes = T * K_TOP
    fc1_bytes = distinct * FC1_EXPERT_BYTES + routes * (H // 2 + H // 16) + routes * (I // 2 + I // 16)
    peak, peak_kind = measured_peak_gbs()
    fc1_gbs = fc1_bytes / (stage_ms["fc1"] * 1e-3) / 1e9
    layer_bytes = layer_algorithmic_bytes(T, distinct)

    # ---- end to end through the host-buffer entry point ----
    for i in range(2):
        layer.forward_host(host_batches[i % n_batches], host_out)
    torch.cuda.synchronize()
    ev0.record()
    for i in range(steps):
        layer.forward_host(host_batches[i % n_batches], host_out)
    ev1.record()
    torch.cuda.synchronize()
    e2e_ms = ev0.elapsed_time(ev1) / steps
    layer.check()
    sampler.stop()
    sampler.join(timeout=2)

    cpu = None
    if not args.no_cpu_baseline:
        layer.close()
        del layer
        torch.cuda.empty_cache()
        r = cpu_port_run(T, min(T, 2), 100, 2)
        cpu = {"value": r["tokens_per_s"], "unit": "tokens/s", "cores": r["cores"], "kind": "port",
               "sample": r["sample"]}

    prefill = T > 256          # the layer switches to its tokens-on-the-MMA-rows kernels above 256 rows
    if not prefill:
        roofline = {"bound": "hbm", "kernel": "expert_gemm_kernel<FC1>", "achieved": fc1_gbs, "peak": peak,
                    "unit": "GB/s", "frac": fc1_gbs / peak, "peak_source": peak_kind,
                    "algorithmic_bytes_per_launch": fc1_bytes, "ms_per_launch": stage_ms["fc1"],
                    "traffic": NCU_FC1_TRAFFIC_PER_EXPERT * distinct,
                    "traffic_source": "ncu dram read+write of one FC1 launch on a 64-expert T=16 case "
                                      "(profiles/expert_gemm_fc1_fc2_E64_T16_ncu_full.md), per expert touched, "
                                      "times the experts touched here"}
    else:
        # prefill: the contraction is what one pays for; FP4 runs at four times the bf16 rate and no
        # FP4 figure is measured on this pool, so the peak is 4 x the measured bf16 burst figure
        fc1_flops = routes * 2.0 * (2 * I) * H
        tf = fc1_flops / (stage_ms["fc1"] * 1e-3) / 1e12
        bf16_peak, bf16_kind = measured_peak_tflops()
        roofline = {"bound": "tensor", "kernel": "expert_gemm_tokens_kernel<FC1>", "achieved": tf,
                    "peak": 4.0 * bf16_peak, "unit": "TFLOP/s", "frac": tf / (4.0 * bf16_peak),
                    "peak_source": f"4 x bf16 burst ({bf16_kind}); nominal dense FP4 is 9000",
                    "frac_of_nominal_fp4": tf / 9000.0,
                    "algorithmic_flops_per_launch": fc1_flops, "ms_per_launch": stage_ms["fc1"],
                    "hbm_gbs": fc1_gbs, "hbm_frac": fc1_gbs / peak,
                    "traffic": NCU_FC1_PREFILL_TRAFFIC_PER_EXPERT * distinct,
                    "traffic_source": "ncu dram read+write of one FC1 launch on a 64-expert T=2048 case "
                                      "(profiles/expert_gemm_tokens_fc1_fc2_E64_T2048_ncu_full.md), per expert "
                                      "touched (weights dominate), times the experts touched here"}

    line = {
        "metric": "moe_layer_tokens_per_s", "value": T / (ms_per_step * 1e-3), "unit": "tokens/s", "n_gpus": 1,
        "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4", "data": "synthetic",
        "config": {"workload": f"glm52_moe_layer_{'prefill' if prefill else 'decode'}_T{T}", "tokens": T, "hidden": H, "experts": E,
                   "top_k": K_TOP, "intermediate": I, "experts_per_gpu": E,
                   "l2": f"no flush: each step streams {layer_bytes / 1e9:.2f} GB of expert weights, far above the 126 MB L2",
                   "distinct_experts_per_step": distinct, "stage_ms": stage_ms,
                   "graph_replay_ms_per_step": graph_ms,
                   "layer_hbm_gbs": layer_bytes / (ms_per_step * 1e-3) / 1e9,
                   "layer_frac_of_peak": layer_bytes / (ms_per_step * 1e-3) / 1e9 / peak},
        "clocks": sampler.summary(),
        "e2e": {"value": T / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": T * H * 2,
                "d2h_bytes_per_step": T * H * 2, "ms_per_step": e2e_ms},
        "gpu_launches": launches,
        "roofline": roofline,
        "cpu_baseline": cpu,
    }
    print(json.dumps(line), flush=True)


def run_ep(args, dist, rank, world, local_rank):
    """N > 1: the same layer and the same global batch, experts sharded e % N over the ranks
    (256/N per GPU), each rank home to T/N rows; rows and results cross NVLink as in-kernel peer
    stores.  Total work is fixed as N grows (strong scaling)."""
    import torch
    from glmrt_b200 import ep as EP
    from glmrt_b200.layer import MoeLayer

    T, steps, warmup = args.tokens, args.steps, max(3, args.warmup)
    sampler = ClockSampler(local_rank)
    sampler.start()
    layer = MoeLayer(H, I, E, K_TOP, max_tokens=T, ep_world=world, ep_rank=rank)
    layer.fill_synthetic(0, 0.02)
    g = torch.Generator(device="cpu").manual_seed(0)
    layer.set_router(torch.randn(E, H, generator=g) * 0.02, torch.zeros(E))
    EP.attach_distributed(layer, dist)
    r0, rn = EP.partition_rows(T, world, rank)
    n_batches = 4
    host_batches = [torch.randn(T, H, generator=g).to(torch.bfloat16)[r0:r0 + rn].contiguous().pin_memory()
                    for _ in range(n_batches)]
    dev_batches = [b.cuda() for b in host_batches]
    out = torch.empty(rn, H, dtype=torch.bfloat16, device="cuda")
    host_out = torch.empty(rn, H, dtype=torch.bfloat16).pin_memory()

    def timed(fn, n):
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        torch.cuda.synchronize()
        ev0.record()
        for i in range(n):
            fn(i)
        ev1.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([ev0.elapsed_time(ev1)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / n

    for i in range(warmup):
        EP.forward_ep(layer, dev_batches[i % n_batches], out)
    layer.check()
    st0 = layer.stats()
    ms_per_step = timed(lambda i: EP.forward_ep(layer, dev_batches[i % n_batches], out), steps)
    st1 = layer.stats()
    launches = int(st1.launches_total - st0.launches_total)

    layer.set_profiling(True)
    stage_sum, distinct_sum = {}, 0
    for i in range(steps):
        EP.forward_ep(layer, dev_batches[i % n_batches], out)
        for k, v in layer.stage_times_ms().items():
            stage_sum[k] = stage_sum.get(k, 0.0) + v
        distinct_sum += layer.stats().distinct_experts
    layer.set_profiling(False)
    stage_ms = {k: v / steps for k, v in stage_sum.items()}
    distinct = distinct_sum / steps
    routes_owned = T * K_TOP / world
    fc1_bytes = distinct * FC1_EXPERT_BYTES + routes_owned * ((H // 2 + H // 16) + (I // 2 + I // 16))
    peak, peak_kind = measured_peak_gbs()
    fc1_gbs = fc1_bytes / (stage_ms["fc1"] * 1e-3) / 1e9

    e2e_ms = timed(lambda i: EP.forward_ep_host(layer, host_batches[i % n_batches], host_out), steps)
    layer.check()
    sampler.stop()
    sampler.join(timeout=2)
    gathered = [None] * world
    dist.all_gather_object(gathered, {"distinct": distinct, "fc1_ms": stage_ms["fc1"], "fc2_ms": stage_ms["fc2"],
                                      "clocks": sampler.summary()})
    if rank == 0:
        total_distinct = sum(x["distinct"] for x in gathered)
        layer_bytes = layer_algorithmic_bytes(T, total_distinct)
        line = {
            "metric": "moe_layer_tokens_per_s", "value": T / (ms_per_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4",
            "data": "synthetic",
            "config": {"workload": f"glm52_moe_layer_{'prefill' if T > 256 else 'decode'}_T{T}", "tokens": T, "hidden": H, "experts": E,
                       "top_k": K_TOP, "intermediate": I, "experts_per_gpu": E // world,
                       "parallelism": f"ep{world}: expert e on rank e % {world}, rows block-partitioned, "
                                      "dispatch/combine = in-kernel NVLink peer stores",
                       "l2": f"no flush: each step streams {layer_bytes / 1e9:.2f} GB of expert weights over "
                             f"{world} GPUs, far above the 126 MB L2",
                       "distinct_experts_per_step": total_distinct, "stage_ms_rank0": stage_ms,
                       "max_over_ranks_imbalance": max(x["distinct"] for x in gathered) /
                                                   max(1e-9, total_distinct / world),
                       "layer_hbm_gbs_aggregate": layer_bytes / (ms_per_step * 1e-3) / 1e9,
                       "layer_frac_of_aggregate_peak": layer_bytes / (ms_per_step * 1e-3) / 1e9 / (peak * world)},
            "clocks": gathered[0]["clocks"],
            "clocks_all_ranks": [x["clocks"] for x in gathered],
            "e2e": {"value": T / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": T * H * 2,
                    "d2h_bytes_per_step": T * H * 2, "ms_per_step": e2e_ms},
            "gpu_launches": launches * world,
            "roofline": {"bound": "hbm", "kernel": "expert_gemm_kernel<FC1> (rank 0)", "achieved": fc1_gbs,
                         "peak": peak, "unit": "GB/s", "frac": fc1_gbs / peak, "peak_source": peak_kind,
                         "algorithmic_bytes_per_launch": fc1_bytes, "ms_per_launch": stage_ms["fc1"],
                         "traffic": NCU_FC1_TRAFFIC_PER_EXPERT * distinct},
            "cpu_baseline": None,
        }
        print(json.dumps(line), flush=True)
    dist.barrier()
    layer.close()
    dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one FC1 launch from the ncu captures summarised
# under profiles/, per expert touched: decode kernel (820.55 MB, 57 experts touched) and prefill
# kernel (1003.59 MB, 64 experts).
NCU_FC1_TRAFFIC_PER_EXPERT = 820.55e6 / 57
NCU_FC1_PREFILL_TRAFFIC_PER_EXPERT = 1003.59e6 / 64


def main():
    global E, ROUTER_BYTES
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--graph", action="store_true",
                    help="also time the steps replayed from CUDA graphs (config.graph_replay_ms_per_step)")
    ap.add_argument("--pair-tiles", default=None, choices=["tc2", "tc2-fc1", "tc2-fc2"],
                    help="large batches: run both / FC1 / FC2 on CTA pairs (cta_group::2) instead of one-CTA tiles")
    ap.add_argument("--experts", type=int, default=E,
                    help="routed experts in the layer (256 = GLM-5.2; smaller values give a profiler-sized case)")
    args = ap.parse_args()
    E = args.experts
    ROUTER_BYTES = E * H * 4
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
