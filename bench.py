"""Benchmark of the routed-MoE expert path: MoE-layer tokens/s on 1..8 B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T] [--impl reference]
                    [--layers L] [--zipf S] [--no-extras]

One "step" is one forward pass of one GLM-5.2-shaped routed-MoE layer (hidden 6144, 256
experts, top-8, expert intermediate 2048, NVFP4 weights, uniform router) over one batch of
T synthetic bf16 N(0,1) rows (default T = 64, the decode-shaped configuration).  Prints ONE
JSON line (rank 0).  Keys beyond the usual ones:

  value     whole-job tokens/s with inputs resident in device memory: blocks of K steps between
            two CUDA events on the launching stream, repeated until at least 0.3 s have been
            timed; the median block counts (max over ranks for N > 1).
  e2e       the same through the host-buffer entry point: pinned HOST buffers in and out,
            host<->device copies inside the timed region.
  roofline  dominant kernel (FC1 expert GEMM): algorithmic bytes per launch / its mean duration
            from CUDA events recorded around it on the launching stream during K further steps.
  cpu_baseline  the CPU oracle (numpy port of the reference's python/reference path) timed on
            this host on a bounded sample of the same workload.
  config.prefill_T8192   the other half of the headline metric, measured in the same run on a
            second lane of the same weights: ms/step, tokens/s, FC1/FC2 TFLOP/s, fraction of FP4 peak.
  config.ep_parity       N > 1: one step's rows gathered on rank 0 and compared with the same batch
            run by a single-GPU layer there ("bit-equal", or the largest per-token relative L2).
  config.stack           N > 1: the expert-parallel decode stack of the reference model: up to 75
            sparse layers with independent weights on one workspace, run back to back.
  config.zipf            N > 1: load-skewed routing sweep (popularity ~ rank^-1.2), T = 1 .. 16384.

--layers L makes the stack the measured workload, --zipf S the sweep.  With --impl reference only
the CPU port runs (no kernel of this repository is used).
"""
from __future__ import annotations

import os
import sys

if "--impl" in sys.argv and "reference" in sys.argv:
    # The CPU arm uses every host core; a launcher's OMP_NUM_THREADS=1 must not reach the BLAS.
    for _v in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[_v] = str(os.cpu_count() or 1)

import argparse
import json
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
NOMINAL_FP4_TFLOPS = 9000.0
MIN_TIMED_S = 0.3


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def layer_algorithmic_bytes(tokens: int, distinct: float) -> float:
    """Bytes one forward must move: weights of the experts actually selected, activations in and
    out, the float32 router weight and the route table."""
    return distinct * EXPERT_BYTES + tokens * (2 * H * 2) + ROUTER_BYTES + tokens * K_TOP * 8


def zipf_bias(router_w: np.ndarray, hidden_rows_f32: np.ndarray, s: float = 1.2, top_k: int = K_TOP,
              iters: int = 200) -> np.ndarray:
    """Router bias under which expert popularity follows rank^-s on rows like `hidden_rows_f32`:
    expert r is to receive a share proportional to (r + 1)^-s of the routes (an expert can take
    a row at most once, so the hottest experts saturate at "every row").  Expert id = popularity
    rank, so e % N spreads the hot experts round-robin over N shards.  Damped fixed-point
    iteration on the selection scores sigmoid(logit) + bias."""
    x = hidden_rows_f32.astype(np.float64)
    score = 1.0 / (1.0 + np.exp(-(x @ router_w.astype(np.float64).T)))
    n = router_w.shape[0]
    target = np.arange(1, n + 1, dtype=np.float64) ** -s
    target = np.minimum(target / target.sum() * top_k, 0.98)
    bias = np.zeros(n)
    for it in range(iters):
        top = np.argpartition(-(score + bias), top_k, axis=1)[:, :top_k]
        share = np.bincount(top.reshape(-1), minlength=n) / x.shape[0]
        eta = 0.03 / (1 + it / 50)
        bias += eta * np.clip(np.log(target + 1e-3) - np.log(share + 1e-3), -2, 2)
        bias -= bias.mean()
    return bias.astype(np.float32)


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
        busy = [m for m, u in self.samples if u > 0] or mhz
        return {"sm_mhz": float(np.median(busy)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(mhz), "samples_under_load": len(busy) if busy is not mhz else 0}


def descriptive_config(tokens: int, world: int) -> dict:
    """The keys both arms (this library and the CPU reference) emit: what was run, not what was measured."""
    return {"workload": f"glm52_moe_layer_{'prefill' if tokens > 256 else 'decode'}_T{tokens}", "tokens": tokens,
            "hidden": H, "experts": E, "top_k": K_TOP, "intermediate": I, "experts_per_gpu": E // max(1, world),
            "router": "uniform (bias 0)", "weights": "NVFP4, seeded synthetic N(0, 0.02)",
            "parity_mode": "O1 (hidden rows and the SwiGLU intermediate pass through the NVFP4 activation "
                           "quantiser, as on the reference's NVFP4 wire)"}


# ------------------------------------------------------------------------------------------
# CPU arm: the oracle port of python/reference (router + moe_forward) on host cores
# ------------------------------------------------------------------------------------------
def cpu_port_run(tokens_total: int, sample_tokens: int, steps: int, warmup: int):
    """Times the numpy port on `sample_tokens` rows of the workload.  Weights of the touched
    experts are drawn, quantised to NVFP4 and pre-dequantised before timing, as the reference's
    baseline plan does; the timed step is router + per-route expert FFNs + combine."""
    from oracle import glmrt_oracle as O
    cores = os.cpu_count() or 1
    limiter = None
    try:
        from threadpoolctl import threadpool_limits
        limiter = threadpool_limits(limits=cores)
    except Exception:
        pass
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
    threads = cores
    try:
        from threadpoolctl import threadpool_info
        threads = max([p.get("num_threads", 1) for p in threadpool_info()] + [1])
    except Exception:
        pass
    del limiter
    return {"tokens_per_s": sample_tokens / dt, "ms_per_step": dt * 1e3, "cores": int(threads),
            "sample": f"{sample_tokens} of {tokens_total} rows ({len(cache)} experts touched), weights "
                      f"pre-dequantised ({prep_s:.1f} s, untimed), {steps} timed steps",
            "prep_s": prep_s}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 500))
    warmup = max(0, min(args.warmup, 50))
    r = cpu_port_run(args.tokens, min(args.tokens, 2), steps, warmup)
    line = {
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": r["tokens_per_s"], "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
        "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "nvfp4", "data": "synthetic",
        "config": descriptive_config(args.tokens, args.gpus),
        "cpu_baseline": {"value": r["tokens_per_s"], "unit": "tokens/s", "cores": r["cores"], "kind": "port",
                         "sample": r["sample"]},
        "e2e": {"value": r["tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm: timing helpers
# ------------------------------------------------------------------------------------------
class Timer:
    """Blocks of `steps` calls between two CUDA events on the current stream; blocks repeat until
    MIN_TIMED_S have been timed (at least 3, at most 200 blocks).  With a process group the block
    time is the max over ranks and every rank runs the same number of blocks."""

    def __init__(self, torch, dist=None):
        self.torch, self.dist = torch, dist

    def block(self, fn, steps):
        torch, dist = self.torch, self.dist
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        ev0.record()
        for i in range(steps):
            fn(i)
        ev1.record()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1)
        if dist is not None:
            dist.barrier()
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def run(self, fn, steps, min_s=MIN_TIMED_S):
        blocks = [self.block(fn, steps)]
        while (sum(blocks) < min_s * 1e3 or len(blocks) < 3) and len(blocks) < 200:
            blocks.append(self.block(fn, steps))
        per_step = sorted(b / steps for b in blocks)
        return {"ms_per_step": per_step[len(per_step) // 2], "min_ms_per_step": per_step[0],
                "blocks": len(blocks), "timed_s": sum(blocks) * 1e-3}


def profile_stages(layer, fwd, steps):
    """Mean device time of each stage over `steps` profiled forwards, and mean distinct experts."""
    layer.set_profiling(True)
    stage_sum, distinct_sum = {}, 0
    for i in range(steps):
        fwd(i)
        for k, v in layer.stage_times_ms().items():
            stage_sum[k] = stage_sum.get(k, 0.0) + v
        distinct_sum += layer.stats().distinct_experts
    layer.set_profiling(False)
    return {k: v / steps for k, v in stage_sum.items()}, distinct_sum / steps


def prefill_numbers(T, world, ms_per_step, stage_ms, distinct):
    """Throughput figures of a prefill-sized step: the contraction is what one pays for."""
    hbm, bf16, kind = measured_peaks()
    routes_here = T * K_TOP / world
    fc1_flops = routes_here * 2.0 * (2 * I) * H
    fc2_flops = routes_here * 2.0 * H * I
    fc1_tf = fc1_flops / (stage_ms["fc1"] * 1e-3) / 1e12
    fc2_tf = fc2_flops / (stage_ms["fc2"] * 1e-3) / 1e12
    gemm_tf = (fc1_flops + fc2_flops) / ((stage_ms["fc1"] + stage_ms["fc2"]) * 1e-3) / 1e12
    layer_flops = T * K_TOP * 2.0 * 3 * I * H + T * 2.0 * E * H
    return {"tokens": T, "ms_per_step": ms_per_step, "tokens_per_s": T / (ms_per_step * 1e-3),
            "stage_ms_rank0": stage_ms, "fc1_tflops_per_gpu": fc1_tf, "fc2_tflops_per_gpu": fc2_tf,
            "gemm_tflops_per_gpu": gemm_tf, "fc1_frac_of_nominal_fp4": fc1_tf / NOMINAL_FP4_TFLOPS,
            "fc2_frac_of_nominal_fp4": fc2_tf / NOMINAL_FP4_TFLOPS,
            "gemm_frac_of_nominal_fp4": gemm_tf / NOMINAL_FP4_TFLOPS,
            "layer_tflops_aggregate": layer_flops / (ms_per_step * 1e-3) / 1e12,
            "layer_frac_of_nominal_fp4_aggregate": layer_flops / (ms_per_step * 1e-3) / 1e12 / (NOMINAL_FP4_TFLOPS * world),
            "fc1_frac_of_4x_measured_bf16": fc1_tf / (4.0 * bf16), "peak_source": kind,
            "fc1_weight_stream_gbs": distinct * FC1_EXPERT_BYTES / (stage_ms["fc1"] * 1e-3) / 1e9,
            "distinct_experts_rank0": distinct}


def make_batches(torch, T, n, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed + 1000)
    return [torch.randn(T, H, generator=g).to(torch.bfloat16) for _ in range(n)]


def router_weight(torch, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(E, H, generator=g) * 0.02


# ------------------------------------------------------------------------------------------
# GPU arm, one GPU
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
    timer = Timer(torch)
    if args.layers:
        return run_stack_single(args, torch, MoeLayer, sampler, timer)
    layer = MoeLayer(H, I, E, K_TOP, max_tokens=T, engine=args.pair_tiles or "tc")
    layer.fill_synthetic(0, 0.02)
    layer.set_router(router_weight(torch), torch.zeros(E))
    if args.zipf:
        return run_zipf(args, torch, None, 0, 1, layer, sampler, timer)
    # a few distinct input batches so that consecutive steps select different experts
    n_batches = 4
    host_batches = [b.pin_memory() for b in make_batches(torch, T, n_batches)]
    dev_batches = [b.cuda() for b in host_batches]
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    host_out = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()

    def fwd(i):
        layer.forward(dev_batches[i % n_batches], out)

    for i in range(warmup):
        fwd(i)
    layer.check()
    st0 = layer.stats()
    fwd(0)
    launches_per_step = int(layer.stats().launches_total - st0.launches_total)

    # ---- device-resident timing ----
    res = timer.run(fwd, steps)
    ms_per_step = res["ms_per_step"]

    # ---- the same steps replayed from CUDA graphs (reported beside the stream-ordered figure) ----
    graph_ms = None
    if args.graph:
        graph_ms = graph_replay_ms(torch, timer, layer, dev_batches, out, steps, warmup)

    # ---- per-kernel timing (events around each kernel on the launching stream) ----
    stage_ms, distinct = profile_stages(layer, fwd, steps)
    routes = T * K_TOP
    fc1_bytes = distinct * FC1_EXPERT_BYTES + routes * (H // 2 + H // 16) + routes * (I // 2 + I // 16)
    peak, bf16_peak, peak_kind = measured_peaks()
    fc1_gbs = fc1_bytes / (stage_ms["fc1"] * 1e-3) / 1e9
    layer_bytes = layer_algorithmic_bytes(T, distinct)

    # ---- end to end through the host-buffer entry point ----
    def fwd_host(i):
        layer.forward_host(host_batches[i % n_batches], host_out)

    for i in range(2):
        fwd_host(i)
    e2e = timer.run(fwd_host, steps)
    layer.check()

    prefill = T > 256          # the layer switches to its tokens-on-the-MMA-rows kernels above 256 rows
    extras = {}
    if not args.no_extras and not prefill:
        extras["prefill_T8192"] = prefill_block_single(torch, timer, layer, 8192, steps, warmup)
        extras["decode_small"] = {f"T{t}": small_decode_block(torch, timer, layer, t, steps, warmup) for t in (1, 8)}
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

    if not prefill:
        roofline = {"bound": "hbm", "kernel": "expert_gemm_kernel<FC1>", "achieved": fc1_gbs, "peak": peak,
                    "unit": "GB/s", "frac": fc1_gbs / peak, "peak_source": peak_kind,
                    "algorithmic_bytes_per_launch": fc1_bytes, "ms_per_launch": stage_ms["fc1"],
                    "traffic": NCU_FC1_TRAFFIC_PER_EXPERT * distinct,
                    "traffic_source": "ncu dram read+write of one FC1 launch on a 64-expert T=16 case "
                                      "(profiles/expert_gemm_fc1_fc2_E64_T16_ncu_full.md), per expert touched, "
                                      "times the experts touched here",
                    "note": "the weights of this kernel's first 48 (work item, 128-row tile) pairs, 38 MB of its "
                            "3.1 GB, are asked into the L2 by extra CTAs of the dispatch kernel before it starts "
                            "(GLMRT_B200_PREFETCH_FC1=0 turns that off); the ncu capture predates that prefetch"}
    else:
        # prefill: the contraction is what one pays for; FP4 runs at four times the bf16 rate and the
        # measured peaks hold a bf16 figure only, so the peak is 4 x the measured bf16 burst figure
        fc1_flops = routes * 2.0 * (2 * I) * H
        tf = fc1_flops / (stage_ms["fc1"] * 1e-3) / 1e12
        roofline = {"bound": "tensor", "kernel": "expert_gemm_tokens_kernel<FC1>", "achieved": tf,
                    "peak": 4.0 * bf16_peak, "unit": "TFLOP/s", "frac": tf / (4.0 * bf16_peak),
                    "peak_source": f"4 x bf16 burst ({peak_kind}); nominal dense FP4 is 9000",
                    "frac_of_nominal_fp4": tf / NOMINAL_FP4_TFLOPS,
                    "algorithmic_flops_per_launch": fc1_flops, "ms_per_launch": stage_ms["fc1"],
                    "hbm_gbs": fc1_gbs, "hbm_frac": fc1_gbs / peak,
                    "traffic": NCU_FC1_PREFILL_TRAFFIC_PER_EXPERT * distinct,
                    "traffic_source": "ncu dram read+write of one FC1 launch on a 64-expert T=2048 case "
                                      "(profiles/expert_gemm_tokens_fc1_fc2_E64_T2048_ncu_full.md), per expert "
                                      "touched (weights dominate), times the experts touched here"}
        extras["prefill"] = prefill_numbers(T, 1, ms_per_step, stage_ms, distinct)

    config = descriptive_config(T, 1)
    config.update({
        "l2": f"no flush: each step streams {layer_bytes / 1e9:.2f} GB of expert weights, far above the 126 MB L2",
        "timing": f"median of {res['blocks']} blocks of {steps} steps ({res['timed_s']:.2f} s timed)",
        "min_block_ms_per_step": res["min_ms_per_step"],
        "distinct_experts_per_step": distinct, "stage_ms": stage_ms,
        "graph_replay_ms_per_step": graph_ms,
        "layer_hbm_gbs": layer_bytes / (ms_per_step * 1e-3) / 1e9,
        "layer_frac_of_peak": layer_bytes / (ms_per_step * 1e-3) / 1e9 / peak})
    config.update(extras)
    line = {
        "metric": "moe_layer_tokens_per_s", "value": T / (ms_per_step * 1e-3), "unit": "tokens/s", "n_gpus": 1,
        "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4", "data": "synthetic",
        "config": config,
        "clocks": sampler.summary(),
        "e2e": {"value": T / (e2e["ms_per_step"] * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": T * H * 2,
                "d2h_bytes_per_step": T * H * 2, "ms_per_step": e2e["ms_per_step"]},
        "gpu_launches": launches_per_step * steps * res["blocks"],
        "gpu_launches_per_step": launches_per_step,
        "roofline": roofline,
        "cpu_baseline": cpu,
    }
    print(json.dumps(line), flush=True)


def graph_replay_ms(torch, timer, layer, dev_batches, out, steps, warmup):
    graphs = []
    for b in dev_batches:
        gph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gph):
            layer.forward(b, out)
        graphs.append(gph)
    for i in range(warmup):
        graphs[i % len(graphs)].replay()
    r = timer.run(lambda i: graphs[i % len(graphs)].replay(), steps)
    layer.check()
    return r["ms_per_step"]


def prefill_block_single(torch, timer, layer, T, steps, warmup):
    """T = 8192 on a second lane of the same weights (a workspace sized for 8192 rows)."""
    lane = layer.create_lane(T)
    batches = [b.cuda() for b in make_batches(torch, T, 2, seed=7)]
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")

    def fwd(i):
        lane.forward(batches[i % 2], out)

    for i in range(warmup):
        fwd(i)
    lane.check()
    res = timer.run(fwd, steps)
    stage_ms, distinct = profile_stages(lane, fwd, min(steps, 20))
    lane.check()
    chunks = int(lane.stats().chunks)
    block = prefill_numbers(T, 1, res["ms_per_step"], stage_ms, distinct)
    block["timing"] = f"median of {res['blocks']} blocks of {steps} steps ({res['timed_s']:.2f} s timed)"
    block["operand_delivery"] = operand_delivery(lane.lib, torch, chunks, stage_ms)
    lane.close()
    del batches, out
    torch.cuda.empty_cache()
    return block


def operand_delivery(lib, torch, chunks, stage_ms):
    """What bounds the token-major expert GEMMs: every CTA must bring 54 KB (FC1: 128 token rows, 128 gate
    and 128 up rows of 128 bytes, three 2 KB scale groups) or 36 KB (FC2) into shared memory per
    256-element K stage.  Bytes delivered / kernel time, beside the rate a probe kernel that issues the
    same copies and consumes nothing reaches on this GPU with an L2-resident working set."""
    import ctypes as C
    gbs, ms = C.c_float(), C.c_float()
    lib.call("glmrt_b200_probe_operand_delivery", C.c_size_t(48 << 20), C.c_uint32(4), C.c_uint32(8),
             C.byref(gbs), C.byref(ms), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    fc1_bytes = chunks * (I // 128) * (H // 256) * 55296
    fc2_bytes = chunks * (H // 128) * (I // 256) * 36864
    fc1 = fc1_bytes / (stage_ms["fc1"] * 1e-3) / 1e9
    fc2 = fc2_bytes / (stage_ms["fc2"] * 1e-3) / 1e9
    return {"probe_l2_to_smem_gbs": float(gbs.value), "work_items_128_tokens": chunks,
            "fc1_bytes_into_smem": fc1_bytes, "fc1_gbs": fc1, "fc1_frac_of_probe": fc1 / float(gbs.value),
            "fc2_bytes_into_smem": fc2_bytes, "fc2_gbs": fc2, "fc2_frac_of_probe": fc2 / float(gbs.value),
            "note": "the probe runs with the tensor pipe idle and the SM clock at its maximum; under the power cap of a "
                    "GEMM the same per-clock rate delivers proportionally less"}


def small_decode_block(torch, timer, layer, T, steps, warmup):
    """Latency of a very small decode batch (the reference's main production case is M = 1),
    stream-ordered and replayed from CUDA graphs; 8 input batches and the weights they select
    rotate, so no step finds its experts in L2."""
    batches = [b.cuda() for b in make_batches(torch, T, 8, seed=11)]
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")

    def fwd(i):
        layer.forward(batches[i % 8], out)

    for i in range(warmup):
        fwd(i)
    res = timer.run(fwd, steps, min_s=0.1)
    stage_ms, distinct = profile_stages(layer, fwd, min(steps, 20))
    g_ms = graph_replay_ms(torch, timer, layer, batches, out, steps, warmup)
    peak, _, _ = measured_peaks()
    lb = layer_algorithmic_bytes(T, distinct)
    return {"ms_per_step": res["ms_per_step"], "graph_replay_ms_per_step": g_ms,
            "tokens_per_s": T / (res["ms_per_step"] * 1e-3), "distinct_experts": distinct, "stage_ms": stage_ms,
            "layer_frac_of_peak": lb / (res["ms_per_step"] * 1e-3) / 1e9 / peak,
            "layer_frac_of_peak_graph": lb / (g_ms * 1e-3) / 1e9 / peak}


# ------------------------------------------------------------------------------------------
# GPU arm, N > 1: expert parallelism
# ------------------------------------------------------------------------------------------
def ep_parity(torch, dist, EP, MoeLayer, layer, rank, world, T, seed=123):
    """One step's rows gathered on rank 0 and compared with a single-GPU layer holding all experts
    (same seeded weights and router) on the same batch."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    r0, rn = EP.partition_rows(T, world, rank)
    mine = x[r0:r0 + rn].contiguous().cuda()
    out = torch.zeros_like(mine)
    EP.forward_ep(layer, mine, out)
    layer.check()
    torch.cuda.synchronize()
    parts = [None] * world
    dist.all_gather_object(parts, out.cpu().view(torch.int16).numpy())
    verdict = None
    if rank == 0:
        from oracle import glmrt_oracle as O   # checker only: per-token relative L2 of two bf16 arrays
        single = MoeLayer(H, I, E, K_TOP, max_tokens=T, engine="tc-ordered")   # one row per route, summed in order, like the exchange
        single.fill_synthetic(0, 0.02)
        single.set_router(router_weight(torch), torch.zeros(E))
        ref = single.forward(x.cuda()).cpu().view(torch.int16).numpy()
        single.check()
        single.close()
        del single
        torch.cuda.empty_cache()
        got = np.concatenate([p for p in parts if p.shape[0] > 0], axis=0)
        if np.array_equal(got, ref):
            verdict = "bit-equal"
        else:
            err = O.rel_l2_per_token(got.view(np.uint16), ref.view(np.uint16))
            verdict = {"max_rel_l2": float(err.max()), "rows_differing": int((got != ref).any(axis=1).sum()),
                       "rows": int(T)}
    box = [verdict]
    dist.broadcast_object_list(box, src=0)
    return box[0]


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
    timer = Timer(torch, dist)
    if args.layers:
        return run_stack_ep(args, torch, dist, EP, MoeLayer, rank, world, sampler, timer, as_block=False)
    layer = MoeLayer(H, I, E, K_TOP, max_tokens=T, ep_world=world, ep_rank=rank)
    layer.fill_synthetic(0, 0.02)
    layer.set_router(router_weight(torch), torch.zeros(E))
    EP.attach_distributed(layer, dist)
    EP.set_global_rows(layer, T)
    if args.zipf:
        return run_zipf(args, torch, dist, rank, world, layer, sampler, timer)
    r0, rn = EP.partition_rows(T, world, rank)
    n_batches = 4
    host_batches = [b[r0:r0 + rn].contiguous().pin_memory() for b in make_batches(torch, T, n_batches)]
    dev_batches = [b.cuda() for b in host_batches]
    out = torch.empty(rn, H, dtype=torch.bfloat16, device="cuda")
    host_out = torch.empty(rn, H, dtype=torch.bfloat16).pin_memory()

    parity = ep_parity(torch, dist, EP, MoeLayer, layer, rank, world, T)
    parity_ok = parity == "bit-equal" or (isinstance(parity, dict) and parity["max_rel_l2"] <= 2e-2 and T > 64)

    def fwd(i):
        EP.forward_ep(layer, dev_batches[i % n_batches], out)

    for i in range(warmup):
        fwd(i)
    layer.check()
    st0 = layer.stats()
    fwd(0)
    launches_per_step = int(layer.stats().launches_total - st0.launches_total)
    res = timer.run(fwd, steps)
    ms_per_step = res["ms_per_step"]
    stage_ms, distinct = profile_stages(layer, fwd, steps)
    routes_owned = T * K_TOP / world
    fc1_bytes = distinct * FC1_EXPERT_BYTES + routes_owned * ((H // 2 + H // 16) + (I // 2 + I // 16))
    peak, _, peak_kind = measured_peaks()
    fc1_gbs = fc1_bytes / (stage_ms["fc1"] * 1e-3) / 1e9

    def fwd_host(i):
        EP.forward_ep_host(layer, host_batches[i % n_batches], host_out)

    e2e = timer.run(fwd_host, steps)
    layer.check()

    extras = {}
    if not args.no_extras and T <= 256:
        extras["prefill_T8192"] = prefill_block_ep(torch, dist, EP, MoeLayer, timer, layer, rank, world, 8192, steps, warmup)
        extras["zipf"] = zipf_sweep(torch, dist, EP, layer, rank, world, timer, 1.2, max_T=args.zipf_max_tokens,
                                    steps=min(steps, 20))
        layer.close()
        del layer
        torch.cuda.empty_cache()
        layer = None
        extras["stack"] = run_stack_ep(args, torch, dist, EP, MoeLayer, rank, world, sampler, timer, as_block=True)
    sampler.stop()
    sampler.join(timeout=2)
    gathered = [None] * world
    dist.all_gather_object(gathered, {"distinct": distinct, "fc1_ms": stage_ms["fc1"], "fc2_ms": stage_ms["fc2"],
                                      "clocks": sampler.summary()})
    if rank == 0:
        total_distinct = sum(x["distinct"] for x in gathered)
        layer_bytes = layer_algorithmic_bytes(T, total_distinct)
        config = descriptive_config(T, world)
        config.update({
            "parallelism": f"ep{world}: expert e on rank e % {world}, rows block-partitioned, "
                           "dispatch/combine = in-kernel NVLink peer stores",
            "ep_parity": parity,
            "l2": f"no flush: each step streams {layer_bytes / 1e9:.2f} GB of expert weights over "
                  f"{world} GPUs, far above the 126 MB L2",
            "timing": f"median of {res['blocks']} blocks of {steps} steps ({res['timed_s']:.2f} s timed), max over ranks",
            "min_block_ms_per_step": res["min_ms_per_step"],
            "distinct_experts_per_step": total_distinct, "stage_ms_rank0": stage_ms,
            "max_over_ranks_imbalance": max(x["distinct"] for x in gathered) / max(1e-9, total_distinct / world),
            "layer_hbm_gbs_aggregate": layer_bytes / (ms_per_step * 1e-3) / 1e9,
            "layer_frac_of_aggregate_peak": layer_bytes / (ms_per_step * 1e-3) / 1e9 / (peak * world)})
        if T > 256:
            extras["prefill"] = prefill_numbers(T, world, ms_per_step, stage_ms, distinct)
        config.update(extras)
        line = {
            "metric": "moe_layer_tokens_per_s", "value": T / (ms_per_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4",
            "data": "synthetic",
            "config": config,
            "clocks": gathered[0]["clocks"],
            "clocks_all_ranks": [x["clocks"] for x in gathered],
            "e2e": {"value": T / (e2e["ms_per_step"] * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": T * H * 2,
                    "d2h_bytes_per_step": T * H * 2, "ms_per_step": e2e["ms_per_step"]},
            "gpu_launches": launches_per_step * steps * res["blocks"] * world,
            "gpu_launches_per_step_per_rank": launches_per_step,
            "roofline": {"bound": "hbm", "kernel": "expert_gemm_kernel<FC1> (rank 0)", "achieved": fc1_gbs,
                         "peak": peak, "unit": "GB/s", "frac": fc1_gbs / peak, "peak_source": peak_kind,
                         "algorithmic_bytes_per_launch": fc1_bytes, "ms_per_launch": stage_ms["fc1"],
                         "traffic": NCU_FC1_TRAFFIC_PER_EXPERT * distinct},
            "cpu_baseline": None,
        }
        print(json.dumps(line), flush=True)
    dist.barrier()
    if layer is not None:
        layer.close()
    dist.destroy_process_group()
    if not parity_ok:
        raise SystemExit(f"expert-parallel output differs from the single-GPU layer: {parity}")


def prefill_block_ep(torch, dist, EP, MoeLayer, timer, layer, rank, world, T, steps, warmup):
    """T = 8192 over the same shards: a second lane (workspace for T / N home rows) of the same weights."""
    r0, rn = EP.partition_rows(T, world, rank)
    cap = EP.partition_rows(T, world, 0)[1]
    lane = layer.create_lane(max(cap, 257))
    EP.attach_distributed(lane, dist)
    EP.set_global_rows(lane, T)
    batches = [b[r0:r0 + rn].contiguous().cuda() for b in make_batches(torch, T, 2, seed=7)]
    out = torch.empty(rn, H, dtype=torch.bfloat16, device="cuda")
    g = torch.Generator(device="cpu").manual_seed(123)
    parity = None
    if T * H * 2 <= (1 << 28):
        parity = ep_parity_lane(torch, dist, EP, MoeLayer, lane, rank, world, T)

    def fwd(i):
        EP.forward_ep(lane, batches[i % 2], out)

    for i in range(warmup):
        fwd(i)
    lane.check()
    res = timer.run(fwd, steps)
    stage_ms, distinct = profile_stages(lane, fwd, min(steps, 20))
    lane.check()
    block = prefill_numbers(T, world, res["ms_per_step"], stage_ms, distinct)
    block["ep_parity"] = parity
    block["timing"] = f"median of {res['blocks']} blocks of {steps} steps ({res['timed_s']:.2f} s timed), max over ranks"
    dist.barrier()
    lane.close()
    del batches, out, g
    torch.cuda.empty_cache()
    return block


def ep_parity_lane(torch, dist, EP, MoeLayer, lane, rank, world, T):
    return ep_parity(torch, dist, EP, MoeLayer, lane, rank, world, T, seed=321)


# ------------------------------------------------------------------------------------------
# The decode stack: L sparse layers with independent weights, one workspace, run back to back
# ------------------------------------------------------------------------------------------
def stack_layers_that_fit(torch, world, want):
    """How many layers' expert shards fit beside a workspace, leaving a margin, on this GPU."""
    free, total = torch.cuda.mem_get_info()
    per_layer = E // world * EXPERT_BYTES + 3 * E * H * 4 + (64 << 20)
    return int(max(1, min(want, (free - (12 << 30)) // per_layer)))


def build_stack(torch, MoeLayer, T_cap, world, rank, n_layers):
    base = MoeLayer(H, I, E, K_TOP, max_tokens=T_cap, ep_world=world, ep_rank=rank)
    stack = [base]
    for _ in range(1, n_layers):
        stack.append(base.create_stacked())
    for li, l in enumerate(stack):
        l.fill_synthetic(li, 0.02)                      # independent seeded weights: seed = layer index
        l.set_router(router_weight(torch, seed=li), torch.zeros(E))
    return stack


def stack_step_fn(forward_one, stack, x, bufs):
    """One step = the layers in order, each reading the previous layer's output."""
    def step(_i=0):
        src = x
        for li, l in enumerate(stack):
            dst = bufs[li % 2]
            forward_one(l, src, dst)
            src = dst
        return src
    return step


def chain_is_healthy(torch, dist, last):
    """Chaining output -> input is only a fair workload if the rows keep a sane scale."""
    rms = torch.tensor([float(last.float().pow(2).mean().sqrt().item()) if last.numel() else 1.0], device="cuda")
    if dist is not None:
        dist.all_reduce(rms, op=dist.ReduceOp.MIN)
    v = float(rms.item())
    return bool(np.isfinite(v) and 1e-3 < v < 1e3), v


def stack_result(T, world, n_layers, want, res, e2e_ms, chained, rms, launches, stage0):
    floor_ms = n_layers * (222.4 * EXPERT_BYTES / world) / (measured_peaks()[0] * 1e9) * 1e3
    return {"layers": n_layers, "layers_wanted": want,
            "note": None if n_layers == want else f"{want} layers do not fit this GPU's memory at {world} GPUs "
                                                  f"({want * E // world * EXPERT_BYTES / 1e9:.0f} GB of weights per GPU); "
                                                  f"{n_layers} run",
            "tokens": T, "ms_per_step": res["ms_per_step"], "ms_per_layer": res["ms_per_step"] / n_layers,
            "tokens_per_s": T / (res["ms_per_step"] * 1e-3),
            "ms_per_step_75_layers": res["ms_per_step"] / n_layers * 75,
            "weight_stream_floor_ms": floor_ms, "frac_of_weight_stream_floor": floor_ms / res["ms_per_step"],
            "e2e_ms_per_step": e2e_ms, "input": "each layer reads the previous layer's output" if chained else
            "every layer reads the step's input rows (a chained pass lost its scale)",
            "output_rms_after_last_layer": rms, "launches_per_step_per_rank": launches,
            "layer0_stage_ms_rank0": stage0,
            "timing": f"median of {res['blocks']} blocks ({res['timed_s']:.2f} s timed), max over ranks"}


def run_stack_ep(args, torch, dist, EP, MoeLayer, rank, world, sampler, timer, as_block):
    T = args.tokens if args.tokens <= 256 else 64
    want = args.layers or 75
    n_layers = stack_layers_that_fit(torch, world, want)
    t = torch.tensor([n_layers], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    n_layers = int(t.item())
    cap = EP.partition_rows(T, world, 0)[1]
    stack = build_stack(torch, MoeLayer, max(cap, 1), world, rank, n_layers)
    EP.attach_distributed(stack[0], dist)       # the exchange buffers belong to the shared workspace
    EP.set_global_rows(stack[0], T)
    r0, rn = EP.partition_rows(T, world, rank)
    host_x = make_batches(torch, T, 1, seed=5)[0][r0:r0 + rn].contiguous().pin_memory()
    x = host_x.cuda()
    bufs = [torch.empty(rn, H, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    host_out = torch.empty(rn, H, dtype=torch.bfloat16).pin_memory()
    step = stack_step_fn(lambda l, s, d: EP.forward_ep(l, s, d), stack, x, bufs)
    last = step()
    stack[0].check()
    chained, rms = chain_is_healthy(torch, dist, last)
    if not chained:
        def step(_i=0):
            for li, l in enumerate(stack):
                EP.forward_ep(l, x, bufs[li % 2])
            return bufs[(len(stack) - 1) % 2]
    steps = max(3, min(args.steps, 20))
    for i in range(3):
        step()
    stack[0].check()
    st0 = stack[0].stats()
    step()
    launches = int(stack[0].stats().launches_total - st0.launches_total)
    res = timer.run(step, steps)

    def step_host(_i=0):
        x.copy_(host_x, non_blocking=True)
        y = step()
        host_out.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e = timer.run(step_host, steps)
    stage0, _ = profile_stages(stack[0], lambda i: step(), 3)
    stack[0].check()
    block = stack_result(T, world, n_layers, want, res, e2e["ms_per_step"], chained, rms, launches, stage0)
    dist.barrier()
    for l in reversed(stack):
        l.close()
    torch.cuda.empty_cache()
    if as_block:
        return block
    sampler.stop()
    sampler.join(timeout=2)
    if rank == 0:
        config = descriptive_config(T, world)
        config["workload"] = f"glm52_moe_decode_stack_{n_layers}_layers_T{T}"
        config["parallelism"] = f"ep{world}: expert e on rank e % {world}"
        config["stack"] = block
        line = {"metric": "moe_stack_tokens_per_s", "value": block["tokens_per_s"], "unit": "tokens/s",
                "n_gpus": world, "steps": steps, "warmup": 3, "ms_per_step": block["ms_per_step"],
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4",
                "data": "synthetic", "config": config, "clocks": sampler.summary(),
                "e2e": {"value": T / (e2e["ms_per_step"] * 1e-3), "unit": "tokens/s",
                        "h2d_bytes_per_step": T * H * 2, "d2h_bytes_per_step": T * H * 2,
                        "ms_per_step": e2e["ms_per_step"]},
                "gpu_launches": launches * steps * res["blocks"] * world, "cpu_baseline": None}
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def run_stack_single(args, torch, MoeLayer, sampler, timer):
    """--layers L on one GPU: as many of the L layers as fit (all 256 experts each are local)."""
    T = args.tokens if args.tokens <= 256 else 64
    want = args.layers
    n_layers = stack_layers_that_fit(torch, 1, want)
    stack = build_stack(torch, MoeLayer, T, 1, 0, n_layers)
    host_x = make_batches(torch, T, 1, seed=5)[0].pin_memory()
    x = host_x.cuda()
    bufs = [torch.empty(T, H, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    host_out = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()
    step = stack_step_fn(lambda l, s, d: l.forward(s, d), stack, x, bufs)
    last = step()
    stack[0].check()
    chained, rms = chain_is_healthy(torch, None, last)
    if not chained:
        def step(_i=0):
            for li, l in enumerate(stack):
                l.forward(x, bufs[li % 2])
            return bufs[(len(stack) - 1) % 2]
    steps = max(3, min(args.steps, 20))
    for i in range(3):
        step()
    st0 = stack[0].stats()
    step()
    launches = int(stack[0].stats().launches_total - st0.launches_total)
    res = timer.run(step, steps)

    def step_host(_i=0):
        x.copy_(host_x, non_blocking=True)
        y = step()
        host_out.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e = timer.run(step_host, steps)
    stage0, _ = profile_stages(stack[0], lambda i: step(), 3)
    block = stack_result(T, 1, n_layers, want, res, e2e["ms_per_step"], chained, rms, launches, stage0)
    sampler.stop()
    sampler.join(timeout=2)
    config = descriptive_config(T, 1)
    config["workload"] = f"glm52_moe_decode_stack_{n_layers}_layers_T{T}"
    config["stack"] = block
    line = {"metric": "moe_stack_tokens_per_s", "value": block["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
            "steps": steps, "warmup": 3, "ms_per_step": block["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4", "data": "synthetic", "config": config,
            "clocks": sampler.summary(),
            "e2e": {"value": T / (e2e["ms_per_step"] * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": T * H * 2,
                    "d2h_bytes_per_step": T * H * 2, "ms_per_step": e2e["ms_per_step"]},
            "gpu_launches": launches * steps * res["blocks"], "cpu_baseline": None}
    print(json.dumps(line), flush=True)
    for l in reversed(stack):
        l.close()


# ------------------------------------------------------------------------------------------
# Load-skewed routing sweep (expert popularity ~ rank^-s)
# ------------------------------------------------------------------------------------------
def zipf_sweep(torch, dist, EP, layer, rank, world, timer, s, max_T, steps):
    """T = 1 .. max_T in powers of two plus the speculative-verify batch T = 16 = 4 x (1 + 3 drafts),
    on a lane sized for the largest T; router bias calibrated so that popularity follows rank^-s.
    Reports tokens/s, the routes the busiest rank received over the mean (max-over-ranks imbalance),
    and what the layer reported when the plan did not fit."""
    rw = router_weight(torch)
    cal = make_batches(torch, 1024, 1, seed=99)[0].float().numpy()
    bias = zipf_bias(rw.numpy(), cal, s)
    sizes = sorted({1 << i for i in range(0, 15) if (1 << i) <= max_T} | {16})
    cap = -(-max(sizes) // world)
    lane = layer.create_lane(max(cap, 1))
    lane.set_router(rw, torch.from_numpy(bias))       # the lane shares the weights: restore below
    if world > 1:
        EP.attach_distributed(lane, dist)
    rows_out = []
    for T in sizes:
        full = make_batches(torch, T, 2, seed=200 + T)
        if world > 1:
            r0, rn = EP.partition_rows(T, world, rank)
            EP.set_global_rows(lane, T)
        else:
            r0, rn = 0, T
        batches = [b[r0:r0 + rn].contiguous().cuda() for b in full]
        out = torch.empty(rn, H, dtype=torch.bfloat16, device="cuda")

        def fwd(i):
            if world > 1:
                EP.forward_ep(lane, batches[i % 2], out)
            else:
                lane.forward(batches[i % 2], out)

        entry = {"tokens": T}
        try:
            problem = ""
            try:
                for i in range(3):
                    fwd(i)
                lane.check()
            except Exception as ex:
                problem = str(ex)[:160]
            if dist is not None:   # all ranks take the same branch
                flag = torch.tensor([1.0 if problem else 0.0], device="cuda")
                dist.all_reduce(flag, op=dist.ReduceOp.MAX)
                if float(flag.item()) != 0.0 and not problem:
                    problem = "another rank reported an error"
            if problem:
                raise RuntimeError(problem)
            res = timer.run(fwd, steps, min_s=0.05)
            lane.check()
            routes_here = float(lane.debug("COUNTERS", np.uint32)[4])      # routes this rank's experts received
            if dist is not None:
                t = torch.tensor([routes_here, routes_here], device="cuda")
                mx = t.clone()
                dist.all_reduce(mx, op=dist.ReduceOp.MAX)
                dist.all_reduce(t, op=dist.ReduceOp.SUM)
                imb = float(mx[0].item()) / max(1e-9, float(t[0].item()) / world)
            else:
                imb = 1.0
            st = lane.stats()
            entry.update({"ms_per_step": res["ms_per_step"], "tokens_per_s": T / (res["ms_per_step"] * 1e-3),
                          "max_over_ranks_routes_imbalance": imb, "distinct_experts_rank0": int(st.distinct_experts),
                          "status": "ok"})
        except Exception as ex:   # a plan that does not fit is reported, never a hang
            entry.update({"status": f"refused: {str(ex)[:160]}"})
        rows_out.append(entry)
        del batches, out
    if dist is not None:
        dist.barrier()
    lane.set_router(rw, torch.zeros(E))
    lane.close()
    torch.cuda.empty_cache()
    counts_note = "expert id = popularity rank, so e % N spreads the hot experts round-robin over the ranks"
    return {"s": s, "calibration": "bias by damped fixed-point iteration on 1024 seeded rows; " + counts_note,
            "sweep": rows_out}


def run_zipf(args, torch, dist, rank, world, layer, sampler, timer):
    if world > 1:
        from glmrt_b200 import ep as EP
    else:
        EP = None
    block = zipf_sweep(torch, dist, EP, layer, rank, world, timer, args.zipf, args.zipf_max_tokens, min(args.steps, 20))
    sampler.stop()
    sampler.join(timeout=2)
    if rank == 0:
        head = [r for r in block["sweep"] if r["tokens"] == 64 and r["status"] == "ok"]
        head = head[0] if head else {"ms_per_step": None, "tokens_per_s": None}
        config = descriptive_config(64, world)
        config["workload"] = f"glm52_moe_layer_zipf_s{args.zipf}_sweep"
        config["router"] = f"bias calibrated for popularity ~ rank^-{args.zipf}"
        config["zipf"] = block
        line = {"metric": "moe_layer_tokens_per_s", "value": head["tokens_per_s"], "unit": "tokens/s",
                "n_gpus": world, "steps": min(args.steps, 20), "warmup": 3, "ms_per_step": head["ms_per_step"],
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4",
                "data": "synthetic", "config": config, "clocks": sampler.summary(), "cpu_baseline": None}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
    layer.close()
    if dist is not None:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one FC1 launch from the ncu captures summarised
# under profiles/, per expert touched: decode kernel (862.55 MB, 60 experts touched) and prefill
# kernel (998.81 MB, 64 experts).
NCU_FC1_TRAFFIC_PER_EXPERT = 862.55e6 / 60
NCU_FC1_PREFILL_TRAFFIC_PER_EXPERT = 998.81e6 / 64


def main():
    global E, ROUTER_BYTES
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="only the main workload: no prefill / small-decode / stack / skew blocks")
    ap.add_argument("--graph", action="store_true",
                    help="also time the steps replayed from CUDA graphs (config.graph_replay_ms_per_step)")
    ap.add_argument("--layers", type=int, default=0,
                    help="measure a stack of this many sparse layers (independent weights, one workspace) instead of one layer")
    ap.add_argument("--zipf", type=float, default=0.0,
                    help="measure the load-skewed routing sweep with this popularity exponent instead of the uniform router")
    ap.add_argument("--zipf-max-tokens", type=int, default=16384)
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
