#!/usr/bin/env python
"""Benchmark of the FP8 block-scale MoE layer (one "step" = one forward of the layer).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workloads (synthetic tensors with the benchmark definition's shapes and distributions):
  decode   T=64,   32 local of 256 experts, DeepSeek-V3 shape   (default at N=1; HBM-bound)
  prefill  T=4096, 32 local experts, 4 experts with ~4x the mean load
  t14107   T=14107, 32 local experts (the shape the reference quotes its best latency on)
  ep       T=8192 per step, 256 experts sharded over the N ranks  (default at N>1)
  qwen3    T=2048, 128 experts of the Qwen3-MoE shape sharded over the N ranks

Prints ONE JSON line on rank 0.  `value` is tokens/s with all inputs resident in HBM;
`e2e` is tokens/s through the public entry point with the step's inputs (logits, fp8 hidden
states, scales) copied from pinned host memory and the bf16 output copied back inside the
timed region (expert weights are model state and stay resident).  `--impl reference` times
the CPU port of the operator definition (oracle/) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from justgoal_b200 import inputs as I  # noqa: E402

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return json.load(open(p)), "measured"
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml as N
            N.nvmlInit()
            self.N = N
            self.h = N.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(N.nvmlDeviceGetMaxClockInfo(self.h, N.NVML_CLOCK_SM))
        except Exception:
            self.N = None

    def _loop(self):
        N = self.N
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20,
                 "hw_thermal_slowdown": 0x40, "hw_power_brake_slowdown": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(int(N.nvmlDeviceGetClockInfo(self.h, N.NVML_CLOCK_SM)))
                r = int(N.nvmlDeviceGetCurrentClocksEventReasons(self.h)) if hasattr(
                    N, "nvmlDeviceGetCurrentClocksEventReasons") else int(
                    N.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.004)

    def start(self):
        if self.N is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()

    def stop(self):
        self._stop.set()
        if self._thr is not None:
            self._thr.join()
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def workload_spec(name, n_gpus):
    if name == "decode":
        return dict(shape=I.DEEPSEEK_V3, T=64, boost=None, ep=False, rsf=2.5)
    if name == "prefill":
        return dict(shape=I.DEEPSEEK_V3, T=4096, boost=((0, 8, 16, 24), PREFILL_BIAS_BOOST), ep=False, rsf=2.5)
    if name == "t14107":      # the token count the reference quotes its best layer latency on (942 us)
        return dict(shape=I.DEEPSEEK_V3, T=14107, boost=None, ep=False, rsf=2.5)
    if name == "ep":
        return dict(shape=I.DEEPSEEK_V3.with_local(256 // n_gpus), T=8192, boost=None, ep=True, rsf=2.5)
    if name == "qwen3":
        return dict(shape=I.QWEN3_MOE.with_local(128 // n_gpus), T=2048, boost=None, ep=True, rsf=1.0)
    raise SystemExit(f"unknown workload {name}")


# bias added to local experts 0, 8, 16, 24 so that they receive ~4x the mean load of the 32
# local experts at T=4096 (calibrated once on the CPU, by bisection, with the seeded logits)
PREFILL_BIAS_BOOST = 0.328


def dist_setup(n_gpus):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if torch.cuda.is_available():
            torch.cuda.set_device(local)
        dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo",
                                device_id=torch.device("cuda", local) if torch.cuda.is_available() else None)
    return rank, world, local


def run_ours(args):
    rank, world, local = dist_setup(args.gpus)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py (impl ours) needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    name = args.workload or ("decode" if world == 1 else "ep")
    spec = workload_spec(name, world)
    if spec["ep"] and world > 1:
        from justgoal_b200 import ep
        return ep.bench(args, spec, name, rank, world, local)
    from justgoal_b200 import MoELayer
    shape, T = spec["shape"], spec["T"]
    layer = MoELayer(shape, dev)
    d = I.make_inputs(shape, T, seed=0, device=dev, routed_scaling_factor=spec["rsf"], bias_boost=spec["boost"])
    op = [d[k] for k in ("routing_logits", "routing_bias", "hidden_states", "hidden_states_scale",
                         "gemm1_weights", "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale",
                         "local_expert_offset", "routed_scaling_factor")]
    K, W = args.steps, max(args.warmup, 3)

    # ---- warm-up, realised routing
    for _ in range(W):
        out = layer.forward(*op)
    torch.cuda.synchronize()
    if layer.status(T) != 0:
        raise SystemExit(f"device error word {layer.status(T)}")
    st = layer.view(T, "status", torch.int32, (8,)).cpu().tolist()
    pairs, active = st[1], st[4]
    work = I.algorithmic_work(shape, T, pairs, active)

    # ---- timed region: K steps, inputs resident in HBM
    sampler = ClockSampler(local)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    sampler.start()
    e0.record()
    for _ in range(K):
        out = layer.forward(*op)
    e1.record()
    torch.cuda.synchronize()
    ms_total = e0.elapsed_time(e1)
    ms_step = ms_total / K

    # ---- the same K steps again with the library's per-stage CUDA events on the launch stream
    # (an event between two kernels removes their programmatic overlap, so the sum of the stages
    # is a little above ms_step; the stage durations feed the roofline of the dominant kernel)
    slots = min(K, 512)
    layer.profile_enable(slots)
    for _ in range(K):
        out = layer.forward(*op)
    torch.cuda.synchronize()
    clocks = sampler.stop()
    # median over the recorded steps: a stage's event pair also spans any host-side stall between
    # its two records, and one such outlier must not move the roofline figure
    per_slot = [layer.profile_read(s) for s in range(slots)]
    stage = {k: sorted(r[k] for r in per_slot)[slots // 2] for k in layer.STAGES}
    layer.profile_enable(0)
    if layer.status(T) != 0:
        raise SystemExit(f"device error word {layer.status(T)} after the timed steps")

    # ---- end to end: host inputs -> device, forward, output -> host, every step
    host_in = [d[k].cpu().pin_memory() for k in ("routing_logits", "hidden_states", "hidden_states_scale")]
    dev_in = [torch.empty_like(d[k]) for k in ("routing_logits", "hidden_states", "hidden_states_scale")]
    host_out = torch.empty(T, shape.hidden, dtype=torch.bfloat16).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = host_out.numel() * host_out.element_size()

    # the caller-facing loop for host-resident inputs: justgoal_b200.HostPipeline (copy in, forward, copy out
    # on three streams, two sets of device buffers).  Every step copies its inputs in and its output out.
    from justgoal_b200 import HostPipeline
    pipe = HostPipeline(layer, T, d["routing_bias"], *op[4:])
    del dev_in

    def e2e_step():
        pipe.step(host_in[0], host_in[1], host_in[2], host_out)

    for _ in range(W):
        e2e_step()
    pipe.drain()
    torch.cuda.synchronize()
    Ke = K
    t0 = time.perf_counter()
    for _ in range(Ke):
        e2e_step()
    pipe.drain()
    wall = time.perf_counter() - t0
    e2e_ms = wall * 1e3 / Ke            # host clock around K pipelined steps, drained on both sides
    assert torch.equal(host_out.view(torch.int16), out.cpu().view(torch.int16))

    # ---- roofline of the dominant kernel (GEMM1: two thirds of the weight bytes)
    peaks, which = measured_peaks()
    H, Iz = shape.hidden, shape.intermediate
    # algorithmic bytes of one GEMM1 launch: fp8 W13 + block scales of the active experts, and
    # the fp8 activations + scales of the routed rows (its outputs are intermediates: excluded)
    g1_bytes = active * 2 * Iz * H + active * (2 * Iz // 128) * (H // 128) * 4 \
        + pairs * H + pairs * (H // 128) * 4
    g1_flops = 4 * pairs * H * Iz
    t_g1 = stage["gemm1"] * 1e-3
    hbm_peak = float(peaks["hbm_gbs"])
    roof = {"kernel": "gemm_kernel<NTOK,G1> (GEMM1 + SwiGLU + requant)", "bound": "hbm",
            "achieved": g1_bytes / t_g1 / 1e9, "peak": hbm_peak, "unit": "GB/s",
            "frac": g1_bytes / t_g1 / 1e9 / hbm_peak, "peak_source": which,
            "traffic": NCU_TRAFFIC.get(name), "bytes_per_launch": g1_bytes, "ms_per_launch": stage["gemm1"],
            "tflops": g1_flops / t_g1 / 1e12}
    layer_roof = {"bytes": work["bytes"], "flops": work["flops"],
                  "hbm_gbs": work["bytes"] / (ms_step * 1e-3) / 1e9,
                  "frac_of_hbm": work["bytes"] / (ms_step * 1e-3) / 1e9 / hbm_peak,
                  "tflops": work["flops"] / (ms_step * 1e-3) / 1e12}

    line = {
        "metric": METRIC, "value": T / (ms_step * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp8_e4m3 x fp8_e4m3 -> f32 (block-scaled), bf16 out", "data": "synthetic",
        "config": {"workload": f"{name}: T={T}, hidden {H}, intermediate {Iz}, {shape.num_local_experts} local of "
                               f"{shape.num_experts} experts, top-{shape.top_k}",
                   "pairs": pairs, "active_experts": active, "token_tile": int(layer.layout(T).token_tile),
                   "l2": "inputs larger than L2 (expert weights streamed per step: %.2f GB)" % (work["weight_bytes"] / 1e9)},
        "e2e": {"value": T / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms},
        "gpu_launches": layer.launches_per_forward(T) * K,
        "clocks": clocks,
        "roofline": roof,
        "layer": layer_roof,
        "stage_ms": stage,
    }
    if not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(shape, d, T, spec, budget_s=args.cpu_budget)
    print(json.dumps(line))


# dram__bytes_read.sum + dram__bytes_write.sum of one GEMM1 launch, from the ncu capture
# summarised under profiles/ (None until a capture of that workload exists)
NCU_TRAFFIC = {"decode": 471.93e6 + 5.57e6, "prefill": 993.29e6 + 79.53e6}


def _to_cpu(d):
    return {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}


def cpu_baseline(shape, d, T, spec, budget_s=20.0, steps=1, warmup=0):
    """Time the CPU port of the operator definition (oracle/) on the host cores, on a bounded
    sample: the first S local experts that received tokens (routing always over all tokens).
    The value is extrapolated to the whole step by the share of (token, expert) pairs covered."""
    from oracle import moe_oracle as O
    dc = _to_cpu(d)
    idx, w = O.route(shape.routing_mode, dc["routing_logits"], dc["routing_bias"], shape.top_k, shape.n_group,
                     shape.topk_group, spec["rsf"])
    off, El = dc["local_expert_offset"], shape.num_local_experts
    counts = [(int((idx == off + e).sum())) for e in range(El)]
    act = [e for e in range(El) if counts[e]]
    total_pairs = sum(counts)

    def step(experts):
        lo, hi = experts[0], experts[-1] + 1
        t0 = time.perf_counter()
        O.moe_forward(dc["routing_logits"], dc["routing_bias"], dc["hidden_states"], dc["hidden_states_scale"],
                      dc["gemm1_weights"][lo:hi], dc["gemm1_weights_scale"][lo:hi], dc["gemm2_weights"][lo:hi],
                      dc["gemm2_weights_scale"][lo:hi], off + lo, spec["rsf"], routing_mode=shape.routing_mode,
                      top_k=shape.top_k, n_group=shape.n_group, topk_group=shape.topk_group)
        return time.perf_counter() - t0

    t1 = step(act[:1])                                   # probe: one expert
    per_step_budget = budget_s / max(1, steps + warmup)
    S = max(1, min(len(act), int(per_step_budget / max(t1, 1e-3))))
    sample = act[:S]
    for _ in range(warmup):
        step(sample)
    ts = [step(sample) for _ in range(steps)]
    t = sum(ts) / len(ts)
    covered = sum(counts[e] for e in range(sample[0], sample[-1] + 1))
    value = T * (covered / max(total_pairs, 1)) / t
    return {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"oracle (PyTorch fp32 CPU port of the definition) on local experts {sample[0]}..{sample[-1]} "
                      f"({covered} of {total_pairs} pairs), {t:.2f} s per step, extrapolated by pair share",
            "s_per_step": t}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    name = args.workload or ("decode" if world == 1 else "ep")
    spec = workload_spec(name, 1 if not (name in ("ep", "qwen3")) else world)
    shape, T = spec["shape"], spec["T"]
    if spec["ep"]:
        # the reference arm covers one rank's share: T tokens against that rank's local experts
        pass
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    d = I.make_inputs(shape, T, seed=0, device=dev, routed_scaling_factor=spec["rsf"], bias_boost=spec["boost"])
    K, W = args.steps, args.warmup
    cb = cpu_baseline(shape, d, T, spec, budget_s=min(150.0, max(20.0, 3.0 * (K + W))), steps=K, warmup=W)
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": cb["s_per_step"] * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32 (CPU, de-quantised fp8)", "data": "synthetic",
            "config": {"workload": f"{name}: T={T}, hidden {shape.hidden}, intermediate {shape.intermediate}, "
                                   f"{shape.num_local_experts} local of {shape.num_experts} experts, top-{shape.top_k}"},
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=[None, "decode", "prefill", "t14107", "ep", "qwen3"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--cpu-budget", type=float, default=20.0)
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
