#!/usr/bin/env python
"""Benchmark of the FP8 block-scale MoE layer (one "step" = one forward of the layer).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workloads (synthetic tensors with the benchmark definition's shapes and distributions):
  ep       T=8192 per step, the full 256-expert DeepSeek-V3 layer: all experts on the one GPU at N=1,
           sharded expert-parallel over the N ranks otherwise          (the headline at every N: one
           scaling series, "strong")
  decode   T=64,   32 local of 256 experts                              (sub-record of the N=1 line)
  prefill  T=4096, 32 local experts, 4 experts with ~4x the mean load   (sub-record of the N=1 line)
  qwen3    T=2048, 128 experts of the Qwen3-MoE shape over the N ranks  (sub-record of the N=8 line)
  t14107   T=14107, 32 local experts (the token count the reference quotes its best latency on)

Prints ONE JSON line on rank 0.  `value` is tokens/s with all inputs resident in HBM; `e2e` is tokens/s
through the public entry point with the step's inputs (logits, fp8 hidden states, scales) copied from
pinned host memory and the bf16 output copied back inside the timed region (expert weights are model
state and stay resident).  `workloads` holds the same measurements for the other configurations.
`parity` compares a sample of the timed configuration's output rows with the CPU oracle (outside the
timed region); a line is only printed when no sampled element fails.  `--impl reference` times the CPU
port of the operator definition (oracle/) on the host cores instead.
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
DTYPE = "fp8_e4m3 x fp8_e4m3 -> f32 (block-scaled), bf16 out"
FP8_PEAK_NOMINAL = 4.5e15          # dense FP8 FLOP/s of one B200 (nominal; the roofline's compute term)
NVLINK_MEASURED = 770e9            # peer copy, bytes/s per direction per GPU on this pool
PARITY_TOKENS = 256                # output rows per rank compared with the oracle
ATOL, RTOL = 1e-2, 1e-2            # the operator's stated output tolerance


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return json.load(open(p)), "measured"
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


def ncu_traffic(workload, kernel):
    """DRAM bytes (read + write) of one launch of `kernel` in `workload`, from the ncu capture summarised under
    profiles/ (None when no capture of that pair exists)."""
    try:
        table = json.load(open(os.path.join(ROOT, "profiles", "dram_traffic.json")))
        rec = table[workload][kernel]
        return float(rec["dram_bytes_read"]) + float(rec["dram_bytes_write"])
    except Exception:
        return None


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
        return self

    def stop(self):
        self._stop.set()
        if self._thr is not None:
            self._thr.join()
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


# bias added to local experts 0, 8, 16, 24 so that they receive ~4x the mean load of the 32
# local experts at T=4096 (calibrated once on the CPU, by bisection, with the seeded logits)
PREFILL_BIAS_BOOST = 0.328


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


def workload_text(name, spec, world):
    """The same string in both arms (ours / reference) and at every N for the expert-parallel series."""
    s, T = spec["shape"], spec["T"]
    if spec["ep"]:
        return (f"{name}: T={T} per step, hidden {s.hidden}, intermediate {s.intermediate}, all {s.num_experts} experts, "
                f"top-{s.top_k}, expert parallel over {world} GPU(s) ({s.num_experts // world} experts per GPU)")
    return (f"{name}: T={T}, hidden {s.hidden}, intermediate {s.intermediate}, {s.num_local_experts} local of "
            f"{s.num_experts} experts, top-{s.top_k}")


def l2_text(weight_bytes):
    return ("inputs larger than L2, no flush: every step streams %.2f GB of expert weights (L2 is 126 MB; the only "
            "bytes a step shares with the one before are its few MB of activations and tables)" % (weight_bytes / 1e9))


def dist_setup():
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


# ----------------------------------------------------------------------------------------------------
# oracle helpers (the checker and the CPU baseline; never inside a timed GPU region)
# ----------------------------------------------------------------------------------------------------
def oracle_partial(shape, tok_cpu, weights, local_offset, rsf, slice_experts=32):
    """fp32 [n, H]: sum over the experts held in `weights` (any device) of the oracle's expert outputs for the
    tokens in `tok_cpu`; the weights travel to the host one slice at a time."""
    from oracle import moe_oracle as O
    idx, w = O.route(shape.routing_mode, tok_cpu["routing_logits"], tok_cpu["routing_bias"], shape.top_k, shape.n_group,
                     shape.topk_group, rsf)
    El = int(weights["gemm1_weights"].shape[0])
    total = torch.zeros(tok_cpu["hidden_states"].shape[0], shape.hidden, dtype=torch.float32)
    for lo in range(0, El, slice_experts):
        hi = min(El, lo + slice_experts)
        hit = ((idx >= local_offset + lo) & (idx < local_offset + hi)).any()
        if not bool(hit):
            continue
        wc = {k: weights[k][lo:hi].cpu() for k in ("gemm1_weights", "gemm1_weights_scale", "gemm2_weights",
                                                    "gemm2_weights_scale")}
        part, _, _ = O.run_experts(tok_cpu["hidden_states"], tok_cpu["hidden_states_scale"], wc["gemm1_weights"],
                                   wc["gemm1_weights_scale"], wc["gemm2_weights"], wc["gemm2_weights_scale"], w, idx,
                                   local_offset + lo, shape.num_experts)
        total += part
    return total


def sample_tokens(d, T, n):
    """Every (T // n)-th token: (index tensor on the CPU, the tokens' inputs on the CPU)."""
    n = min(n, T)
    sel = torch.arange(n) * (T // n)
    dev_sel = sel.to(d["routing_logits"].device)
    tok = {"routing_logits": d["routing_logits"][dev_sel].cpu(), "routing_bias": d["routing_bias"].cpu(),
           "hidden_states": d["hidden_states"].view(torch.uint8)[dev_sel].cpu().view(torch.float8_e4m3fn),
           "hidden_states_scale": d["hidden_states_scale"][:, dev_sel].contiguous().cpu()}
    return sel, tok


def parity_report(got_rows_bf16, want_f32):
    from oracle import moe_oracle as O
    rep = O.compare_output(got_rows_bf16, want_f32.to(torch.bfloat16), ATOL, RTOL)
    return {"tokens": int(got_rows_bf16.shape[0]), "fail_frac": rep["fail_frac"], "max_abs": rep["max_abs"],
            "finite": rep["finite"], "atol": ATOL, "rtol": RTOL, "against": "CPU oracle of the whole layer"}


def cpu_baseline(shape, d, T, spec, budget_s=20.0, steps=1, warmup=0, all_pairs=None):
    """Time the CPU port of the operator definition (oracle/) on the host cores, on a bounded sample: the
    first S experts held in `d` that received tokens (routing always over all tokens).  The value is extrapolated
    to the whole step by the share of (token, expert) pairs covered; `all_pairs` is that base when `d` holds
    only a prefix of the step's experts."""
    from oracle import moe_oracle as O
    tok = {k: d[k].cpu() for k in ("routing_logits", "routing_bias", "hidden_states", "hidden_states_scale")}
    idx, w = O.route(shape.routing_mode, tok["routing_logits"], tok["routing_bias"], shape.top_k, shape.n_group,
                     shape.topk_group, spec["rsf"])
    off, El = int(d["local_expert_offset"]), int(d["gemm1_weights"].shape[0])
    counts = torch.bincount((idx - off).clamp(-1, El).flatten() + 1, minlength=El + 2)[1:El + 1].tolist()
    act = [e for e in range(El) if counts[e]]
    total_pairs = all_pairs if all_pairs is not None else sum(counts)

    def step(experts):
        lo, hi = experts[0], experts[-1] + 1
        wc = [d[k][lo:hi].cpu() for k in ("gemm1_weights", "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale")]
        t0 = time.perf_counter()
        O.moe_forward(tok["routing_logits"], tok["routing_bias"], tok["hidden_states"], tok["hidden_states_scale"],
                      *wc, off + lo, spec["rsf"], routing_mode=shape.routing_mode,
                      top_k=shape.top_k, n_group=shape.n_group, topk_group=shape.topk_group)
        return time.perf_counter() - t0

    def fixed():                                         # routing + de-quantising the tokens: paid once per step
        wc = [d[k][0:0].cpu() for k in ("gemm1_weights", "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale")]
        t0 = time.perf_counter()
        O.moe_forward(tok["routing_logits"], tok["routing_bias"], tok["hidden_states"], tok["hidden_states_scale"],
                      *wc, off, spec["rsf"], routing_mode=shape.routing_mode,
                      top_k=shape.top_k, n_group=shape.n_group, topk_group=shape.topk_group)
        return time.perf_counter() - t0

    t_fixed = min(fixed(), fixed())
    t1 = max(step(act[:1]) - t_fixed, 1e-3)              # probe: one expert
    per_step_budget = budget_s / max(1, steps + warmup)
    S = max(1, min(len(act), int((per_step_budget - t_fixed) / t1)))
    sample = act[:S]
    for _ in range(warmup):
        step(sample)
    ts = [step(sample) for _ in range(steps)]
    t = sum(ts) / len(ts)
    covered = sum(counts[e] for e in range(sample[0], sample[-1] + 1))
    # whole step = the once-per-step part + the per-expert part scaled by the share of pairs the sample covered
    t_whole = t_fixed + max(t - t_fixed, 0.0) * (max(total_pairs, 1) / max(covered, 1))
    return {"value": T / t_whole, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"oracle (PyTorch fp32 CPU port of the definition) on experts {off + sample[0]}..{off + sample[-1]} "
                      f"({covered} of the step's {total_pairs} (token, expert) pairs): {t:.2f} s per sampled step, of "
                      f"which {t_fixed:.2f} s routing and token de-quantisation (counted once); the expert part is "
                      f"extrapolated by pair share to {t_whole:.1f} s for the whole step",
            "s_per_step": t, "s_whole_step": t_whole}


# ----------------------------------------------------------------------------------------------------
# one GPU
# ----------------------------------------------------------------------------------------------------
WARM_MS = 60.0      # untimed steps run for at least this long before the timed region (and never fewer than --warmup)


def measure_single(name, spec, K, W, dev, local, parity=True):
    """All measurements of one single-GPU workload; returns (record, inputs dict)."""
    from justgoal_b200 import HostPipeline, MoELayer
    shape, T = spec["shape"], spec["T"]
    layer = MoELayer(shape, dev)
    d = I.make_inputs(shape, T, seed=0, device=dev, routed_scaling_factor=spec["rsf"], bias_boost=spec["boost"])
    op = [d[k] for k in ("routing_logits", "routing_bias", "hidden_states", "hidden_states_scale",
                         "gemm1_weights", "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale",
                         "local_expert_offset", "routed_scaling_factor")]
    t_w = time.perf_counter()
    for _ in range(W):
        out = layer.forward(*op)
    torch.cuda.synchronize()
    # A step of the small workloads is ~0.15 ms: W of them end before a GPU that sat idle (input generation, the CPU
    # baseline of the workload before) is back at its clocks.  Untimed steps go on until WARM_MS have passed.
    while (time.perf_counter() - t_w) * 1e3 < WARM_MS:
        for _ in range(W):
            out = layer.forward(*op)
        torch.cuda.synchronize()
    if layer.status(T) != 0:
        raise SystemExit(f"{name}: device error word {layer.status(T)}")
    st = layer.view(T, "status", torch.int32, (8,)).cpu().tolist()
    pairs, active = st[1], st[4]
    work = I.algorithmic_work(shape, T, pairs, active)

    # ---- timed region: K steps, inputs resident in HBM
    sampler = ClockSampler(local).start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(K):
        out = layer.forward(*op)
    e1.record()
    torch.cuda.synchronize()
    ms_step = e0.elapsed_time(e1) / K

    # ---- the same K steps again with the library's per-stage CUDA events on the launch stream (an event
    # between two kernels removes their programmatic overlap, so the stages sum to a little more than ms_step)
    slots = min(K, 512)
    layer.profile_enable(slots)
    for _ in range(K):
        out = layer.forward(*op)
    torch.cuda.synchronize()
    clocks = sampler.stop()
    per_slot = [layer.profile_read(s) for s in range(slots)]
    stage = {k: sorted(r[k] for r in per_slot)[slots // 2] for k in layer.STAGES}     # medians
    layer.profile_enable(0)
    if layer.status(T) != 0:
        raise SystemExit(f"{name}: device error word {layer.status(T)} after the timed steps")

    # ---- end to end: host inputs -> device, forward, output -> host, every step (HostPipeline: three streams,
    # two sets of device buffers; every step still moves its own bytes)
    host_in = [d[k].cpu().pin_memory() for k in ("routing_logits", "hidden_states", "hidden_states_scale")]
    host_out = torch.empty(T, shape.hidden, dtype=torch.bfloat16).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = host_out.numel() * host_out.element_size()
    pipe = HostPipeline(layer, T, d["routing_bias"], *op[4:])
    for _ in range(W):
        pipe.step(host_in[0], host_in[1], host_in[2], host_out)
    pipe.drain()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(K):
        pipe.step(host_in[0], host_in[1], host_in[2], host_out)
    pipe.drain()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / K
    assert torch.equal(host_out.view(torch.int16), out.cpu().view(torch.int16))

    # ---- roofline of the dominant kernel (GEMM1: two thirds of the weight bytes and of the flops)
    peaks, which = measured_peaks()
    hbm_peak = float(peaks["hbm_gbs"])
    H, Iz = shape.hidden, shape.intermediate
    g1_bytes = active * 2 * Iz * H + active * (2 * Iz // 128) * (H // 128) * 4 + pairs * H + pairs * (H // 128) * 4
    g1_flops = 4 * pairs * H * Iz
    t_g1 = stage["gemm1"] * 1e-3
    ntok = int(layer.layout(T).token_tile)
    kernel = f"gemm_kernel<{ntok},true>"
    g1_hbm_t, g1_fp8_t = g1_bytes / (hbm_peak * 1e9), g1_flops / FP8_PEAK_NOMINAL
    if g1_hbm_t >= g1_fp8_t:
        roof = {"kernel": kernel + " (GEMM1 + SwiGLU + requant)", "bound": "hbm", "achieved": g1_bytes / t_g1 / 1e9,
                "peak": hbm_peak, "unit": "GB/s", "frac": g1_bytes / t_g1 / 1e9 / hbm_peak, "peak_source": which}
    else:
        roof = {"kernel": kernel + " (GEMM1 + SwiGLU + requant)", "bound": "tensor", "achieved": g1_flops / t_g1 / 1e12,
                "peak": FP8_PEAK_NOMINAL / 1e12, "unit": "TFLOP/s", "frac": g1_flops / t_g1 / FP8_PEAK_NOMINAL,
                "peak_source": "nominal dense FP8 (MEASURED_PEAKS.json holds bf16 only: %.0f TFLOP/s)" % peaks["bf16_tflops"]}
    roof.update({"traffic": ncu_traffic(name, kernel), "bytes_per_launch": g1_bytes, "flops_per_launch": g1_flops,
                 "ms_per_launch": stage["gemm1"], "t_hbm_ms": g1_hbm_t * 1e3, "t_fp8_ms": g1_fp8_t * 1e3,
                 "tflops": g1_flops / t_g1 / 1e12, "gbs": g1_bytes / t_g1 / 1e9})
    t_hbm, t_fp8 = work["bytes"] / (hbm_peak * 1e9), work["flops"] / FP8_PEAK_NOMINAL
    layer_roof = {"bytes": work["bytes"], "flops": work["flops"], "t_hbm_ms": t_hbm * 1e3, "t_fp8_ms": t_fp8 * 1e3,
                  "frac_of_roof": max(t_hbm, t_fp8) / (ms_step * 1e-3), "bound": "hbm" if t_hbm >= t_fp8 else "tensor",
                  "hbm_gbs": work["bytes"] / (ms_step * 1e-3) / 1e9, "tflops": work["flops"] / (ms_step * 1e-3) / 1e12}
    rec = {"workload": workload_text(name, spec, 1), "ms_per_step": ms_step, "value": T / (ms_step * 1e-3), "unit": UNIT,
           "e2e": {"value": T / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                   "ms_per_step": e2e_ms},
           "gpu_launches": layer.launches_per_forward(T) * K, "clocks": clocks, "roofline": roof, "layer": layer_roof,
           "stage_ms": stage, "pairs": pairs, "active_experts": active, "token_tile": ntok,
           "l2": l2_text(work["weight_bytes"]),
           "warmup_note": "untimed steps ran for at least %d ms (never fewer than the warm-up count)" % WARM_MS}
    if parity:
        sel, tok = sample_tokens(d, T, PARITY_TOKENS)
        want = oracle_partial(shape, tok, d, int(d["local_expert_offset"]), spec["rsf"])
        rec["parity"] = parity_report(out[sel.to(dev)].cpu(), want)
        if rec["parity"]["fail_frac"] != 0.0 or not rec["parity"]["finite"]:
            raise SystemExit(f"{name}: output differs from the oracle: {rec['parity']}")
    return rec, d


def run_ours(args):
    rank, world, local = dist_setup()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py (impl ours) needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))      # torchrun sets one thread; the oracle legs use more
    name = args.workload or "ep"
    spec = workload_spec(name, world)
    K, W = args.steps, max(args.warmup, 3)
    if world > 1:
        if not spec["ep"]:
            raise SystemExit(f"workload {name} is single-GPU")
        return run_expert_parallel(args, name, spec, rank, world, local, K, W)
    rec, d = measure_single(name, spec, K, W, dev, local)
    line = {"metric": METRIC, "value": rec["value"], "unit": UNIT, "n_gpus": 1, "steps": K, "warmup": W,
            "ms_per_step": rec["ms_per_step"], "higher_is_better": True,
            "scaling": "strong" if spec["ep"] else "weak", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
            "config": {"workload": rec["workload"], "l2": rec["l2"], "warmup_note": rec["warmup_note"]}}
    for k in ("e2e", "gpu_launches", "clocks", "roofline", "layer", "stage_ms", "pairs", "active_experts", "token_tile",
              "parity"):
        line[k] = rec[k]
    if not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(spec["shape"], d, spec["T"], spec, budget_s=args.cpu_budget)
    del d
    torch.cuda.empty_cache()
    if args.workload is None:
        # the other single-GPU configurations of the benchmark, same measurements, in the same line
        line["workloads"] = {}
        for sub in ("decode", "prefill"):
            srec, sd = measure_single(sub, workload_spec(sub, 1), K, W, dev, local)
            del sd
            torch.cuda.empty_cache()
            line["workloads"][sub] = srec
            line["gpu_launches"] += srec["gpu_launches"]
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------------
# expert parallel (N > 1): one step = one forward of the whole layer over T tokens, T/N per rank
# ----------------------------------------------------------------------------------------------------
def measure_expert_parallel(name, spec, rank, world, local, K, W):
    import torch.distributed as dist
    from justgoal_b200 import HostPipeline
    from justgoal_b200.ep import ExpertParallelMoE, plan_dispatch

    dev = torch.device("cuda", local)
    shape, T = spec["shape"], spec["T"]
    per = T // world
    tokens = I.make_tokens(shape, T, seed=0, device=dev)
    sl = slice(rank * per, (rank + 1) * per)
    logits = tokens["routing_logits"][sl].contiguous()
    bias = tokens["routing_bias"]
    hidden = tokens["hidden_states"].view(torch.uint8)[sl].contiguous().view(torch.float8_e4m3fn)
    hscale = tokens["hidden_states_scale"][:, sl].contiguous()
    weights = I.make_weights(shape, 0, dev, rank * shape.num_local_experts)
    # Exchange: this library's kernels over peer memory when the node can map it and one step of it agrees
    # with the collective form on the real inputs; else the NCCL form (B200MOE_EP_EXCHANGE=nccl|p2p forces one).
    want = os.environ.get("B200MOE_EP_EXCHANGE", "auto")
    ep_nccl = ExpertParallelMoE(shape, weights, device=dev)
    ep, exchange, why = ep_nccl, "nccl", "forced" if want == "nccl" else ""
    if want != "nccl":
        ok = torch.ones(1, device=dev)
        try:
            ep_p2p = ExpertParallelMoE(shape, weights, device=dev, exchange="p2p", capacity=per)
            a = ep_nccl.forward(logits, bias, hidden, hscale, spec["rsf"])
            b = ep_p2p.forward(logits, bias, hidden, hscale, spec["rsf"])
            torch.cuda.synchronize()
            if ep_p2p.peer.error_word() != 0 or not torch.allclose(a.float(), b.float(), atol=1e-2, rtol=1e-2):
                ok.zero_(); why = "peer-memory step differs from the NCCL step"
        except Exception as e:           # noqa: BLE001 - any failure to set the mapping up means: use NCCL
            ok.zero_(); why = f"peer-memory setup failed: {type(e).__name__}"
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok) > 0:
            ep, exchange = ep_p2p, "p2p"
        elif want == "p2p":
            raise SystemExit(f"B200MOE_EP_EXCHANGE=p2p but {why or 'another rank failed'}")

    def sync_time(fn, steps):
        for _ in range(W):
            fn()
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize(); dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    out = None

    def step():
        nonlocal out
        out = ep.forward(logits, bias, hidden, hscale, spec["rsf"])

    sync_time(step, 2)           # untimed: first use of the barrier / all-reduce / event path itself
    sampler = ClockSampler(local).start()
    ms_step = sync_time(step, K)
    clocks = sampler.stop()
    ep.check_status()

    # ---- parity: PARITY_TOKENS of every rank's tokens against the oracle of the WHOLE layer.  Every rank computes
    # the oracle's partial sum over ITS experts for all sampled tokens of all ranks; the partials are added across
    # the ranks in fp32 and rounded once.
    n_s = min(PARITY_TOKENS, per)
    sel = torch.arange(n_s, device=dev) * (per // n_s)
    gather = lambda t: [torch.empty_like(t) for _ in range(world)]                 # noqa: E731
    s_log, s_hid, s_sc = logits[sel].contiguous(), hidden.view(torch.uint8)[sel].contiguous(), hscale[:, sel].contiguous()
    g_log, g_hid, g_sc = gather(s_log), gather(s_hid), gather(s_sc)
    dist.all_gather(g_log, s_log)
    dist.all_gather(g_hid, s_hid)
    dist.all_gather(g_sc, s_sc)
    tok = {"routing_logits": torch.cat(g_log).cpu(), "routing_bias": bias.cpu(),
           "hidden_states": torch.cat(g_hid).cpu().view(torch.float8_e4m3fn),
           "hidden_states_scale": torch.cat(g_sc, dim=1).cpu()}
    part = oracle_partial(shape, tok, weights, rank * shape.num_local_experts, spec["rsf"]).to(dev)
    dist.all_reduce(part)
    par = parity_report(out[sel].cpu(), part[rank * n_s:(rank + 1) * n_s].cpu())
    bad = torch.tensor([par["fail_frac"], par["max_abs"], 0.0 if par["finite"] else 1.0], device=dev, dtype=torch.float64)
    dist.all_reduce(bad, op=dist.ReduceOp.MAX)
    par.update(tokens=n_s * world, fail_frac=float(bad[0]), max_abs=float(bad[1]), finite=bool(bad[2] == 0))

    ep.last_plan = plan_dispatch(ep.backend.route(logits, bias, spec["rsf"])[0], shape.num_local_experts, world)
    nv = ep.nvlink_bytes()
    ep.phase_events = []
    for _ in range(min(K, 10)):
        step()
    phases = ep.phase_ms()
    ep.phase_events = None
    allp = [None] * world
    dist.all_gather_object(allp, phases)
    phases_max = {k: max(p_[k] for p_ in allp) for k in phases}
    phases_min = {k: min(p_[k] for p_ in allp) for k in phases}

    # ---- end to end: host-resident inputs through the package's HostPipeline around the expert-parallel step
    host_in = [t.cpu().pin_memory() for t in (logits, hidden, hscale)]
    host_out = torch.empty(per, shape.hidden, dtype=torch.bfloat16).pin_memory()
    pipe = HostPipeline(ep.backend.layer, per, bias, None, None, None, None, 0, spec["rsf"],
                        forward_fn=lambda lg, hd, sc, o: ep.forward(lg, bias, hd, sc, spec["rsf"]))

    def e2e_round(steps):
        for _ in range(steps):
            pipe.step(host_in[0], host_in[1], host_in[2], host_out)
        pipe.drain()

    e2e_round(W)
    torch.cuda.synchronize(); dist.barrier()
    t0 = time.perf_counter()
    e2e_round(K)
    te = torch.tensor([(time.perf_counter() - t0) * 1e3 / K], device=dev)
    dist.barrier()
    dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_ms = float(te)
    ep.check_status()
    h2d = sum(t.numel() * t.element_size() for t in host_in) * world
    d2h = host_out.numel() * host_out.element_size() * world

    # realised work over all ranks
    n_recv = torch.tensor([sum(ep.last_plan.recv_counts)], device=dev, dtype=torch.float64)
    idx, _ = ep.backend.route(logits, bias, spec["rsf"])
    pairs = torch.tensor([float(idx.numel())], device=dev, dtype=torch.float64)
    link = torch.tensor([float(max(nv["dispatch_send"] + nv["combine_send"], nv["dispatch_recv"] + nv["combine_recv"]))],
                        device=dev, dtype=torch.float64)
    dist.all_reduce(pairs); dist.all_reduce(n_recv); dist.all_reduce(link, op=dist.ReduceOp.MAX)
    peaks, which = measured_peaks()
    hbm_peak = float(peaks["hbm_gbs"])
    H, Iz = shape.hidden, shape.intermediate
    flops = 6 * float(pairs) * H * Iz
    w_bytes_rank = shape.num_local_experts * 3 * H * Iz
    t_hbm, t_fp8, t_nv = w_bytes_rank / (hbm_peak * 1e9), flops / world / FP8_PEAK_NOMINAL, float(link) / NVLINK_MEASURED
    rec = {
        "workload": workload_text(name, spec, world), "ms_per_step": ms_step, "value": T / (ms_step * 1e-3), "unit": UNIT,
        "exchange": exchange, "exchange_note": why,
        "e2e": {"value": T / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms},
        "gpu_launches": ep.launches_per_step() * K * world, "clocks": clocks, "parity": par,
        "roofline": {"kernel": "whole step, slowest rank", "bound": "hbm", "peak_source": which,
                     "achieved": w_bytes_rank / (ms_step * 1e-3) / 1e9, "peak": hbm_peak, "unit": "GB/s",
                     "frac": w_bytes_rank / (ms_step * 1e-3) / 1e9 / hbm_peak, "traffic": None,
                     "t_hbm_ms": t_hbm * 1e3, "t_fp8_ms": t_fp8 * 1e3, "t_nvlink_ms": t_nv * 1e3},
        "layer": {"flops": flops, "tflops": flops / (ms_step * 1e-3) / 1e12, "pairs": float(pairs),
                  "rows_dispatched": float(n_recv), "max_link_bytes_per_rank": float(link),
                  "frac_of_roof": max(t_hbm, t_fp8, t_nv) / (ms_step * 1e-3)},
        "phase_ms_rank0": phases, "phase_ms_max_over_ranks": phases_max, "phase_ms_min_over_ranks": phases_min,
        "l2": l2_text(w_bytes_rank)}
    if par["fail_frac"] != 0.0 or not par["finite"]:
        raise SystemExit(f"{name}: expert-parallel output differs from the oracle: {par}")
    return rec


def run_expert_parallel(args, name, spec, rank, world, local, K, W):
    import torch.distributed as dist
    rec = measure_expert_parallel(name, spec, rank, world, local, K, W)
    line = {"metric": METRIC, "value": rec["value"], "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": DTYPE, "data": "synthetic",
            "config": {"workload": rec["workload"], "l2": rec["l2"], "exchange": rec["exchange"],
                       "exchange_note": rec["exchange_note"]}}
    for k in ("e2e", "gpu_launches", "clocks", "parity", "roofline", "layer", "phase_ms_rank0", "phase_ms_max_over_ranks",
              "phase_ms_min_over_ranks"):
        line[k] = rec[k]
    if args.workload is None and (world == 8 or os.environ.get("B200MOE_BENCH_QWEN3")):     # configs[4] is an 8-GPU configuration
        torch.cuda.empty_cache()
        q = measure_expert_parallel("qwen3", workload_spec("qwen3", world), rank, world, local, K, W)
        line["workloads"] = {"qwen3": q}
        line["gpu_launches"] += q["gpu_launches"]
    if rank == 0:
        print(json.dumps(line))
    dist.barrier()
    dist.destroy_process_group()


# ----------------------------------------------------------------------------------------------------
# reference arm: the CPU port of the definition on the host cores, whole layer, bounded sample
# ----------------------------------------------------------------------------------------------------
def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    torch.set_num_threads(os.cpu_count() or 1)          # torchrun exports OMP_NUM_THREADS=1
    name = args.workload or "ep"
    spec = workload_spec(name, 1)                       # the WHOLE layer on the host, whatever N the GPU arm used
    shape, T = spec["shape"], spec["T"]
    K, W = args.steps, args.warmup
    budget = min(150.0, max(20.0, 3.0 * (K + W)))
    # tokens in full; weights of a prefix of the experts only (more than the bounded sample can cover)
    n_w = min(shape.num_local_experts, 48)
    d = I.make_tokens(shape, T, seed=0, device="cpu", bias_boost=spec["boost"])
    d.update(I.make_weights(shape.with_local(n_w), 0, "cpu", 0))
    d["local_expert_offset"], d["routed_scaling_factor"] = 0, spec["rsf"]
    all_pairs = T * shape.top_k if shape.num_local_experts == shape.num_experts else None
    cb = cpu_baseline(shape, d, T, spec, budget_s=budget, steps=K, warmup=W, all_pairs=all_pairs)
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": T / cb["value"] * 1e3, "higher_is_better": True,
            "scaling": "strong" if spec["ep"] else "weak",
            "vs_baseline": None, "dtype": "f32 (CPU, de-quantised fp8)", "data": "synthetic",
            "config": {"workload": workload_text(name, workload_spec(name, world), world)},
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
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
