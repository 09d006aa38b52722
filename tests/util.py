"""Helpers shared by the parity tests."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")
sys.path.insert(0, GOLDEN)

from justgoal_b200 import inputs as I  # noqa: E402
from oracle import moe_oracle as O  # noqa: E402
import make_golden  # noqa: E402

ATOL, RTOL = 1e-2, 1e-2   # output tolerance stated for the operator: |got - want| <= ATOL + RTOL*|want|


def golden_case(name):
    """(shape, inputs dict on CPU, golden npz) of a committed fixture; the inputs are re-drawn
    from the seeds and verified against the checksums stored with the fixture."""
    shape, d = make_golden.build_inputs(name)
    g = np.load(os.path.join(GOLDEN, name + ".npz"))
    assert abs(float(d["routing_logits"].double().sum()) - float(g["logits_checksum"])) < 1e-6
    assert int(d["hidden_states"].view(torch.uint8).long().sum()) == int(g["hidden_checksum"])
    assert int(d["gemm1_weights"].view(torch.uint8).long().sum()) == int(g["w13_checksum"])
    return shape, d, g


def run_oracle(shape, d, keep_inter=False):
    return O.moe_forward(d["routing_logits"], d["routing_bias"], d["hidden_states"], d["hidden_states_scale"],
                         d["gemm1_weights"], d["gemm1_weights_scale"], d["gemm2_weights"],
                         d["gemm2_weights_scale"], d["local_expert_offset"], d["routed_scaling_factor"],
                         routing_mode=shape.routing_mode, top_k=shape.top_k, n_group=shape.n_group,
                         topk_group=shape.topk_group, keep_inter=keep_inter)


def to_cuda(d):
    return {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}


TENSOR_ORDER = ("routing_logits", "routing_bias", "hidden_states", "hidden_states_scale", "gemm1_weights",
                "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale", "local_expert_offset",
                "routed_scaling_factor")


def op_args(d):
    return [d[k] for k in TENSOR_ORDER]


def ulp_diff(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in units of the last place between two positive fp32 tensors."""
    return (a.contiguous().view(torch.int32).long() - b.contiguous().view(torch.int32).long()).abs()


def routing_margin_ulp(shape, logits, bias):
    """Per token, the smallest gap (in ulp of the biased score) between a selected and a rejected
    candidate in the oracle's selection -- used to explain a set mismatch, if one ever shows."""
    s = 1.0 / (1.0 + torch.exp(-logits.float()))
    v = s + (bias.float() if bias is not None else 0)
    srt = torch.sort(v, dim=1, descending=True).values
    gaps = ulp_diff(srt[:, :-1].clamp_min(1e-30), srt[:, 1:].clamp_min(1e-30))
    return gaps.min(dim=1).values


def collect(q, procs, n, seconds):
    """n results from the workers' queue; fails at once when a worker has died instead of waiting out
    the whole time limit."""
    import queue
    import time
    out, deadline = [], time.time() + seconds
    while len(out) < n:
        try:
            out.append(q.get(timeout=1.0))
        except queue.Empty:
            dead = [p.exitcode for p in procs if p.exitcode not in (None, 0)]
            if dead:
                raise AssertionError(f"worker exited with {dead} before reporting")
            if time.time() > deadline:
                raise AssertionError("workers did not report in time")
    return out
