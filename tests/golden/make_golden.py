"""Generate the golden fixtures that pin oracle/moe_oracle.py.

Run in a container where `flashinfer-python` (0.6.11.post2 here) is importable:

    python tests/golden/make_golden.py [case ...]

For every case below it draws the seeded synthetic inputs (justgoal_b200/inputs.py), runs the
PUBLISHED PyTorch reference of the operator definition
(flashinfer/trace/templates/moe.py: `_trtllm_fp8_block_scale_moe_ds_routing_reference`,
`_trtllm_fp8_block_scale_moe_renormalize_naive_routing_reference`) on the CPU, and stores its
bf16 output (as raw int16 bits) in tests/golden/<case>.npz.  The published functions return
only the layer output; the routing ids / weights stored beside it are produced by running
the same published routing statements (they are the first lines of those functions) through
`torch.topk`, i.e. by the oracle's `route_*`, and are cross-checked here by feeding them to
the published `_fp8_moe_run_experts` and requiring the identical layer output.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from justgoal_b200 import inputs as I  # noqa: E402
from oracle import moe_oracle as O  # noqa: E402

CASES = {
    # name: (shape, T, seed, local_expert_offset, weight std)
    "tiny_ds_t33": (I.TINY_DS, 33, 1, 0, 0.05),
    "tiny_ds_t7_off16": (I.TINY_DS, 7, 2, 16, 0.05),
    "tiny_renorm_t20": (I.TINY_RENORM, 20, 3, 8, 0.08),
    "ds_v3_t16": (I.DEEPSEEK_V3, 16, 0, 0, 0.02),   # configs[0] of the benchmark definition
    # the other routing methods of the operator family
    "tiny_default_t20": (I.TINY_DEFAULT, 20, 4, 8, 0.08),
    "tiny_renormalize_t20": (I.TINY_RENORMALIZE, 20, 5, 8, 0.08),
    "tiny_llama4_t40": (I.TINY_LLAMA4, 40, 6, 8, 0.08),
    "tiny_topk_t20": (I.TINY_TOPK, 20, 7, 8, 0.08),
}

PUBLISHED = {     # routing mode -> name of the published reference function
    I.ROUTING_RENORM_NAIVE: "_trtllm_fp8_block_scale_moe_renormalize_naive_routing_reference",
    I.ROUTING_DEFAULT: "_trtllm_fp8_block_scale_moe_default_routing_reference",
    I.ROUTING_RENORMALIZE: "_trtllm_fp8_block_scale_moe_renormalize_routing_reference",
    I.ROUTING_LLAMA4: "_trtllm_fp8_block_scale_moe_llama4_routing_reference",
    I.ROUTING_TOPK: "_trtllm_fp8_block_scale_moe_topk_routing_reference",
}


def build_inputs(name):
    shape, T, seed, off, std = CASES[name]
    d = I.make_tokens(shape, T, seed)
    d.update(I.make_weights(shape, seed, "cpu", off, std=std))
    d["local_expert_offset"] = off
    d["routed_scaling_factor"] = 2.5 if shape.routing_mode == I.ROUTING_DS else 1.0
    return shape, d


def main():
    from flashinfer.trace.templates import moe as FM
    here = os.path.dirname(os.path.abspath(__file__))
    for name in (sys.argv[1:] or list(CASES)):
        shape, d = build_inputs(name)
        args = (d["routing_logits"], d["routing_bias"], d["hidden_states"], d["hidden_states_scale"],
                d["gemm1_weights"], d["gemm1_weights_scale"], d["gemm2_weights"], d["gemm2_weights_scale"])
        if shape.routing_mode == I.ROUTING_DS:
            ref = FM._trtllm_fp8_block_scale_moe_ds_routing_reference(
                *args, shape.top_k, shape.n_group, shape.topk_group,
                d["local_expert_offset"], d["routed_scaling_factor"])
            idx, w = O.route_ds(d["routing_logits"], d["routing_bias"], shape.top_k, shape.n_group,
                                shape.topk_group, d["routed_scaling_factor"])
        else:
            ref = getattr(FM, PUBLISHED[shape.routing_mode])(
                *args, shape.top_k, d["local_expert_offset"], d["routed_scaling_factor"])
            idx, w = O.route(shape.routing_mode, d["routing_logits"], d["routing_bias"], shape.top_k, shape.n_group,
                             shape.topk_group, d["routed_scaling_factor"])
        chk = FM._fp8_moe_run_experts(*args[2:], w, idx, d["local_expert_offset"], shape.num_experts)
        assert torch.equal(chk.view(torch.int16), ref.view(torch.int16)), name
        order = torch.argsort(idx, dim=1)
        np.savez_compressed(
            os.path.join(here, name + ".npz"),
            output_bf16_bits=ref.view(torch.int16).numpy(),
            topk_idx_sorted=idx.gather(1, order).to(torch.int32).numpy(),
            topk_w_sorted=w.gather(1, order).numpy(),
            logits_checksum=np.float64(d["routing_logits"].double().sum().item()),
            hidden_checksum=np.int64(d["hidden_states"].view(torch.uint8).long().sum().item()),
            w13_checksum=np.int64(d["gemm1_weights"].view(torch.uint8).long().sum().item()),
        )
        print(name, "absmean", float(ref.float().abs().mean()), "absmax", float(ref.float().abs().max()))


if __name__ == "__main__":
    main()
