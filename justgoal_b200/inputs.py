"""Seeded synthetic inputs for the FP8 block-scale MoE layer.

The reference corpus was measured on the flashinfer-bench workloads of the definition
`moe_fp8_block_scale_ds_routing_topk8_ng8_kg4_e32_h7168_i2048` (README.md:51-56); those
tensors are not available offline, so the bench and the tests draw tensors with the
definition's shapes and dtypes and the distributions the benchmark configuration states:
logits ~ N(0,1) fp32, bias ~ N(0,0.1) bf16, hidden ~ N(0,1) quantised to e4m3 per 1x128
group (scale = amax/448, stored [H/128, T]), weights ~ N(0,0.02) quantised per 128x128
block.  One torch.Generator per tensor, seeded seed*1000 + tensor id (+ expert id).
"""
from __future__ import annotations

from dataclasses import dataclass, replace

import torch

BLOCK = 128
FP8_MAX = 448.0

ROUTING_DS = 0
ROUTING_RENORM_NAIVE = 1     # softmax -> top-k -> renormalise
ROUTING_DEFAULT = 2          # softmax -> top-k
ROUTING_RENORMALIZE = 3      # top-k -> softmax over the selected logits
ROUTING_LLAMA4 = 4           # top-1 -> sigmoid
ROUTING_TOPK = 5             # top-k, uniform weights


@dataclass(frozen=True)
class MoEShape:
    """Static description of one rank's share of an MoE layer."""
    hidden: int = 7168
    intermediate: int = 2048
    num_experts: int = 256          # global
    num_local_experts: int = 32
    top_k: int = 8
    n_group: int = 8
    topk_group: int = 4
    routing_mode: int = ROUTING_DS

    def with_local(self, n):
        return replace(self, num_local_experts=n)


DEEPSEEK_V3 = MoEShape()
QWEN3_MOE = MoEShape(hidden=4096, intermediate=1536, num_experts=128, num_local_experts=16,
                     top_k=8, n_group=1, topk_group=1, routing_mode=ROUTING_RENORM_NAIVE)
# A tiny shape with the DeepSeek routing structure, for fast tests and the smoke run.
TINY_DS = MoEShape(hidden=512, intermediate=256, num_experts=64, num_local_experts=16,
                   top_k=8, n_group=8, topk_group=4, routing_mode=ROUTING_DS)
TINY_RENORM = MoEShape(hidden=384, intermediate=128, num_experts=32, num_local_experts=8,
                       top_k=4, n_group=1, topk_group=1, routing_mode=ROUTING_RENORM_NAIVE)
TINY_DEFAULT = replace(TINY_RENORM, routing_mode=ROUTING_DEFAULT)
TINY_RENORMALIZE = replace(TINY_RENORM, routing_mode=ROUTING_RENORMALIZE)
TINY_LLAMA4 = replace(TINY_RENORM, top_k=1, routing_mode=ROUTING_LLAMA4)
TINY_TOPK = replace(TINY_RENORM, routing_mode=ROUTING_TOPK)


def _gen(seed, tensor_id, device):
    g = torch.Generator(device=device)
    g.manual_seed(int(seed) * 1000 + int(tensor_id))
    return g


def quantize_rows_1x128(x: torch.Tensor):
    """[T, H] float -> (e4m3 [T, H], scales fp32 [H/128, T]); scale = amax/448 per (row, 128 cols)."""
    T, H = x.shape
    xb = x.float().reshape(T, H // BLOCK, BLOCK)
    amax = xb.abs().amax(dim=2)
    scale = torch.where(amax > 0, amax / FP8_MAX, torch.ones_like(amax))
    q = (xb / scale.unsqueeze(-1)).reshape(T, H).to(torch.float8_e4m3fn)
    return q, scale.t().contiguous()


def quantize_blocks_128x128(w: torch.Tensor):
    """[N, K] float -> (e4m3 [N, K], scales fp32 [N/128, K/128])."""
    N, K = w.shape
    wb = w.float().reshape(N // BLOCK, BLOCK, K // BLOCK, BLOCK)
    amax = wb.abs().amax(dim=(1, 3))
    scale = torch.where(amax > 0, amax / FP8_MAX, torch.ones_like(amax))
    q = (wb / scale[:, None, :, None]).reshape(N, K).to(torch.float8_e4m3fn)
    return q, scale.contiguous()


def make_tokens(shape: MoEShape, T: int, seed: int = 0, device="cpu", bias_boost=None):
    """Per-step tensors: routing_logits, routing_bias, hidden_states, hidden_states_scale.

    bias_boost: optional (expert_ids, delta) added to the bias of those global experts
    (the skewed-load prefill configuration)."""
    E, H = shape.num_experts, shape.hidden
    logits = torch.randn(T, E, generator=_gen(seed, 1, device), device=device, dtype=torch.float32)
    if shape.routing_mode == ROUTING_RENORM_NAIVE:
        bias = torch.zeros(E, device=device, dtype=torch.float32)    # the Qwen3-MoE configuration states no bias
    else:
        bias = torch.randn(E, generator=_gen(seed, 2, device), device=device, dtype=torch.float32) * 0.1
    if bias_boost is not None:
        ids, delta = bias_boost
        bias[torch.as_tensor(list(ids), device=device)] += float(delta)
    bias = bias.to(torch.bfloat16)
    x = torch.randn(T, H, generator=_gen(seed, 3, device), device=device, dtype=torch.float32)
    hs, hs_scale = quantize_rows_1x128(x)
    return {"routing_logits": logits, "routing_bias": bias,
            "hidden_states": hs, "hidden_states_scale": hs_scale}


def make_weights(shape: MoEShape, seed: int = 0, device="cpu", local_expert_offset: int = 0, std=0.02):
    """Expert weights of the local experts, generated one expert at a time (the fp32 draws of
    32 DeepSeek experts would not fit comfortably otherwise).  The generator of an expert is
    keyed on its GLOBAL id, so every expert-parallel split sees the same model."""
    H, I, El = shape.hidden, shape.intermediate, shape.num_local_experts
    w13 = torch.empty(El, 2 * I, H, dtype=torch.float8_e4m3fn, device=device)
    s13 = torch.empty(El, 2 * I // BLOCK, H // BLOCK, dtype=torch.float32, device=device)
    w2 = torch.empty(El, H, I, dtype=torch.float8_e4m3fn, device=device)
    s2 = torch.empty(El, H // BLOCK, I // BLOCK, dtype=torch.float32, device=device)
    for le in range(El):
        ge = local_expert_offset + le
        a = torch.randn(2 * I, H, generator=_gen(seed, 100 + 2 * ge, device), device=device) * std
        w13[le], s13[le] = quantize_blocks_128x128(a)
        b = torch.randn(H, I, generator=_gen(seed, 101 + 2 * ge, device), device=device) * std
        w2[le], s2[le] = quantize_blocks_128x128(b)
    return {"gemm1_weights": w13, "gemm1_weights_scale": s13,
            "gemm2_weights": w2, "gemm2_weights_scale": s2}


def make_inputs(shape: MoEShape, T: int, seed: int = 0, device="cpu", local_expert_offset: int = 0,
                routed_scaling_factor: float = 2.5, bias_boost=None):
    d = make_tokens(shape, T, seed, device, bias_boost)
    d.update(make_weights(shape, seed, device, local_expert_offset))
    d["local_expert_offset"] = int(local_expert_offset)
    d["routed_scaling_factor"] = float(routed_scaling_factor)
    return d


def algorithmic_work(shape: MoEShape, T: int, num_pairs: int, active_experts: int) -> dict:
    """FLOPs and HBM bytes one call must do, from the REALISED routing: 6*P*H*I flops; fp8
    weights and block scales of the experts that received a token, the step's inputs and the
    bf16 output.  Intermediates are excluded."""
    H, I, E = shape.hidden, shape.intermediate, shape.num_experts
    w_bytes = active_experts * 3 * H * I
    s_bytes = active_experts * (3 * H * I // (BLOCK * BLOCK)) * 4
    io = T * H + T * (H // BLOCK) * 4 + T * E * 4 + 2 * E + T * H * 2
    return {"flops": 6 * num_pairs * H * I, "bytes": w_bytes + s_bytes + io,
            "weight_bytes": w_bytes, "io_bytes": io + s_bytes}
