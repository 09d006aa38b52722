"""CPU oracle for the FP8 block-scale MoE layer (test infrastructure, NOT the product).

This is a restatement, in plain PyTorch on the CPU, of the arithmetic that defines the
operator `moe_fp8_block_scale_ds_routing_topk8_ng8_kg4_e32_h7168_i2048` which every
`moe_fp8_fwd` solution of the reference corpus implements (the `"definition"` field of
e.g. goal_full_shape/fable-5.1/moe_fp8_fwd/<def>/solution.json:3).  The reference corpus
ships no CPU/PyTorch implementation of the layer; the definition's arithmetic lives in the
third-party flashinfer-bench harness, un-vendored and un-pinned by the reference
(README.md:51-56,60-66).  The same definition family is published in the wheel
`flashinfer-python 0.6.11.post2` (flashinfer/trace/templates/moe.py,
`_trtllm_fp8_block_scale_moe_ds_routing_reference`,
`_trtllm_fp8_block_scale_moe_renormalize_naive_routing_reference` and the four other routing
methods of the family); this file restates that published algorithm and is pinned against
outputs of those functions through the fixtures in tests/golden/ (made by
tests/golden/make_golden.py).

Only tests/, __graft_entry__.smoke() and the CPU-baseline legs of bench.py may import this
module, and only as the checker.  The product path never calls it.

What the reference kernels state about the same arithmetic (used to cross-check the
restatement):
  * routing: fp32 sigmoid, + bias, group score = sum of the two largest biased scores of a
    group, keep `topk_group` groups, pick `top_k` experts among kept groups, weights from the
    UNBIASED sigmoid normalised by (sum + 1e-20) and multiplied by the routed scaling factor
    (goal_full_shape/fable-5.1/moe_fp8_fwd/<def>/moe_common.cuh:266-365,
     goal_full_shape/opus-4.8/moe_fp8_fwd/<def>/main.py:24-70);
  * block scales: activations per (token, 128 columns), stored [H/128, T]; weights per
    128x128 block (goal_full_shape/opus-4.8/moe_fp8_fwd/<def>/main.py:125-132,181-187);
  * SwiGLU: silu(second half of GEMM1 output) * first half
    (goal_full_shape/opus-4.8/moe_fp8_fwd/<def>/main.py:138-156);
  * combine: fp32 sum over the token's local experts of weight * expert output, one final
    rounding to bf16; tokens without a local expert give a zero row
    (kda05_reproduction_full_shape/fable-5.1/moe_fp8_fwd/<def>/fable51_moe_v94/kernel.cu:3207-3217).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

BLOCK = 128

ROUTING_DS = 0            # DeepSeek-V3: sigmoid + bias, group-limited top-k
ROUTING_RENORM_NAIVE = 1  # softmax -> top-k -> renormalise (Qwen3-MoE shape)
ROUTING_DEFAULT = 2       # softmax -> top-k
ROUTING_RENORMALIZE = 3   # top-k on the logits -> softmax over the selected
ROUTING_LLAMA4 = 4        # top-1 -> sigmoid
ROUTING_TOPK = 5          # top-k, uniform weights


@dataclass
class OracleResult:
    output_f32: torch.Tensor      # [T, H] fp32, before the final cast
    output: torch.Tensor          # [T, H] bf16
    topk_idx: torch.Tensor        # [T, top_k] int64, global expert ids (unordered within a row)
    topk_w: torch.Tensor          # [T, top_k] fp32, aligned with topk_idx
    expert_tokens: dict           # local expert -> LongTensor of token ids (ascending)
    inter: dict                   # local expert -> (G1 [n,2I] fp32, C [n,I] fp32, O [n,H] fp32) when keep_inter


@torch.no_grad()
def route_ds(routing_logits, routing_bias, top_k, n_group, topk_group, routed_scaling_factor):
    """DeepSeek-V3 group-limited routing (definition's `ds_routing`).

    Returns (topk_idx [T,top_k] int64, topk_w [T,top_k] fp32).  Same operations, in the same
    order and precision, as the published definition; the order of ids inside a row is
    whatever torch.topk(sorted=False) gives, so callers compare rows as sets.
    """
    logits = routing_logits.to(torch.float32)
    T, E = logits.shape
    if routing_bias is None:
        bias = torch.zeros(E, dtype=torch.float32, device=logits.device)
    else:
        bias = routing_bias.to(torch.float32).reshape(-1)
    s = 1.0 / (1.0 + torch.exp(-logits))
    s_with_bias = s + bias
    group_size = E // int(n_group)
    grouped = s_with_bias.view(T, int(n_group), group_size)
    top2, _ = torch.topk(grouped, k=2, dim=2, largest=True, sorted=False)
    group_scores = top2.sum(dim=2)
    _, group_idx = torch.topk(group_scores, k=int(topk_group), dim=1, largest=True, sorted=False)
    group_mask = torch.zeros_like(group_scores)
    group_mask.scatter_(1, group_idx, 1.0)
    score_mask = group_mask.unsqueeze(2).expand(T, int(n_group), group_size).reshape(T, E)
    neg = torch.finfo(torch.float32).min
    pruned = s_with_bias.masked_fill(score_mask == 0, neg)
    _, topk_idx = torch.topk(pruned, k=int(top_k), dim=1, largest=True, sorted=False)
    sel = torch.zeros_like(s)
    sel.scatter_(1, topk_idx, 1.0)
    raw = s * sel
    denom = raw.sum(dim=1, keepdim=True) + 1e-20
    weights = (raw / denom) * routed_scaling_factor
    return topk_idx, weights.gather(1, topk_idx)


@torch.no_grad()
def route_renorm_naive(routing_logits, routing_bias, top_k, routed_scaling_factor):
    """Softmax over all experts -> top-k -> renormalise the selected probabilities."""
    logits = routing_logits.to(torch.float32)
    if routing_bias is not None:
        logits = logits + routing_bias.to(torch.float32).reshape(-1)
    s = torch.softmax(logits, dim=-1)
    _, topk_idx = torch.topk(s, k=int(top_k), dim=1, largest=True, sorted=False)
    g = s.gather(1, topk_idx)
    w = g / (g.sum(dim=1, keepdim=True) + 1e-20)
    return topk_idx, w * routed_scaling_factor


def _biased_logits(routing_logits, routing_bias):
    logits = routing_logits.to(torch.float32)
    if routing_bias is not None:
        logits = logits + routing_bias.to(torch.float32).reshape(-1)
    return logits


@torch.no_grad()
def route_default(routing_logits, routing_bias, top_k, routed_scaling_factor):
    """Softmax over all experts -> top-k; the weights are the selected probabilities
    (published as `..._default_routing_reference`, flashinfer/trace/templates/moe.py:186-224)."""
    s = torch.softmax(_biased_logits(routing_logits, routing_bias), dim=-1)
    _, topk_idx = torch.topk(s, k=int(top_k), dim=1, largest=True, sorted=False)
    return topk_idx, s.gather(1, topk_idx) * routed_scaling_factor


@torch.no_grad()
def route_renormalize(routing_logits, routing_bias, top_k, routed_scaling_factor):
    """Top-k on the logits -> softmax over the selected logits (`..._renormalize_routing_reference`,
    same file :226-265)."""
    logits = _biased_logits(routing_logits, routing_bias)
    _, topk_idx = torch.topk(logits, k=int(top_k), dim=1, largest=True, sorted=False)
    return topk_idx, torch.softmax(logits.gather(1, topk_idx), dim=-1) * routed_scaling_factor


@torch.no_grad()
def route_llama4(routing_logits, routing_bias, top_k, routed_scaling_factor):
    """Top-1 on the logits, weight = sigmoid of that logit (`..._llama4_routing_reference`, :267-306)."""
    logits = _biased_logits(routing_logits, routing_bias)
    topk_idx = logits.argmax(dim=-1, keepdim=True)
    top1 = logits.gather(1, topk_idx)
    return topk_idx, (1.0 / (1.0 + torch.exp(-top1))) * routed_scaling_factor


@torch.no_grad()
def route_topk(routing_logits, routing_bias, top_k, routed_scaling_factor):
    """Top-k on the logits, every selected expert weighs factor / top_k (`..._topk_routing_reference`,
    :350-390)."""
    logits = _biased_logits(routing_logits, routing_bias)
    _, topk_idx = torch.topk(logits, k=int(top_k), dim=1, largest=True, sorted=False)
    w = torch.full(topk_idx.shape, routed_scaling_factor / int(top_k), dtype=torch.float32)
    return topk_idx, w


def route(routing_mode, routing_logits, routing_bias, top_k, n_group, topk_group, routed_scaling_factor):
    """Dispatch on the routing mode; (topk_idx int64 [T, top_k], topk_w fp32 [T, top_k])."""
    rsf = float(routed_scaling_factor)
    if routing_mode == ROUTING_DS:
        return route_ds(routing_logits, routing_bias, top_k, n_group, topk_group, rsf)
    fn = {ROUTING_RENORM_NAIVE: route_renorm_naive, ROUTING_DEFAULT: route_default,
          ROUTING_RENORMALIZE: route_renormalize, ROUTING_LLAMA4: route_llama4, ROUTING_TOPK: route_topk}.get(routing_mode)
    if fn is None:
        raise ValueError(f"unknown routing_mode {routing_mode}")
    return fn(routing_logits, routing_bias, top_k, rsf)


def _dequant_weight(w_fp8, scale):
    """[N, K] fp8 with [N/128, K/128] block scales -> fp32."""
    w = w_fp8.to(torch.float32)
    s = torch.repeat_interleave(scale.to(torch.float32), BLOCK, dim=0)
    s = torch.repeat_interleave(s, BLOCK, dim=1)
    return w * s


def dequant_hidden(hidden_states, hidden_states_scale):
    """[T, H] fp8 with scales [H/128, T] -> fp32 [T, H]."""
    T, H = hidden_states.shape
    a = hidden_states.to(torch.float32)
    s = hidden_states_scale.to(torch.float32).permute(1, 0).contiguous()  # [T, H/128]
    s = s.unsqueeze(-1).repeat(1, 1, BLOCK).reshape(T, H)
    return a * s


@torch.no_grad()
def run_experts(hidden_states, hidden_states_scale, gemm1_weights, gemm1_weights_scale,
                gemm2_weights, gemm2_weights_scale, topk_w, topk_idx, local_expert_offset,
                num_experts_global, keep_inter=False):
    """Dequantise, then per local expert: fp32 GEMM1 -> SwiGLU -> fp32 GEMM2 -> weighted
    fp32 index_add.  No intermediate re-quantisation.  Only experts that received a token
    are dequantised (the result equals dequantising all of them)."""
    T, H = hidden_states.shape
    E_local, two_i, _ = gemm1_weights.shape
    I = two_i // 2
    A = dequant_hidden(hidden_states, hidden_states_scale)
    out = torch.zeros((T, H), dtype=torch.float32)
    expert_tokens, inter = {}, {}
    start = int(local_expert_offset)
    for le in range(E_local):
        ge = start + le
        if ge < 0 or ge >= num_experts_global:
            continue
        hit = (topk_idx == ge)
        sel = hit.any(dim=1)
        if not bool(sel.any()):
            continue
        tok = torch.nonzero(sel, as_tuple=False).squeeze(1)
        expert_tokens[le] = tok
        W13 = _dequant_weight(gemm1_weights[le], gemm1_weights_scale[le])
        W2 = _dequant_weight(gemm2_weights[le], gemm2_weights_scale[le])
        A_e = A.index_select(0, tok)
        G1 = A_e.matmul(W13.t())
        X1, X2 = G1[:, :I], G1[:, I:]
        C = (X2 / (1.0 + torch.exp(-X2))) * X1
        O = C.matmul(W2.t())
        w_e = (topk_w.index_select(0, tok) * hit.index_select(0, tok).float()).sum(dim=1)
        out.index_add_(0, tok, O * w_e.unsqueeze(1))
        if keep_inter:
            inter[le] = (G1, C, O)
    return out, expert_tokens, inter


@torch.no_grad()
def moe_forward(routing_logits, routing_bias, hidden_states, hidden_states_scale,
                gemm1_weights, gemm1_weights_scale, gemm2_weights, gemm2_weights_scale,
                local_expert_offset, routed_scaling_factor, *, routing_mode=ROUTING_DS,
                top_k=8, n_group=8, topk_group=4, keep_inter=False) -> OracleResult:
    """The whole layer for one rank's experts; all tensors on the CPU."""
    E_global = routing_logits.shape[1]
    idx, w = route(routing_mode, routing_logits, routing_bias, top_k, n_group, topk_group, routed_scaling_factor)
    out, et, inter = run_experts(hidden_states, hidden_states_scale, gemm1_weights, gemm1_weights_scale,
                                 gemm2_weights, gemm2_weights_scale, w, idx, local_expert_offset,
                                 E_global, keep_inter=keep_inter)
    return OracleResult(out, out.to(torch.bfloat16), idx, w, et, inter)


def compare_output(got_bf16: torch.Tensor, want_bf16: torch.Tensor, atol=1e-2, rtol=1e-2) -> dict:
    """Tolerance report used by every parity test: |got-want| <= atol + rtol*|want|."""
    g = got_bf16.detach().to("cpu", torch.float32)
    w = want_bf16.detach().to("cpu", torch.float32)
    if g.numel() == 0:
        return {"max_abs": 0.0, "mean_abs": 0.0, "fail_frac": 0.0, "n": 0, "finite": True}
    d = (g - w).abs()
    bad = d > (atol + rtol * w.abs())
    return {"max_abs": float(d.max()), "mean_abs": float(d.mean()),
            "fail_frac": float(bad.float().mean()), "n": g.numel(),
            "finite": bool(torch.isfinite(g).all())}


def routing_sets_equal(idx_a: torch.Tensor, idx_b: torch.Tensor) -> torch.Tensor:
    """Per-token equality of the selected expert sets (order inside a row is irrelevant)."""
    a = torch.sort(idx_a.to(torch.int64).cpu(), dim=1).values
    b = torch.sort(idx_b.to(torch.int64).cpu(), dim=1).values
    return (a == b).all(dim=1)
