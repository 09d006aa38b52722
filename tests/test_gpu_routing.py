"""GPU: routing kernel through the C ABI (b200moe_route) against the oracle: selected expert
SETS must be identical per token; weights within 4 ulp (the definition sums 256 mostly-zero
terms in an unspecified order, so the last bits of the normaliser are not pinned)."""
import dataclasses

import pytest
import torch

import util
from util import I, O

pytestmark = pytest.mark.gpu


def _check(shape, T, seed, rsf, bias_none=False):
    from justgoal_b200 import MoELayer
    d = I.make_tokens(shape, T, seed)
    bias = None if bias_none else d["routing_bias"]
    idx_o, w_o = O.route(shape.routing_mode, d["routing_logits"], bias, shape.top_k, shape.n_group,
                         shape.topk_group, rsf)
    layer = MoELayer(shape)
    idx, w = layer.route(d["routing_logits"].cuda(), None if bias is None else bias.cuda(), rsf)
    torch.cuda.synchronize()
    idx, w = idx.cpu().long(), w.cpu()
    eq = O.routing_sets_equal(idx, idx_o)
    if not bool(eq.all()):
        bad = torch.nonzero(~eq).flatten()
        margins = util.routing_margin_ulp(shape, d["routing_logits"][bad], bias)
        pytest.fail(f"{len(bad)} of {T} tokens differ in their expert set; oracle score margins (ulp): "
                    f"{margins.tolist()[:16]}")
    so, sg = torch.argsort(idx_o, dim=1), torch.argsort(idx, dim=1)
    wo, wg = w_o.gather(1, so), w.gather(1, sg)
    tol_ulp = 4 if shape.routing_mode == I.ROUTING_DS else 64   # softmax normaliser: longer sums
    assert int(util.ulp_diff(wg, wo).max()) <= tol_ulp
    assert int(idx.min()) >= 0 and int(idx.max()) < shape.num_experts


@pytest.mark.parametrize("T", [1, 7, 64, 4096])
def test_deepseek_routing_sets_bit_exact(T):
    _check(I.DEEPSEEK_V3, T, seed=T, rsf=2.5)


def test_deepseek_routing_large_and_no_bias():
    _check(I.DEEPSEEK_V3, 16384, seed=11, rsf=2.5)
    _check(I.DEEPSEEK_V3, 333, seed=12, rsf=1.0, bias_none=True)


def test_tiny_group_structure():
    _check(I.TINY_DS, 257, seed=5, rsf=2.5)


@pytest.mark.parametrize("shape", [I.QWEN3_MOE, I.TINY_RENORM])
def test_softmax_topk_renormalise(shape):
    _check(shape, 2048, seed=3, rsf=1.0)


@pytest.mark.parametrize("shape", [I.TINY_DEFAULT, I.TINY_RENORMALIZE, I.TINY_LLAMA4, I.TINY_TOPK,
                                   dataclasses.replace(I.QWEN3_MOE, routing_mode=I.ROUTING_RENORMALIZE)])
def test_other_routing_methods_of_the_family(shape):
    """softmax -> top-k, top-k -> softmax, Llama-4 top-1 -> sigmoid, plain top-k: sets exact, weights within
    the softmax tolerance, with a bias and without."""
    _check(shape, 1500, seed=9, rsf=1.5)
    _check(shape, 33, seed=10, rsf=1.0, bias_none=True)
