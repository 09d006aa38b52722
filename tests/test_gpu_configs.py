"""GPU: the benchmark configurations at full size (DeepSeek-V3 shape, 32 local of 256 experts)
against the oracle, plus size-independent properties.  Inputs are drawn on the GPU (the CPU
draw of 1.4 GB of weights takes minutes) and copied to the host for the oracle."""
import pytest
import torch

import util
from util import I, O

pytestmark = pytest.mark.gpu

PREFILL_BOOST = ((0, 8, 16, 24), 0.328)


@pytest.fixture(scope="module")
def ds_weights():
    return I.make_weights(I.DEEPSEEK_V3, seed=0, device="cuda")


def _inputs(T, weights, seed=0, boost=None, offset=0):
    d = I.make_tokens(I.DEEPSEEK_V3, T, seed, "cuda", boost)
    d.update(weights)
    d["local_expert_offset"] = offset
    d["routed_scaling_factor"] = 2.5
    return d


def _cpu(d):
    return {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}


def _check_against_oracle(T, weights, boost=None, seed=0, tile=0):
    from justgoal_b200 import MoELayer
    shape = I.DEEPSEEK_V3
    d = _inputs(T, weights, seed, boost)
    layer = MoELayer(shape)
    if tile:
        layer.set_token_tile(tile)
    out = layer.forward(*util.op_args(d))
    torch.cuda.synchronize()
    assert layer.status(T) == 0
    assert not tile or int(layer.layout(T).token_tile) == tile
    r = util.run_oracle(shape, _cpu(d))
    idx = layer.view(T, "topk_idx", torch.int32, (T, shape.top_k)).cpu()
    assert bool(O.routing_sets_equal(idx, r.topk_idx).all())
    rep = O.compare_output(out, r.output, util.ATOL, util.RTOL)
    assert rep["finite"] and rep["fail_frac"] == 0.0, rep
    return rep


def test_decode_t64(ds_weights):
    _check_against_oracle(64, ds_weights)


@pytest.mark.parametrize("tile", [0, 32, 64])
def test_mid_t901(ds_weights, tile):
    """Ragged counts at full size: the tile the layer picks for 901 tokens (128), and the 32- and 64-token kernel
    families forced through set_token_tile (several token tiles per expert, claimed chunks)."""
    _check_against_oracle(901, ds_weights, seed=7, tile=tile)


def test_token_tile_choice():
    """16 tokens while an expert expects about seven rows or fewer, 128 from about nine, 32 in between."""
    from justgoal_b200 import MoELayer
    layer = MoELayer(I.DEEPSEEK_V3)
    got = {T: int(layer.layout(T).token_tile) for T in (1, 64, 224, 256, 288, 320, 901, 4096)}
    assert got == {1: 16, 64: 16, 224: 16, 256: 32, 288: 32, 320: 128, 901: 128, 4096: 128}


def test_prefill_t4096_skewed(ds_weights):
    _check_against_oracle(4096, ds_weights, boost=PREFILL_BOOST)


def test_scaling_factor_doubling_is_exact(ds_weights):
    """out(2*f) == 2*out(f) bit for bit: the factor enters once, as a power-of-two multiple."""
    from justgoal_b200 import MoELayer
    d = _inputs(4096, ds_weights, 0, PREFILL_BOOST)
    layer = MoELayer(I.DEEPSEEK_V3)
    a = layer.forward(*util.op_args(d)).clone()
    d["routed_scaling_factor"] = 5.0
    b = layer.forward(*util.op_args(d))
    torch.cuda.synchronize()
    assert torch.equal((a.float() * 2).to(torch.bfloat16).view(torch.int16), b.view(torch.int16))


def _permuted(d, perm):
    d2 = dict(d)
    d2["routing_logits"] = d["routing_logits"][perm].contiguous()
    d2["hidden_states"] = d["hidden_states"].view(torch.uint8)[perm].contiguous().view(torch.float8_e4m3fn)
    d2["hidden_states_scale"] = d["hidden_states_scale"][:, perm].contiguous()
    return d2


def test_token_permutation_equivariance(ds_weights):
    """Permuting the tokens permutes the output rows.  With one token tile per expert (T=64) the
    result is bit-identical: columns of a tile do not interact and the combine order is by
    expert.  With several tiles per expert a token may move to another tile, whose K range is
    cut differently by the stream-K schedule (another fp32 summation order), so there only
    the last bf16 bit of a few elements may move."""
    from justgoal_b200 import MoELayer
    layer = MoELayer(I.DEEPSEEK_V3)
    for T, exact in ((64, True), (1000, False)):
        d = _inputs(T, ds_weights, 3)
        a = layer.forward(*util.op_args(d)).clone()
        perm = torch.randperm(T, generator=torch.Generator().manual_seed(1)).cuda()
        b = layer.forward(*util.op_args(_permuted(d, perm)))
        torch.cuda.synchronize()
        if exact:
            assert torch.equal(a[perm].view(torch.int16), b.view(torch.int16))
        else:
            differs = (a[perm].view(torch.int16) != b.view(torch.int16)).float().mean().item()
            assert differs < 2e-3, differs
            rep = O.compare_output(b, a[perm], 1e-3, 8e-3)      # one bf16 ulp = 2^-8 relative
            assert rep["fail_frac"] == 0.0, rep


def test_nonzero_expert_offset_matches_shifted_weights(ds_weights):
    """local_expert_offset = 32 with the same 32 weight tensors: only tokens routed to experts
    32..63 contribute; checked against the oracle."""
    from justgoal_b200 import MoELayer
    shape = I.DEEPSEEK_V3
    d = _inputs(256, ds_weights, 5, offset=32)
    layer = MoELayer(shape)
    out = layer.forward(*util.op_args(d))
    torch.cuda.synchronize()
    r = util.run_oracle(shape, _cpu(d))
    rep = O.compare_output(out, r.output, util.ATOL, util.RTOL)
    assert rep["fail_frac"] == 0.0, rep


def _share_check(shape, T, offset, rsf, seed):
    """One rank's share of an expert-parallel configuration (its local experts, all T tokens)."""
    from justgoal_b200 import MoELayer
    d = I.make_tokens(shape, T, seed, "cuda")
    d.update(I.make_weights(shape, seed, "cuda", offset))
    d["local_expert_offset"] = offset
    d["routed_scaling_factor"] = rsf
    layer = MoELayer(shape)
    out = layer.forward(*util.op_args(d))
    torch.cuda.synchronize()
    assert layer.status(T) == 0
    r = util.run_oracle(shape, _cpu(d))
    idx = layer.view(T, "topk_idx", torch.int32, (T, shape.top_k)).cpu()
    assert bool(O.routing_sets_equal(idx, r.topk_idx).all())
    rep = O.compare_output(out, r.output, util.ATOL, util.RTOL)
    assert rep["finite"] and rep["fail_frac"] == 0.0, rep


def test_ep_share_deepseek_128_local_experts():
    """The 2-GPU expert-parallel share of the 256-expert layer: 128 local experts, second rank."""
    _share_check(I.DEEPSEEK_V3.with_local(128), 512, 128, 2.5, seed=21)


def test_ep_share_qwen3_shape():
    """Qwen3-MoE shape (hidden 4096, intermediate 1536, 128 experts, 16 per rank, softmax top-8,
    renormalised, no groups), one rank's share of the 8-GPU configuration at its full T=2048."""
    _share_check(I.QWEN3_MOE, 2048, 48, 1.0, seed=22)


def test_sm_pair_kernels_match_the_single_sm_kernels():
    """The cta_group::2 family (B200MOE_PAIR=1: two CTAs of a cluster share every weight tile) computes the same
    arithmetic as the default single-SM family; the two MMA forms need not order their internal sums alike, so
    the outputs agree to a bf16 unit in the last place, not bit for bit.  Run in child processes because the
    switch is read once per process."""
    import os
    import subprocess
    import sys
    code = r"""
import sys, torch
sys.path.insert(0, %r); sys.path.insert(0, %r)
import util
from util import I
from justgoal_b200 import MoELayer
outs = []
for shape, T, seed in ((I.TINY_RENORM, 700, 31), (I.TINY_DS, 2000, 5)):
    d = I.make_inputs(shape, T, seed=seed)
    layer = MoELayer(shape)
    out = layer.forward(*util.op_args(util.to_cuda(d)))
    torch.cuda.synchronize()
    assert layer.status(T) == 0 and int(layer.layout(T).token_tile) == 128
    outs.append(out.cpu())
torch.save(outs, sys.argv[1])
""" % (util.ROOT, os.path.join(util.ROOT, "tests"))
    import tempfile
    res = {}
    with tempfile.TemporaryDirectory() as tmp:
        for pair in ("0", "1"):
            path = os.path.join(tmp, f"out{pair}.pt")
            env = dict(os.environ, B200MOE_PAIR=pair)
            r = subprocess.run([sys.executable, "-c", code, path], env=env, capture_output=True, text=True, timeout=600)
            assert r.returncode == 0, r.stderr[-2000:]
            res[pair] = torch.load(path)
    for a, b in zip(res["0"], res["1"]):
        a, b = a.float(), b.float()
        assert bool(((a - b).abs() <= 2.0 ** -7 * torch.maximum(a.abs(), b.abs()) + 1e-4).all())
        assert float((a != b).float().mean()) < 0.05
