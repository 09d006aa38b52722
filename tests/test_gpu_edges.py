"""Ragged and boundary cases of the CUDA path against the oracle: one token, the first size past the
fused small-T front end, several permutation slices, every token colliding on the same experts,
ragged last tiles.  Output tolerance as stated for the operator; integer structures exact."""
import pytest
import torch

import util
from util import I, O

pytestmark = pytest.mark.gpu


def _forward(shape, d, layer=None):
    from justgoal_b200 import MoELayer
    layer = layer or MoELayer(shape)
    out = layer.forward(*util.op_args(util.to_cuda(d)))
    torch.cuda.synchronize()
    T = int(d["hidden_states"].shape[0])
    assert layer.status(T) == 0
    return layer, out


def _check_output(shape, d, out):
    want = util.run_oracle(shape, d).output
    rep = O.compare_output(out, want, util.ATOL, util.RTOL)
    assert rep["fail_frac"] == 0.0, rep


def _check_tables(shape, d, layer, T):
    """counts, segment alignment, ascending tokens inside every expert segment, padding rows = -1,
    pair_row pointing back at the pair's token."""
    r = util.run_oracle(shape, d, keep_inter=True)
    El, K = shape.num_local_experts, shape.top_k
    rows_cap = int(layer.layout(T).rows_cap)
    counts = layer.view(T, "counts", torch.int32, (El,)).cpu()
    row0 = layer.view(T, "expert_row0", torch.int32, (El + 1,)).cpu()
    row_token = layer.view(T, "row_token", torch.int32, (rows_cap,)).cpu()
    pair_row = layer.view(T, "pair_row", torch.int32, (T, K)).cpu()
    topk = layer.view(T, "topk_idx", torch.int32, (T, K)).cpu()
    want = torch.tensor([len(r.expert_tokens.get(e, [])) for e in range(El)], dtype=torch.int32)
    assert torch.equal(counts, want)
    for e in range(El):
        a, c = int(row0[e]), int(counts[e])
        assert a % 16 == 0 and int(row0[e + 1]) - a == (c + 15) // 16 * 16
        if c:
            assert torch.equal(row_token[a:a + c].long(), r.expert_tokens[e])
        assert bool((row_token[a + c:int(row0[e + 1])] == -1).all())
    off = int(d["local_expert_offset"])
    local = (topk >= off) & (topk < off + El)
    t_of_pair = torch.arange(T).unsqueeze(1).expand(T, K)
    assert torch.equal(row_token[pair_row[local].long()].long(), t_of_pair[local])


def test_single_token():
    shape = I.TINY_DS
    d = I.make_inputs(shape, 1, seed=21)
    layer, out = _forward(shape, d)
    _check_output(shape, d, out)


@pytest.mark.parametrize("tile", [0, 16, 32, 64])
@pytest.mark.parametrize("T", [128, 129, 257])
def test_around_the_fused_front_end_boundary(T, tile):
    """T = 128 is the last size of the fused permute + gather launch, 129 the first of the sliced
    permutation (two slices of 1024 pairs), 257 crosses into a third slice.  Run with the tile the layer picks
    (128 tokens here) and with every narrow kernel family forced (several token tiles per expert)."""
    from justgoal_b200 import MoELayer
    shape = I.TINY_DS
    d = I.make_inputs(shape, T, seed=22 + T)
    layer = MoELayer(shape)
    layer.set_token_tile(tile)
    layer, out = _forward(shape, d, layer)
    _check_output(shape, d, out)
    _check_tables(shape, d, layer, T)


def test_many_slices_top4():
    """top-4 shape, 700 tokens = 2800 pairs = 3 slices; a token's pairs straddle slice borders."""
    shape = I.TINY_RENORM
    d = I.make_inputs(shape, 700, seed=31)
    layer, out = _forward(shape, d)
    _check_output(shape, d, out)
    _check_tables(shape, d, layer, 700)


def test_all_tokens_collide_on_the_same_experts():
    """Identical routing rows: every token picks the same top-k experts, so a few experts receive T
    rows each (several token tiles with a ragged last one) and all others none."""
    shape = I.TINY_DS
    T = 300
    d = I.make_inputs(shape, T, seed=41)
    d["routing_logits"] = d["routing_logits"][:1].repeat(T, 1).contiguous()
    layer, out = _forward(shape, d)
    _check_output(shape, d, out)
    _check_tables(shape, d, layer, T)
    counts = layer.view(T, "counts", torch.int32, (shape.num_local_experts,)).cpu()
    assert set(counts.tolist()) <= {0, T}


def test_small_forwards_back_to_back_without_a_host_wait():
    """Up to 128 tokens the forward is four launches and nothing else on the stream, each allowed to start under
    the tail of the one before: the front end of call n+1 overlaps the combine of call n, clears the head of the
    workspace itself, meets at two words owned by the handle, and GEMM1 schedules itself from the routing result
    while the front end still gathers.  Twelve forwards with two alternating token sets and sizes are queued with
    no host wait in between; every result must match the oracle and the error word must stay clear."""
    from justgoal_b200 import MoELayer
    shape = I.TINY_DS
    layer = MoELayer(shape)
    cases = [I.make_inputs(shape, T, seed=seed) for T, seed in ((64, 61), (7, 62), (128, 63))]
    args = [util.op_args(util.to_cuda(d)) for d in cases]
    outs = []
    for n in range(12):
        outs.append((n % 3, layer.forward(*args[n % 3]).clone()))
    torch.cuda.synchronize()
    for T in (64, 7, 128):
        assert layer.status(T) == 0
    want = [util.run_oracle(shape, d).output for d in cases]
    for k, out in outs:
        rep = O.compare_output(out, want[k], util.ATOL, util.RTOL)
        assert rep["fail_frac"] == 0.0, (k, rep)
    # the same inputs give the same bits every time (fixed summation order, whoever was quick or slow)
    for k in range(3):
        same = [o for kk, o in outs if kk == k]
        assert all(torch.equal(same[0].view(torch.int16), o.view(torch.int16)) for o in same[1:])


@pytest.mark.parametrize("shape_name,T,tile", [("TINY_DS", 64, 16), ("TINY_DS", 150, 32), ("TINY_DS", 400, 64),
                                               ("TINY_RENORM", 20, 16), ("TINY_RENORM", 130, 32)])
def test_fused_combine_equals_the_combine_kernel_bit_for_bit(shape_name, T, tile):
    """With the fused combine switched on and narrow token tiles the forward has no combine launch: the GEMM2 unit
    that delivers a token's last row sums the token's rows in its epilogue.  forward_routed keeps the separate combine kernel; both add the same
    rows in the same order, so the bf16 outputs must be identical - including tokens without a local expert (zero
    rows) and a hidden size that is not a multiple of 256 (TINY_RENORM: the last unit has one weight tile)."""
    from justgoal_b200 import MoELayer
    shape = getattr(I, shape_name)
    d = I.make_inputs(shape, T, seed=70 + T)
    layer = MoELayer(shape)
    layer.set_token_tile(tile)                         # every narrow kernel family, whatever the layer would pick
    assert layer.launches_per_forward(T) == (4 if T <= 128 else 6)
    layer.set_fused_combine(True)                      # off by default
    assert layer.launches_per_forward(T) == (3 if T <= 128 else 5)
    _, out = _forward(shape, d, layer)
    assert int(layer.layout(T).token_tile) == tile
    _check_output(shape, d, out)
    K = shape.top_k
    idx = layer.view(T, "topk_idx", torch.int32, (T, K)).clone()
    w = layer.view(T, "topk_w", torch.float32, (T, K)).clone()
    dc = util.to_cuda(d)
    out2 = layer.forward_routed(idx, w, dc["hidden_states"], dc["hidden_states_scale"], dc["gemm1_weights"],
                                dc["gemm1_weights_scale"], dc["gemm2_weights"], dc["gemm2_weights_scale"],
                                int(d["local_expert_offset"]), out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    assert layer.status(T) == 0
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16))


def test_tma_gathered_token_rows_give_the_same_bits():
    """Optional form of GEMM1 for 128-token tiles: the token rows come from hidden_states by four-row TMA gathers
    through the token-of-row table instead of from a gathered copy (no gather launch).  Ragged last tiles, padding
    rows (token -1: the gather reads zeros) and rows of the next expert inside a tile are all in this case."""
    from justgoal_b200 import MoELayer
    shape, T = I.TINY_DS, 600
    d = I.make_inputs(shape, T, seed=91)
    layer = MoELayer(shape)
    assert int(layer.layout(T).token_tile) == 128
    _, out1 = _forward(shape, d, layer)
    out1 = out1.clone()
    n1 = layer.launches_per_forward(T)
    layer.set_tma_gather(True)
    assert layer.launches_per_forward(T) == n1 - 1
    layer.workspace(T).fill_(0xFF)          # stale token ids past the last row must be harmless
    _, out2 = _forward(shape, d, layer)
    assert torch.equal(out1.view(torch.int16), out2.view(torch.int16))
    _check_output(shape, d, out2)


def test_workspace_reuse_across_sizes():
    """One layer object, shrinking and growing token counts back to back (workspace buckets, stale
    tables from the larger call must not leak into the smaller one)."""
    from justgoal_b200 import MoELayer
    shape = I.TINY_DS
    layer = MoELayer(shape)
    for T, seed in ((513, 51), (5, 52), (130, 53), (64, 54)):
        d = I.make_inputs(shape, T, seed=seed)
        _, out = _forward(shape, d, layer)
        _check_output(shape, d, out)


def test_ep_combine_kernel_matches_restatement():
    """b200moe_ep_combine: fp32 sum in rank order of the fp16 partial rows a token's ranks sent back."""
    from justgoal_b200 import MoELayer
    shape = I.TINY_DS
    layer = MoELayer(shape)
    T, world, H = 37, 4, shape.hidden
    g = torch.Generator().manual_seed(61)
    has = torch.rand(world, T, generator=g) < 0.6
    has[:, 5] = False                                     # a token nobody computed: zeros
    row_of = torch.full((world, T), -1, dtype=torch.int32)
    row_of[has] = torch.arange(int(has.sum()), dtype=torch.int32)
    back = torch.randn(int(has.sum()), H, generator=g).to(torch.float16)
    got = layer.ep_combine(back.cuda(), row_of.cuda(), T).cpu()
    want = torch.zeros(T, H, dtype=torch.float32)
    for r in range(world):
        sel = row_of[r] >= 0
        want[sel] += back[row_of[r][sel].long()].float()
    assert torch.equal(got.view(torch.int16), want.to(torch.bfloat16).view(torch.int16))
    assert bool((got[5].float() == 0).all())


def test_forward_routed_bf16_and_fp16_are_the_rounded_fp32_result():
    from justgoal_b200 import MoELayer
    shape = I.TINY_DS
    T = 45
    d = util.to_cuda(I.make_inputs(shape, T, seed=62))
    layer = MoELayer(shape)
    idx, w = layer.route(d["routing_logits"], d["routing_bias"], d["routed_scaling_factor"])
    args = (idx, w, d["hidden_states"], d["hidden_states_scale"], d["gemm1_weights"], d["gemm1_weights_scale"],
            d["gemm2_weights"], d["gemm2_weights_scale"], d["local_expert_offset"])
    f32 = layer.forward_routed(*args).clone()
    b16 = layer.forward_routed(*args, out_dtype=torch.bfloat16).clone()
    h16 = layer.forward_routed(*args, out_dtype=torch.float16)
    torch.cuda.synchronize()
    assert torch.equal(b16.view(torch.int16), f32.to(torch.bfloat16).view(torch.int16))
    assert torch.equal(h16.view(torch.int16), f32.to(torch.float16).view(torch.int16))


def test_ep_pack_unpack_round_trip():
    """b200moe_ep_pack / _unpack: the wire row is [fp8 row | scales | ids | weights] padded to 16 bytes;
    unpacking returns the operator's layouts (scales K-block major) for exactly the packed tokens."""
    from justgoal_b200 import MoELayer
    shape = I.TINY_DS
    T = 50
    d = util.to_cuda(I.make_inputs(shape, T, seed=63))
    layer = MoELayer(shape)
    idx, w = layer.route(d["routing_logits"], d["routing_bias"], d["routed_scaling_factor"])
    send = torch.tensor([3, 3, 49, 0, 17, 20, 21, 48], dtype=torch.int64, device="cuda")
    wire = layer.ep_pack(d["hidden_states"], d["hidden_states_scale"], idx, w, send)
    H, K, KB = shape.hidden, shape.top_k, shape.hidden // 128
    assert wire.shape == (send.numel(), (H + 4 * KB + 8 * K + 15) // 16 * 16) == (send.numel(), layer.ep_row_bytes())
    assert torch.equal(wire[:, :H], d["hidden_states"].view(torch.uint8)[send])
    x, sc, i2, w2 = layer.ep_unpack(wire)
    torch.cuda.synchronize()
    assert torch.equal(x.view(torch.uint8), d["hidden_states"].view(torch.uint8)[send])
    assert torch.equal(sc, d["hidden_states_scale"][:, send])
    assert torch.equal(i2, idx[send]) and torch.equal(w2, w[send])


def test_host_pipeline_returns_every_steps_own_result():
    """HostPipeline overlaps copies and forwards of consecutive steps over two sets of device buffers:
    each step's host output must be that step's own result, bit for bit."""
    from justgoal_b200 import HostPipeline, MoELayer
    shape, T = I.TINY_DS, 40
    layer = MoELayer(shape)
    base = util.to_cuda(I.make_inputs(shape, T, seed=70))
    static = [base[k] for k in ("routing_bias", "gemm1_weights", "gemm1_weights_scale", "gemm2_weights",
                                "gemm2_weights_scale", "local_expert_offset", "routed_scaling_factor")]
    steps = []
    for i in range(5):
        tok = I.make_tokens(shape, T, seed=71 + i, device="cpu")
        steps.append(dict(logits=tok["routing_logits"].pin_memory(), hidden=tok["hidden_states"].pin_memory(),
                          scale=tok["hidden_states_scale"].pin_memory(),
                          out=torch.empty(T, shape.hidden, dtype=torch.bfloat16).pin_memory()))
    pipe = HostPipeline(layer, T, *static)
    for s in steps:
        pipe.step(s["logits"], s["hidden"], s["scale"], s["out"])
    pipe.drain()
    for s in steps:
        want = layer.forward(s["logits"].cuda(), static[0], s["hidden"].cuda(), s["scale"].cuda(), *static[1:])
        torch.cuda.synchronize()
        assert torch.equal(s["out"].view(torch.int16), want.cpu().view(torch.int16))
