"""GPU (one device): the expert-parallel step - push, barrier, slot unpack, local experts with the result rows
stored straight into the owners' buffers, owner-side sum; and the pack / unpack / combine kernels of the
all-to-all form - with one process playing all ranks in turn, against the oracle of the WHOLE layer.
Same bar as every parity test: |got - want| <= 1e-2 + 1e-2 |want|, no failing element.  Also: a barrier
whose peer never arrives gives up after its wait limit, reports through the status word, and the next
barrier on the same buffers works."""
import ctypes as C

import pytest
import torch

import util
from util import I, O

pytestmark = pytest.mark.gpu

TINY_ALL = I.MoEShape(hidden=512, intermediate=256, num_experts=64, num_local_experts=64, top_k=8, n_group=8,
                      topk_group=4, routing_mode=I.ROUTING_DS)


def _split_tokens(tokens, sizes):
    out, a = [], 0
    for n in sizes:
        sl = slice(a, a + n)
        out.append((tokens["routing_logits"][sl].cuda(), tokens["routing_bias"].cuda(),
                    tokens["hidden_states"].view(torch.uint8)[sl].cuda().view(torch.float8_e4m3fn),
                    tokens["hidden_states_scale"][:, sl].contiguous().cuda()))
        a += n
    return out


def _oracle_by_slices(shape_all, tokens, weights_of_rank, world, rsf):
    """fp32 sum over ALL experts, one rank's slice of the weights on the host at a time, one rounding."""
    El = shape_all.num_experts // world
    idx, w = O.route(shape_all.routing_mode, tokens["routing_logits"], tokens["routing_bias"], shape_all.top_k,
                     shape_all.n_group, shape_all.topk_group, rsf)
    total = None
    for r in range(world):
        wr = {k: v.cpu() for k, v in weights_of_rank(r).items()}
        part, _, _ = O.run_experts(tokens["hidden_states"], tokens["hidden_states_scale"], wr["gemm1_weights"],
                                   wr["gemm1_weights_scale"], wr["gemm2_weights"], wr["gemm2_weights_scale"], w, idx,
                                   r * El, shape_all.num_experts)
        total = part if total is None else total + part
    return total.to(torch.bfloat16)


def _check(got_list, want, what):
    got = torch.cat(got_list).cpu()
    rep = O.compare_output(got, want, util.ATOL, util.RTOL)
    assert rep["finite"] and rep["fail_frac"] == 0.0, (what, rep)


@pytest.mark.parametrize("world", [2, 4])
def test_all_ranks_on_one_device_match_the_oracle(world):
    from ep_emu import EmulatedRanks
    T, rsf, std, seed = 300, 2.5, 0.05, 9
    shape = TINY_ALL.with_local(TINY_ALL.num_experts // world)
    tokens = I.make_tokens(TINY_ALL, T, seed=seed)
    w_cpu = [I.make_weights(shape, seed, "cpu", r * shape.num_local_experts, std=std) for r in range(world)]
    w_gpu = [{k: v.cuda() for k, v in w.items()} for w in w_cpu]
    # ragged: the last rank brings fewer tokens than the slots hold
    per = T // world
    sizes = [per] * (world - 1) + [per - 7]
    toks = _split_tokens(tokens, sizes)
    used = sum(sizes)
    sub = {k: (v[:used] if k != "hidden_states_scale" else v[:, :used].contiguous()) for k, v in tokens.items()
           if k != "routing_bias"}
    sub["routing_bias"] = tokens["routing_bias"]
    want = _oracle_by_slices(TINY_ALL, sub, lambda r: w_cpu[r], world, rsf)
    emu = EmulatedRanks(TINY_ALL, world, w_gpu, cap=per)
    _check(emu.step_peer(toks, rsf), want, "peer-memory exchange, step 1")
    _check(emu.step_peer(toks, rsf), want, "peer-memory exchange, step 2 (slots reused, epochs grow)")
    _check(emu.step_alltoall(toks, rsf), want, "all-to-all form")
    _check(emu.step_peer_long(toks, rsf), want, "peer-memory exchange through the stand-alone entry points")
    # a step in which rank 0 brings no token at all
    toks0 = [(toks[0][0][:0], toks[0][1], toks[0][2][:0], toks[0][3][:, :0].contiguous())] + toks[1:]
    outs = emu.step_peer(toks0, rsf)
    assert outs[0].shape[0] == 0
    sub2 = {k: (v[per:used] if k != "hidden_states_scale" else v[:, per:used].contiguous()) for k, v in tokens.items()
            if k != "routing_bias"}
    sub2["routing_bias"] = tokens["routing_bias"]
    _check(outs[1:], _oracle_by_slices(TINY_ALL, sub2, lambda r: w_cpu[r], world, rsf), "rank 0 empty")


def _host_has_gb(n):
    try:
        for line in open("/proc/meminfo"):
            if line.startswith("MemAvailable"):
                return int(line.split()[1]) / 1e6 >= n
    except OSError:
        pass
    return False


@pytest.mark.parametrize("name", ["deepseek_v3_8_ranks", "qwen3_8_ranks"])
def test_full_size_expert_parallel_shapes_on_one_device(name):
    """The benchmark's expert-parallel configurations at their real shapes, 8 ranks played on one GPU:
    DeepSeek-V3 (256 experts, 32 per rank) on 512 tokens; the Qwen3-MoE shape (128 experts, 16 per rank,
    softmax routing) on 2048 tokens."""
    from ep_emu import EmulatedRanks
    if not _host_has_gb(24):
        pytest.skip("needs 24 GB of host memory for the oracle")
    world = 8
    if name == "deepseek_v3_8_ranks":
        shape_all, T, rsf = I.DEEPSEEK_V3.with_local(256), 512, 2.5
    else:
        shape_all, T, rsf = I.QWEN3_MOE.with_local(128), 2048, 1.0
    shape = shape_all.with_local(shape_all.num_experts // world)
    tokens = I.make_tokens(shape_all, T, seed=3)
    w_gpu = [I.make_weights(shape, 3, "cuda", r * shape.num_local_experts) for r in range(world)]
    per = T // world
    toks = _split_tokens(tokens, [per] * world)
    emu = EmulatedRanks(shape_all, world, w_gpu, cap=per)
    got_peer = emu.step_peer(toks, rsf)
    got_a2a = emu.step_alltoall(toks, rsf)
    want = _oracle_by_slices(shape_all, tokens, lambda r: w_gpu[r], world, rsf)
    _check(got_peer, want, name + " peer-memory exchange")
    _check(got_a2a, want, name + " all-to-all form")


def test_barrier_gives_up_when_the_peer_never_arrives():
    """World of 2 on one device; the peer's flag is never written.  With a 2 ms limit the barrier kernel must
    return by itself, leave 7 in the status word (read through b200moe_status), and a later barrier whose flag
    is there must pass on the same buffers."""
    from justgoal_b200 import MoELayer, _lib
    from justgoal_b200.ep import PeerExchange
    shape = TINY_ALL.with_local(32)
    layer = MoELayer(shape)
    layer.set_wait_limit(2e-3)
    n = PeerExchange.buffer_bytes(layer, shape, 8, 2)
    bufs = [torch.zeros(n, dtype=torch.uint8, device="cuda") for _ in range(2)]
    px = PeerExchange(layer, shape, 8, None, None, local_buffers=bufs, rank=0)
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    px.barrier()                              # epoch 1: flags[1] stays 0
    t1.record()
    torch.cuda.synchronize()                  # the kernel came back by itself
    assert 1.0 < t0.elapsed_time(t1) < 500.0
    assert px.error_word() == 7
    word = C.c_int(0)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = _lib.lib.b200moe_status(layer._h, C.c_void_p(px.status.data_ptr()), stream, C.byref(word))
    assert rc == -5 and word.value == 7       # B200MOE_E_KERNEL
    assert int(px.flags[0]) == 1              # its own arrival was published to both buffers
    assert int(bufs[1][:4].view(torch.int32)[0]) == 1
    px.clear_error()
    px.flags[1] = 2                           # the peer arrives for the next epoch
    px.barrier()
    torch.cuda.synchronize()
    assert px.error_word() == 0
