"""GPU, 2 ranks on 2 GPUs over NCCL: the expert-parallel layer (routing, dispatch all-to-all,
local experts through b200moe_forward_routed, combine all-to-all) against the single-process
oracle of the whole layer.  Skipped on a box with fewer than two GPUs."""
import os
import socket
import sys

import pytest
import torch

import util
from util import I, O

pytestmark = pytest.mark.gpu

SHAPE_ALL = I.MoEShape(hidden=512, intermediate=256, num_experts=64, num_local_experts=64, top_k=8, n_group=8,
                       topk_group=4, routing_mode=I.ROUTING_DS)
T_TOTAL, RSF, STD = 300, 2.5, 0.05


def _worker(rank, world, port, out_q, exchange):
    import torch.distributed as dist
    sys.path.insert(0, util.ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from justgoal_b200.ep import ExpertParallelMoE
        shape = SHAPE_ALL.with_local(SHAPE_ALL.num_experts // world)
        tokens = I.make_tokens(SHAPE_ALL, T_TOTAL, seed=9)
        per = T_TOTAL // world
        sl = slice(rank * per, (rank + 1) * per)
        weights = {k: v.cuda() for k, v in I.make_weights(shape, 9, "cpu", rank * shape.num_local_experts, std=STD).items()}
        ep = ExpertParallelMoE(shape, weights, exchange=exchange, capacity=per if exchange == "p2p" else None)
        out = ep.forward(tokens["routing_logits"][sl].cuda(), tokens["routing_bias"].cuda(),
                         tokens["hidden_states"].view(torch.uint8)[sl].cuda().view(torch.float8_e4m3fn),
                         tokens["hidden_states_scale"][:, sl].contiguous().cuda(), RSF)
        torch.cuda.synchronize()
        # route, [pack, unpack | push, barrier, barrier], the local experts (5 or 6 launches), owner-side sum
        assert ep.launches_per_step() in ((10, 11) if ep.peer is not None else (9, 10))
        if ep.peer is not None:
            # a second step on the same buffers (slots are reused, epochs grow), then the barriers' status
            out = ep.forward(tokens["routing_logits"][sl].cuda(), tokens["routing_bias"].cuda(),
                             tokens["hidden_states"].view(torch.uint8)[sl].cuda().view(torch.float8_e4m3fn),
                             tokens["hidden_states_scale"][:, sl].contiguous().cuda(), RSF)
            torch.cuda.synchronize()
            assert ep.peer.error_word() == 0
        out_q.put((rank, out.float().cpu().numpy()))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("exchange", ["nccl", "p2p"])
def test_two_gpu_expert_parallel_matches_oracle(exchange):
    import torch.multiprocessing as mp
    world = 2
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, exchange)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(util.collect(q, procs, world, 240), key=lambda r: r[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    tokens = I.make_tokens(SHAPE_ALL, T_TOTAL, seed=9)
    weights = I.make_weights(SHAPE_ALL, 9, "cpu", 0, std=STD)
    d = dict(tokens); d.update(weights); d["local_expert_offset"] = 0; d["routed_scaling_factor"] = RSF
    want = util.run_oracle(SHAPE_ALL, d)
    got = torch.cat([torch.from_numpy(r[1]) for r in results]).to(torch.bfloat16)
    rep = O.compare_output(got, want.output, util.ATOL, util.RTOL)
    assert rep["finite"] and rep["fail_frac"] == 0.0, rep
