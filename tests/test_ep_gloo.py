"""CPU, world_size 2 over gloo: the expert-parallel exchange (dispatch plan, all-to-all, combine)
with the oracle standing in for the local routing and expert math.  The two ranks together must
reproduce the single-process oracle of the whole layer on all tokens."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import util
from util import I, O

SHAPE_ALL = I.MoEShape(hidden=512, intermediate=256, num_experts=64, num_local_experts=64, top_k=8, n_group=8,
                       topk_group=4, routing_mode=I.ROUTING_DS)
T_TOTAL, RSF, STD = 26, 2.5, 0.05


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_q):
    sys.path.insert(0, util.ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from justgoal_b200.ep import ExpertParallelMoE
        shape = SHAPE_ALL.with_local(SHAPE_ALL.num_experts // world)
        tokens = I.make_tokens(SHAPE_ALL, T_TOTAL, seed=9)
        per = T_TOTAL // world
        sl = slice(rank * per, (rank + 1) * per)
        weights = I.make_weights(shape, 9, "cpu", rank * shape.num_local_experts, std=STD)

        class OracleBackend:
            """The five per-rank steps on the CPU: the oracle for routing and experts, plain torch
            restatements of the pack / unpack / combine kernels (same wire format)."""
            KB = shape.hidden // 128

            def route(self, logits, bias, rsf):
                idx, w = O.route_ds(logits, bias, shape.top_k, shape.n_group, shape.topk_group, rsf)
                return idx.to(torch.int32), w

            def pack(self, hidden, hscale, idx, w, send_token):
                rows = [hidden.view(torch.uint8)[send_token],
                        hscale.t()[send_token].contiguous().view(torch.uint8).reshape(len(send_token), -1),
                        idx[send_token].contiguous().view(torch.uint8).reshape(len(send_token), -1),
                        w[send_token].contiguous().view(torch.uint8).reshape(len(send_token), -1)]
                wire = torch.cat(rows, dim=1)
                pad = (-wire.shape[1]) % 16
                return torch.nn.functional.pad(wire, (0, pad)).contiguous()

            def unpack(self, wire):
                H, K, KB = shape.hidden, shape.top_k, self.KB
                x = wire[:, :H].contiguous().view(torch.float8_e4m3fn)
                sc = wire[:, H:H + 4 * KB].contiguous().view(torch.float32).t().contiguous()
                idx = wire[:, H + 4 * KB:H + 4 * KB + 4 * K].contiguous().view(torch.int32)
                w = wire[:, H + 4 * KB + 4 * K:H + 4 * KB + 8 * K].contiguous().view(torch.float32)
                return x, sc, idx, w

            def experts(self, idx, w, hidden, hscale):
                out, _, _ = O.run_experts(hidden, hscale, weights["gemm1_weights"], weights["gemm1_weights_scale"],
                                          weights["gemm2_weights"], weights["gemm2_weights_scale"], w, idx.long(),
                                          rank * shape.num_local_experts, shape.num_experts)
                return out.to(torch.float16)                   # partial rows travel as fp16

            def combine(self, back, row_of, T):
                acc = torch.zeros(T, back.shape[1], dtype=torch.float32)     # fp32 sum in rank order, one rounding
                for r in range(row_of.shape[0]):
                    has = row_of[r] >= 0
                    acc[has] += back[row_of[r][has].long()].float()
                return acc.to(torch.bfloat16)

        ep = ExpertParallelMoE(shape, weights, backend=OracleBackend())
        out = ep.forward(tokens["routing_logits"][sl], tokens["routing_bias"],
                         tokens["hidden_states"].view(torch.uint8)[sl].view(torch.float8_e4m3fn),
                         tokens["hidden_states_scale"][:, sl].contiguous(), RSF)
        plan = ep.last_plan
        assert ep.launches_per_step() == 0          # no kernel of the library behind the oracle backend
        out_q.put((rank, out.float().numpy(), plan.send_counts, plan.recv_counts, plan.send_token.tolist()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_ranks_reproduce_the_single_process_layer(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(util.collect(q, procs, world, 240), key=lambda r: r[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # whole layer in one process
    tokens = I.make_tokens(SHAPE_ALL, T_TOTAL, seed=9)
    weights = I.make_weights(SHAPE_ALL, 9, "cpu", 0, std=STD)
    d = dict(tokens); d.update(weights); d["local_expert_offset"] = 0; d["routed_scaling_factor"] = RSF
    want = util.run_oracle(SHAPE_ALL, d)
    got = torch.cat([torch.from_numpy(r[1]) for r in results]).to(torch.bfloat16)
    per = T_TOTAL // world                                   # tokens beyond world*per belong to no rank
    rep = O.compare_output(got, want.output[:world * per], 1e-2, 1e-2)    # fp16 partial rows on the wire
    assert rep["fail_frac"] == 0.0, rep
    # plan invariants: what rank a sends to b is what b receives from a; no (token, rank) pair twice
    per = T_TOTAL // world
    for a in range(world):
        for b in range(world):
            assert results[a][2][b] == results[b][3][a]
        sent = results[a][4]
        off = 0
        for b in range(world):
            seg = sent[off:off + results[a][2][b]]
            assert seg == sorted(set(seg)) and all(0 <= t < per for t in seg)
            # token t is sent to rank b exactly when one of its experts lives there
            idx = want.topk_idx[a * per:(a + 1) * per]
            need = sorted(torch.nonzero(((idx // (SHAPE_ALL.num_experts // world)) == b).any(dim=1)).flatten().tolist())
            assert seg == need
            off += results[a][2][b]
