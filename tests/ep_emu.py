"""One process plays every rank of the expert-parallel step on ONE GPU (test infrastructure).

The ranks' kernels - exactly the ones a multi-GPU run launches, through the same Python wrappers and
C-ABI entry points - are issued in turn on one stream.  "Peer" buffers are plain allocations on this
device.  No kernel ever waits for another kernel: before a rank's barrier kernel runs, the flags its peers
would have written are set from the host side of the stream, so the barrier finds them and returns."""
import torch

from justgoal_b200 import MoELayer
from justgoal_b200.ep import PeerExchange, plan_dispatch, send_counts_of


class EmulatedRanks:
    def __init__(self, shape_all, world, weights, cap):
        """`weights[r]`: rank r's expert weights (CUDA); `cap`: token slots per rank in the peer buffers."""
        self.world, self.cap = world, cap
        self.shape = shape_all.with_local(shape_all.num_experts // world)
        self.weights = weights
        self.layers = [MoELayer(self.shape) for _ in range(world)]
        n = PeerExchange.buffer_bytes(self.layers[0], self.shape, cap, world)
        self.bufs = [torch.zeros(n, dtype=torch.uint8, device="cuda") for _ in range(world)]
        self.px = [PeerExchange(self.layers[r], self.shape, cap, None, None, local_buffers=self.bufs, rank=r)
                   for r in range(world)]

    def offset(self, r):
        return r * self.shape.num_local_experts

    def _barrier(self, r):
        px = self.px[r]
        px.flags[:self.world].fill_(px.epoch + 1)      # what the peers' barrier kernels would have stored
        px.barrier()

    def step_peer(self, toks, rsf):
        """toks[r] = (logits, bias, hidden fp8, hidden_scale [H/128, T_r]) of rank r; returns bf16 outputs per rank."""
        W = self.world
        routed = []
        for r in range(W):
            lg, bias, hid, sc = toks[r]
            idx, w = self.layers[r].route(lg, bias, rsf)
            routed.append(idx)
            self.px[r].push(hid, sc, idx, w)
        for r in range(W):
            self._barrier(r)
        for r in range(W):
            self.px[r].experts_to_peers(self.weights[r], self.offset(r))
        for r in range(W):
            self._barrier(r)
        outs = [self.px[r].combine(routed[r], int(toks[r][2].shape[0])) for r in range(W)]
        torch.cuda.synchronize()
        for r in range(W):
            assert self.px[r].error_word() == 0
            assert self.layers[r].status(W * self.cap) == 0
        return outs

    def step_peer_long(self, toks, rsf):
        """The same exchange through the stand-alone entry points: slot unpack copy, b200moe_forward_routed with
        fp16 partial rows, b200moe_ep_return."""
        W = self.world
        routed = []
        for r in range(W):
            lg, bias, hid, sc = toks[r]
            idx, w = self.layers[r].route(lg, bias, rsf)
            routed.append(idx)
            self.px[r].push(hid, sc, idx, w)
        for r in range(W):
            self._barrier(r)
        for r in range(W):
            x, sc, i, w = self.px[r].unpack()
            part = self.layers[r].forward_routed(i, w, x, sc, self.weights[r]["gemm1_weights"],
                                                 self.weights[r]["gemm1_weights_scale"], self.weights[r]["gemm2_weights"],
                                                 self.weights[r]["gemm2_weights_scale"], self.offset(r),
                                                 out_dtype=torch.float16)
            self.px[r].give_back(part, i)
        for r in range(W):
            self._barrier(r)
        outs = [self.px[r].combine(routed[r], int(toks[r][2].shape[0])) for r in range(W)]
        torch.cuda.synchronize()
        return outs

    def step_alltoall(self, toks, rsf):
        """The library-collective form of the step with the two all-to-alls done by device copies."""
        W, El = self.world, self.shape.num_local_experts
        routed, counts = [], []
        for r in range(W):
            lg, bias, hid, sc = toks[r]
            idx, w = self.layers[r].route(lg, bias, rsf)
            routed.append((idx, w))
            counts.append(send_counts_of(idx, El, W))
        counts = torch.stack(counts)                                   # [source, destination]
        plans, wires = [], []
        for r in range(W):
            idx, w = routed[r]
            plan = plan_dispatch(idx, El, W, recv_counts=counts[:, r].contiguous())
            plans.append(plan)
            wires.append(self.layers[r].ep_pack(toks[r][2], toks[r][3], idx, w, plan.send_token))
        starts = [[sum(plans[q].send_counts[:d]) for d in range(W)] for q in range(W)]
        parts = []
        for r in range(W):                                             # dispatch: what every rank q sends to r
            recv = torch.cat([wires[q][starts[q][r]:starts[q][r] + plans[q].send_counts[r]] for q in range(W)])
            assert recv.shape[0] == sum(plans[r].recv_counts)
            if recv.shape[0]:
                x, sc, i, w = self.layers[r].ep_unpack(recv)
                parts.append(self.layers[r].forward_routed(i, w, x, sc, self.weights[r]["gemm1_weights"],
                                                           self.weights[r]["gemm1_weights_scale"],
                                                           self.weights[r]["gemm2_weights"],
                                                           self.weights[r]["gemm2_weights_scale"], self.offset(r),
                                                           out_dtype=torch.float16))
            else:
                parts.append(torch.zeros(0, self.shape.hidden, dtype=torch.float16, device="cuda"))
        outs = []
        for q in range(W):                                             # combine: rows come back in send order
            back = []
            for r in range(W):
                first = sum(plans[r].recv_counts[:q])
                back.append(parts[r][first:first + plans[r].recv_counts[q]])
            back = torch.cat(back)
            outs.append(self.layers[q].ep_combine(back, plans[q].row_of, int(toks[q][2].shape[0])))
        torch.cuda.synchronize()
        return outs
