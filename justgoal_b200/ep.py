"""Expert-parallel MoE layer: experts sharded over the ranks of one node, tokens sharded evenly.

The reference corpus has no distributed code; its operator is ONE rank's share of a layer
(`local_expert_offset`, 32 local of 256 experts: goal_full_shape/fable-5.1/moe_fp8_fwd/<def>/
moe_common.cuh:14-15).  This module supplies the two exchanges around that share:

  route own tokens -> DISPATCH (ONE all-to-all of packed rows: fp8 row + scales + the token's top-k
  ids/weights, one copy per (token, destination rank); b200moe_ep_pack / _unpack) -> local experts
  (b200moe_forward_routed: fp16 row = partial sum over the local experts of a received token) -> COMBINE
  (all-to-all of the fp16 partial rows back to the token's owner) -> b200moe_ep_combine: fp32 sum over
  the destination ranks in rank order, one rounding to bf16.

One process per GPU, `torch.distributed` (NCCL over NVLink) for the exchange.  The exchange logic
is independent of where the per-rank compute runs: `backend` defaults to the CUDA library
(`CudaBackend`); the CPU tests run the same exchange over gloo with a backend built on the oracle.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from .inputs import MoEShape


@dataclass
class DispatchPlan:
    """Who gets which of my tokens.  `send_token[i]` is the local token of the i-th sent row; rows
    are grouped by destination rank (ascending), tokens ascending inside a group.  `row_of[r, t]`
    is the sent row that carries token t to rank r (-1: rank r owns none of its experts) - the same
    row index holds rank r's partial result in the buffer the combine all-to-all fills."""
    send_token: torch.Tensor        # int64 [n_send]
    send_counts: list               # rows per destination rank
    recv_counts: list               # rows per source rank
    row_of: torch.Tensor            # int32 [world, T]


def _dispatch_mask(topk_idx: torch.Tensor, experts_per_rank: int, world: int):
    T, dev = topk_idx.shape[0], topk_idx.device
    dst = torch.div(topk_idx.long(), experts_per_rank, rounding_mode="floor").clamp_(0, world - 1)   # [T, K]
    mask = torch.zeros(world, T, dtype=torch.int32, device=dev)
    mask.scatter_(0, dst.t().contiguous(), 1)                     # mask[r, t] = 1 iff token t has an expert on rank r
    within = torch.cumsum(mask, dim=1, dtype=torch.int32)         # inclusive rank of token t among rank r's rows
    send_counts = within[:, -1].contiguous() if T else torch.zeros(world, dtype=torch.int32, device=dev)
    return mask, within, send_counts


def send_counts_of(topk_idx: torch.Tensor, experts_per_rank: int, world: int) -> torch.Tensor:
    """int32 [world]: rows this rank's tokens send to every rank (what plan_dispatch exchanges)."""
    return _dispatch_mask(topk_idx, experts_per_rank, world)[2]


def plan_dispatch(topk_idx: torch.Tensor, experts_per_rank: int, world: int, group=None,
                  recv_counts: torch.Tensor = None) -> DispatchPlan:
    """De-duplicated per (token, destination rank): a token with several experts on one rank is
    sent there once.  One host synchronisation (the split sizes NCCL needs on the host).
    `recv_counts` (int32 [world], rows every rank sends to this one) replaces the counts all-to-all when
    the caller already knows it - a single process that plays several ranks does."""
    T, dev = topk_idx.shape[0], topk_idx.device
    mask, within, send_counts = _dispatch_mask(topk_idx, experts_per_rank, world)
    if recv_counts is None:
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=group)
    else:
        recv_counts = recv_counts.to(device=dev, dtype=send_counts.dtype)
    both = torch.stack([send_counts, recv_counts]).cpu()          # the one host sync of a step
    send, recv = both[0].tolist(), both[1].tolist()
    n_send = sum(send)
    first = torch.cumsum(send_counts, 0, dtype=torch.int32) - send_counts          # first row of each destination
    row_of = torch.where(mask.bool(), within - 1 + first[:, None], torch.full_like(within, -1))
    # token of every sent row: scatter the token ids to their rows (non-pairs go to a spare slot)
    slot = torch.where(row_of >= 0, row_of, torch.full_like(row_of, n_send)).long().reshape(-1)
    tok_ids = torch.arange(T, device=dev, dtype=torch.int64).repeat(world)
    send_token = torch.empty(n_send + 1, dtype=torch.int64, device=dev).scatter_(0, slot, tok_ids)[:n_send]
    return DispatchPlan(send_token, send, recv, row_of)


def _a2a(x: torch.Tensor, out_rows: int, in_splits, out_splits, group):
    out = torch.empty((out_rows,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_to_all_single(out, x, out_splits, in_splits, group=group)
    return out


class CudaBackend:
    """The per-rank compute of a step on the CUDA library: routing, packing / unpacking of the dispatch
    rows, the local experts, the owner-side combine.  The CPU tests of the exchange pass an object with
    the same five methods built on the oracle."""

    def __init__(self, shape: MoEShape, weights: dict, offset: int, device=None):
        from .main import MoELayer
        self.layer, self.w, self.offset = MoELayer(shape, device), weights, offset

    def route(self, logits, bias, rsf):
        return self.layer.route(logits, bias, rsf)

    def pack(self, hidden, hscale, idx, w, send_token):
        return self.layer.ep_pack(hidden, hscale, idx, w, send_token)

    def unpack(self, wire):
        return self.layer.ep_unpack(wire)

    def experts(self, idx, w, hidden, hscale):
        """fp16 [n, H]: per received token the partial sum over this rank's experts."""
        return self.layer.forward_routed(idx, w, hidden, hscale, self.w["gemm1_weights"], self.w["gemm1_weights_scale"],
                                         self.w["gemm2_weights"], self.w["gemm2_weights_scale"], self.offset,
                                         out_dtype=torch.float16)

    def combine(self, back, row_of, T):
        return self.layer.ep_combine(back, row_of, T)


class PeerExchange:
    """The exchange over peer memory (NVLink stores + flag barriers, csrc/ep_p2p.cuh) instead of NCCL
    all-to-alls: no host synchronisation and no library collective in a step.  One symmetric buffer per
    rank (torch symmetric memory supplies the mapping and the peer addresses; the kernels are this
    library's): flags | status word | wire [world][cap] rows | back [world][cap][H] fp16."""

    FLAGS_BYTES = 4096          # flags uint32[16] at 0, device status int at 1024

    @staticmethod
    def buffer_bytes(layer, shape: MoEShape, cap: int, world: int) -> int:
        wire_bytes = world * int(cap) * layer.ep_row_bytes()
        back_off = (PeerExchange.FLAGS_BYTES + wire_bytes + 255) // 256 * 256
        return back_off + world * int(cap) * shape.hidden * 2

    def __init__(self, layer, shape: MoEShape, cap: int, group, device, local_buffers=None, rank=None):
        """`local_buffers` (a list of `world` zeroed uint8 tensors of `buffer_bytes` bytes on THIS device, entry r
        standing in for rank r's buffer) with `rank` builds the exchange without symmetric memory or a process
        group: one process then plays every rank in turn on one GPU (tests)."""
        import ctypes as C
        from . import _lib
        self._lib, self._C = _lib, C
        self.layer, self.shape, self.cap = layer, shape, int(cap)
        device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        if local_buffers is None:
            self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        else:
            self.rank, self.world = int(rank), len(local_buffers)
        self.row_bytes = layer.ep_row_bytes()
        wire_bytes = self.world * self.cap * self.row_bytes
        back_bytes = self.world * self.cap * shape.hidden * 2
        self.wire_off = self.FLAGS_BYTES
        self.back_off = (self.wire_off + wire_bytes + 255) // 256 * 256
        total = self.back_off + back_bytes
        assert total == self.buffer_bytes(layer, shape, cap, self.world)
        if local_buffers is None:
            import torch.distributed._symmetric_memory as symm
            self.buf = symm.empty(total, dtype=torch.uint8, device=device)
            self.buf.zero_()
            self.handle = symm.rendezvous(self.buf, group if group is not None else dist.group.WORLD)
            bases = [int(p) for p in self.handle.buffer_ptrs]
        else:
            if any(b.numel() < total or b.dtype != torch.uint8 or not b.is_cuda for b in local_buffers):
                raise ValueError("local_buffers must be CUDA uint8 tensors of at least buffer_bytes() bytes")
            self.buf, self.handle = local_buffers[self.rank], None
            bases = [int(b.data_ptr()) for b in local_buffers]
        arr = C.c_void_p * self.world
        self.peer_flags = arr(*bases)
        self.peer_wire = arr(*[b + self.wire_off for b in bases])
        self.peer_back = arr(*[b + self.back_off for b in bases])
        self.status = self.buf[1024:1028].view(torch.int32)
        self.wire = self.buf[self.wire_off:self.wire_off + wire_bytes].view(self.world * self.cap, self.row_bytes)
        self.back = self.buf[self.back_off:self.back_off + back_bytes].view(torch.float16).view(
            self.world * self.cap, shape.hidden)
        self.flags = self.buf[:64].view(torch.int32)          # uint32[16] arrival flags, entry r written by rank r
        self.epoch = 0
        torch.cuda.synchronize(device)
        if local_buffers is None:
            dist.barrier(group)       # every rank's flags are zero before anyone's first barrier kernel

    def _stream(self):
        return self._C.c_void_p(torch.cuda.current_stream(self.buf.device).cuda_stream)

    def _check(self, rc, what):
        self._lib.check(rc, what)

    def barrier(self):
        self.epoch += 1
        self._check(self._lib.lib.b200moe_ep_barrier(self.layer._h, self.peer_flags, self.world, self.rank, self.epoch,
                                                     self.status.data_ptr(), self._stream()), "b200moe_ep_barrier")

    def push(self, hidden, hscale, idx, w):
        T = int(hidden.shape[0])
        if T > self.cap:
            raise ValueError(f"{T} tokens exceed the exchange capacity {self.cap}")
        self._keep = (hidden.contiguous(), hscale.contiguous(), idx.contiguous(), w.contiguous())
        h, sc, i, ww = self._keep
        self._check(self._lib.lib.b200moe_ep_push(self.layer._h, h.data_ptr(), sc.data_ptr(), i.data_ptr(), ww.data_ptr(),
                                                  T, self.cap, self.world, self.rank, self.peer_wire, self._stream()),
                    "b200moe_ep_push")

    def unpack(self):
        s, n, dev = self.shape, self.world * self.cap, self.buf.device
        x = torch.empty(n, s.hidden, dtype=torch.float8_e4m3fn, device=dev)
        sc = torch.empty(s.hidden // 128, n, dtype=torch.float32, device=dev)
        idx = torch.empty(n, s.top_k, dtype=torch.int32, device=dev)
        w = torch.empty(n, s.top_k, dtype=torch.float32, device=dev)
        self._check(self._lib.lib.b200moe_ep_unpack_slots(self.layer._h, self.wire.data_ptr(), n, x.data_ptr(),
                                                          sc.data_ptr(), idx.data_ptr(), w.data_ptr(), self._stream()),
                    "b200moe_ep_unpack_slots")
        return x, sc, idx, w

    def experts_to_peers(self, weights, offset):
        """The local experts over all wire slots, read in place (no unpack copy); the last kernel stores every
        present slot's fp16 partial row straight into its owner's back slot (b200moe_forward_routed_slots)."""
        n = self.world * self.cap
        ws = self.layer.workspace(n)
        ptrs = [weights[k].data_ptr() for k in ("gemm1_weights", "gemm1_weights_scale", "gemm2_weights",
                                               "gemm2_weights_scale")]
        self._check(self._lib.lib.b200moe_forward_routed_slots(self.layer._h, self.wire.data_ptr(), *ptrs, self.cap,
                                                               self.world, self.rank, int(offset), self.peer_back,
                                                               ws.data_ptr(), ws.numel(), self._stream()),
                    "b200moe_forward_routed_slots")

    def give_back(self, part, idx_slots):
        self._check(self._lib.lib.b200moe_ep_return(self.layer._h, part.data_ptr(), idx_slots.data_ptr(), self.cap,
                                                    self.world, self.rank, self.peer_back, self._stream()),
                    "b200moe_ep_return")

    def combine(self, idx, T):
        out = torch.empty(T, self.shape.hidden, dtype=torch.bfloat16, device=self.buf.device)
        self._check(self._lib.lib.b200moe_ep_combine_slots(self.layer._h, self.back.data_ptr(), idx.data_ptr(), T, self.cap,
                                                           self.world, out.data_ptr(), self._stream()),
                    "b200moe_ep_combine_slots")
        return out

    def error_word(self) -> int:
        """Device status of the barriers (0 = fine, 7 = a wait for a peer ran out).  Synchronises."""
        return int(self.status.item())

    def clear_error(self):
        self.status.zero_()


class ExpertParallelMoE:
    def __init__(self, shape: MoEShape, weights: dict, group=None, backend=None, device=None, exchange="nccl",
                 capacity=None):
        """`shape.num_local_experts` experts per rank, rank r owning experts [r*E_local, (r+1)*E_local);
        `weights` = this rank's gemm1/gemm2 weights and scales."""
        self.shape, self.group = shape, group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if shape.num_local_experts * self.world != shape.num_experts:
            raise ValueError("num_local_experts * world_size must equal num_experts")
        self.offset = self.rank * shape.num_local_experts
        self.backend = backend or CudaBackend(shape, weights, self.offset, device)
        self.last_plan = None
        # exchange = "nccl": three all-to-alls per step (works with any backend, CPU tests included);
        # "p2p": this library's kernels over peer memory, `capacity` = the most tokens a rank brings to a step
        self.peer = None
        if exchange == "p2p":
            if backend is not None or capacity is None:
                raise ValueError("the peer-memory exchange needs the CUDA backend and a capacity")
            self.peer = PeerExchange(self.backend.layer, shape, capacity, group, device)
        elif exchange != "nccl":
            raise ValueError("exchange must be 'nccl' or 'p2p'")

    # ---- one step
    @torch.no_grad()
    def forward(self, routing_logits, routing_bias, hidden_states, hidden_states_scale, routed_scaling_factor):
        """Inputs are this rank's tokens (hidden_states_scale is [H/128, T_local]); returns bf16
        [T_local, H], the full layer output for those tokens.  Three all-to-alls per step: split sizes,
        dispatch rows, partial result rows."""
        s, g, be = self.shape, self.group, self.backend
        T, H = hidden_states.shape
        mark = self._mark
        mark("start")
        if self.peer is not None:
            px = self.peer
            idx, w = be.route(routing_logits, routing_bias, routed_scaling_factor)
            mark("route")
            px.push(hidden_states, hidden_states_scale, idx, w)
            mark("push")
            px.barrier()
            mark("barrier1")
            px.experts_to_peers(be.w, be.offset)      # reads the slots in place; result rows go straight home
            mark("experts")
            px.barrier()
            mark("barrier2")
            out = px.combine(idx, T)
            mark("combine")
            return out
        idx, w = be.route(routing_logits, routing_bias, routed_scaling_factor)
        idx = idx.to(torch.int32)
        mark("route")
        plan = plan_dispatch(idx, s.num_local_experts, self.world, g)
        self.last_plan = plan
        n_recv = sum(plan.recv_counts)
        self._last_recv = int(n_recv)
        mark("plan")
        # DISPATCH: one packed row per (token, destination rank)
        wire = be.pack(hidden_states, hidden_states_scale, idx, w, plan.send_token)
        wire = _a2a(wire, n_recv, plan.send_counts, plan.recv_counts, g)
        x_recv, sc_recv, idx_recv, w_recv = be.unpack(wire)
        mark("dispatch")
        # LOCAL EXPERTS: partial sum over this rank's experts for every received token, as fp16 rows
        if n_recv:
            part = be.experts(idx_recv, w_recv, x_recv, sc_recv)
        else:
            part = torch.zeros(0, H, dtype=torch.float16, device=hidden_states.device)
        mark("experts")
        # COMBINE: fp16 partial rows back to the owners, fp32 sum over destination ranks, one rounding
        back = _a2a(part, plan.send_token.numel(), plan.recv_counts, plan.send_counts, g)
        out = be.combine(back, plan.row_of, T)
        mark("combine")
        return out

    def launches_per_step(self) -> int:
        """Kernels of this library one step launches on one rank.  Peer-memory form: route, push, barrier, count,
        permute, [gather from the wire slots unless GEMM1 gathers by TMA], GEMM1, GEMM2, combine (stores into the
        owners' slots), barrier, owner-side sum; collective form: route, pack, unpack, count, permute, [gather],
        GEMM1, GEMM2, combine, owner-side sum."""
        layer = getattr(self.backend, "layer", None)
        if layer is None:               # a backend that is not this library (the CPU tests' oracle backend)
            return 0
        if self.peer is not None:       # route, push, barrier | local experts over all slots | barrier, owner-side sum
            return 5 + layer.launches_routed(self.peer.world * self.peer.cap)
        # route, pack, unpack | local experts over the rows received in the last step | owner-side sum
        return 4 + layer.launches_routed(max(1, getattr(self, "_last_recv", 1)))

    def check_status(self):
        """Raises if a barrier of the peer-memory exchange gave up waiting for a peer since the last check (the
        outputs of that step are then invalid).  Synchronises the device, so call it where a synchronisation
        is acceptable - e.g. once per batch of steps - not inside a latency-critical loop."""
        if self.peer is not None:
            word = self.peer.error_word()
            if word != 0:
                self.peer.clear_error()
                raise RuntimeError(f"expert-parallel exchange: device error word {word} "
                                   "(7 = a rank gave up waiting for a peer's barrier flag)")

    # ---- optional phase timing (CUDA events on the current stream; off unless `phase_events` is a list)
    phase_events = None

    def _mark(self, name):
        if self.phase_events is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self.phase_events.append((name, e))

    def phase_ms(self):
        """Durations between consecutive marks of the steps recorded since `phase_events = []`."""
        torch.cuda.synchronize()
        acc, n = {}, 0
        ev = self.phase_events or []
        for (n0, e0), (n1, e1) in zip(ev, ev[1:]):
            if n1 == "start":
                continue
            acc[n1] = acc.get(n1, 0.0) + e0.elapsed_time(e1)
            n += n1 == "combine"
        return {k: v / max(n, 1) for k, v in acc.items()}

    def nvlink_bytes(self):
        """Bytes this rank sent to / received from OTHER ranks in the last step: the figure the NVLink
        term of the roofline uses."""
        p, s = self.last_plan, self.shape
        if p is None:
            return None
        remote_send = sum(c for d, c in enumerate(p.send_counts) if d != self.rank)
        remote_recv = sum(c for d, c in enumerate(p.recv_counts) if d != self.rank)
        row = (s.hidden + 4 * (s.hidden // 128) + 8 * s.top_k + 15) // 16 * 16
        return {"dispatch_send": remote_send * row, "combine_send": remote_recv * 2 * s.hidden,
                "dispatch_recv": remote_recv * row, "combine_recv": remote_send * 2 * s.hidden}
