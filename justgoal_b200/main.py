"""Operator entry point with the reference's signature.

`run(...)` keeps the argument list, dtypes, layouts and return value of the reference
solutions' `main.py::run` (goal_full_shape/fable-5.1/moe_fp8_fwd/<def>/main.py:102-117,
non destination-passing) and `run_dps(..., output)` the destination-passing twin
(kda05_reproduction_full_shape/fable-5.1/moe_fp8_fwd/<def>/fable51_moe_v94/main.py:196-209).
All work happens in libb200moe.so through its C ABI on the caller's current CUDA stream;
torch is only used for tensors, the stream handle and the workspace allocation.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from .inputs import MoEShape, ROUTING_DS, ROUTING_RENORM_NAIVE  # noqa: F401


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _contig(t):
    return t if t.is_contiguous() else t.contiguous()


def _scalar(v, kind):
    if isinstance(v, torch.Tensor):
        v = v.item()
    return kind(v)


class MoELayer:
    """One rank's share of an MoE layer of a fixed shape: a library handle plus workspaces
    cached per token count (the reference caches per (T, device): GF main.py:68-94)."""

    def __init__(self, shape: MoEShape, device=None):
        if not torch.cuda.is_available():
            raise _lib.B200MoEError("b200moe needs a CUDA device (no CPU fallback exists)")
        self.shape = shape
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        cfg = _lib.Config(shape.hidden, shape.intermediate, shape.num_experts, shape.num_local_experts,
                          shape.top_k, shape.n_group, shape.topk_group, shape.routing_mode)
        self._h = C.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib.b200moe_create(C.byref(cfg), C.byref(self._h)), "b200moe_create")
        self._ws = {}

    def __del__(self):
        h = getattr(self, "_h", None)
        if h and _lib is not None and getattr(_lib, "lib", None) is not None:   # may run at interpreter exit
            _lib.lib.b200moe_destroy(h)
            self._h = None

    # ------------------------------------------------------------------ workspace
    def workspace(self, T: int) -> torch.Tensor:
        """Workspace for a forward over T tokens.  Buffers are cached per power-of-two bucket of T
        (sizes grow monotonically with T, so the bucket's buffer serves every smaller count), which
        keeps memory bounded when the token count changes from call to call."""
        bucket = 64
        while bucket < T:
            bucket *= 2
        ws = self._ws.get(bucket)
        if ws is None:
            n = C.c_size_t()
            _lib.check(_lib.lib.b200moe_workspace_bytes(self._h, bucket, C.byref(n)), "b200moe_workspace_bytes")
            ws = torch.empty(max(int(n.value), 256), dtype=torch.uint8, device=self.device)
            assert ws.data_ptr() % 256 == 0
            self._ws[bucket] = ws
        return ws

    def layout(self, T: int) -> _lib.WsLayout:
        L = _lib.WsLayout()
        _lib.check(_lib.lib.b200moe_workspace_layout(self._h, T, C.byref(L)), "b200moe_workspace_layout")
        return L

    def view(self, T: int, name: str, dtype, shape):
        """A typed view of one intermediate buffer of the workspace (tests / debugging)."""
        L = self.layout(T)
        off = getattr(L, name)
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self.workspace(T)[off:off + nbytes].view(dtype).view(*shape)

    def launches_per_forward(self, T: int) -> int:
        n = C.c_int()
        _lib.check(_lib.lib.b200moe_launches_per_forward(self._h, T, C.byref(n)))
        return int(n.value)

    STAGES = ("route", "permute", "gather", "gemm1", "gemm2", "combine")

    def profile_enable(self, slots: int):
        _lib.check(_lib.lib.b200moe_profile_enable(self._h, int(slots)), "b200moe_profile_enable")

    def profile_read(self, slot: int) -> dict:
        ms = (C.c_float * 6)()
        _lib.check(_lib.lib.b200moe_profile_read(self._h, int(slot), ms), "b200moe_profile_read")
        return dict(zip(self.STAGES, [float(x) for x in ms]))

    def launches_routed(self, T: int) -> int:
        """Kernel launches of forward_routed (or the slot form) over T tokens (slots)."""
        n = C.c_int(0)
        _lib.check(_lib.lib.b200moe_launches_routed(self._h, T, C.byref(n)))
        return n.value

    def set_token_tile(self, tokens: int):
        """Token tile of the GEMMs: 0 = chosen from the token count (default), else 16, 32, 64 or 128 for every call
        (tuning and tests).  Workspaces are sized per tile, so the cached ones are dropped."""
        _lib.check(_lib.lib.b200moe_set_token_tile(self._h, int(tokens)), "b200moe_set_token_tile")
        self._ws.clear()

    def set_tma_gather(self, on: bool):
        """128-token tiles only: GEMM1 gathers its token rows by TMA instead of reading a gathered copy (same bits;
        off by default, measured slower)."""
        _lib.check(_lib.lib.b200moe_set_tma_gather(self._h, 1 if on else 0), "b200moe_set_tma_gather")

    def set_fused_combine(self, on: bool):
        """Narrow token tiles only: let the GEMM2 epilogue add a token's rows up instead of a combine launch (same
        bits; off by default, measured slower at 64 tokens)."""
        _lib.check(_lib.lib.b200moe_set_fused_combine(self._h, 1 if on else 0), "b200moe_set_fused_combine")

    def set_wait_limit(self, seconds: float):
        """Limit of this layer's waits on another rank (barrier flags of the peer-memory exchange)."""
        _lib.check(_lib.lib.b200moe_set_wait_limit_ns(self._h, int(seconds * 1e9)), "b200moe_set_wait_limit_ns")

    def status(self, T: int) -> int:
        word = C.c_int(0)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = _lib.lib.b200moe_status(self._h, _ptr(self.workspace(T)), C.c_void_p(stream), C.byref(word))
        if rc not in (0, -5):
            _lib.check(rc, "b200moe_status")
        return int(word.value)

    # ------------------------------------------------------------------ operator
    def forward(self, routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
                routed_scaling_factor, output=None):
        s = self.shape
        T = int(hidden_states.shape[0])
        self._check(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                    gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, T)
        if output is None:
            output = torch.empty(T, s.hidden, dtype=torch.bfloat16, device=hidden_states.device)
        elif output.shape != (T, s.hidden) or output.dtype != torch.bfloat16 or not output.is_contiguous():
            raise ValueError("output must be a contiguous bf16 [T, hidden] tensor")
        if T == 0:
            return output
        ws = self.workspace(T)
        tensors = [_contig(t) if t is not None else None for t in (
            routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
            gemm1_weights_scale, gemm2_weights, gemm2_weights_scale)]
        stream = torch.cuda.current_stream(hidden_states.device).cuda_stream
        rc = _lib.lib.b200moe_forward(self._h, *[_ptr(t) for t in tensors], T,
                                      _scalar(local_expert_offset, int), _scalar(routed_scaling_factor, float),
                                      _ptr(output), _ptr(ws), ws.numel(), C.c_void_p(stream))
        _lib.check(rc, "b200moe_forward")
        return output

    def forward_routed(self, topk_idx, topk_w, hidden_states, hidden_states_scale, gemm1_weights,
                       gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset, output=None,
                       out_dtype=torch.float32):
        """Expert part only: the sum over the local experts as fp32 (no rounding), bf16, or fp16 rows (the form
        partial rows travel in between the ranks of an expert-parallel layer)."""
        s = self.shape
        T = int(hidden_states.shape[0])
        if output is None:
            output = torch.empty(T, s.hidden, dtype=out_dtype, device=hidden_states.device)
        kinds = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
        if output.dtype not in kinds or not output.is_contiguous():
            raise ValueError("output must be a contiguous fp32, bf16 or fp16 [T, hidden] tensor")
        if T == 0:
            return output
        if topk_idx.dtype != torch.int32 or topk_w.dtype != torch.float32:
            raise ValueError("topk_idx must be int32 and topk_w float32")
        ws = self.workspace(T)
        tensors = [_contig(t) for t in (topk_idx, topk_w, hidden_states, hidden_states_scale, gemm1_weights,
                                        gemm1_weights_scale, gemm2_weights, gemm2_weights_scale)]
        stream = torch.cuda.current_stream(hidden_states.device).cuda_stream
        rc = _lib.lib.b200moe_forward_routed(self._h, *[_ptr(t) for t in tensors], T,
                                             _scalar(local_expert_offset, int), _ptr(output),
                                             kinds[output.dtype], _ptr(ws),
                                             ws.numel(), C.c_void_p(stream))
        _lib.check(rc, "b200moe_forward_routed")
        return output

    def ep_row_bytes(self) -> int:
        n = C.c_int(0)
        _lib.check(_lib.lib.b200moe_ep_row_bytes(self._h, C.byref(n)), "b200moe_ep_row_bytes")
        return int(n.value)

    def ep_pack(self, hidden_states, hidden_states_scale, topk_idx, topk_w, send_token):
        """uint8 [n, ep_row_bytes()]: the dispatch rows of the tokens `send_token` (int64 [n])."""
        n, T = int(send_token.numel()), int(hidden_states.shape[0])
        if topk_idx.dtype != torch.int32 or topk_w.dtype != torch.float32 or send_token.dtype != torch.int64:
            raise ValueError("topk_idx int32, topk_w float32, send_token int64")
        wire = torch.empty(n, self.ep_row_bytes(), dtype=torch.uint8, device=hidden_states.device)
        stream = torch.cuda.current_stream(hidden_states.device).cuda_stream
        rc = _lib.lib.b200moe_ep_pack(self._h, _ptr(_contig(hidden_states)), _ptr(_contig(hidden_states_scale)),
                                      _ptr(_contig(topk_idx)), _ptr(_contig(topk_w)), _ptr(_contig(send_token)), n, T,
                                      _ptr(wire), C.c_void_p(stream))
        _lib.check(rc, "b200moe_ep_pack")
        return wire

    def ep_unpack(self, wire):
        """(hidden fp8 [n, H], scales float [H/128, n], topk_idx int32 [n, K], topk_w float [n, K])."""
        s, n, dev = self.shape, int(wire.shape[0]), wire.device
        x = torch.empty(n, s.hidden, dtype=torch.float8_e4m3fn, device=dev)
        sc = torch.empty(s.hidden // 128, n, dtype=torch.float32, device=dev)
        idx = torch.empty(n, s.top_k, dtype=torch.int32, device=dev)
        w = torch.empty(n, s.top_k, dtype=torch.float32, device=dev)
        stream = torch.cuda.current_stream(dev).cuda_stream
        rc = _lib.lib.b200moe_ep_unpack(self._h, _ptr(_contig(wire)), n, _ptr(x), _ptr(sc), _ptr(idx), _ptr(w),
                                        C.c_void_p(stream))
        _lib.check(rc, "b200moe_ep_unpack")
        return x, sc, idx, w

    def ep_combine(self, partial_rows, row_of, num_tokens):
        """Owner-rank side of the expert-parallel combine: bf16 [T, hidden] = per token the fp32 sum, in
        rank order, of the fp16 partial rows `partial_rows[row_of[r, t]]` (row_of int32 [world, T], -1 = none)."""
        s = self.shape
        world = int(row_of.shape[0])
        if partial_rows.dtype != torch.float16 or row_of.dtype != torch.int32 or row_of.shape[1] != num_tokens:
            raise ValueError("partial_rows must be fp16 [n, hidden] and row_of int32 [world, T]")
        out = torch.empty(num_tokens, s.hidden, dtype=torch.bfloat16, device=partial_rows.device)
        stream = torch.cuda.current_stream(partial_rows.device).cuda_stream
        rc = _lib.lib.b200moe_ep_combine(self._h, _ptr(_contig(partial_rows)), _ptr(_contig(row_of)), world,
                                         int(num_tokens), _ptr(out), C.c_void_p(stream))
        _lib.check(rc, "b200moe_ep_combine")
        return out

    def route(self, routing_logits, routing_bias, routed_scaling_factor):
        s = self.shape
        T = int(routing_logits.shape[0])
        idx = torch.empty(T, s.top_k, dtype=torch.int32, device=routing_logits.device)
        w = torch.empty(T, s.top_k, dtype=torch.float32, device=routing_logits.device)
        if T:
            stream = torch.cuda.current_stream(routing_logits.device).cuda_stream
            rb = None if routing_bias is None else _contig(routing_bias)
            rc = _lib.lib.b200moe_route(self._h, _ptr(_contig(routing_logits)), _ptr(rb), T,
                                        _scalar(routed_scaling_factor, float), _ptr(idx), _ptr(w),
                                        C.c_void_p(stream))
            _lib.check(rc, "b200moe_route")
        return idx, w

    def permute_noalloc(self, topk_idx, topk_w, local_expert_offset, expert_row0, row_token, row_w):
        """Expert-sorted row map into caller-provided tensors through the entry point that keeps its
        scratch in a static device array (for hosts that must not allocate device memory); at most
        `_lib.NOALLOC_MAX_TOKENS` tokens, calls on one device must not overlap."""
        T = int(topk_idx.shape[0])
        dev = topk_idx.device
        for name, t, dt in (("topk_idx", topk_idx, torch.int32), ("topk_w", topk_w, torch.float32),
                            ("expert_row0", expert_row0, torch.int32), ("row_token", row_token, torch.int32),
                            ("row_w", row_w, torch.float32)):
            if t.dtype != dt or not t.is_cuda or t.device != dev:
                raise ValueError(f"{name} must be a {dt} CUDA tensor on {dev}")
        for name, t in (("expert_row0", expert_row0), ("row_token", row_token), ("row_w", row_w)):
            if not t.is_contiguous():
                raise ValueError(f"{name} must be contiguous (it is written in place)")
        if tuple(topk_idx.shape) != (T, self.shape.top_k) or tuple(topk_w.shape) != (T, self.shape.top_k):
            raise ValueError("topk_idx / topk_w must be [T, top_k]")
        if expert_row0.numel() < self.shape.num_local_experts + 1:
            raise ValueError("expert_row0 needs num_local_experts + 1 entries")
        stream = torch.cuda.current_stream(dev).cuda_stream
        rc = _lib.lib.b200moe_permute_noalloc(self._h, _ptr(_contig(topk_idx)), _ptr(_contig(topk_w)), T,
                                              _scalar(local_expert_offset, int), _ptr(expert_row0),
                                              _ptr(row_token), _ptr(row_w), min(int(row_token.numel()), int(row_w.numel())),
                                              C.c_void_p(stream))
        _lib.check(rc, "b200moe_permute_noalloc")

    def _check(self, logits, bias, hs, hss, w13, s13, w2, s2, T):
        s = self.shape
        H, I, E, El = s.hidden, s.intermediate, s.num_experts, s.num_local_experts
        f8 = torch.float8_e4m3fn
        want = [("routing_logits", logits, (T, E), torch.float32),
                ("hidden_states", hs, (T, H), f8),
                ("hidden_states_scale", hss, (H // 128, T), torch.float32),
                ("gemm1_weights", w13, (El, 2 * I, H), f8),
                ("gemm1_weights_scale", s13, (El, 2 * I // 128, H // 128), torch.float32),
                ("gemm2_weights", w2, (El, H, I), f8),
                ("gemm2_weights_scale", s2, (El, H // 128, I // 128), torch.float32)]
        if bias is not None:
            want.append(("routing_bias", bias, (E,), torch.bfloat16))
        for name, t, shape, dt in want:
            if tuple(t.shape) != shape or t.dtype != dt:
                raise ValueError(f"{name}: expected {dt} {shape}, got {t.dtype} {tuple(t.shape)}")
            if not t.is_cuda:
                raise ValueError(f"{name} must be a CUDA tensor")


def quantize_1x128(x: torch.Tensor):
    """bf16 [T, H] on the GPU -> (e4m3 [T, H], float scales [H/128, T]): the operator's `hidden_states` and
    `hidden_states_scale` inputs, made by the library's quantiser kernel on the current stream."""
    if x.dtype != torch.bfloat16 or x.dim() != 2 or not x.is_cuda:
        raise ValueError("x must be a CUDA bf16 [T, H] tensor")
    x = _contig(x)
    T, H = int(x.shape[0]), int(x.shape[1])
    q = torch.empty(T, H, dtype=torch.float8_e4m3fn, device=x.device)
    sc = torch.empty(H // 128, T, dtype=torch.float32, device=x.device)
    stream = torch.cuda.current_stream(x.device).cuda_stream
    _lib.check(_lib.lib.b200moe_quantize_1x128(_ptr(x), T, H, _ptr(q), _ptr(sc), C.c_void_p(stream)),
               "b200moe_quantize_1x128")
    return q, sc


_layers = {}


def _layer_for(routing_logits, hidden_states, gemm1_weights, top_k=8, n_group=8, topk_group=4,
               routing_mode=ROUTING_DS) -> MoELayer:
    shape = MoEShape(hidden=int(hidden_states.shape[1]), intermediate=int(gemm1_weights.shape[1]) // 2,
                     num_experts=int(routing_logits.shape[1]), num_local_experts=int(gemm1_weights.shape[0]),
                     top_k=top_k, n_group=n_group, topk_group=topk_group, routing_mode=routing_mode)
    key = (shape, hidden_states.device.index)
    layer = _layers.get(key)
    if layer is None:
        layer = _layers[key] = MoELayer(shape, hidden_states.device)
    return layer


class HostPipeline:
    """Steady-state loop for callers whose per-step inputs live in pinned host memory: the copy in, the
    forward and the copy out run on three streams over `depth` sets of device buffers, so step i+1's
    inputs travel while step i computes and step i-1's output travels back.  Every step still copies its
    own inputs to the device and its own output to the host; only the overlap is added.

        pipe = HostPipeline(layer, T, routing_bias, weights..., local_expert_offset, routed_scaling_factor)
        for logits, hidden, scale, out in steps:      # pinned host tensors
            pipe.step(logits, hidden, scale, out)
        pipe.drain()                                  # all outputs have landed
    """

    def __init__(self, layer: "MoELayer", num_tokens, routing_bias, gemm1_weights, gemm1_weights_scale,
                 gemm2_weights, gemm2_weights_scale, local_expert_offset, routed_scaling_factor, depth=2,
                 forward_fn=None):
        """`forward_fn(logits, hidden, scale, out) -> tensor` replaces `layer.forward` (the expert-parallel
        layer passes its own step); it runs on the pipeline's compute stream."""
        s, dev, T = layer.shape, layer.device, int(num_tokens)
        self.layer, self.T, self.depth, self.n = layer, T, int(depth), 0
        self.forward_fn = forward_fn
        self.static = (routing_bias, gemm1_weights, gemm1_weights_scale, gemm2_weights, gemm2_weights_scale,
                       local_expert_offset, routed_scaling_factor)
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(dev) for _ in range(3))
        mk = lambda *shape, dtype: torch.empty(*shape, dtype=dtype, device=dev)   # noqa: E731
        self.slots = [dict(logits=mk(T, s.num_experts, dtype=torch.float32),
                           hidden=mk(T, s.hidden, dtype=torch.float8_e4m3fn),
                           scale=mk(s.hidden // 128, T, dtype=torch.float32),
                           out=mk(T, s.hidden, dtype=torch.bfloat16),
                           loaded=torch.cuda.Event(), computed=torch.cuda.Event(), stored=torch.cuda.Event())
                      for _ in range(self.depth)]

    @torch.no_grad()
    def step(self, host_logits, host_hidden, host_scale, host_out):
        b = self.slots[self.n % self.depth]
        reuse = self.n >= self.depth
        bias, w13, s13, w2, s2, off, rsf = self.static
        with torch.cuda.stream(self.s_in):
            if reuse:
                self.s_in.wait_event(b["computed"])      # the forward that read this slot's inputs is done
            b["logits"].copy_(host_logits, non_blocking=True)
            b["hidden"].view(torch.uint8).copy_(host_hidden.view(torch.uint8), non_blocking=True)
            b["scale"].copy_(host_scale, non_blocking=True)
            b["loaded"].record()
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(b["loaded"])
            if reuse:
                self.s_run.wait_event(b["stored"])       # this slot's previous output has left the device
            if self.forward_fn is None:
                o = self.layer.forward(b["logits"], bias, b["hidden"], b["scale"], w13, s13, w2, s2, off, rsf,
                                       output=b["out"])
            else:
                o = self.forward_fn(b["logits"], b["hidden"], b["scale"], b["out"])
                if o.data_ptr() != b["out"].data_ptr():
                    o.record_stream(self.s_out)          # allocated on the compute stream, read on the copy stream
            b["computed"].record()
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(b["computed"])
            host_out.copy_(o, non_blocking=True)
            b["stored"].record()
        self.n += 1

    def drain(self):
        for st in (self.s_in, self.s_run, self.s_out):
            st.synchronize()


@torch.no_grad()
def run(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights, gemm1_weights_scale,
        gemm2_weights, gemm2_weights_scale, local_expert_offset, routed_scaling_factor):
    """DeepSeek-V3 routing (top-8 of 8 groups, 4 groups kept), returns bf16 [T, hidden]."""
    layer = _layer_for(routing_logits, hidden_states, gemm1_weights)
    return layer.forward(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                         gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
                         routed_scaling_factor)


@torch.no_grad()
def run_dps(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights, gemm1_weights_scale,
            gemm2_weights, gemm2_weights_scale, local_expert_offset, routed_scaling_factor, output):
    """Destination-passing twin of `run`: writes into `output` and returns it."""
    layer = _layer_for(routing_logits, hidden_states, gemm1_weights)
    return layer.forward(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                         gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
                         routed_scaling_factor, output=output)
