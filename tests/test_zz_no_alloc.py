"""GPU: the allocation-free permutation entry point (b200moe_permute_noalloc).

It exists for hosts that cannot allocate device memory when they need the expert-sorted row
map (frozen allocators in serving loops, plugins inside a runtime that owns the memory); its
scratch is a fixed array inside the library.  The test calls it twice in a row through the C
ABI, on two different inputs, and compares every output with what the regular entry point
(b200moe_forward_routed, whose tables are read from its caller-provided workspace) produces:
integers and copied weights, so the comparison is exact.  The second call also proves that
what the first call left in the shared array does not leak into the next result.
This file sorts last so that a `pytest -x` run has finished all other tests before it."""
import ctypes as C

import pytest
import torch

import util
from util import I

pytestmark = pytest.mark.gpu


def _reference_tables(layer, shape, d, idx, w):
    """Tables the existing entry point leaves in its workspace for the same routing."""
    T = idx.shape[0]
    dc = util.to_cuda(d)
    layer.forward_routed(idx, w, dc["hidden_states"], dc["hidden_states_scale"], dc["gemm1_weights"],
                         dc["gemm1_weights_scale"], dc["gemm2_weights"], dc["gemm2_weights_scale"],
                         d["local_expert_offset"])
    torch.cuda.synchronize()
    L = layer.layout(T)
    El, rows_cap = shape.num_local_experts, int(L.rows_cap)
    row0 = layer.view(T, "expert_row0", torch.int32, (El + 1,)).clone()
    tok = layer.view(T, "row_token", torch.int32, (rows_cap,)).clone()
    rw = layer.view(T, "row_w", torch.float32, (rows_cap,)).clone()
    return row0, tok, rw, rows_cap


def test_noalloc_permute_matches_regular_entry_point_twice_in_a_row():
    from justgoal_b200 import MoELayer
    shape = I.TINY_DS
    layer = MoELayer(shape)
    El = shape.num_local_experts
    for T, seed, off in ((33, 21, 0), (50, 22, 16)):          # two calls in a row, different inputs
        d = I.make_inputs(shape, T, seed=seed, local_expert_offset=off)
        idx, w = layer.route(d["routing_logits"].cuda(), d["routing_bias"].cuda(), 2.5)
        want_row0, want_tok, want_w, rows_cap = _reference_tables(layer, shape, d, idx, w)
        row0 = torch.full((El + 1,), -7, dtype=torch.int32, device="cuda")
        tok = torch.full((rows_cap,), -7, dtype=torch.int32, device="cuda")
        rw = torch.full((rows_cap,), -7.0, dtype=torch.float32, device="cuda")
        layer.permute_noalloc(idx, w, off, row0, tok, rw)
        torch.cuda.synchronize()
        n = int(want_row0[-1])
        assert n > 0
        assert torch.equal(row0, want_row0)
        assert torch.equal(tok[:n], want_tok[:n])
        assert torch.equal(rw[:n], want_w[:n])
        assert bool((tok[n:] == -7).all())                    # nothing written past the last segment


def test_noalloc_rejects_sizes_beyond_the_static_array():
    from justgoal_b200 import MoELayer, _lib
    shape = I.TINY_DS
    layer = MoELayer(shape)
    T = _lib.NOALLOC_MAX_TOKENS + 1
    idx = torch.zeros(T, shape.top_k, dtype=torch.int32, device="cuda")
    w = torch.zeros(T, shape.top_k, dtype=torch.float32, device="cuda")
    row0 = torch.zeros(shape.num_local_experts + 1, dtype=torch.int32, device="cuda")
    tok = torch.zeros(T * 8 + 1024, dtype=torch.int32, device="cuda")
    rw = torch.zeros(T * 8 + 1024, dtype=torch.float32, device="cuda")
    with pytest.raises(_lib.B200MoEError, match="NOALLOC_MAX_TOKENS"):
        layer.permute_noalloc(idx, w, 0, row0, tok, rw)
    # capacity of the caller's row arrays is checked too
    with pytest.raises(_lib.B200MoEError):
        layer.permute_noalloc(idx[:64], w[:64], 0, row0, tok[:8], rw[:8])
