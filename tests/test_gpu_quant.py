"""GPU: the activation quantiser (bf16 -> e4m3 + 1x128 scales, the step before the operator) through the
C ABI, BIT-EXACT against the host statement of the same arithmetic (justgoal_b200.inputs.quantize_rows_1x128:
scale = amax/448 per (token, 128 columns), 1.0 for an all-zero group, round to nearest even)."""
import pytest
import torch

import util
from util import I

pytestmark = pytest.mark.gpu


def _case(T, H, seed, spread=1.0):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(T, H, generator=g) * spread).to(torch.bfloat16)
    if T:
        x[0, :128] = 0                      # an all-zero group: scale 1.0, bytes 0
        x[T - 1, H - 128:] *= 1e-3          # a tiny group
        x[T // 2, 5] = 3.0e4                # one large outlier: the rest of its group lands in the subnormals
    return x


@pytest.mark.parametrize("T,H", [(1, 128), (7, 384), (64, 7168), (333, 4096), (4096, 7168)])
def test_quantiser_bit_exact(T, H):
    from justgoal_b200 import quantize_1x128
    x = _case(T, H, seed=T + H)
    q_ref, s_ref = I.quantize_rows_1x128(x)
    q, s = quantize_1x128(x.cuda())
    torch.cuda.synchronize()
    assert s.shape == (H // 128, T) and q.shape == (T, H)
    assert torch.equal(s.cpu().view(torch.int32), s_ref.view(torch.int32))
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))


def test_quantiser_feeds_the_operator():
    """bf16 activations -> quantiser kernel -> layer: same output as with host-quantised inputs."""
    from justgoal_b200 import MoELayer, quantize_1x128
    shape = I.TINY_DS
    d = I.make_inputs(shape, 50, seed=77)
    x = torch.randn(50, shape.hidden, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    d["hidden_states"], d["hidden_states_scale"] = I.quantize_rows_1x128(x)
    dc = util.to_cuda(d)
    layer = MoELayer(shape)
    want = layer.forward(*util.op_args(dc)).clone()
    dc["hidden_states"], dc["hidden_states_scale"] = quantize_1x128(x.cuda())
    got = layer.forward(*util.op_args(dc))
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    rep = util.O.compare_output(got, util.run_oracle(shape, d).output, util.ATOL, util.RTOL)
    assert rep["fail_frac"] == 0.0, rep


def test_quantiser_rejects_bad_shapes():
    from justgoal_b200 import _lib
    assert _lib.lib.b200moe_quantize_1x128(None, 4, 100, None, None, None) == -1      # H not a multiple of 128
    assert _lib.lib.b200moe_quantize_1x128(None, 4, 128, None, None, None) == -1      # null pointers
    assert _lib.lib.b200moe_quantize_1x128(None, 0, 128, None, None, None) == 0       # nothing to do
