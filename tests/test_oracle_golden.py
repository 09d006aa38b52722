"""CPU: the oracle restatement against the committed golden vectors (outputs of the published
PyTorch reference of the operator definition, see tests/golden/make_golden.py)."""
import numpy as np
import pytest
import torch

import util
from util import O

CASES = ["tiny_ds_t33", "tiny_ds_t7_off16", "tiny_renorm_t20", "ds_v3_t16",
         "tiny_default_t20", "tiny_renormalize_t20", "tiny_llama4_t40", "tiny_topk_t20"]


@pytest.mark.parametrize("name", CASES)
def test_oracle_matches_golden(name):
    shape, d, g = util.golden_case(name)
    r = util.run_oracle(shape, d)
    # routing: identical expert sets, weights bit-identical (same torch ops on the same machine class)
    order = torch.argsort(r.topk_idx, dim=1)
    idx = r.topk_idx.gather(1, order).to(torch.int32).numpy()
    w = r.topk_w.gather(1, order).numpy()
    assert np.array_equal(idx, g["topk_idx_sorted"])
    assert np.allclose(w, g["topk_w_sorted"], rtol=1e-6, atol=0)
    # output: bit-identical bf16
    got = r.output.view(torch.int16).numpy()
    want = g["output_bf16_bits"]
    assert got.shape == want.shape
    same = (got == want).mean()
    rep = O.compare_output(r.output, torch.from_numpy(want).view(torch.bfloat16), atol=1e-3, rtol=1e-3)
    assert rep["fail_frac"] == 0.0, rep
    assert same > 0.999, same


def test_rows_without_local_expert_are_zero():
    shape, d, g = util.golden_case("tiny_ds_t7_off16")
    r = util.run_oracle(shape, d)
    off, El = d["local_expert_offset"], shape.num_local_experts
    local = ((r.topk_idx >= off) & (r.topk_idx < off + El)).any(dim=1)
    assert bool((r.output_f32[~local] == 0).all())


def test_weights_sum_to_scaling_factor():
    shape, d, g = util.golden_case("tiny_ds_t33")
    r = util.run_oracle(shape, d)
    assert torch.allclose(r.topk_w.sum(dim=1), torch.full((33,), 2.5), rtol=1e-5)


def test_compare_output_reports_failures():
    a = torch.zeros(4, 4, dtype=torch.bfloat16)
    b = a.clone(); b[0, 0] = 1.0
    rep = O.compare_output(a, b)
    assert rep["fail_frac"] == pytest.approx(1 / 16)
