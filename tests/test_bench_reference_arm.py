"""CPU: the reference arm of the benchmark (`bench.py --impl reference`: the oracle port timed on the host cores)
prints one JSON line with the contract's keys, for the decode configuration and for the whole-layer configuration
the scaling series runs on, without a GPU."""
import json
import os
import subprocess
import sys

import pytest

import util


def _run(*flags):
    r = subprocess.run([sys.executable, os.path.join(util.ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                        "--warmup", "0", *flags], capture_output=True, text=True, timeout=900,
                       env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    return json.loads(lines[0])


@pytest.mark.parametrize("flags,workload,scaling", [(("--workload", "decode"), "decode: T=64", "weak"),
                                                    ((), "ep: T=8192", "strong")])
def test_reference_arm_line(flags, workload, scaling):
    line = _run(*flags)
    assert line["impl"] == "reference" and line["metric"] == "moe_layer_tokens_per_s" and line["unit"] == "tokens/s"
    assert line["config"]["workload"].startswith(workload) and line["scaling"] == scaling
    assert line["higher_is_better"] is True and line["value"] > 0 and line["gpu_launches"] == 0
    cb = line["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == line["value"] and "pairs" in cb["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
