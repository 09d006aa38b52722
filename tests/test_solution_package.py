"""CPU: the flashinfer-bench packaging.  The committed manifests must be current with the tree, unpack
into a directory whose main.py imports on its own, expose the reference's entry-point signatures, and their
CUDA sources must compile for sm_100a into a library that exports the operator (no GPU needed for any of it)."""
import ctypes
import importlib.util
import inspect
import json
import os
import subprocess
import sys

import pytest

import util

SOL = os.path.join(util.ROOT, "solution")
ARGS = ["routing_logits", "routing_bias", "hidden_states", "hidden_states_scale", "gemm1_weights",
        "gemm1_weights_scale", "gemm2_weights", "gemm2_weights_scale", "local_expert_offset",
        "routed_scaling_factor"]


def _unpack(manifest, dst):
    for src in manifest["sources"]:
        path = os.path.join(dst, src["path"])
        os.makedirs(os.path.dirname(path), exist_ok=True)
        open(path, "w").write(src["content"])
    spec = importlib.util.spec_from_file_location("packed_solution_main", os.path.join(dst, "main.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_manifests_are_current():
    assert subprocess.run([sys.executable, os.path.join(SOL, "make_solution.py"), "--check"]).returncode == 0


@pytest.mark.parametrize("name,dps", [("solution.json", False), ("solution_dps.json", True)])
def test_manifest_fields_and_entry_point(name, dps, tmp_path):
    m = json.load(open(os.path.join(SOL, name)))
    assert m["definition"] == "moe_fp8_block_scale_ds_routing_topk8_ng8_kg4_e32_h7168_i2048"
    assert m["spec"]["language"] == "python" and m["spec"]["destination_passing_style"] is dps
    assert m["spec"]["dependencies"] == [] and "B200" in m["spec"]["target_hardware"][0]
    file, func = m["spec"]["entry_point"].split("::")
    assert file in [s["path"] for s in m["sources"]]
    mod = _unpack(m, str(tmp_path))
    fn = getattr(mod, func)
    assert list(inspect.signature(fn).parameters) == ARGS + (["output"] if dps else [])


def test_packed_sources_compile_and_export_the_operator(tmp_path, monkeypatch):
    m = json.load(open(os.path.join(SOL, "solution.json")))
    mod = _unpack(m, str(tmp_path / "src"))
    monkeypatch.setenv("B200MOE_BUILD_DIR", str(tmp_path / "build"))
    so = mod._build()
    assert os.path.isfile(so) and mod._build() == so          # the second call finds the cached build
    lib = ctypes.CDLL(so)
    for sym in ("b200moe_create", "b200moe_workspace_bytes", "b200moe_forward", "b200moe_strerror"):
        assert hasattr(lib, sym)
