"""Pack the library into flashinfer-bench solution manifests (the format of the reference's
goal_full_shape/fable-5.1/moe_fp8_fwd/<def>/solution.json: name, definition, author, spec{language,
target_hardware, entry_point, dependencies, destination_passing_style}, sources[{path, content}]).

    python solution/make_solution.py        # writes solution/solution.json and solution/solution_dps.json

Both manifests carry the same flat source set: this directory's main.py, the CUDA sources of
justgoal_b200/csrc/ and include/b200moe.h.  `--check` only verifies that the committed manifests are
up to date with the tree (exit code 1 if not).
"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
DEFINITION = "moe_fp8_block_scale_ds_routing_topk8_ng8_kg4_e32_h7168_i2048"
CSRC = ["b200moe.cu", "common.cuh", "routing.cuh", "permute.cuh", "front.cuh", "ep_p2p.cuh", "gemm.cuh", "gemm_pair.cuh", "quant.cuh"]


def sources():
    files = [("main.py", os.path.join(HERE, "main.py")), ("b200moe.h", os.path.join(ROOT, "include", "b200moe.h"))]
    files += [(f, os.path.join(ROOT, "justgoal_b200", "csrc", f)) for f in CSRC]
    return [{"path": name, "content": open(path).read()} for name, path in files]


def manifest(dps: bool):
    return {
        "name": "justgoal_b200_moe_fp8" + ("_dps" if dps else ""),
        "definition": DEFINITION,
        "author": "justgoal_b200",
        "spec": {"language": "python", "target_hardware": ["NVIDIA B200"],
                 "entry_point": "main.py::run_dps" if dps else "main.py::run", "dependencies": [],
                 "destination_passing_style": dps},
        "sources": sources(),
        "description": "Hand-written sm_100a kernels behind a C ABI: warp-per-token DeepSeek-V3 routing, stable "
                       "counting-sort permutation, tcgen05 FP8 grouped GEMMs with per-128-K promotion in fp32, "
                       "SwiGLU + two-term e4m3 requantisation, weighted combine with one bf16 rounding.",
    }


def main():
    out = {"solution.json": manifest(False), "solution_dps.json": manifest(True)}
    stale = False
    for name, m in out.items():
        path = os.path.join(HERE, name)
        text = json.dumps(m, indent=1) + "\n"
        if "--check" in sys.argv:
            stale |= not os.path.exists(path) or open(path).read() != text
        else:
            open(path, "w").write(text)
    if "--check" in sys.argv and stale:
        print("solution manifests are out of date: run python solution/make_solution.py")
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
