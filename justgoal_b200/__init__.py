"""B200-native FP8 block-scale MoE layer behind the reference's operator entry point.

`run` / `run_dps` keep the reference solutions' `main.py::run` signature; `MoELayer` is the
handle-based form for other shapes (e.g. the Qwen3-MoE shape) and for expert parallelism;
`HostPipeline` overlaps the host<->device copies of consecutive steps with the forward.
They are resolved on first use, which loads libb200moe.so and raises if it is missing (build
it with `python -m justgoal_b200.build`): there is no CPU or PyTorch fallback.
"""
from .inputs import (DEEPSEEK_V3, QWEN3_MOE, TINY_DS, TINY_RENORM, MoEShape, ROUTING_DS,  # noqa: F401
                     ROUTING_RENORM_NAIVE)

_LAZY = {"MoELayer": "main", "HostPipeline": "main", "run": "main", "run_dps": "main", "quantize_1x128": "main",
         "B200MoEError": "_lib"}


def __getattr__(name):
    mod = _LAZY.get(name)
    if mod is None:
        raise AttributeError(f"module 'justgoal_b200' has no attribute {name!r}")
    import importlib
    return getattr(importlib.import_module("." + mod, __name__), name)
