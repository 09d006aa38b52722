"""B200-native FP8 block-scale MoE layer behind the reference's operator entry point.

`run` / `run_dps` keep the reference solutions' `main.py::run` signature; `MoELayer` is the
handle-based form for other shapes (e.g. the Qwen3-MoE shape) and for expert parallelism.
Importing this package loads libb200moe.so and raises if it is missing: there is no CPU or
PyTorch fallback.
"""
from .inputs import (DEEPSEEK_V3, QWEN3_MOE, TINY_DS, TINY_RENORM, MoEShape, ROUTING_DS,  # noqa: F401
                     ROUTING_RENORM_NAIVE)
from .main import MoELayer, run, run_dps  # noqa: F401
from ._lib import B200MoEError  # noqa: F401
