"""ferrox_b200: a single-GPU inference engine for Qwen2-MoE on B200 (sm_100a).

Public entry points: :class:`Engine` (``from_folder``, ``from_random``, ``step``,
``generate``), :func:`write_random_model`, the registries
(:func:`register_architecture`, :func:`register_part`) and the command line
(``python -m ferrox_b200``, ``bin/ferrox``, ``bin/trace_run``).
"""
from .config.registry import known_architectures, register_architecture, resolve  # noqa: F401
from .config.schema import ConfigError  # noqa: F401
from .models import qwen2_moe as _qwen2_moe  # noqa: F401  (registers the architecture)
from .parts.base import register_part  # noqa: F401
from .weights.loader import WeightsError  # noqa: F401
from .weights.random_init import write_random_model  # noqa: F401
from .weights.safetensors_io import SafetensorsError  # noqa: F401


def __getattr__(name):
    # the engine pulls in the kernel library; keep plain imports light
    if name in ("Engine", "StepEntry"):
        from .engine import batch, engine

        return {"Engine": engine.Engine, "StepEntry": batch.StepEntry}[name]
    raise AttributeError(name)


__version__ = "0.1.0"
