"""A small, whole Llama inference library for one B200: configuration, weights,
parts, cache, step function, generation and hand-written sm_100a kernels."""
from .api import (LoadedModel, build_engine, build_model, generate, generate_with_stats, init_random,  # noqa: F401
                  load_model)
from .engine import Engine, StepEntry  # noqa: F401
from .kernels.options import KernelOptions  # noqa: F401
from .sampling import GREEDY, SamplingParams  # noqa: F401

__all__ = ["LoadedModel", "build_engine", "build_model", "generate", "generate_with_stats", "init_random",
           "load_model", "Engine", "StepEntry", "SamplingParams", "GREEDY", "KernelOptions"]
