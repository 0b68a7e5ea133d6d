"""Sampling options (the kernel lives in ``csrc/sampling.cu``, its Python face in ``kernels.ops.sample``)."""
from .params import GREEDY, SamplingParams, request_seed, uniform_from_counter  # noqa: F401
