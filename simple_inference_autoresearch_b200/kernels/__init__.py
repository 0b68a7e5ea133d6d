"""CUDA kernels of the library: build/load (``build``) and their Python face (``ops``)."""
from . import build, ops  # noqa: F401
