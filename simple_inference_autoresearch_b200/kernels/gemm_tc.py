"""bfloat16 matrix products on the 5th-generation tensor cores (tcgen05 + TMEM, fed by TMA).

``try_linear`` runs the product when the shape is one the unit takes (K a multiple
of 8, 16-byte aligned operands) and returns False otherwise, so that the caller
uses the CUDA-core kernel.
"""

from __future__ import annotations

import ctypes

import torch

from . import build

_state = {}
#: cap of the split along K for products with few output tiles (1 disables it)
max_splits = 8
_fn = None
enabled = True


def _bind():
    global _fn
    if _fn is None:
        lib = build.load_unit("gemm_tc")
        f = lib.siar_gemm_tc_bf16
        c = ctypes
        f.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int,
                      c.c_void_p, c.c_int, c.c_void_p]
        f.restype = c.c_int
        _fn = f
    return _fn


def _device_state(device: torch.device):
    key = device.index if device.index is not None else torch.cuda.current_device()
    st = _state.get(key)
    if st is None:
        st = {"sms": torch.cuda.get_device_properties(device).multi_processor_count}
        _state[key] = st
    return st


def try_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = 0) -> bool:
    """out[M, N] = x[M, K] @ w[N, K]^T; False when the shape is refused (nothing launched).
    ``epilogue=1``: w's rows alternate (gate, up) and out[M, N/2] = silu(gate) * up."""
    if not enabled:
        return False
    from . import ops

    fn = _bind()
    m, k = x.shape
    n = w.shape[0]
    st = _device_state(x.device)
    err = fn(x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, int(out.dtype == torch.float32), max_splits,
             int(epilogue), ops.status_word(x.device).data_ptr(), st["sms"], torch.cuda.current_stream().cuda_stream)
    if err == -1:
        return False
    if err != 0:
        raise RuntimeError(f"siar_gemm_tc_bf16 failed to launch: CUDA error {err}")
    ops.launch_count += 1
    return True
