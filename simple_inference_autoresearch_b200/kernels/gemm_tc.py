"""bfloat16 matrix products on the 5th-generation tensor cores (tcgen05 + TMEM, fed by TMA).

``try_linear`` runs the product when the shape is one the unit takes (K a multiple
of 8, 16-byte aligned operands) and returns False otherwise, so that the caller
uses the CUDA-core kernel.
"""

from __future__ import annotations

import ctypes

import torch

from . import build

from .options import DEFAULT, KernelOptions

_state = {}
_fn = None
_fn_fused = None


def _bind():
    global _fn
    if _fn is None:
        lib = build.load_unit("gemm_tc")
        f = lib.siar_gemm_tc_bf16
        c = ctypes
        f.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int,
                      c.c_void_p, c.c_int, c.c_void_p, c.c_int]
        f.restype = c.c_int
        _fn = f
    return _fn


def _bind_fused():
    global _fn_fused
    if _fn_fused is None:
        f = build.load_unit("gemm_tc").siar_gemm_tc_bf16_fused
        c = ctypes
        f.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int,
                      c.c_void_p, c.c_int, c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_void_p, c.c_float,
                      c.c_void_p, c.c_int]
        f.restype = c.c_int
        _fn_fused = f
    return _fn_fused


def _device_state(device: torch.device):
    key = device.index if device.index is not None else torch.cuda.current_device()
    st = _state.get(key)
    if st is None:
        st = {"sms": torch.cuda.get_device_properties(device).multi_processor_count}
        _state[key] = st
    return st


def try_linear(x, w: torch.Tensor, out: torch.Tensor, epilogue: int = 0, normed=None, ss_out=None,
               options: KernelOptions = DEFAULT) -> bool:
    """out[M, N] = x[M, K] @ w[N, K]^T; False when the shape is refused (nothing launched).
    ``epilogue=1``: w's rows alternate (gate, up) and out[M, N/2] = silu(gate) * up.
    ``epilogue=2``: out (float32) += the product; for at most 16 rows ``ss_out`` [M, ceil(N/128)]
    also receives partial sums of squares of the new rows of out (more than 128 rows: no sums;
    17..128 rows are refused).
    ``normed`` (an ``ops.NormedResidual`` of at most 16 rows; x is None): the kernel makes the
    activations rmsnorm(residual) * weight itself.
    ``options``: ``use_tc_gemm`` False refuses everything; ``max_splits`` and ``pair_mode`` as in ``KernelOptions``."""
    if not options.use_tc_gemm:
        return False
    from . import ops

    n = w.shape[0]
    dev = w.device
    st = _device_state(dev)
    status = ops.status_word(dev).data_ptr()
    stream = torch.cuda.current_stream().cuda_stream
    if normed is not None or epilogue == 2:
        if normed is not None:
            m, k = normed.residual.shape
            assert k == w.shape[1] and normed.ss_parts.shape[0] == m and normed.ss_parts.is_contiguous()
            extra = (normed.residual.data_ptr(), normed.ss_parts.data_ptr(), normed.ss_parts.shape[1],
                     normed.weight.data_ptr(), float(normed.eps))
            xp = None
        else:
            m, k = x.shape
            extra = (None, None, 0, None, 0.0)
            xp = x.data_ptr()
        err = _bind_fused()(xp, w.data_ptr(), out.data_ptr(), m, n, k, int(out.dtype == torch.float32),
                            options.max_splits, int(epilogue), status, st["sms"], stream, *extra,
                            None if ss_out is None else ss_out.data_ptr(), options.pair_mode)
    else:
        m, k = x.shape
        err = _bind()(x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, int(out.dtype == torch.float32),
                      options.max_splits, int(epilogue), status, st["sms"], stream, options.pair_mode)
    if err == -1:
        return False
    if err != 0:
        raise RuntimeError(f"the tensor-core product failed to launch: CUDA error {err}")
    ops.launch_count += 1
    return True
