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
                      c.c_void_p, c.c_int, c.c_void_p, c.c_int, c.c_int]
        f.restype = c.c_int
        _fn = f
    return _fn


def _bind_fused():
    global _fn_fused
    if _fn_fused is None:
        f = build.load_unit("gemm_tc").siar_gemm_tc_bf16_fused
        c = ctypes
        f.argtypes = [c.c_void_p, c.c_void_p, c.c_void_p, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int, c.c_int,
                      c.c_void_p, c.c_int, c.c_void_p,
                      c.c_void_p, c.c_int, c.c_float,                         # ss_in, its parts, eps
                      c.c_void_p, c.c_int, c.c_void_p, c.c_void_p, c.c_int,   # ss_out, its parts, rb_out, next_w, next_w_f32
                      c.c_int, c.c_int]
        f.restype = c.c_int
        _fn_fused = f
    return _fn_fused


def ss_parts(m: int, n: int, k: int, device, options: KernelOptions = DEFAULT) -> int:
    """Parts per row of the sum of squares that an adding product [m, k] x [n, k]^T leaves for the norm
    that follows (the second dimension of ``ss_out``); 0 when a product of these sizes cannot."""
    if not options.use_tc_gemm:
        return 0
    f = build.load_unit("gemm_tc").siar_gemm_tc_ss_parts
    f.argtypes = [ctypes.c_int] * 7
    f.restype = ctypes.c_int
    return int(f(m, n, k, options.max_splits, _device_state(torch.device(device))["sms"], options.pair_mode,
                 options.tile_n))


def _device_state(device: torch.device):
    key = device.index if device.index is not None else torch.cuda.current_device()
    st = _state.get(key)
    if st is None:
        st = {"sms": torch.cuda.get_device_properties(device).multi_processor_count}
        _state[key] = st
    return st


def try_linear(x, w: torch.Tensor, out: torch.Tensor, epilogue: int = 0, normed=None, ss_out=None, rb_out=None,
               next_w=None, options: KernelOptions = DEFAULT) -> bool:
    """out[M, N] = x[M, K] @ w[N, K]^T; False when the shape is refused (nothing launched).
    ``epilogue=1``: w's rows alternate (gate, up) and out[M, N/2] = silu(gate) * up.
    ``epilogue=2``: out (float32) += the product.  With ``ss_out`` [M, ss_parts(...)] float32, ``rb_out``
    [M, N] bfloat16 and ``next_w`` [N] (the weight of the RMSNorm that follows) the kernel also leaves
    the rows' sums of squares of the new ``out`` in parts and bf16(out * next_w): what the product
    after that norm needs in place of the normed activations.
    ``normed`` (an ``ops.NormedResidual`` whose ``scaled`` is such a tensor; x is None): the product's
    rows are multiplied by the norm's factors rsqrt(mean square + eps) on the accumulators.
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
        consumer = (None, 0, 0.0)
        producer = (None, 0, None, None, 0)
        if normed is not None:
            x = normed.scaled
            assert x.dtype == torch.bfloat16 and x.is_contiguous() and normed.ss_parts.is_contiguous()
            assert normed.ss_parts.shape[0] == x.shape[0] and normed.ss_parts.dtype == torch.float32
            consumer = (normed.ss_parts.data_ptr(), normed.ss_parts.shape[1], float(normed.eps))
        m, k = x.shape
        assert k == w.shape[1]
        if ss_out is not None:
            assert rb_out is not None and next_w is not None and next_w.numel() == n and next_w.is_contiguous()
            assert ss_out.dtype == torch.float32 and ss_out.shape[0] == m and ss_out.is_contiguous()
            assert rb_out.dtype == torch.bfloat16 and rb_out.shape == (m, n) and rb_out.is_contiguous()
            assert next_w.dtype in (torch.float32, torch.bfloat16) and next_w.data_ptr() % 16 == 0
            producer = (ss_out.data_ptr(), ss_out.shape[1], rb_out.data_ptr(), next_w.data_ptr(),
                        int(next_w.dtype == torch.float32))
        err = _bind_fused()(x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, int(out.dtype == torch.float32),
                            options.max_splits, int(epilogue), status, st["sms"], stream, *consumer, *producer,
                            options.pair_mode, options.tile_n)
    else:
        m, k = x.shape
        err = _bind()(x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, int(out.dtype == torch.float32),
                      options.max_splits, int(epilogue), status, st["sms"], stream, options.pair_mode, options.tile_n)
    if err == -1:
        return False
    if err != 0:
        raise RuntimeError(f"the tensor-core product failed to launch: CUDA error {err}")
    ops.launch_count += 1
    return True
