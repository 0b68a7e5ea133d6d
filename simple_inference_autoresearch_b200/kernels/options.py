"""Which kernel runs where there is a choice: one immutable object instead of switches.

An ``Engine`` carries a ``KernelOptions``; a step hands it to the parts through the step
context, and the parts pass it to the functions of ``ops``.  Two engines in one process can
therefore differ, and a test compares two paths by building two engines (or by passing two
option objects to a kernel's function), never by flipping a module-level switch.  The
reference chooses its paths by environment variables read at import (``USE_TRITON``,
ops/rmsnorm.py:38; ``USE_CUDA_GRAPH``, model/llama.py:48-50).

Every choice changes rounding only: the results of all paths agree within the tolerances the
tests state.
"""

from __future__ import annotations

from dataclasses import dataclass, replace


@dataclass(frozen=True)
class KernelOptions:
    #: the products of a decode step add into the residual stream and make the next product's
    #: normed input themselves (no norm kernel between them); False: separate norm kernels
    fuse_residual_stream: bool = True
    #: prompts' attention on the tcgen05 kernel where its sizes allow; False: the warp-level kernel
    use_tc_attention: bool = True
    #: bfloat16 attention on the warp-level tensor-core kernels where their sizes allow; False:
    #: the CUDA-core kernels (this also rules out the tcgen05 kernel)
    use_mma_attention: bool = True
    #: a decode step's rotary encoding and cache write inside its attention kernel
    fuse_decode_rope: bool = True
    #: bfloat16 products on the tcgen05 kernels; False: the CUDA-core product
    use_tc_gemm: bool = True
    #: cap of the split along K for products with few output tiles (1 disables it; at most 8)
    max_splits: int = 8
    #: products of many rows on pairs of SMs (cta_group::2): 0 never, 1 from 4,096 rows on, 2 always
    pair_mode: int = 1
    #: output columns per tile of products of many rows (the persistent kernel): 0 = the width whose
    #: waves of tiles come out most even, or one of 128, 160, 192, 224, 256
    tile_n: int = 0
    #: a debugging mode: before every launch that follows the batch description and the block table
    #: into the cache (rotary + cache write, attention), the host reads them back and checks every
    #: index the kernels will form (slots, row ranges, lengths, pages) against the tensors' sizes, and
    #: raises with the first offender.  It synchronises, so it is off while a step is captured.
    check_arguments: bool = False

    def __post_init__(self):
        if self.tile_n not in (0, 128, 160, 192, 224, 256):
            raise ValueError(f"tile_n must be 0 or one of 128, 160, 192, 224, 256, got {self.tile_n}")
        if not 1 <= self.max_splits <= 8:
            raise ValueError(f"max_splits must be 1..8, got {self.max_splits}")
        if self.pair_mode not in (0, 1, 2):
            raise ValueError(f"pair_mode must be 0, 1 or 2, got {self.pair_mode}")

    def but(self, **changes) -> "KernelOptions":
        """A copy with some fields changed."""
        return replace(self, **changes)


DEFAULT = KernelOptions()
